"""The drop-in `fused_lut_linear_cuda` API (reference tensor layout) on the GPU against the golden vectors
produced by the reference's own PyTorch code, and against the CPU oracle at a second shape."""
import numpy as np
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, bf16_from_bits, check_status

pytestmark = pytest.mark.gpu


def test_hard_functional_against_reference_vectors(golden):
    import fused_lut_linear_cuda as F
    x = bf16_from_bits(golden["x"]).cuda().requires_grad_(True)
    pal = bf16_from_bits(golden["palette"]).cuda().requires_grad_(True)
    idx = torch.from_numpy(golden["indices"]).cuda()
    dy = bf16_from_bits(golden["dy"]).cuda()
    y = F.fused_lut_linear(x, pal, idx, None, int(golden["GS"]))
    y.backward(dy)
    check_status()
    assert_close(y, bf16_from_bits(golden["y_hard"]), "y vs torch_hard_forward")
    assert_close(x.grad, bf16_from_bits(golden["dx_hard"]), "dX vs autograd")
    assert_close(pal.grad, torch.from_numpy(golden["dpal_hard"]), "dPalette vs autograd", rel=2e-2)
    # larger batch goes through the tiled kernel instead of the small-M one
    xb = torch.cat([x.detach()] * 3)
    yb = F.fused_lut_linear(xb, pal.detach(), idx, None, int(golden["GS"]))
    assert_close(yb[: x.shape[0]], bf16_from_bits(golden["y_hard"]), "y (tiled kernel)")


def test_soft_functional_against_reference_vectors(golden):
    import fused_lut_linear_cuda as F
    x = bf16_from_bits(golden["x"]).cuda().requires_grad_(True)
    pal = bf16_from_bits(golden["palette"]).cuda().requires_grad_(True)
    lg = torch.from_numpy(golden["logits"]).cuda().requires_grad_(True)
    nz = torch.from_numpy(golden["noise"]).cuda()
    dy = bf16_from_bits(golden["dy"]).cuda()
    y = F.fused_lut_linear_soft(x, pal, lg, None, int(golden["GS"]), float(golden["tau"]), noise=nz)
    y.backward(dy)
    check_status()
    assert_close(y, bf16_from_bits(golden["y_soft"]), "y vs torch_soft_forward")
    assert_close(x.grad, bf16_from_bits(golden["dx_soft"]), "dX vs torch_soft_backward")
    assert lg.grad.dtype == torch.float16 and lg.grad.shape == lg.shape
    assert_close(lg.grad, torch.from_numpy(golden["dlogits_4kn"]), "dLogits vs torch_soft_backward (fp16)", rel=1e-2)
    assert_close(pal.grad, torch.from_numpy(golden["dpal_soft"]), "dPalette vs torch_soft_backward (bf16 out)", rel=2e-2)


def test_soft_functional_larger_shape_and_seed_counter():
    import fused_lut_linear_cuda as F
    M, K, N, GS, tau = 384, 512, 1024, 256, 0.9
    g = torch.Generator().manual_seed(21)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    pal = (torch.randn(N // GS, 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
    lg = torch.randn(4, K, N, generator=g).to(torch.float16)
    xs, ps, ls = x.cuda().requires_grad_(True), pal.cuda().requires_grad_(True), lg.cuda().requires_grad_(True)
    before = F._SOFT_STEP_SEED
    y = F.fused_lut_linear_soft(xs, ps, ls, None, GS, tau)
    assert F._SOFT_STEP_SEED == before + 1
    y.backward(dy.cuda())
    check_status()
    noise = O.gumbel_hash(F._SOFT_STEP_SEED, N, K)
    want = O.linear_step(x, dy, O.to_nk_logits(lg), noise, pal, tau, GS, K, lora=None, ste=True)
    assert_close(y, want["y"], "y")
    assert_close(xs.grad, want["dx"], "dX")
    assert_close(ls.grad, O.from_nk_logits(want["dlogits"]), "dLogits (fp16)", rel=1e-2)
    assert_close(ps.grad, want["dpalette"], "dPalette (bf16)", rel=2e-2)
    # pure soft forward (no straight-through estimator)
    y2 = F.fused_lut_linear_soft(x.cuda(), pal.cuda(), lg.cuda(), None, GS, tau, noise=O.from_nk_logits(noise).cuda(), ste=False)
    want2 = O.linear_step(x, None, O.to_nk_logits(lg), noise, pal, tau, GS, K, lora=None, ste=False)
    assert_close(y2, want2["y"], "y (pure soft)")


def test_reference_module_runs_on_this_backend(golden):
    """A module written like the reference's PalettizedLinear.forward dispatch (scripts/qwen_model.py:147-196)
    calls the two functionals with the reference's positional arguments."""
    import fused_lut_linear_cuda as F
    x = bf16_from_bits(golden["x"]).cuda()
    pal = bf16_from_bits(golden["palette"]).cuda()
    idx = torch.from_numpy(golden["indices"]).cuda()
    lg = torch.full((4,) + tuple(idx.shape), -10.0, dtype=torch.float16, device="cuda")
    for k in range(4):
        lg[k][idx == k] = 10.0          # one-hot initialisation, scripts/qwen_model.py:135-143
    y_hard = F.fused_lut_linear(x, pal, idx, None, 256)
    y_soft = F.fused_lut_linear_soft(x, pal, lg, None, 256, 1.0)
    check_status()
    assert torch.equal(y_hard, y_soft)   # same hard indices -> identical bits
