"""The reference extension's lower-level functions (scripts/fused_lut_linear_cuda.py:721-732) served by this library, the bias
epilogue / bias gradient, and the packed-index cache of the drop-in module, against the CPU oracle.

These functions pass P, W_soft / W_hard and dW between calls as tensors in the reference's layouts: logits (4, K, N) fp16,
P (4, K, N) or (K, N, 4) fp16, W (K, N) bf16, palette (N / gs, 4) bf16, noise from the counter-based sampler."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu

K, N, GS, M, TAU = 256, 512, 256, 160, 0.8


def _inputs(seed=3):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    pal = (torch.randn(N // GS, 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
    lg = torch.randn(4, K, N, generator=g).to(torch.float16)
    return x, dy, pal, lg


def _oracle_soft(pal, lg, seed):
    noise = O.gumbel_hash(seed, N, K)                      # [N, K, 4], index (k * N + n) * 4 + p
    p, w_soft, hard, w_hard = O.soft_weights(O.to_nk_logits(lg), noise, pal, TAU, GS, K)
    return p, w_soft, hard, w_hard


def test_soft_forward_functions():
    import fused_lut_linear_cuda as F
    ext = F._get_module()
    x, dy, pal, lg = _inputs()
    seed = 77
    p, w_soft, _, _ = _oracle_soft(pal, lg, seed)          # p [N, K, 4], w_soft [N, K]
    xs, ps, ls = x.cuda(), pal.cuda(), lg.cuda()
    y, P4, W = ext.fused_lut_linear_soft_fwd(xs, ps, ls, GS, TAU, seed)
    check_status()
    assert P4.shape == (4, K, N) and P4.dtype == torch.float16 and W.shape == (K, N) and W.dtype == torch.bfloat16
    assert_close(P4.permute(2, 1, 0), p, "P planar", rel=2e-3)
    assert_close(W.t(), w_soft, "W_soft", rel=1e-2)
    assert_close(y, x.float() @ W.float().cpu(), "y = x @ W")
    Pa, W2 = ext.fused_lut_linear_soft_fwd_aos(xs, ps, ls, GS, TAU, seed)
    assert Pa.shape == (K, N, 4) and torch.equal(Pa.permute(2, 0, 1), P4) and torch.equal(W2, W)
    # sum of P is 1, W_soft inside the palette range (the reference's own checks, scripts/test_triton_soft_forward.py:168-189)
    assert (Pa.float().sum(-1) - 1).abs().max().item() < 2e-3
    lo, hi = pal.float().min(-1).values, pal.float().max(-1).values
    Wg = W.float().cpu().reshape(K, N // GS, GS)
    assert (Wg >= lo[None, :, None] - 1e-3).all() and (Wg <= hi[None, :, None] + 1e-3).all()
    # with_hard: hard index = argmax of the noised probabilities
    Pa3, Ws3, Wh3 = ext.fused_lut_linear_soft_fwd_with_hard(xs, ps, ls, GS, TAU, seed)
    check_status()
    assert torch.equal(Pa3, Pa) and torch.equal(Ws3, W)
    hard_noisy = Pa.float().argmax(-1).cpu()                                   # (K, N), first maximum
    want_wh = O.dequantize(hard_noisy.t().contiguous(), pal, GS, K)            # [N, K]
    # fp16 rounding of P can merge two near-equal maxima; compare where the top two differ clearly
    top2 = Pa.float().cpu().topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 2e-3
    assert torch.equal(Wh3.cpu().t()[clear.t()], want_wh[clear.t()])
    assert clear.float().mean().item() > 0.95


def test_batched_equals_per_layer_with_layer_seeds():
    """scripts/test_batched_compute_pw.py:237-260: layer i of the batched call uses step_seed ^ (i * 0x9E3779B9)."""
    import fused_lut_linear_cuda as F
    ext = F._get_module()
    shapes = [(256, 512), (128, 256), (256, 768)]
    g = torch.Generator().manual_seed(9)
    lgs = [torch.randn(4, k, n, generator=g).to(torch.float16).cuda() for k, n in shapes]
    pals = [(torch.randn(n // GS, 4, generator=g) * 0.02).to(torch.bfloat16).cuda() for k, n in shapes]
    step_seed = 1234
    flat = ext.fused_compute_P_W_batched(lgs, pals, GS, TAU, step_seed)
    check_status()
    assert len(flat) == 6
    for i, (lg, pal) in enumerate(zip(lgs, pals)):
        seed_i = step_seed ^ ((i * 0x9E3779B9) & 0xFFFFFFFF)
        Pa, W = ext.fused_lut_linear_soft_fwd_aos(None, pal, lg, GS, TAU, seed_i)
        assert torch.equal(flat[2 * i], Pa) and torch.equal(flat[2 * i + 1], W)
    # the module-walking helper
    class PalettizedLinear(torch.nn.Module):     # recognised by name and attributes
        def __init__(self, lg, pal):
            super().__init__()
            self.index_logits, self.palette, self.group_size, self._use_cuda = lg, pal, GS, True
    net = torch.nn.Sequential(*[PalettizedLinear(a, b) for a, b in zip(lgs, pals)])
    pairs = F.fused_compute_P_W_batched(net, TAU, step_seed)
    assert len(pairs) == 3 and all(torch.equal(pairs[i][0], flat[2 * i]) for i in range(3))


def test_soft_backward_functions():
    import fused_lut_linear_cuda as F
    import plz_ops as ops
    ext = F._get_module()
    x, dy, pal, lg = _inputs(5)
    seed = 5
    xs, dys, ps, ls = x.cuda(), dy.cuda(), pal.cuda(), lg.cuda()
    Pa, W = ext.fused_lut_linear_soft_fwd_aos(xs, ps, ls, GS, TAU, seed)
    P4 = Pa.permute(2, 0, 1).contiguous()
    # oracle on the SAME fp16-rounded P (the reference's backward reads the stored fp16 P)
    p_nk4 = Pa.float().cpu().permute(1, 0, 2).contiguous()
    w_fwd = W.t().contiguous().cpu()
    _, want_dl, want_dpal, want_dw = O.soft_backward(x, dy, w_fwd, p_nk4, pal, GS, K)
    gw = ops.weight_grad(xs, dys, "kn")
    check_status()
    assert_close(gw.t(), want_dw, "grad_W = x^T grad_y (K, N) fp32")
    assert_close(ops.weight_grad(xs, dys, "nk"), want_dw, "grad_W [N, K]")
    want_dl_4kn = O.from_nk_logits(want_dl)
    for name, out in (("soft_bwd (fp32 dW, planar P)", ext.fused_lut_linear_soft_bwd(gw, P4, ps, GS)),
                      ("soft_bwd_elementwise (bf16 dW, AoS P)", ext.soft_bwd_elementwise(gw.to(torch.bfloat16), Pa, ps, GS)),
                      ("soft_bwd_fused (planar P)", ext.fused_lut_linear_soft_bwd_fused(dys, xs, P4, ps, GS)),
                      ("soft_bwd_fused_aos", ext.fused_lut_linear_soft_bwd_fused_aos(dys, xs, Pa, ps, GS))):
        gl, gp = out
        check_status()
        assert gl.shape == (4, K, N) and gl.dtype == torch.float16 and gp.shape == (N // GS, 4) and gp.dtype == torch.bfloat16
        tol = 2e-2 if "bf16 dW" in name else 1e-2
        assert_close(gl, want_dl_4kn, f"{name}: grad_logits", rel=tol)
        assert_close(gp, want_dpal, f"{name}: grad_palette", rel=2e-2)


def test_hard_functions_and_bias():
    import fused_lut_linear_cuda as F
    ext = F._get_module()
    x, dy, pal, _ = _inputs(8)
    g = torch.Generator().manual_seed(8)
    idx = torch.randint(0, 4, (K, N), generator=g).to(torch.int8)
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    w_nk = O.dequantize(idx.t().long().contiguous(), pal, GS, K)
    want_y = (x.float() @ w_nk.float().t() + bias.float()).to(torch.bfloat16)
    xs, dys, ps, ids, bs = x.cuda(), dy.cuda(), pal.cuda(), idx.cuda(), bias.cuda()
    y = ext.fused_lut_linear_fwd(xs, ps, ids, bs, GS)
    check_status()
    assert_close(y, want_y, "y with bias (fp32 add in the epilogue)")
    gx, gp, gb = ext.fused_lut_linear_bwd(dys, xs, ps, ids, bs, GS, True, True)
    check_status()
    want_dx, want_dpal = O.hard_backward(x, dy, idx.t().long().contiguous(), pal, GS, K)
    assert_close(gx, want_dx, "grad_x")
    assert_close(gp, want_dpal, "grad_palette", rel=2e-2)
    assert_close(gb, dy.float().sum(0), "grad_bias", rel=1e-2)
    gx2, gp2, gb2 = ext.fused_lut_linear_bwd(dys, xs, ps, ids, None, GS, False, False)
    assert gx2 is None and gp2 is None and gb2 is None
    # autograd path with a trainable bias, ragged M and an odd number of row blocks for the column sum
    xb = torch.cat([xs] * 5)[:777].requires_grad_(True)
    bp = bs.clone().requires_grad_(True)
    yb = F.fused_lut_linear(xb, ps, ids, bp, GS)
    dyb = torch.cat([dys] * 5)[:777]
    yb.backward(dyb)
    check_status()
    assert_close(bp.grad, dyb.float().sum(0), "bias.grad", rel=1e-2)
    assert_close(yb[:M], want_y, "y with bias, larger batch")


def test_pack_cache_is_not_fooled_by_temporaries():
    """Two different same-shape index tensors of a dtype that needs a conversion, back to back: the conversion's temporary
    may land on the address the previous call's temporary had, which must not return the previous packed weights."""
    import fused_lut_linear_cuda as F
    x, _, pal, _ = _inputs(12)
    xs, ps = x.cuda(), pal.cuda()
    g = torch.Generator().manual_seed(12)
    for trial in range(4):
        idx = torch.randint(0, 4, (K, N), generator=g)                 # int64
        y = F.fused_lut_linear(xs, ps, idx.cuda(), None, GS)           # converted inside; temporary freed on return
        want = O.hard_forward(x, O.dequantize(idx.t().contiguous(), pal, GS, K))
        assert_close(y, want, f"int64 indices, call {trial}")
        idx_t = torch.randint(0, 4, (N, K), generator=g).to(torch.int8).cuda().t()   # int8 but not contiguous
        y = F.fused_lut_linear(xs, ps, idx_t, None, GS)
        want = O.hard_forward(x, O.dequantize(idx_t.t().long().cpu().contiguous(), pal, GS, K))
        assert_close(y, want, f"strided int8 indices, call {trial}")
    # a frozen int8 buffer is cached, and the cache follows in-place updates (version counter) and the tensor's lifetime
    buf = torch.randint(0, 4, (K, N), generator=g).to(torch.int8).cuda()
    n0 = len(F._PACK_CACHE)
    y1 = F.fused_lut_linear(xs, ps, buf, None, GS)
    y1b = F.fused_lut_linear(xs, ps, buf, None, GS)
    assert len(F._PACK_CACHE) == n0 + 1 and torch.equal(y1, y1b)
    buf.copy_(torch.randint(0, 4, (K, N), generator=g).to(torch.int8))
    y2 = F.fused_lut_linear(xs, ps, buf, None, GS)
    assert_close(y2, O.hard_forward(x, O.dequantize(buf.t().long().cpu().contiguous(), pal, GS, K)), "after an in-place update")
    del buf
    assert len(F._PACK_CACHE) == n0
    check_status()
