"""Soft forward + full backward (native layout, explicit Gumbel noise) on the GPU against the CPU oracle."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, assert_close_rows, check_status

pytestmark = pytest.mark.gpu


def _inputs(M, N, K, seed=0, rank=16):
    import synth
    return synth.make_linear_inputs(M, N, K, seed=seed, rank=rank)


def _run(d, tau, ste, lora=True, noise="tensor", seed=0):
    import palettized_linear as PL
    c = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    lo = (c["lora_a"], c["lora_b"], d["lora_scale"]) if lora else None
    nz = {"tensor": c["noise"], "hash": "hash", "none": None}[noise]
    return PL.linear_step(c["x"], c["dy"], c["palette"].reshape(-1, 4), c["logits"], nz, tau, lora=lo, ste=ste, seed=seed)


def _oracle(d, tau, ste, lora=True, noise=None):
    lo = (d["lora_a"], d["lora_b"], d["lora_scale"]) if lora else None
    return O.linear_step(d["x"], d["dy"], d["logits"], noise, d["palette"], tau, 1, 256, lora=lo, ste=ste)


@pytest.mark.parametrize("M,N,K,tau,ste", [(128, 256, 256, 1.0, True), (300, 512, 512, 1.0, True),
                                           (512, 768, 1024, 0.5, True), (300, 512, 512, 2.0, False)])
def test_linear_step_matches_oracle(M, N, K, tau, ste):
    d = _inputs(M, N, K, seed=M + N)
    got = _run(d, tau, ste)
    check_status()
    want = _oracle(d, tau, ste, noise=d["noise"])
    import numpy as np
    hard = O.pack_rows(want["hard"].to(torch.uint8).numpy())
    assert np.array_equal(got["packed"].cpu().numpy(), hard), "hard indices must be bit exact"
    assert_close(got["y"], want["y"], "y")
    assert_close(got["dx"], want["dx"], "dX")
    assert_close(got["dlogits"], want["dlogits"], "dLogits")
    assert_close(got["dpalette"], want["dpalette"], "dPalette")
    assert_close(got["da"], want["da"], "dA")
    assert_close(got["db"], want["db"], "dB")
    # the same bound per palette group / per LoRA row, so that small-magnitude rows are checked on their own scale
    assert_close_rows(got["dpalette"], want["dpalette"], "dPalette per group")
    assert_close_rows(got["da"], want["da"], "dA per rank row")
    assert_close_rows(got["db"], want["db"], "dB per weight row")


def test_linear_step_without_lora_and_noise():
    d = _inputs(200, 256, 512, seed=3)
    got = _run(d, 1.3, True, lora=False, noise="none")
    check_status()
    want = _oracle(d, 1.3, True, lora=False, noise=None)
    for k in ("y", "dx", "dlogits", "dpalette"):
        assert_close(got[k], want[k], k)


def test_linear_step_counter_based_noise():
    d = _inputs(200, 256, 512, seed=4)
    got = _run(d, 1.0, True, noise="hash", seed=77)
    check_status()
    want = _oracle(d, 1.0, True, noise=O.gumbel_hash(77, 256, 512))
    for k in ("y", "dx", "dlogits", "dpalette"):
        assert_close(got[k], want[k], k)


def test_backward_is_deterministic():
    d = _inputs(300, 512, 512, seed=5)
    a = _run(d, 1.0, True)
    b = _run(d, 1.0, True)
    for k in ("y", "dx", "dlogits", "dpalette"):
        assert torch.equal(a[k], b[k]), k


def test_module_autograd_matches_functional():
    import palettized_linear as PL
    d = _inputs(64 * 3, 256, 256, seed=6)
    m = PL.PalettizedLinear(256, 256, rank=16, lora_scale=1.0)
    with torch.no_grad():
        m.palette.copy_(d["palette"].cuda()); m.index_logits.copy_(d["logits"].cuda())
        m.lora_A.copy_(d["lora_a"].cuda()); m.lora_B.copy_(d["lora_b"].cuda())
    m.noise = d["noise"].cuda()
    m.train()
    x = d["x"].cuda().reshape(3, 64, 256).requires_grad_(True)
    y = m(x)
    y.backward(d["dy"].cuda().reshape(3, 64, 256))
    check_status()
    want = _oracle(d, 1.0, True, noise=d["noise"])
    assert_close(y.reshape(-1, 256), want["y"], "y")
    assert_close(x.grad.reshape(-1, 256), want["dx"], "dX")
    assert_close(m.index_logits.grad, want["dlogits"], "dLogits")
    assert_close(m.palette.grad.reshape(-1, 4), want["dpalette"], "dPalette (bf16)", rel=2e-2)
    assert_close(m.lora_A.grad, want["da"], "dA (bf16)", rel=2e-2)
    m.eval(); m.extract_hard_indices()
    ye = m(d["x"].cuda())
    assert_close(ye, want["y"], "eval y")


@pytest.mark.parametrize("limit", [3, 7])
def test_persistent_schedule_with_few_ctas(limit):
    """Few CTAs: every CTA walks several tiles of the weight-gradient kernel and the last round is cut into
    half tiles; all outputs must still match the oracle."""
    import plz_native as P
    d = _inputs(300, 1024, 768, seed=11)
    P.lib().plz_set_cta_limit(limit)
    try:
        got = _run(d, 1.0, True)
        check_status()
    finally:
        P.lib().plz_set_cta_limit(0)
    want = _oracle(d, 1.0, True, noise=d["noise"])
    for k in ("y", "dx", "dlogits", "dpalette", "da", "db"):
        assert_close(got[k], want[k], k)
