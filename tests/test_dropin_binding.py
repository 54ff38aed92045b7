"""plz_dropin.install() makes `import fused_lut_linear_cuda` resolve to this package and the Triton modules fail to import,
which is what sends the reference's PalettizedLinear to this library (scripts/qwen_model.py:104-130).

CPU part: the binding itself -- with a caller restated in tests/ref_like_module.py, and, where a reference checkout is
available (PLZ_REFERENCE_DIR), with the reference's own qwen_model.PalettizedLinear.  GPU part: forward + backward through
the bound modules against the CPU oracle."""
import os
import sys

import pytest
import torch

import plz_oracle as O

REF = os.environ.get("PLZ_REFERENCE_DIR")
HAVE_REF = bool(REF) and os.path.isdir(os.path.join(REF or "", "scripts"))


@pytest.fixture
def dropin(built_lib):
    import plz_dropin
    mod = plz_dropin.install()
    yield mod
    plz_dropin.uninstall()
    for n in ("qwen_model", "palettize_core"):
        sys.modules.pop(n, None)


def _inputs(K=256, N=512, gs=256, seed=7):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 4, (K, N), generator=g)
    pal = (torch.randn(N // gs, 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
    return idx, pal


def test_install_routes_the_imports(dropin):
    import fused_lut_linear_cuda as F
    import plz_dropin
    assert F is dropin and os.path.dirname(os.path.abspath(F.__file__)) == os.path.dirname(os.path.abspath(plz_dropin.__file__))
    with pytest.raises(ImportError):
        import triton_soft_forward  # noqa: F401
    with pytest.raises(ImportError):
        from triton_hard_forward import triton_hard_linear  # noqa: F401
    from ref_like_module import RefLikePalettizedLinear
    idx, pal = _inputs()
    m = RefLikePalettizedLinear(idx, pal, 256)
    assert plz_dropin.is_bound(m)
    assert len([n for n in dir(F._get_module()) if not n.startswith("_")]) == 10


def test_uninstall_restores(built_lib):
    import plz_dropin
    before = {n: sys.modules.get(n, "absent") for n in ("fused_lut_linear_cuda", "triton_soft_forward", "triton_hard_forward")}
    plz_dropin.install()
    plz_dropin.uninstall()
    after = {n: sys.modules.get(n, "absent") for n in before}
    assert before == after


@pytest.mark.skipif(not HAVE_REF, reason="needs a checkout of the reference (PLZ_REFERENCE_DIR)")
def test_reference_module_binds_to_this_library(dropin):
    """The reference's own file, imported unchanged; its scripts directory goes to sys.path[0] as qwen_model.py:27 does."""
    import plz_dropin
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(REF, "scripts"))
    try:
        import qwen_model
        assert os.path.abspath(qwen_model.__file__).startswith(os.path.abspath(REF))
        idx, pal = _inputs()
        lin = torch.nn.Linear(256, 512, bias=False)
        m = qwen_model.PalettizedLinear(lin, idx, 2, 4, 256, False, initial_palette=pal, use_soft_indices=True)
        assert m._use_cuda and not m._use_triton
        assert m._hard_kernel is dropin.fused_lut_linear and m._soft_kernel is dropin.fused_lut_linear_soft
        assert plz_dropin.is_bound(m)
        wrapped = qwen_model.QwenLoRA(m, rank=16, alpha=32, init="random")
        assert plz_dropin.is_bound(wrapped.base) and wrapped.scaling == 2.0
        # the batched helper finds the module by its attributes
        assert dropin.fused_compute_P_W_batched(torch.nn.Sequential(), 1.0, 1) == []
    finally:
        sys.path.remove(os.path.join(REF, "scripts"))


def _check_bound_module(make_module, make_lora, dev):
    """Eval (hard) and train (soft, one-hot logits => same weights) forward + backward through the bound module, LoRA on top,
    against the oracle's hard forward/backward plus the eager LoRA arithmetic on CPU."""
    from helpers import assert_close, check_status
    K, N, gs, M = 256, 512, 256, 200
    idx, pal = _inputs(K, N, gs)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(2, M // 2, K, generator=g).to(torch.bfloat16)
    dy = torch.randn(2, M // 2, N, generator=g).to(torch.bfloat16)
    m = make_module(idx.to(dev), pal.to(dev), gs)
    wrapped = make_lora(m, K, N).to(dev)
    w_nk = O.dequantize(idx.t().contiguous(), pal, gs, K)
    a, b, s = wrapped.lora_A.detach().cpu(), wrapped.lora_B.detach().cpu(), wrapped.scaling
    xf = x.reshape(-1, K)
    want_base = O.hard_forward(xf, w_nk)
    want_y = want_base + (((xf @ a) @ b.T) * s)
    want_dx_base, want_dpal = O.hard_backward(xf, dy.reshape(-1, N), idx.t().contiguous(), pal, gs, K)
    for mode in ("eval", "train"):
        wrapped.train(mode == "train")
        for p_ in wrapped.parameters():
            p_.grad = None
        xg = x.to(dev).requires_grad_(True)
        y = wrapped(xg)
        y.backward(dy.to(dev))
        check_status()
        assert_close(y.reshape(-1, N), want_y, f"{mode}: y")
        want_dx = want_dx_base.float() + ((dy.reshape(-1, N).float() @ b.float()) @ a.float().T) * s
        assert_close(xg.grad.reshape(-1, K), want_dx, f"{mode}: dX")
        assert_close(m.palette.grad, want_dpal, f"{mode}: dPalette", rel=2e-2)
        assert wrapped.lora_A.grad is not None and wrapped.lora_B.grad is not None
        if mode == "train":
            assert m.index_logits.grad is not None and m.index_logits.grad.dtype == torch.float16
            assert torch.isfinite(m.index_logits.grad.float()).all()


@pytest.mark.gpu
def test_bound_stand_in_module_forward_backward(dropin):
    from ref_like_module import RefLikeLoRA, RefLikePalettizedLinear
    import plz_dropin
    made = []

    def mk(idx, pal, gs):
        m = RefLikePalettizedLinear(idx, pal, gs)
        assert plz_dropin.is_bound(m)
        made.append(m)
        return m
    _check_bound_module(mk, lambda m, K, N: RefLikeLoRA(m, K, N), torch.device("cuda", 0))


@pytest.mark.gpu
@pytest.mark.skipif(not HAVE_REF, reason="needs a checkout of the reference (PLZ_REFERENCE_DIR)")
def test_bound_reference_module_forward_backward(dropin):
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(REF, "scripts"))
    try:
        import qwen_model

        def mk(idx, pal, gs):
            lin = torch.nn.Linear(idx.shape[0], idx.shape[1], bias=False)
            return qwen_model.PalettizedLinear(lin, idx, idx.shape[1] // gs, 4, gs, False, initial_palette=pal,
                                               use_soft_indices=True).to(idx.device)
        def lora(m, K, N):
            w = qwen_model.QwenLoRA(m, rank=16, alpha=32, init="random")
            with torch.no_grad():   # the reference initialises B to zero; give the branch something to do
                w.lora_B.copy_((torch.randn(N, 16, generator=torch.Generator().manual_seed(5)) * 0.01).to(torch.bfloat16))
            return w
        _check_bound_module(mk, lora, torch.device("cuda", 0))
    finally:
        sys.path.remove(os.path.join(REF, "scripts"))
