"""Hard forward / backward of the palettized Linear on the GPU against the CPU oracle."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


def _make(M, N, K, gs_n, gs_k, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
    pal = (torch.randn((N // gs_n) * (K // gs_k), 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
    return x, dy, idx, pal


def _weight(idx, pal, N, K, gs_n, gs_k):
    import plz_ops as ops
    return ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, gs_n, gs_k)


SHAPES = [
    # M, N, K, gs_n, gs_k
    (128, 256, 64, 1, 64),        # one tile, one stage
    (128, 256, 512, 1, 256),      # pipeline wraps
    (100, 512, 256, 1, 256),      # ragged M inside one 128-row tile
    (300, 768, 1024, 1, 256),     # two M tiles per CTA, ragged
    (512, 1024, 512, 256, 512),   # reference grouping: one palette per 256 output columns
    (257, 320, 192, 1, 64),       # N not a multiple of the 256-wide tile
]


@pytest.mark.parametrize("M,N,K,gs_n,gs_k", SHAPES)
def test_hard_forward(M, N, K, gs_n, gs_k):
    import plz_ops as ops
    x, dy, idx, pal = _make(M, N, K, gs_n, gs_k)
    w = _weight(idx, pal, N, K, gs_n, gs_k)
    y, _ = ops.hard_forward(w, x.cuda())
    check_status()
    assert_close(y, O.hard_forward(x, O.dequantize(idx.long(), pal, gs_n, gs_k)), "y")


@pytest.mark.parametrize("M,N,K,gs_n,gs_k", SHAPES)
def test_backward_dx(M, N, K, gs_n, gs_k):
    import plz_ops as ops
    if N % 64:
        pytest.skip("dX needs N % 64 == 0")
    x, dy, idx, pal = _make(M, N, K, gs_n, gs_k, seed=1)
    w = _weight(idx, pal, N, K, gs_n, gs_k)
    dx, _ = ops.backward_dx(w, dy.cuda())
    check_status()
    want, _ = O.hard_backward(x, dy, idx.long(), pal, gs_n, gs_k)
    assert_close(dx, want, "dX")


@pytest.mark.parametrize("M,N,K,gs_n,gs_k", [(128, 256, 256, 1, 256), (300, 512, 512, 1, 256), (200, 512, 256, 256, 256),
                                             (512, 1024, 512, 256, 512)])
def test_hard_palette_gradient(M, N, K, gs_n, gs_k):
    import plz_ops as ops
    x, dy, idx, pal = _make(M, N, K, gs_n, gs_k, seed=2)
    w = _weight(idx, pal, N, K, gs_n, gs_k)
    dpal = ops.backward_dw_hard(w, x.cuda(), dy.cuda())
    check_status()
    _, want = O.hard_backward(x, dy, idx.long(), pal, gs_n, gs_k)
    assert_close(dpal, want, "dPalette")


@pytest.mark.parametrize("rank", [16, 32])
def test_hard_forward_with_lora(rank):
    import plz_ops as ops
    M, N, K = 300, 512, 512
    x, dy, idx, pal = _make(M, N, K, 1, 256, seed=4)
    g = torch.Generator().manual_seed(8)
    a = (torch.randn(rank, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    b = (torch.randn(N, rank, generator=g) * 0.05).to(torch.bfloat16)
    w = _weight(idx, pal, N, K, 1, 256)
    lora = (a.cuda(), b.cuda(), 2.0)
    y, t = ops.hard_forward(w, x.cuda(), lora)
    dx, dt = ops.backward_dx(w, dy.cuda(), lora)
    da, db = ops.lora_backward(x.cuda(), dy.cuda(), t, dt)
    check_status()
    wd = O.dequantize(idx.long(), pal, 1, 256)
    want_y = (x.float() @ wd.float().t() + O.lora_forward(x, a, b, 2.0)).to(torch.bfloat16)
    dxl, want_da, want_db = O.lora_backward(x, dy, a, b, 2.0)
    assert_close(y, want_y, "y + LoRA")
    assert_close(t, (x.float() @ a.float().t() * 2.0), "t = s x A^T")
    assert_close(dx, (dy.float() @ wd.float() + dxl), "dX + LoRA")
    assert_close(da, want_da, "dA")
    assert_close(db, want_db, "dB")


def test_forward_is_deterministic():
    import plz_ops as ops
    x, dy, idx, pal = _make(300, 512, 512, 1, 256, seed=6)
    w = _weight(idx, pal, 512, 512, 1, 256)
    xc = x.cuda()
    y1 = ops.hard_forward(w, xc)[0].clone()
    y2 = ops.hard_forward(w, xc)[0]
    assert torch.equal(y1, y2)


def test_empty_batch_is_a_no_op():
    import plz_ops as ops
    x, dy, idx, pal = _make(1, 256, 64, 1, 64)
    w = _weight(idx, pal, 256, 64, 1, 64)
    y, _ = ops.hard_forward(w, torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (0, 256)


@pytest.mark.parametrize("limit", [1, 3, 5])
def test_persistent_schedule_with_few_ctas(limit):
    """Restrict the persistent kernels to a few CTAs so that every CTA walks several tiles (and the last,
    partially filled round is cut into half tiles): results must not change."""
    import plz_native as P
    import plz_ops as ops
    M, N, K = 1100, 1024, 512
    x, dy, idx, pal = _make(M, N, K, 1, 256, seed=9)
    g = torch.Generator().manual_seed(10)
    a = (torch.randn(16, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    b = (torch.randn(N, 16, generator=g) * 0.05).to(torch.bfloat16)
    w = _weight(idx, pal, N, K, 1, 256)
    lora = (a.cuda(), b.cuda(), 1.0)
    P.lib().plz_set_cta_limit(limit)
    try:
        y, t = ops.hard_forward(w, x.cuda(), lora)
        dx, dt = ops.backward_dx(w, dy.cuda(), lora)
        dpal = ops.backward_dw_hard(w, x.cuda(), dy.cuda())
        check_status()
    finally:
        P.lib().plz_set_cta_limit(0)
    wd = O.dequantize(idx.long(), pal, 1, 256)
    dxl, _, _ = O.lora_backward(x, dy, a, b, 1.0)
    assert_close(y, (x.float() @ wd.float().t() + O.lora_forward(x, a, b, 1.0)), "y")
    assert_close(dx, (dy.float() @ wd.float() + dxl), "dX")
    assert_close(dpal, O.hard_backward(x, dy, idx.long(), pal, 1, 256)[1], "dPalette")


@pytest.mark.parametrize("N,K,gs_n,gs_k", [(768, 512, 1, 256), (512, 256, 256, 256), (1024, 512, 256, 512), (320, 192, 1, 64)])
def test_in_gemm_decode_is_bit_exact(N, K, gs_n, gs_k):
    """x = I makes every output the sum of ONE weight times 1 plus zeros, which is exact in fp32 and in the bf16 store:
    y = I W^T must equal the gathered weights bit for bit (decode inside the forward GEMM), and dX = I W likewise (decode
    inside the dX GEMM), for both palette groupings."""
    import plz_ops as ops
    g = torch.Generator().manual_seed(N + K)
    idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
    pal = (torch.randn((N // gs_n) * (K // gs_k), 4, generator=g) * 0.02).to(torch.bfloat16)
    pal[pal == 0] = 0.0078125
    w = _weight(idx, pal, N, K, gs_n, gs_k)
    wd = O.dequantize(idx.long(), pal, gs_n, gs_k)                       # [N, K] bf16, pure gather
    assert torch.equal(ops.dequantize(w).cpu(), wd)
    eye_k = torch.eye(K, dtype=torch.bfloat16, device="cuda")
    y, _ = ops.hard_forward(w, eye_k)                                     # [K, N] = W^T
    check_status()
    assert torch.equal(y.cpu(), wd.t()), "forward GEMM decode"
    if N % 64 == 0:
        eye_n = torch.eye(N, dtype=torch.bfloat16, device="cuda")
        dx, _ = ops.backward_dx(w, eye_n)                                 # [N, K] = W
        check_status()
        assert torch.equal(dx.cpu(), wd), "dX GEMM decode"
    # the small-M kernels: 16 rows of the identity at a time
    for k0 in range(0, K, 16):
        for rows in ((16, 1) if k0 == 0 else (16,)):
            ys = ops.hard_forward_smallm(w, eye_k[k0:k0 + rows].contiguous())  # [rows, N]
            assert torch.equal(ys.cpu(), wd[:, k0:k0 + rows].t()), f"small-M decode, columns {k0}..{k0 + rows}"
    y64 = ops.hard_forward_smallm(w, eye_k[:64].contiguous())
    assert torch.equal(y64.cpu(), wd[:, :64].t()), "small-M (17..64 rows) decode"
    check_status()
