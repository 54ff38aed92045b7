"""Backward of the ops around the MLP Linears: SwiGLU and RMSNorm element-wise kernels against the CPU oracle, and the
recomputing backward of act = silu(h Wg^T) * (h Wu^T), h = rmsnorm(x), against torch autograd on the dequantized weights."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N", [(1, 8), (37, 264), (512, 9728)])
def test_swiglu_backward(M, N):
    import plz_ops as ops
    g = torch.Generator().manual_seed(M + N)
    gate = (torch.randn(M, N, generator=g) * 2).to(torch.bfloat16)
    up = torch.randn(M, N, generator=g).to(torch.bfloat16)
    dact = torch.randn(M, N, generator=g).to(torch.bfloat16)
    dg, du = ops.swiglu_backward(gate.cuda(), up.cuda(), dact.cuda())
    check_status()
    wg, wu = O.swiglu_backward(gate, up, dact)
    assert_close(dg, wg, "dGate", rel=5e-3)
    assert_close(du, wu, "dUp", rel=5e-3)
    # and torch autograd of the same expression
    gt, ut = gate.float().requires_grad_(), up.float().requires_grad_()
    (torch.nn.functional.silu(gt) * ut).backward(dact.float())
    assert_close(wg, gt.grad, "oracle dGate vs autograd", rel=1e-5)
    assert_close(wu, ut.grad, "oracle dUp vs autograd", rel=1e-5)


@pytest.mark.parametrize("M,K,with_weight", [(1, 64, True), (33, 2560, True), (300, 9728, True), (64, 1000, False), (5, 10240, True)])
def test_rmsnorm_backward(M, K, with_weight):
    import plz_ops as ops
    g = torch.Generator().manual_seed(M + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dh = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16) if with_weight else None
    rstd = ops.rms_rstd(x.cuda(), 1e-6)
    dx, dw = ops.rmsnorm_backward(x.cuda(), dh.cuda(), rstd, w.cuda() if w is not None else None)
    check_status()
    wx, ww = O.rmsnorm_backward(x, w, dh, 1e-6)
    assert_close(dx, wx, "dX", rel=5e-3)
    if with_weight:
        assert_close(dw, ww, "dWeight", rel=1e-4)
    xt = x.float().requires_grad_()
    wt = w.float().requires_grad_() if w is not None else None
    O.rmsnorm(xt, wt, 1e-6).backward(dh.float())
    assert_close(wx, xt.grad, "oracle dX vs autograd", rel=1e-5)
    if with_weight:
        assert_close(ww, wt.grad, "oracle dWeight vs autograd", rel=1e-5)


def test_mlp_front_backward_against_autograd():
    """Composite chain (two recomputed LUT GEMMs, SwiGLU backward, two dX products, RMSNorm backward): four bf16 roundings
    of intermediates lie between the inputs and dX, so the bound is 2e-2 / cosine 0.9998 instead of the single-GEMM 1e-2."""
    import plz_ops as ops
    M, N, K = 384, 768, 512
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    nw = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16)
    dact = torch.randn(M, N, generator=g).to(torch.bfloat16)
    ws, dense = [], []
    for _ in range(2):
        idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
        pal = (torch.randn(N * (K // 256), 4, generator=g) * 0.05).sort(-1).values.to(torch.bfloat16)
        ws.append(ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, 1, 256))
        dense.append(O.dequantize(idx.long(), pal, 1, 256).float())
    xc = x.cuda()
    rstd = ops.rms_rstd(xc, 1e-6)
    dx, dg, dgate, dup = ops.mlp_front_backward(ws[0], ws[1], xc, rstd, nw.cuda(), dact.cuda())
    check_status()
    xt, wt = x.float().requires_grad_(), nw.float().requires_grad_()
    O.mlp_gate_up(xt, dense[0], dense[1], wt, 1e-6).backward(dact.float())
    assert_close(dx, xt.grad, "dX", rel=2e-2, cos=0.9998)
    assert_close(dg, wt.grad, "dNormWeight", rel=2e-2, cos=0.9998)
    h = O.rmsnorm(x, nw, 1e-6)
    wg, wu = O.swiglu_backward(h @ dense[0].t(), h @ dense[1].t(), dact)
    assert_close(dgate, wg, "dGate", rel=1e-2)
    assert_close(dup, wu, "dUp", rel=1e-2)


@pytest.mark.parametrize("M,N,K", [(300, 384, 512), (1000, 1280, 768)])
def test_gate_up_forward_keeps_preactivations(M, N, K):
    """keep=True: same act as the plain fused launch bit for bit, gate / up equal to the single-matrix norm-folded forward,
    and the backward from the kept tensors equals the recomputing backward."""
    import plz_ops as ops
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    nw = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16).cuda()
    dact = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    ws = []
    for _ in range(2):
        idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
        pal = (torch.randn(N * (K // 256), 4, generator=g) * 0.05).sort(-1).values.to(torch.bfloat16)
        ws.append(ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, 1, 256))
    rstd = ops.rms_rstd(x, 1e-6)
    act0 = ops.mlp_gate_up_forward(ws[0], ws[1], x, rstd, nw)
    act, gate, up = ops.mlp_gate_up_forward(ws[0], ws[1], x, rstd, nw, keep=True)
    check_status()
    assert torch.equal(act, act0)
    assert_close(gate, ops.hard_forward_norm(ws[0], x, rstd, nw), "kept gate", rel=4e-3)
    assert_close(up, ops.hard_forward_norm(ws[1], x, rstd, nw), "kept up", rel=4e-3)
    a = ops.mlp_front_backward(ws[0], ws[1], x, rstd, nw, dact, gate=gate, up=up)
    b = ops.mlp_front_backward(ws[0], ws[1], x, rstd, nw, dact)
    for u, v, name in zip(a, b, ("dX", "dG", "dGate", "dUp")):
        assert_close(u, v, name + " kept vs recomputed", rel=1e-2)
