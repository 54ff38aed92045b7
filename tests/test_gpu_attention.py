"""Causal grouped-query attention (tcgen05 kernels) against a plain PyTorch fp32 reference of the same op, forward and
backward.  The reference project has no attention code (it calls transformers' decoder layer), so the checker here is the
textbook formula in fp32, softmax(q k^T / sqrt(d) + causal mask) v with the kv heads repeated over their query group, which is
what transformers' eager attention computes; tolerance: the bf16 contract of the GEMM tests (max rel err 1e-2, cosine 0.9999)."""
import pytest
import torch

from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


def _ref(q, k, v, do, B, S, Hq, Hkv, D):
    qf = q.float().reshape(B, S, Hq, D).transpose(1, 2).clone().requires_grad_(True)      # [B, Hq, S, D]
    kf = k.float().reshape(B, S, Hkv, D).transpose(1, 2).clone().requires_grad_(True)
    vf = v.float().reshape(B, S, Hkv, D).transpose(1, 2).clone().requires_grad_(True)
    g = Hq // Hkv
    kr, vr = kf.repeat_interleave(g, dim=1), vf.repeat_interleave(g, dim=1)
    s = (qf @ kr.transpose(-1, -2)) * D ** -0.5
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ vr
    o.backward(do.float().reshape(B, S, Hq, D).transpose(1, 2))
    back = lambda t, H: t.transpose(1, 2).reshape(B * S, H * D)
    return back(o.detach(), Hq), lse.detach(), back(qf.grad, Hq), back(kf.grad, Hkv), back(vf.grad, Hkv)


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 4, 1), (1, 512, 8, 2), (3, 384, 4, 4), (1, 1152, 2, 1)])
def test_attention_forward_backward(B, S, Hq, Hkv):
    import plz_ops as ops
    D = 128
    g = torch.Generator().manual_seed(B * 100 + S + Hq)
    q = torch.randn(B * S, Hq * D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(B * S, Hkv * D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(B * S, Hkv * D, generator=g).to(torch.bfloat16).cuda()
    do = torch.randn(B * S, Hq * D, generator=g).to(torch.bfloat16).cuda()
    o, lse = ops.attention_forward(q, k, v, B, S, Hq, Hkv)
    check_status()
    want_o, want_lse, want_dq, want_dk, want_dv = _ref(q, k, v, do, B, S, Hq, Hkv, D)
    assert_close(o, want_o, "o")
    assert_close(lse, want_lse, "log-sum-exp", rel=1e-3)
    dq, dk, dv = ops.attention_backward(q, k, v, o, do, lse, B, S, Hq, Hkv)
    check_status()
    assert_close(dq, want_dq, "dQ")
    assert_close(dk, want_dk, "dK")
    assert_close(dv, want_dv, "dV")
    # deterministic: no atomics anywhere
    o2, _ = ops.attention_forward(q, k, v, B, S, Hq, Hkv)
    dq2, dk2, dv2 = ops.attention_backward(q, k, v, o, do, lse, B, S, Hq, Hkv)
    assert torch.equal(o, o2) and torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


def test_attention_on_slices_of_a_fused_projection():
    """q, k, v as column slices of ONE [M, (Hq + 2 Hkv) * 128] matrix (a fused qkv projection output): rows are pitched."""
    import plz_ops as ops
    B, S, Hq, Hkv, D = 2, 256, 4, 2, 128
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16).cuda()
    q, k, v = qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:]
    o, lse = ops.attention_forward(q, k, v, B, S, Hq, Hkv)
    check_status()
    o2, lse2 = ops.attention_forward(q.contiguous(), k.contiguous(), v.contiguous(), B, S, Hq, Hkv)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)


def test_attention_argument_checks():
    import plz_native as P
    import plz_ops as ops
    q = torch.zeros(100, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(P.PlzError):
        ops.attention_forward(q, q, q, 1, 100, 1, 1)            # S not a multiple of 128
    q = torch.zeros(128, 3 * 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(128, 2 * 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(P.PlzError):
        ops.attention_forward(q, k, k, 1, 128, 3, 2)            # 3 query heads over 2 kv heads
