"""Element-wise kernels of the decoder layer: each against a torch fp32 restatement of the transformers module it stands
for (Qwen3RMSNorm, apply_rotary_pos_emb with rotate_half, silu(gate) * up), and the fused forms against the unfused ones
bit for bit."""
import pytest
import torch

from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


def _rms_ref(x, w, eps):
    xf = x.float()
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16)
    return w * xn            # bf16 * bf16, as Qwen3RMSNorm returns weight * hidden.to(input_dtype)


@pytest.mark.parametrize("M,K", [(1, 2560), (5, 256), (700, 2560), (3000, 1024)])
def test_rmsnorm_forward(M, K):
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(M)
    x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(K, generator=g, device=dev)).to(torch.bfloat16)
    h, rstd = ops.rmsnorm_forward(x, w, 1e-6)
    check_status()
    assert_close(h, _rms_ref(x, w, 1e-6), "rmsnorm", rel=1e-2, cos=0.9999)
    assert_close(rstd, torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6), "rstd", rel=1e-5, cos=0.999999)


@pytest.mark.parametrize("M", [3, 64, 2000])
def test_add_rmsnorm_equals_add_then_rmsnorm(M):
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(M)
    K = 2560
    x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    y = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(K, generator=g, device=dev)).to(torch.bfloat16)
    s, h = ops.add_rmsnorm_forward(x, y, w, 1e-6)
    s_ref = ops.add(x, y)
    h_ref, _ = ops.rmsnorm_forward(s_ref, w, 1e-6)
    check_status()
    assert torch.equal(s, s_ref) and torch.equal(s, (x.float() + y.float()).to(torch.bfloat16))
    # a row's sum of squares is added in a different order by a block than by a warp: equal up to one bf16 step
    assert_close(h, h_ref, "fused norm", rel=8e-3, cos=0.99999)


def _rope_ref(x, w, cos, sin, H, S, eps):
    T = x.shape[0]
    xf = x.float().view(T, H, 128)
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16)
    y = (w * xn).float()
    pos = torch.arange(T, device=x.device) % S
    c = torch.cat([cos[pos], cos[pos]], -1)[:, None, :]
    s = torch.cat([sin[pos], sin[pos]], -1)[:, None, :]
    rot = torch.cat([-y[..., 64:], y[..., :64]], -1)
    return (y * c + rot * s).reshape(T, H * 128)


def test_qknorm_rope_forward_and_pair_launch():
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(2)
    B, S, Hq, Hk = 3, 40, 4, 2
    xq = torch.randn(B * S, Hq * 128, generator=g, device=dev).to(torch.bfloat16)
    xk = torch.randn(B * S, Hk * 128, generator=g, device=dev).to(torch.bfloat16)
    wq = (1 + 0.1 * torch.randn(128, generator=g, device=dev)).to(torch.bfloat16)
    wk = (1 + 0.1 * torch.randn(128, generator=g, device=dev)).to(torch.bfloat16)
    cos, sin = ops.rope_tables(S, 128, 1e6, dev)
    q = ops.qknorm_rope_forward(xq, wq, cos, sin, Hq, S)
    k = ops.qknorm_rope_forward(xk, wk, cos, sin, Hk, S)
    q2, k2 = ops.qknorm_rope_forward2(xq, wq, Hq, xk, wk, Hk, cos, sin, S)
    check_status()
    assert torch.equal(q, q2) and torch.equal(k, k2)
    assert_close(q, _rope_ref(xq, wq, cos, sin, Hq, S, 1e-6), "q norm + rope", rel=1e-2, cos=0.9999)
    assert_close(k, _rope_ref(xk, wk, cos, sin, Hk, S, 1e-6), "k norm + rope", rel=1e-2, cos=0.9999)
    # a decode step: S = 1 with the table rows of its position, output into a pitched cache slot
    pos = 17
    cache = torch.zeros(B, S, Hk * 128, dtype=torch.bfloat16, device=dev)
    xs = xk.view(B, S, -1)[:, pos].contiguous()
    ops.qknorm_rope_forward(xs, wk, cos[pos:pos + 1], sin[pos:pos + 1], Hk, 1, out=cache[:, pos])
    check_status()
    assert torch.equal(cache[:, pos], k.view(B, S, -1)[:, pos])
    assert cache[:, :pos].abs().sum() == 0 and cache[:, pos + 1:].abs().sum() == 0


def test_qknorm_rope_backward_matches_autograd():
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    B, S, H = 2, 24, 3
    x = torch.randn(B * S, H * 128, generator=g, device=dev).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(128, generator=g, device=dev)).to(torch.bfloat16)
    dy = torch.randn(B * S, H * 128, generator=g, device=dev).to(torch.bfloat16)
    cos, sin = ops.rope_tables(S, 128, 1e6, dev)
    dx, dw = ops.qknorm_rope_backward(x, w, cos, sin, dy, H, S)
    check_status()
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    xv = xf.view(B * S, H, 128)
    y = wf * (xv * torch.rsqrt(xv.pow(2).mean(-1, keepdim=True) + 1e-6))
    pos = torch.arange(B * S, device=dev) % S
    c = torch.cat([cos[pos], cos[pos]], -1)[:, None, :]
    s = torch.cat([sin[pos], sin[pos]], -1)[:, None, :]
    out = y * c + torch.cat([-y[..., 64:], y[..., :64]], -1) * s
    out.reshape(B * S, -1).backward(dy.float())
    assert_close(dx, xf.grad, "d x", rel=1e-2, cos=0.9999)
    assert_close(dw, wf.grad, "d weight", rel=1e-2, cos=0.9999)


def test_swiglu_and_add():
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(4)
    a = torch.randn(77, 512, generator=g, device=dev).to(torch.bfloat16)
    b = torch.randn(77, 512, generator=g, device=dev).to(torch.bfloat16)
    c = torch.randn(77, 512, generator=g, device=dev).to(torch.bfloat16)
    act = ops.swiglu_forward(a, b)
    want = torch.nn.functional.silu(a.float()).to(torch.bfloat16).float() * b.float()
    assert_close(act, want, "swiglu", rel=1e-2, cos=0.9999)
    assert torch.equal(ops.add(a, b), (a.float() + b.float()).to(torch.bfloat16))
    assert torch.equal(ops.add(a, b, c), (a.float() + b.float() + c.float()).to(torch.bfloat16))
    check_status()
