"""RMSNorm and SwiGLU folded into the hard forward, against the CPU oracle and against transformers' own modules."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


def _weights(N, K, seed):
    import plz_ops as ops
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
    pal = (torch.randn(N * (K // 256), 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
    w = ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, 1, 256)
    return w, O.dequantize(idx.long(), pal, 1, 256)


@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (300, 1024, 512), (1100, 2560, 1024)])
def test_rmsnorm_folded_into_the_forward(M, N, K):
    import plz_ops as ops
    g = torch.Generator().manual_seed(M)
    x = (torch.randn(M, K, generator=g) * 3).to(torch.bfloat16)
    gamma = (1 + 0.2 * torch.randn(K, generator=g)).to(torch.bfloat16)
    w, wd = _weights(N, K, 1)
    rstd = ops.rms_rstd(x.cuda(), 1e-6)
    assert_close(rstd, torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6), "rstd", rel=1e-5, cos=0.999999)
    y = ops.hard_forward_norm(w, x.cuda(), rstd, gamma.cuda())
    check_status()
    assert_close(y, O.rmsnorm(x, gamma) @ wd.float().t(), "y = rmsnorm(x) W^T")
    y_plain = ops.hard_forward_norm(w, x.cuda(), None, None)
    assert torch.equal(y_plain, ops.hard_forward(w, x.cuda())[0])   # no factors: same bits as the plain forward


@pytest.mark.parametrize("M,N,K,norm", [(128, 256, 256, False), (300, 1024, 512, True), (1100, 2560, 1024, True)])
def test_gate_up_swiglu_in_one_launch(M, N, K, norm):
    import plz_ops as ops
    g = torch.Generator().manual_seed(M + 1)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.2 * torch.randn(K, generator=g)).to(torch.bfloat16)
    wg, wgd = _weights(N, K, 2)
    wu, wud = _weights(N, K, 3)
    # palettes of ~0.02 give tiny pre-activations; scale x so that silu is exercised in its non-linear range
    x = (x.float() * 8).to(torch.bfloat16)
    rstd = ops.rms_rstd(x.cuda(), 1e-6) if norm else None
    act = ops.mlp_gate_up_forward(wg, wu, x.cuda(), rstd, gamma.cuda() if norm else None)
    check_status()
    assert_close(act, O.mlp_gate_up(x, wgd, wud, gamma if norm else None, normalize=norm), "silu(gate) * up")


def test_against_transformers_qwen3_modules():
    """The HuggingFace modules the reference runs around its Linears (transformers Qwen3RMSNorm + Qwen3MLP), with the
    MLP's three Linears set to the dequantized palettized weights."""
    tr = pytest.importorskip("transformers")
    from transformers.models.qwen3.modeling_qwen3 import Qwen3MLP, Qwen3RMSNorm
    import plz_ops as ops
    H, I, M = 512, 1024, 200
    cfg = tr.Qwen3Config(hidden_size=H, intermediate_size=I, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                         head_dim=128, rms_norm_eps=1e-6, vocab_size=128)
    g = torch.Generator().manual_seed(5)
    norm, mlp = Qwen3RMSNorm(H, eps=1e-6), Qwen3MLP(cfg)
    wg, wgd = _weights(I, H, 11)
    wu, wud = _weights(I, H, 12)
    wdn, wdd = _weights(H, I, 13)
    with torch.no_grad():
        norm.weight.copy_(1 + 0.1 * torch.randn(H, generator=g))
        mlp.gate_proj.weight.copy_(wgd.float()); mlp.up_proj.weight.copy_(wud.float()); mlp.down_proj.weight.copy_(wdd.float())
    x = (torch.randn(M, H, generator=g) * 6).to(torch.bfloat16)
    with torch.no_grad():
        want = mlp(norm(x.float()))
    xc = x.cuda()
    act = ops.mlp_gate_up_forward(wg, wu, xc, ops.rms_rstd(xc, 1e-6), norm.weight.detach().to(torch.bfloat16).cuda())
    y, _ = ops.hard_forward(wdn, act)
    check_status()
    assert_close(y, want, "down(silu(gate(norm(x))) * up(norm(x)))", rel=2e-2, cos=0.9995)
