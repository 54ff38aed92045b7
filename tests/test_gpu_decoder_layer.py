"""The palettized decoder layer (all kernels of this library) against transformers' Qwen3DecoderLayer in fp32 on the CPU
with the same weights (dequantized palettes + merged LoRA), forward and backward.

The reference project pins nothing at this boundary (it calls the HuggingFace layer as a black box), so the HuggingFace
module at the installed version is the checker by construction.  The bf16 pipeline is compared with an fp32 one across
fourteen chained ops, hence the looser bound than for a single GEMM: max rel err 3e-2, cosine 0.999."""
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


def _hf_layer(cfg, P):
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    from transformers.models.qwen3.modeling_qwen3 import Qwen3DecoderLayer, Qwen3RotaryEmbedding
    hc = Qwen3Config(hidden_size=cfg.hidden, num_attention_heads=cfg.n_heads, num_key_value_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                     intermediate_size=cfg.intermediate, rms_norm_eps=cfg.eps, rope_theta=cfg.rope_theta, num_hidden_layers=1,
                     vocab_size=64, attention_bias=False, attention_dropout=0.0, max_position_embeddings=4096)
    hc._attn_implementation = "sdpa"
    layer = Qwen3DecoderLayer(hc, 0).float()
    import plz_ops as ops
    dense = {}
    with torch.no_grad():
        for name, mod in (("q", layer.self_attn.q_proj), ("k", layer.self_attn.k_proj), ("v", layer.self_attn.v_proj), ("o", layer.self_attn.o_proj),
                          ("gate", layer.mlp.gate_proj), ("up", layer.mlp.up_proj), ("down", layer.mlp.down_proj)):
            lp = P.lin[name]
            w = ops.dequantize(lp.w).float().cpu()
            w_eff = w + lp.scale * (lp.lora_b.float().cpu() @ lp.lora_a.float().cpu())
            mod.weight.copy_(w_eff)
            dense[name] = mod
        layer.input_layernorm.weight.copy_(P.input_ln.float().cpu())
        layer.post_attention_layernorm.weight.copy_(P.post_ln.float().cpu())
        layer.self_attn.q_norm.weight.copy_(P.q_norm.float().cpu())
        layer.self_attn.k_norm.weight.copy_(P.k_norm.float().cpu())
    return layer, Qwen3RotaryEmbedding(hc), dense


@pytest.mark.parametrize("B,S", [(2, 128), (1, 384)])
def test_layer_matches_transformers(B, S):
    import decoder_layer as DL
    import plz_ops as ops
    cfg = DL.LayerConfig(hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, intermediate=512, lora_rank=16, lora_scale=2.0)
    dev = torch.device("cuda", 0)
    P = DL.random_layer(cfg, dev, seed=3)
    g = torch.Generator().manual_seed(B + S)
    x = torch.randn(B * S, cfg.hidden, generator=g).to(torch.bfloat16)
    dy = torch.randn(B * S, cfg.hidden, generator=g).to(torch.bfloat16)
    cos, sin = ops.rope_tables(S, cfg.head_dim, cfg.rope_theta, dev)
    y, ctx = DL.layer_forward(cfg, P, x.to(dev), B, S, cos, sin)
    dx, grads = DL.layer_backward(cfg, P, ctx, dy.to(dev), B, S, cos, sin)
    check_status()

    layer, rot, dense = _hf_layer(cfg, P)
    xf = x.float().reshape(B, S, cfg.hidden).clone().requires_grad_(True)
    pos = torch.arange(S)[None, :].expand(B, S)
    out = layer(xf, attention_mask=None, position_ids=pos, position_embeddings=rot(xf, pos))
    out = out[0] if isinstance(out, tuple) else out
    out.backward(dy.float().reshape(B, S, cfg.hidden))
    tol = dict(rel=3e-2, cos=0.999)
    assert_close(y, out.detach().reshape(B * S, -1), "layer output", **tol)
    assert_close(dx, xf.grad.reshape(B * S, -1), "input gradient", **tol)
    assert_close(grads["input_ln"], layer.input_layernorm.weight.grad, "d input_layernorm", **tol)
    assert_close(grads["post_ln"], layer.post_attention_layernorm.weight.grad, "d post_attention_layernorm", **tol)
    assert_close(grads["q_norm"], layer.self_attn.q_norm.weight.grad, "d q_norm", **tol)
    assert_close(grads["k_norm"], layer.self_attn.k_norm.weight.grad, "d k_norm", **tol)
    for name in DL.LINEARS:
        lp = P.lin[name]
        dw = dense[name].weight.grad                                          # [N, K] fp32, gradient of W + s B A
        idx = ops.unpack_indices(lp.w.packed, lp.w.K, n_major=True).long().cpu()
        N, K = idx.shape
        grp = (torch.arange(N)[:, None] * (K // 256) + torch.arange(K)[None, :] // 256)
        want_dpal = torch.zeros(N * (K // 256) * 4).index_add_(0, (grp * 4 + idx).reshape(-1), dw.reshape(-1)).reshape(-1, 4)
        dpal, da, db = grads[name]
        assert_close(dpal, want_dpal, f"{name}: dPalette", **tol)
        assert_close(da, lp.scale * (lp.lora_b.float().cpu().t() @ dw), f"{name}: dA", **tol)
        assert_close(db, lp.scale * (dw @ lp.lora_a.float().cpu().t()), f"{name}: dB", **tol)


def test_stack_of_layers_runs_and_is_deterministic():
    import decoder_layer as DL
    import plz_ops as ops
    cfg = DL.LayerConfig(hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, intermediate=512)
    dev = torch.device("cuda", 0)
    layers = [DL.random_layer(cfg, dev, seed=s) for s in range(3)]
    B, S = 2, 256
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(B * S, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
    dy = torch.randn(B * S, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
    cos, sin = ops.rope_tables(S, cfg.head_dim, cfg.rope_theta, dev)
    y1, dx1, g1 = DL.stack_forward_backward(cfg, layers, x, dy, B, S, cos, sin)
    y2, dx2, g2 = DL.stack_forward_backward(cfg, layers, x, dy, B, S, cos, sin)
    check_status()
    assert torch.isfinite(y1.float()).all() and torch.isfinite(dx1.float()).all()
    assert torch.equal(y1, y2) and torch.equal(dx1, dx2)
    # norm-weight gradients are fp32 atomic column sums: equal up to summation order
    assert len(g1) == 3 and torch.allclose(g1[0]["input_ln"], g2[0]["input_ln"], rtol=1e-4, atol=1e-4)
