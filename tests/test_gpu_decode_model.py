"""Whole-model inference (prefill + token decode against the key / value cache) against transformers' Qwen3ForCausalLM in
fp32 on the CPU with the same (dequantized) weights, and the decode-attention kernel against a direct softmax.

The reference project holds no test at this boundary (it calls the HuggingFace model); the HuggingFace implementation at the
installed version is the checker.  A bf16 pipeline is compared with an fp32 one: max rel err 3e-2, cosine 0.999."""
import pytest
import torch

from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,Hq,Hkv", [(1, 2049, 32, 8), (3, 130, 4, 2), (8, 777, 8, 8), (64, 96, 8, 2), (2, 1, 16, 2), (2, 333, 16, 2)])
def test_decode_attention_matches_softmax(B, T, Hq, Hkv):
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(T)
    Tmax = T + 5
    q = torch.randn(B, Hq * 128, generator=g, device=dev).to(torch.bfloat16)
    kc = torch.randn(B, Tmax, Hkv * 128, generator=g, device=dev).to(torch.bfloat16)
    vc = torch.randn(B, Tmax, Hkv * 128, generator=g, device=dev).to(torch.bfloat16)
    out = ops.attention_decode(q, kc, vc, T, Hq, Hkv)
    check_status()
    qf = q.float().view(B, Hkv, Hq // Hkv, 128)
    kf = kc[:, :T].float().view(B, T, Hkv, 128).permute(0, 2, 1, 3)          # [B, Hkv, T, 128]
    vf = vc[:, :T].float().view(B, T, Hkv, 128).permute(0, 2, 1, 3)
    p = torch.softmax(qf @ kf.transpose(-1, -2) * 128 ** -0.5, dim=-1)
    want = (p @ vf).reshape(B, Hq * 128)
    assert_close(out, want, "decode attention", rel=1e-2, cos=0.9999)


def test_embed_gather():
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    table = torch.randn(1000, 256, device=dev).to(torch.bfloat16)
    ids = torch.randint(0, 1000, (7, 33), device=dev)
    assert torch.equal(ops.embed_gather(table, ids), table[ids.reshape(-1)])


def _hf_model(cfg, model):
    import plz_ops as ops
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    from transformers.models.qwen3.modeling_qwen3 import Qwen3ForCausalLM
    hc = Qwen3Config(hidden_size=cfg.hidden, num_attention_heads=cfg.n_heads, num_key_value_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                     intermediate_size=cfg.intermediate, rms_norm_eps=cfg.eps, rope_theta=cfg.rope_theta, num_hidden_layers=cfg.n_layers,
                     vocab_size=cfg.vocab, attention_bias=False, attention_dropout=0.0, max_position_embeddings=4096,
                     tie_word_embeddings=True, use_sliding_window=False)
    hc._attn_implementation = "sdpa"
    hf = Qwen3ForCausalLM(hc).float().eval()
    with torch.no_grad():
        hf.model.embed_tokens.weight.copy_(model.embed.float().cpu())
        hf.model.norm.weight.copy_(model.final_norm.float().cpu())
        for L, hl in zip(model.layers, hf.model.layers):
            for name, mod in (("q", hl.self_attn.q_proj), ("k", hl.self_attn.k_proj), ("v", hl.self_attn.v_proj), ("o", hl.self_attn.o_proj),
                              ("gate", hl.mlp.gate_proj), ("up", hl.mlp.up_proj), ("down", hl.mlp.down_proj)):
                mod.weight.copy_(ops.dequantize(L[name]).float().cpu())
            hl.input_layernorm.weight.copy_(L["input_ln"].float().cpu())
            hl.post_attention_layernorm.weight.copy_(L["post_ln"].float().cpu())
            hl.self_attn.q_norm.weight.copy_(L["q_norm"].float().cpu())
            hl.self_attn.k_norm.weight.copy_(L["k_norm"].float().cpu())
    hf.tie_weights()
    return hf


@pytest.mark.parametrize("B", [2, 20])
def test_prefill_and_decode_match_transformers(B):
    import decode_model as DM
    cfg = DM.ModelConfig(hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, intermediate=512, n_layers=2, vocab=512)
    dev = torch.device("cuda", 0)
    model = DM.PalettizedQwen.random(cfg, dev, seed=5, max_positions=512)
    # a livelier embedding than the 0.02 init so that the logits are not all alike
    model.embed = (torch.randn(cfg.vocab, cfg.hidden, device=dev) * 0.5).to(torch.bfloat16)
    S, steps = 128, 3
    ids = torch.randint(0, cfg.vocab, (B, S + steps), device=dev)
    cache = model.new_cache(B, S + steps)
    _, logits0 = model.prefill(ids[:, :S], cache)
    got = [logits0]
    for t in range(steps):
        got.append(model.decode_step(ids[:, S + t].contiguous(), cache))
    check_status()
    assert cache.length == S + steps

    hf = _hf_model(cfg, model)
    with torch.no_grad():
        want = hf(ids.cpu()).logits                        # full causal pass: position p predicts from tokens 0..p
    tol = dict(rel=3e-2, cos=0.999)
    assert_close(got[0], want[:, S - 1], "prefill logits", **tol)
    for t in range(steps):
        assert_close(got[1 + t], want[:, S + t], f"decode step {t} logits", **tol)


def test_decode_graph_replays_the_eager_step():
    import decode_model as DM
    cfg = DM.ModelConfig(hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, intermediate=512, n_layers=2, vocab=512)
    dev = torch.device("cuda", 0)
    model = DM.PalettizedQwen.random(cfg, dev, seed=6, max_positions=512)
    B, S = 4, 128
    ids = torch.randint(0, cfg.vocab, (B, S + 1), device=dev)
    cache = model.new_cache(B, S + 1)
    model.prefill(ids[:, :S], cache, want_logits=False)
    step_ids = ids[:, S].contiguous()
    eager = model.decode_logits(step_ids, cache, S)
    graph, out = model.decode_graph(step_ids, cache, S)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    check_status()
    # the small-M kernels meet their K groups in shared memory in no fixed order: equal up to the last bf16 bit
    assert_close(out, eager, "graph replay", rel=1e-2, cos=0.9999)
