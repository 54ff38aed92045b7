"""Inference through a whole Qwen3-shaped model whose Linears are hard-palettized: prefill of a prompt batch and token
decode against a bf16 key / value cache, every op a kernel of libplz.so.

This is the hard (eval) path of the reference's wrapped model (scripts/qwen_model.py:164-192 inside the HuggingFace layers,
scripts/qwen_model.py:897-951): embed_tokens -> n_layers x [RMSNorm, q/k/v, q/k norm + RoPE, attention, o, residual, RMSNorm,
gate/up, SwiGLU, down, residual] -> final RMSNorm -> logits against the tied embedding table.

  prefill      token batches of B x S (S a multiple of 128): tcgen05 LUT GEMMs and the causal attention kernel; keys (after
               RoPE) and values go into the cache.
  decode_step  one token per sequence: the small-M LUT kernels (q/k/v and gate/up each one launch), the new key / value
               written straight into the cache by the kernels that produce them, attention over the cache, logits by the dense
               GEMM against the embedding table.  All pointers of a step are fixed once the position is known, so a step can
               be captured in a CUDA graph and replayed (decode_graph).
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)

import plz_native as P  # noqa: E402
import plz_ops as ops  # noqa: E402
from decoder_layer import LINEARS, LayerConfig  # noqa: E402


@dataclass
class ModelConfig(LayerConfig):
    n_layers: int = 36
    vocab: int = 151936


@dataclass
class KVCache:
    k: torch.Tensor      # bf16 [n_layers, B, T_max, n_kv_heads * head_dim], keys after q/k norm and RoPE
    v: torch.Tensor
    length: int = 0      # positions filled


class PalettizedQwen:
    def __init__(self, cfg: ModelConfig, layers, embed: torch.Tensor, final_norm: torch.Tensor, max_positions: int = 4096):
        """layers: list of dicts with the seven PackedWeight under LINEARS and bf16 vectors 'input_ln', 'post_ln', 'q_norm', 'k_norm'."""
        self.cfg, self.layers, self.embed, self.final_norm = cfg, layers, embed, final_norm
        self.cos, self.sin = ops.rope_tables(max_positions, cfg.head_dim, cfg.rope_theta, embed.device)
        self.fused_mlp = False    # prefill: gate + up + SwiGLU as ONE single-CTA launch instead of two CTA-pair GEMMs + an element-wise
                                  # pass; measured slower at 8 x 2048 tokens (4.0 against 3.4 ms per layer), so off

    @classmethod
    def random(cls, cfg: ModelConfig, device, seed: int = 0, max_positions: int = 4096):
        """Random-init model: indices uniform, palettes sorted N(0, 0.02^2) 4-tuples (one per row and 256 input columns), norm
        weights 1 + N(0, 0.1^2), embedding N(0, 0.02^2)."""
        g = torch.Generator(device=device).manual_seed(seed)
        layers = []
        for _ in range(cfg.n_layers):
            L = {}
            for name, (N, K) in cfg.shapes().items():
                idx = torch.randint(0, 4, (N, K), generator=g, device=device, dtype=torch.uint8)
                pal = (torch.randn(N * (K // 256), 4, generator=g, device=device) * 0.02).sort(-1).values.to(torch.bfloat16)
                L[name] = ops.PackedWeight(ops.pack_indices(idx.view(torch.int8), n_major=True), pal, N, K, 1, 256)
                del idx
            for name, n in (("input_ln", cfg.hidden), ("post_ln", cfg.hidden), ("q_norm", cfg.head_dim), ("k_norm", cfg.head_dim)):
                L[name] = (1.0 + 0.1 * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)
            layers.append(L)
        embed = (torch.randn(cfg.vocab, cfg.hidden, generator=g, device=device) * 0.02).to(torch.bfloat16)
        fin = (1.0 + 0.1 * torch.randn(cfg.hidden, generator=g, device=device)).to(torch.bfloat16)
        return cls(cfg, layers, embed, fin, max_positions)

    def weight_bytes(self) -> int:
        """Bytes of packed indices and palettes of all layers (what a decode step must read, the embedding table aside)."""
        return sum(L[n].packed.numel() * L[n].packed.element_size() + L[n].palette.numel() * 2 for L in self.layers for n in LINEARS)

    def new_cache(self, B: int, T_max: int) -> KVCache:
        c = self.cfg
        shape = (c.n_layers, B, T_max, c.n_kv_heads * c.head_dim)
        dev = self.embed.device
        return KVCache(torch.zeros(shape, dtype=torch.bfloat16, device=dev), torch.zeros(shape, dtype=torch.bfloat16, device=dev), 0)

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        """Final RMSNorm and the tied-embedding head: bf16 [rows, vocab]."""
        hn, _ = ops.rmsnorm_forward(h, self.final_norm, self.cfg.eps)
        return self.head(hn)

    def head(self, hn: torch.Tensor) -> torch.Tensor:
        """Logits bf16 [rows, vocab] of already normalised hidden states (tied embedding table)."""
        return ops.dense_forward(self.embed, hn)[0]

    def decode_logits(self, ids: torch.Tensor, cache: KVCache, pos: int | None = None) -> torch.Tensor:
        """One decode step up to the logits, with the small kernels of the chain allowed to start under their predecessors
        (programmatic dependent launch; the weights are read-only here). Does not advance cache.length."""
        lib = P.lib()
        lib.plz_set_smallm_overlap(1)
        try:
            return self.head(self.decode_hidden(ids, cache, pos)[1])
        finally:
            lib.plz_set_smallm_overlap(0)

    # ---- prefill -------------------------------------------------------------------------------------------------
    def prefill(self, ids: torch.Tensor, cache: KVCache, want_logits: bool = True):
        """ids int64 [B, S] (S a multiple of 128) into an EMPTY cache. Returns (hidden bf16 [B * S, hidden], logits of the last
        position of every sequence bf16 [B, vocab] or None)."""
        c = self.cfg
        B, S = ids.shape
        assert cache.length == 0 and S <= cache.k.shape[2] and S % 128 == 0
        cos, sin = self.cos[:S], self.sin[:S]
        h = ops.embed_gather(self.embed, ids)
        h1, _ = ops.rmsnorm_forward(h, self.layers[0]["input_ln"], c.eps)
        n = len(self.layers)
        for li, L in enumerate(self.layers):
            q_raw = ops.hard_forward(L["q"], h1)[0]
            k_raw = ops.hard_forward(L["k"], h1)[0]
            v = ops.hard_forward(L["v"], h1)[0]
            q, k = ops.qknorm_rope_forward2(q_raw, L["q_norm"], c.n_heads, k_raw, L["k_norm"], c.n_kv_heads, cos, sin, S, c.eps)
            a, _ = ops.attention_forward(q, k, v, B, S, c.n_heads, c.n_kv_heads, c.head_dim)
            cache.k[li, :, :S].copy_(k.view(B, S, -1))
            cache.v[li, :, :S].copy_(v.view(B, S, -1))
            o = ops.hard_forward(L["o"], a)[0]
            if self.fused_mlp:
                # gate and up in one launch with the RMSNorm folded in and the SwiGLU epilogue: act is the only [M, N] tensor written
                x2 = ops.add(h, o)
                act = ops.mlp_gate_up_forward(L["gate"], L["up"], x2, ops.rms_rstd(x2, c.eps), L["post_ln"])
            else:
                x2, h2 = ops.add_rmsnorm_forward(h, o, L["post_ln"], c.eps)
                act = ops.swiglu_forward(ops.hard_forward(L["gate"], h2)[0], ops.hard_forward(L["up"], h2)[0])
            d = ops.hard_forward(L["down"], act)[0]
            # the residual add closes the layer and the same pass applies the next layer's (or the final) norm
            h, h1 = ops.add_rmsnorm_forward(x2, d, self.layers[li + 1]["input_ln"] if li + 1 < n else self.final_norm, c.eps)
        cache.length = S
        last = self.head(h1.view(B, S, -1)[:, -1].contiguous()) if want_logits else None
        return h, last

    # ---- decode --------------------------------------------------------------------------------------------------
    def _small(self, ws, x, outs=None):
        if x.shape[0] <= 16:
            return ops.hard_forward_smallm_multi(ws, x, outs)
        return [ops.hard_forward_smallm(w, x, out=(outs[i] if outs is not None else None)) for i, w in enumerate(ws)]

    def decode_hidden(self, ids: torch.Tensor, cache: KVCache, pos: int | None = None):
        """One token per sequence (ids int64 [B]) at position pos (default: cache.length): writes its key / value into the cache
        and returns (final hidden state, its final RMSNorm), bf16 [B, hidden] each. Does not advance cache.length."""
        c = self.cfg
        B = ids.shape[0]
        pos = cache.length if pos is None else pos
        assert pos < cache.k.shape[2] and pos < self.cos.shape[0]
        cos, sin = self.cos[pos:pos + 1], self.sin[pos:pos + 1]
        h = ops.embed_gather(self.embed, ids)
        h1, _ = ops.rmsnorm_forward(h, self.layers[0]["input_ln"], c.eps)
        n = len(self.layers)
        for li, L in enumerate(self.layers):
            q_raw, k_raw, _ = self._small([L["q"], L["k"], L["v"]], h1, [None, None, cache.v[li, :, pos]])
            q, _ = ops.qknorm_rope_forward2(q_raw, L["q_norm"], c.n_heads, k_raw, L["k_norm"], c.n_kv_heads, cos, sin, 1, c.eps,
                                            out_k=cache.k[li, :, pos])
            a = ops.attention_decode(q, cache.k[li], cache.v[li], pos + 1, c.n_heads, c.n_kv_heads, c.head_dim)
            x2, h2 = ops.add_rmsnorm_forward(h, self._small([L["o"]], a)[0], L["post_ln"], c.eps)
            gate, up = self._small([L["gate"], L["up"]], h2)
            d = self._small([L["down"]], ops.swiglu_forward(gate, up))[0]
            # the residual add closes the layer and the same pass applies the next layer's (or the final) norm
            h, h1 = ops.add_rmsnorm_forward(x2, d, self.layers[li + 1]["input_ln"] if li + 1 < n else self.final_norm, c.eps)
        return h, h1

    def decode_step(self, ids: torch.Tensor, cache: KVCache) -> torch.Tensor:
        """Logits bf16 [B, vocab] of the next token after ids (int64 [B]); advances the cache by one position."""
        out = self.decode_logits(ids, cache)
        cache.length += 1
        return out

    def decode_graph(self, ids: torch.Tensor, cache: KVCache, pos: int):
        """A CUDA graph of one decode step at a fixed position (ids is read at replay, so the caller may overwrite it in place
        between replays). Returns (graph, logits tensor the replays write)."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.decode_logits(ids, cache, pos)      # warm-up outside the capture (lazy module state, allocator)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.decode_logits(ids, cache, pos)
        return g, out
