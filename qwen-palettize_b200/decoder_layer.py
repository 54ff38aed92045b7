"""A Qwen3-style decoder layer whose seven Linears are hard-palettized (2-bit indices, one palette per output row and 256
input columns) with a LoRA branch each, forward and backward, as explicit sequences of libplz.so calls.

The reference trains through the HuggingFace decoder layer with its Linears swapped for PalettizedLinear + QwenLoRA
(scripts/qwen_model.py:769-794, 897-951) and calls it as a black box (scripts/train_qwen.py:1259-1266); this is that layer
with every op on this library's kernels:

    h1 = rmsnorm(x) -> q, k, v projections (tcgen05 LUT GEMMs + LoRA block) -> per-head q/k RMSNorm + rotary embedding
       -> causal GQA attention -> o projection -> + x -> rmsnorm -> gate, up -> silu(gate) * up -> down -> + residual

Semantics: transformers' Qwen3DecoderLayer (RMSNorm eps, q_norm / k_norm over the head dimension, rotate_half RoPE,
SwiGLU); LoRA as in scripts/qwen_model.py:291-304.  The backward is written out by hand (no autograd): it returns the input
gradient and the gradients of every trainable tensor -- palettes (hard mode: gradient of the gather), LoRA factors, norm
weights.  torch supplies memory only.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)

import plz_ops as ops  # noqa: E402

LINEARS = ("q", "k", "v", "o", "gate", "up", "down")


@dataclass
class LayerConfig:
    hidden: int = 2560
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 9728
    eps: float = 1e-6
    rope_theta: float = 1e6
    lora_rank: int = 16
    lora_scale: float = 2.0      # alpha / rank of the reference (scripts/train_qwen.py:749-750)

    def shapes(self):
        """name -> (out features N, in features K)."""
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        return {"q": (q, self.hidden), "k": (kv, self.hidden), "v": (kv, self.hidden), "o": (self.hidden, q),
                "gate": (self.intermediate, self.hidden), "up": (self.intermediate, self.hidden), "down": (self.hidden, self.intermediate)}


@dataclass
class PalettizedLoraLinear:
    w: ops.PackedWeight
    lora_a: torch.Tensor   # bf16 [r, K]
    lora_b: torch.Tensor   # bf16 [N, r]
    scale: float

    @property
    def lora(self):
        return (self.lora_a, self.lora_b, self.scale)


@dataclass
class LayerParams:
    lin: dict                       # name -> PalettizedLoraLinear
    input_ln: torch.Tensor          # bf16 [hidden]
    post_ln: torch.Tensor           # bf16 [hidden]
    q_norm: torch.Tensor            # bf16 [head_dim]
    k_norm: torch.Tensor            # bf16 [head_dim]


def random_layer(cfg: LayerConfig, device, seed: int = 0) -> LayerParams:
    """Random-init layer with the distributions of the benchmark configurations: indices uniform, palettes sorted
    N(0, 0.02^2) 4-tuples, LoRA A ~ N(0, 1/K), B ~ N(0, 0.01^2), norm weights 1 + N(0, 0.1^2)."""
    g = torch.Generator(device=device).manual_seed(seed)
    lin = {}
    for name, (N, K) in cfg.shapes().items():
        idx = torch.randint(0, 4, (N, K), generator=g, device=device, dtype=torch.uint8)
        pal = (torch.randn(N * (K // 256), 4, generator=g, device=device) * 0.02).sort(-1).values.to(torch.bfloat16)
        w = ops.PackedWeight(ops.pack_indices(idx.view(torch.int8), n_major=True), pal, N, K, 1, 256)
        a = (torch.randn(cfg.lora_rank, K, generator=g, device=device) * K ** -0.5).to(torch.bfloat16)
        b = (torch.randn(N, cfg.lora_rank, generator=g, device=device) * 0.01).to(torch.bfloat16)
        lin[name] = PalettizedLoraLinear(w, a, b, cfg.lora_scale)
    nw = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)
    return LayerParams(lin, nw(cfg.hidden), nw(cfg.hidden), nw(cfg.head_dim), nw(cfg.head_dim))


@dataclass
class LayerCtx:
    """Activations a layer keeps for its backward."""
    t: dict = field(default_factory=dict)   # tensors by name


class HardLinears:
    """The seven Linears of a layer with frozen 2-bit indices (hard mode): forward, and in the backward the input gradient plus
    the gradients of the palette and of the LoRA factors, kept in `grads[name] = (dPalette, dA, dB)`.

    layer_forward / layer_backward take any object with these two methods, so the same layer runs its Linears in another
    mode (soft training with index logits: distill_step.SoftLinears; dense teacher weights: distill_step.DenseLinears)."""

    def __init__(self, P: LayerParams):
        self.P, self.grads = P, {}

    def fwd(self, name: str, x: torch.Tensor):
        """(y bf16 [M, N], t = the LoRA intermediate kept for the backward, or None)."""
        L = self.P.lin[name]
        return ops.hard_forward(L.w, x, L.lora)

    def bwd(self, name: str, x_in: torch.Tensor, t_in, d_out: torch.Tensor) -> torch.Tensor:
        L = self.P.lin[name]
        dxi, dti = ops.backward_dx(L.w, d_out, L.lora)
        self.grads[name] = ops.backward_dw_hard_lora(L.w, x_in, d_out, t_in, dti)
        return dxi


def layer_forward(cfg: LayerConfig, P, x: torch.Tensor, B: int, S: int, cos: torch.Tensor, sin: torch.Tensor, keep: bool = True, lin=None):
    """x bf16 [B * S, hidden] -> (y bf16 [B * S, hidden], ctx or None). P supplies the norm weights (input_ln, post_ln, q_norm,
    k_norm); lin the Linears (default: HardLinears(P))."""
    lin = lin if lin is not None else HardLinears(P)
    h1, rstd1 = ops.rmsnorm_forward(x, P.input_ln, cfg.eps)
    q_raw, t_q = lin.fwd("q", h1)
    k_raw, t_k = lin.fwd("k", h1)
    v, t_v = lin.fwd("v", h1)
    q, k = ops.qknorm_rope_forward2(q_raw, P.q_norm, cfg.n_heads, k_raw, P.k_norm, cfg.n_kv_heads, cos, sin, S, cfg.eps)
    a, lse = ops.attention_forward(q, k, v, B, S, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
    o, t_o = lin.fwd("o", a)
    x2, h2, rstd2 = ops.add_rmsnorm_forward(x, o, P.post_ln, cfg.eps, want_rstd=True)
    gate, t_g = lin.fwd("gate", h2)
    up, t_u = lin.fwd("up", h2)
    act = ops.swiglu_forward(gate, up)
    d, t_d = lin.fwd("down", act)
    y = ops.add(x2, d)
    if not keep:
        return y, None
    ctx = LayerCtx(dict(x=x, h1=h1, rstd1=rstd1, q_raw=q_raw, k_raw=k_raw, v=v, q=q, k=k, a=a, lse=lse, x2=x2, h2=h2, rstd2=rstd2,
                        gate=gate, up=up, act=act, t_q=t_q, t_k=t_k, t_v=t_v, t_o=t_o, t_g=t_g, t_u=t_u, t_d=t_d))
    return y, ctx


def layer_backward(cfg: LayerConfig, P, ctx: LayerCtx, dy: torch.Tensor, B: int, S: int, cos: torch.Tensor, sin: torch.Tensor, lin=None):
    """dy bf16 [B * S, hidden] -> (dx, grads): grads holds fp32 vectors for 'input_ln', 'post_ln', 'q_norm', 'k_norm' and whatever
    the Linears' object left in its `grads` (HardLinears: grads[name] = (dPalette fp32 [groups, 4], dA fp32 [r, K], dB fp32 [N, r]))."""
    lin = lin if lin is not None else HardLinears(P)
    c, g = ctx.t, {}
    dact = lin.bwd("down", c["act"], c["t_d"], dy)
    dgate, dup = ops.swiglu_backward(c["gate"], c["up"], dact)
    dh2 = ops.add(lin.bwd("gate", c["h2"], c["t_g"], dgate), lin.bwd("up", c["h2"], c["t_u"], dup))
    dx2n, g["post_ln"] = ops.rmsnorm_backward(c["x2"], dh2, c["rstd2"], P.post_ln)
    dx2 = ops.add(dy, dx2n)
    da = lin.bwd("o", c["a"], c["t_o"], dx2)
    dq, dk, dv = ops.attention_backward(c["q"], c["k"], c["v"], c["a"], da, c["lse"], B, S, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
    dq_raw, g["q_norm"] = ops.qknorm_rope_backward(c["q_raw"], P.q_norm, cos, sin, dq, cfg.n_heads, S, cfg.eps)
    dk_raw, g["k_norm"] = ops.qknorm_rope_backward(c["k_raw"], P.k_norm, cos, sin, dk, cfg.n_kv_heads, S, cfg.eps)
    dh1 = ops.add(lin.bwd("q", c["h1"], c["t_q"], dq_raw), lin.bwd("k", c["h1"], c["t_k"], dk_raw), lin.bwd("v", c["h1"], c["t_v"], dv))
    dx1n, g["input_ln"] = ops.rmsnorm_backward(c["x"], dh1, c["rstd1"], P.input_ln)
    dx = ops.add(dx2, dx1n)
    g.update(getattr(lin, "grads", {}))
    return dx, g


def stack_forward_backward(cfg: LayerConfig, layers, x: torch.Tensor, dy: torch.Tensor, B: int, S: int, cos, sin):
    """Forward through `layers` keeping activations, then backward from dy: (y, dx, [grads per layer])."""
    ctxs, h = [], x
    for P in layers:
        h, ctx = layer_forward(cfg, P, h, B, S, cos, sin, keep=True)
        ctxs.append(ctx)
    y, d, grads = h, dy, []
    for P, ctx in zip(reversed(layers), reversed(ctxs)):
        d, g = layer_backward(cfg, P, ctx, d, B, S, cos, sin)
        grads.append(g)
        ctx.t.clear()
    return y, d, grads[::-1]
