"""PalettizedLinear in the native layout (weights [N, K], 2-bit indices packed along K, one palette per
output row and 256 input columns, index logits fp32 [N, K, 4]) with the LoRA branch built in.

`linear_step` is the hot path as one call -- soft forward (straight-through or pure soft) plus the full
backward -- exactly the sequence of library calls a training step makes per Linear:

    soft_select   logits -> packed argmax indices (or W_soft)          one pass over the logits
    hard_fwd      y  = x W^T + (s x A^T) B^T                           tcgen05, weights decoded in-kernel
    bwd_dx        dX = dY W + (s dY B) A                               tcgen05, weights decoded in-kernel
    bwd_dw_soft   dW = x^T dY on tcgen05, epilogue -> dLogits, dPalette (dW never stored)
    lora_bwd      dA, dB

Module counterpart of the reference's PalettizedLinear + QwenLoRA (scripts/qwen_model.py:65-304).
"""
from __future__ import annotations

import os
import sys

import torch
from torch import nn

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)

import plz_ops as ops  # noqa: E402


def linear_step(x, dy, palette, logits, noise, tau, lora=None, ste=True, packed=None, seed=0, gs_n=1, gs_k=256,
                want=("y", "dx", "dlogits", "dpalette", "da", "db"), dp_scatter=None):
    """x bf16 [M, K]; dy bf16 [M, N] or None (forward only); palette bf16 [N/gs_n, K/gs_k, 4];
    logits fp32 [N, K, 4]; noise: fp32 [N, K, 4], None or 'hash'; lora = (A [r, K], B [N, r], scale) or None.
    `packed` is an optional preallocated uint8 [N, K/4] buffer for the hard indices.
    Returns a dict with the requested outputs (dlogits fp32 [N, K, 4], dpalette fp32 [groups, 4],
    da fp32 [r, K], db fp32 [N, r]) plus 'packed'.
    dp_scatter: a dp.LogitGradScatter (data-parallel ranks, straight-through path with LoRA): the weight-gradient launch
    stores its dLogits partials into the owners' staging buffers, the exchange runs beside the dX product, and the
    returned gradients are already summed over the ranks."""
    N, K, _ = logits.shape
    if packed is None:
        packed = ops.empty_packed(N, K, x.device)
    w = ops.PackedWeight(packed, palette, N, K, gs_n, gs_k)
    out = {"packed": packed}
    w_soft = ops.soft_select(w, logits, "nk4", noise=noise, tau=tau, seed=seed, want_packed=True, want_soft=not ste)
    if ste:
        y, t = ops.hard_forward(w, x, lora)
    else:
        y, t = ops.dense_forward(w_soft, x, lora)
    out["y"] = y
    if dy is None:
        return out
    fused_lora = ste and lora is not None and ("da" in want or "db" in want) and ("dlogits" in want or "dpalette" in want)
    if fused_lora and dp_scatter is not None and dp_scatter.world > 1:
        dt = ops.lora_dt(lora, dy)
        dpal, da, db = dp_scatter.dw(w, x, dy, logits, noise, tau, seed=seed, lora_ws=(t, dt))
        handle = dp_scatter.start([dpal, da, db])
        if "dx" in want:
            out["dx"] = ops.backward_dx_with_dt(w, dy, lora, dt)
        out.update(dlogits=dp_scatter.finish(handle), dpalette=dpal, da=da, db=db)
        return out
    if fused_lora:
        # dt first, then the weight-gradient launch also produces dA and dB, then dX with the dt already there
        dt = ops.lora_dt(lora, dy)
        dlog, dpal, da, db = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=tau, seed=seed,
                                                  want_dlogits="dlogits" in want, want_dpalette="dpalette" in want, lora_ws=(t, dt))
        out.update(dlogits=dlog, dpalette=dpal, da=da, db=db)
        if "dx" in want:
            out["dx"] = ops.backward_dx_with_dt(w, dy, lora, dt)
        return out
    if "dx" in want:
        dx, dt = ops.backward_dx(w, dy, lora) if ste else ops.dense_backward_dx(w_soft, dy, lora)
        out["dx"] = dx
    else:
        dt = None
    if "dlogits" in want or "dpalette" in want:
        dlog, dpal = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=tau, seed=seed,
                                          want_dlogits="dlogits" in want, want_dpalette="dpalette" in want)
        out["dlogits"], out["dpalette"] = dlog, dpal
    if lora is not None and ("da" in want or "db" in want):
        if dt is None:
            _, dt = ops.backward_dx(w, dy, lora)
        out["da"], out["db"] = ops.lora_backward(x, dy, t, dt)
    return out


class _PalettizedLoraFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, palette, logits, lora_a, lora_b, noise, cfg):
        tau, scale, ste, seed, gs_n, gs_k = cfg
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        N, K, _ = logits.shape
        lora = (lora_a.detach(), lora_b.detach(), scale) if lora_a is not None else None
        w = ops.PackedWeight(ops.empty_packed(N, K, x.device), palette.detach().contiguous(), N, K, gs_n, gs_k)
        w_soft = ops.soft_select(w, logits.detach(), "nk4", noise=noise, tau=tau, seed=seed, want_packed=True,
                                 want_soft=not ste)
        y, t = ops.hard_forward(w, x2, lora) if ste else ops.dense_forward(w_soft, x2, lora)
        ctx.save_for_backward(x2, palette, logits, lora_a, lora_b, w.packed, w_soft, t,
                              noise if isinstance(noise, torch.Tensor) else None)
        ctx.cfg = cfg
        ctx.noise_tag = noise if isinstance(noise, str) else None
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, palette, logits, lora_a, lora_b, packed, w_soft, t, noise_t = ctx.saved_tensors
        tau, scale, ste, seed, gs_n, gs_k = ctx.cfg
        noise = noise_t if noise_t is not None else ctx.noise_tag
        N, K, _ = logits.shape
        dy2 = dy.reshape(-1, N).contiguous()
        lora = (lora_a.detach(), lora_b.detach(), scale) if lora_a is not None else None
        w = ops.PackedWeight(packed, palette.detach().contiguous(), N, K, gs_n, gs_k)
        dx, dt = ops.backward_dx(w, dy2, lora) if ste else ops.dense_backward_dx(w_soft, dy2, lora)
        dlog = dpal = da = db = None
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            dlog, dpal = ops.backward_dw_soft(w, x2, dy2, logits.detach(), "nk4", noise=noise, tau=tau, seed=seed,
                                              want_dlogits=ctx.needs_input_grad[2], want_dpalette=ctx.needs_input_grad[1])
            if dpal is not None:
                dpal = dpal.reshape(palette.shape).to(palette.dtype)
        if lora is not None and (ctx.needs_input_grad[3] or ctx.needs_input_grad[4]):
            da, db = ops.lora_backward(x2, dy2, t, dt)
            da, db = da.to(lora_a.dtype), db.to(lora_b.dtype)
        return dx.reshape(ctx.x_shape), dpal, dlog, da, db, None, None


class PalettizedLinear(nn.Module):
    """Trainable 2-bit palettized Linear with LoRA, native layout.

    Parameters (names keep the substrings the reference's optimizer grouping looks for,
    scripts/train_qwen.py:512-521): palette bf16 [N, K/256, 4]; index_logits fp32 [N, K, 4];
    lora_A bf16 [r, K]; lora_B bf16 [N, r].  Buffer: packed uint8 [N, K/4] (hard indices for eval).
    Training mode runs the soft path (straight-through by default), eval mode the hard path."""

    def __init__(self, in_features, out_features, rank=16, lora_scale=1.0, group_k=256, device="cuda"):
        super().__init__()
        N, K = out_features, in_features
        self.in_features, self.out_features, self.group_k, self.rank = K, N, group_k, rank
        self.lora_scale, self.tau, self.ste, self.step_seed = float(lora_scale), 1.0, True, 0
        self.noise = "hash"  # counter-based sampler; tests may set an explicit fp32 [N, K, 4] tensor
        self.palette = nn.Parameter(torch.zeros(N, K // group_k, 4, dtype=torch.bfloat16, device=device))
        self.index_logits = nn.Parameter(torch.zeros(N, K, 4, dtype=torch.float32, device=device))
        if rank:
            self.lora_A = nn.Parameter(torch.zeros(rank, K, dtype=torch.bfloat16, device=device))
            self.lora_B = nn.Parameter(torch.zeros(N, rank, dtype=torch.bfloat16, device=device))
        else:
            self.lora_A = self.lora_B = None
        self.register_buffer("packed", torch.zeros(N, K // 4, dtype=torch.uint8, device=device))

    @torch.no_grad()
    def extract_hard_indices(self):
        """argmax of the logits -> packed buffer (scripts/qwen_model.py:198-209)."""
        w = ops.PackedWeight(self.packed, self.palette.detach(), self.out_features, self.in_features, 1, self.group_k)
        ops.soft_select(w, self.index_logits.detach(), "nk4", want_packed=True)

    def forward(self, x):
        N, K = self.out_features, self.in_features
        if self.training:
            self.step_seed = (self.step_seed + 1) & 0xFFFFFFFF
            cfg = (float(self.tau), self.lora_scale, self.ste, self.step_seed, 1, self.group_k)
            return _PalettizedLoraFn.apply(x, self.palette, self.index_logits, self.lora_A, self.lora_B, self.noise, cfg)
        x2 = x.reshape(-1, K).contiguous()
        w = ops.PackedWeight(self.packed, self.palette.detach(), N, K, 1, self.group_k)
        lora = (self.lora_A.detach(), self.lora_B.detach(), self.lora_scale) if self.lora_A is not None else None
        if lora is None and x2.shape[0] <= 64:
            y = ops.hard_forward_smallm(w, x2)
        else:
            y = ops.hard_forward(w, x2, lora)[0]
        return y.reshape(*x.shape[:-1], N)
