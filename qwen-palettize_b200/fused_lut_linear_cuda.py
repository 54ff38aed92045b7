"""Drop-in replacement for the reference's `fused_lut_linear_cuda` module (scripts/fused_lut_linear_cuda.py).

Same names, argument order, dtypes and gradients as the reference, so that the reference's
`PalettizedLinear` (scripts/qwen_model.py:123-130) picks this file up unchanged when its directory
comes first on sys.path:

    fused_lut_linear(x, palette, indices, bias=None, group_size=256)              :821-829
    fused_lut_linear_soft(x, palette, logits, bias=None, group_size=256, tau=1.0) :973-994
    CUDAFusedLUTLinear / CUDAFusedLUTLinearSoft (autograd Functions)              :755, :846
    GROUP_SIZE, _SOFT_STEP_SEED, _next_soft_step_seed()                           :752, :837-843

Tensors stay in the reference's runtime layout (x (M, K) bf16; indices (K, N) int8; palette (N/gs, 4)
bf16; logits (4, K, N) fp16).  The work is done by libplz.so: packed 2-bit indices decoded inside the
tcgen05 GEMMs, the weight gradient fused with the logit/palette gradients.  There is no CPU path and
no alternative backend; a missing library or a non-CUDA tensor raises.

Differences from the reference's CUDA wrapper, all on the side of its PyTorch/Triton semantics:
  * the hard index under soft training is argmax of the plain logits (scripts/triton_soft_forward.py:160-168),
    not of the noised probabilities (scripts/fused_lut_kernel.cu:1996-2003);
  * dW is accumulated in fp32 and never stored; P is recomputed in fp32 in the backward from the logits and
    the same counter-based noise instead of being saved as fp16 (10 bytes per weight less to keep);
  * kernels run on the current torch stream, not on stream 0.
Keyword-only extras (defaults reproduce the reference): `noise` -- an explicit (4, K, N) fp32 Gumbel tensor
instead of the counter-based sampler; `ste=False` -- forward with W_soft instead of the straight-through W_hard.
"""
from __future__ import annotations

import os
import sys
import weakref

import torch
from torch import Tensor

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)

import plz_native as _P  # noqa: E402
import plz_ops as _ops  # noqa: E402

GROUP_SIZE = 256
SMALL_M = 64  # at or below this many rows the HBM-bound small-M kernel is used

_SOFT_STEP_SEED = 0


def _next_soft_step_seed() -> int:
    """Global step counter for the Gumbel seed, one increment per soft forward call
    (scripts/fused_lut_linear_cuda.py:837-843)."""
    global _SOFT_STEP_SEED
    _SOFT_STEP_SEED = (_SOFT_STEP_SEED + 1) & 0xFFFFFFFF
    return _SOFT_STEP_SEED


def _get_module():
    """The reference returns its JIT-built pybind extension here (scripts/fused_lut_linear_cuda.py:742-749); this returns
    an object with the same ten functions, served by libplz.so (raises if the library has not been built)."""
    _P.lib()
    return _Extension


# Packed copies of frozen index buffers. An entry belongs to ONE caller tensor object: it holds a weak reference to that
# tensor and its version counter, and is dropped when the tensor is collected. Only the caller's own int8 / uint8
# contiguous tensor is cached (the module's `indices_int8` buffer); anything that needs a conversion is a temporary
# whose address the allocator may hand to the next layer's temporary, so it is packed on every call.
_PACK_CACHE: dict = {}


def _packed_for(indices: Tensor) -> Tensor:
    if indices.dtype not in (torch.int8, torch.uint8) or not indices.is_contiguous():
        tmp = indices if indices.dtype in (torch.int8, torch.uint8) else indices.to(torch.int8)
        return _ops.pack_indices(tmp.contiguous(), n_major=False)
    key = id(indices)
    hit = _PACK_CACHE.get(key)
    if hit is not None and hit[0]() is indices and hit[1] == indices._version and hit[2] == indices.data_ptr():
        return hit[3]
    packed = _ops.pack_indices(indices, n_major=False)
    _PACK_CACHE[key] = (weakref.ref(indices, lambda _r, k=key: _PACK_CACHE.pop(k, None)), indices._version,
                        indices.data_ptr(), packed)
    return packed


def _check_common(x: Tensor, palette: Tensor, K: int, N: int, group_size: int):
    if not x.is_cuda:
        raise RuntimeError("fused_lut_linear_cuda: CUDA tensors only (there is no CPU implementation)")
    if x.dtype != torch.bfloat16 or palette.dtype != torch.bfloat16:
        raise RuntimeError("x and palette must be bfloat16")
    if x.dim() != 2 or x.shape[1] != K:
        raise RuntimeError(f"x must be (M, {K}), got {tuple(x.shape)}")
    if palette.dim() != 2 or palette.shape[1] != 4:
        raise RuntimeError(f"palette last dim must be 4, got {tuple(palette.shape)}")
    if N % group_size != 0 or N // group_size != palette.shape[0]:
        raise RuntimeError(f"G mismatch: N//GS={N // group_size} vs palette.size(0)={palette.shape[0]}")


def _bias_bf16(bias: Tensor, N: int) -> Tensor:
    if bias.dim() != 1 or bias.shape[0] != N:
        raise RuntimeError(f"bias must be ({N},), got {tuple(bias.shape)}")
    return bias.detach().to(torch.bfloat16).contiguous()


def _forward_weight(w, x):
    if x.shape[0] <= SMALL_M:
        return _ops.hard_forward_smallm(w, x)
    return _ops.hard_forward(w, x)[0]


class CUDAFusedLUTLinear(torch.autograd.Function):
    """forward(ctx, x, palette, indices, bias, group_size) -> y; gradients to x, palette, (bias).
    Mirrors scripts/fused_lut_linear_cuda.py:755-818."""

    @staticmethod
    def forward(ctx, x, palette, indices, bias, group_size):
        x = x.contiguous()
        palette = palette.contiguous()
        K, N = indices.shape
        _check_common(x, palette, K, N, group_size)
        w = _ops.PackedWeight(_packed_for(indices), palette.detach(), N, K, group_size, K)
        if bias is not None:
            y = _ops.hard_forward_bias(w, x, _bias_bf16(bias, N))   # added in fp32 inside the GEMM epilogue
        else:
            y = _forward_weight(w, x)
        ctx.save_for_backward(x, palette, w.packed)
        ctx.dims = (N, K, group_size)
        ctx.has_bias = bias is not None
        ctx.bias_requires_grad = bias is not None and bias.requires_grad
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, palette, packed = ctx.saved_tensors
        N, K, gs = ctx.dims
        grad_y = grad_y.contiguous()
        w = _ops.PackedWeight(packed, palette.detach(), N, K, gs, K)
        grad_x = _ops.backward_dx(w, grad_y)[0] if ctx.needs_input_grad[0] else None
        grad_palette = None
        if ctx.needs_input_grad[1]:
            grad_palette = _ops.backward_dw_hard(w, x, grad_y).to(palette.dtype)
        grad_bias = _ops.col_sum(grad_y).to(grad_y.dtype) if (ctx.has_bias and ctx.bias_requires_grad) else None
        return grad_x, grad_palette, None, grad_bias, None


def fused_lut_linear(x: Tensor, palette: Tensor, indices: Tensor, bias: Tensor | None = None,
                     group_size: int = GROUP_SIZE) -> Tensor:
    """Functional interface -- supports autograd."""
    return CUDAFusedLUTLinear.apply(x, palette, indices, bias, group_size)


class CUDAFusedLUTLinearSoft(torch.autograd.Function):
    """forward(ctx, x, palette, logits, bias, group_size, tau[, noise, ste]) -> y
    backward -> (grad_x, grad_palette, grad_logits (4, K, N) fp16, grad_bias, None, None[, None, None]).
    Mirrors scripts/fused_lut_linear_cuda.py:846-970 (straight-through estimator :908-912)."""

    @staticmethod
    def forward(ctx, x, palette, logits, bias, group_size, tau, noise=None, ste=True):
        x = x.contiguous()
        palette = palette.contiguous()
        logits = logits.contiguous()
        assert logits.dim() == 3 and logits.shape[0] == 4, f"logits first dim must be 4, got {tuple(logits.shape)}"
        _, K, N = logits.shape
        _check_common(x, palette, K, N, group_size)
        if logits.dtype not in (torch.float16, torch.float32):
            raise RuntimeError("logits must be float16 (reference layout) or float32")
        seed = _next_soft_step_seed()
        nz = noise if noise is not None else "hash"
        w = _ops.PackedWeight(_ops.empty_packed(N, K, x.device), palette.detach(), N, K, group_size, K)
        w_soft = _ops.soft_select(w, logits.detach(), "4kn", noise=nz, tau=tau, seed=seed, want_packed=True,
                                  want_soft=not ste)
        if ste and bias is not None:
            y = _ops.hard_forward_bias(w, x, _bias_bf16(bias, N))
        elif ste:
            y = _forward_weight(w, x)
        else:
            y = _ops.dense_forward(w_soft, x)[0]
            if bias is not None:
                y = y + bias.to(y.dtype)
        ctx.save_for_backward(x, palette, logits, w.packed, w_soft if not ste else None,
                              noise if noise is not None else None)
        ctx.cfg = (N, K, group_size, float(tau), seed, ste)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, palette, logits, packed, w_soft, noise = ctx.saved_tensors
        N, K, gs, tau, seed, ste = ctx.cfg
        grad_y = grad_y.contiguous()
        w = _ops.PackedWeight(packed, palette.detach(), N, K, gs, K)
        grad_x = None
        if ctx.needs_input_grad[0]:
            grad_x = _ops.backward_dx(w, grad_y)[0] if ste else _ops.dense_backward_dx(w_soft, grad_y)[0]
        grad_palette = grad_logits = None
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            grad_logits, grad_palette = _ops.backward_dw_soft(
                w, x, grad_y, logits.detach(), "4kn", noise=noise if noise is not None else "hash", tau=tau, seed=seed,
                want_dlogits=ctx.needs_input_grad[2], want_dpalette=ctx.needs_input_grad[1])
            if grad_palette is not None:
                grad_palette = grad_palette.to(palette.dtype)
        grad_bias = _ops.col_sum(grad_y).to(grad_y.dtype) if (ctx.has_bias and ctx.needs_input_grad[3]) else None
        return grad_x, grad_palette, grad_logits, grad_bias, None, None, None, None


def fused_lut_linear_soft(x: Tensor, palette: Tensor, logits: Tensor, bias: Tensor | None = None,
                          group_size: int = GROUP_SIZE, tau: float = 1.0, *, noise: Tensor | None = None,
                          ste: bool = True) -> Tensor:
    """Soft (Gumbel-Softmax) functional interface -- supports autograd."""
    return CUDAFusedLUTLinearSoft.apply(x, palette, logits, bias, group_size, tau, noise, ste)


# ─── the reference extension's function surface (scripts/fused_lut_linear_cuda.py:721-732) ─────────────────────────────
def _soft_item(palette: Tensor, logits: Tensor, group_size: int, seed: int, **outs):
    _, K, N = logits.shape
    if palette.dim() != 2 or palette.shape[1] != 4 or N % group_size or N // group_size != palette.shape[0]:
        raise RuntimeError(f"G mismatch: N//GS={N // max(group_size, 1)} vs palette {tuple(palette.shape)}")
    if logits.dtype != torch.float16 or logits.dim() != 3 or logits.shape[0] != 4:
        raise RuntimeError("logits must be (4, K, N) fp16")
    d = dict(N=N, K=K, gs_n=group_size, gs_k=K, palette=palette.contiguous(), logits=logits.contiguous(), logits_layout="4kn",
             noise="hash", seed=int(seed) & 0xFFFFFFFF)
    d.update(outs)
    return d


class _Extension:
    """The ten functions the reference's extension module exports, with its argument order, shapes and dtypes.
    P and W are real tensors here, as in the reference; the library's own training path never materialises them."""

    @staticmethod
    def fused_lut_linear_fwd(x, palette, indices, bias, group_size):
        """-> y (M, N) bf16  (:74-117)"""
        with torch.no_grad():
            return CUDAFusedLUTLinear.apply(x, palette, indices, bias, int(group_size))

    @staticmethod
    def fused_lut_linear_bwd(grad_y, x, palette, indices, bias, group_size, needs_grad_x, needs_grad_palette):
        """-> [grad_x (M, K) bf16, grad_palette (G, 4) bf16, grad_bias (N,) bf16]; entries not asked for are None  (:119-185)"""
        K, N = indices.shape
        x, grad_y, palette = x.contiguous(), grad_y.contiguous(), palette.contiguous()
        _check_common(x, palette, K, N, int(group_size))
        w = _ops.PackedWeight(_packed_for(indices), palette, N, K, int(group_size), K)
        gx = _ops.backward_dx(w, grad_y)[0] if needs_grad_x else None
        gp = _ops.backward_dw_hard(w, x, grad_y).to(torch.bfloat16) if needs_grad_palette else None
        gb = _ops.col_sum(grad_y).to(torch.bfloat16) if bias is not None else None
        return [gx, gp, gb]

    @staticmethod
    def fused_lut_linear_soft_fwd(x, palette, logits, group_size, tau, step_seed):
        """-> [y = x @ W, P (4, K, N) fp16, W (K, N) bf16 = soft weights]  (:239-275)"""
        _, K, N = logits.shape
        P4 = torch.empty(4, K, N, dtype=torch.float16, device=logits.device)
        W = torch.empty(K, N, dtype=torch.bfloat16, device=logits.device)
        _ops.soft_weights([_soft_item(palette, logits, int(group_size), step_seed, P=(P4, "4kn"), w_soft=(W, "kn"))], float(tau))
        y = _ops.dense_backward_dx(W, x.contiguous())[0]   # reduction over the rows of a row-major (K, N) operand
        return [y, P4, W]

    @staticmethod
    def fused_lut_linear_soft_fwd_aos(x, palette, logits, group_size, tau, step_seed):
        """-> [P_aos (K, N, 4) fp16, W (K, N) bf16]; no matmul  (:372-405)"""
        _, K, N = logits.shape
        Pa = torch.empty(K, N, 4, dtype=torch.float16, device=logits.device)
        W = torch.empty(K, N, dtype=torch.bfloat16, device=logits.device)
        _ops.soft_weights([_soft_item(palette, logits, int(group_size), step_seed, P=(Pa, "kn4"), w_soft=(W, "kn"))], float(tau))
        return [Pa, W]

    @staticmethod
    def fused_lut_linear_soft_fwd_with_hard(x, palette, logits, group_size, tau, step_seed):
        """-> [P_aos, W_soft, W_hard]; the hard index is the argmax of P, i.e. of the noised logits, as in the
        reference kernel (scripts/fused_lut_kernel.cu:1996-2003)  (:636-660)"""
        _, K, N = logits.shape
        Pa = torch.empty(K, N, 4, dtype=torch.float16, device=logits.device)
        Ws = torch.empty(K, N, dtype=torch.bfloat16, device=logits.device)
        Wh = torch.empty(K, N, dtype=torch.bfloat16, device=logits.device)
        _ops.soft_weights([_soft_item(palette, logits, int(group_size), step_seed, P=(Pa, "kn4"), w_soft=(Ws, "kn"),
                                      w_hard=(Wh, "kn"))], float(tau), hard_from_noisy=True)
        return [Pa, Ws, Wh]

    @staticmethod
    def _bwd_from(grad_w, dw_layout, P, p_layout, palette, group_size):
        if p_layout == "4kn":
            _, K, N = P.shape
        else:
            K, N, _ = P.shape
        gl = torch.empty(4, K, N, dtype=torch.float16, device=P.device)
        gp = _ops.soft_bwd_elementwise(N, K, int(group_size), K, palette.contiguous(), grad_w, dw_layout, P, p_layout, gl, "4kn")
        return [gl, gp.to(torch.bfloat16)]

    @staticmethod
    def fused_lut_linear_soft_bwd(grad_W, P, palette, group_size):
        """grad_W (K, N) fp32, P (4, K, N) fp16 -> [grad_logits (4, K, N) fp16, grad_palette (G, 4) bf16]  (:283-323)"""
        return _Extension._bwd_from(grad_W.contiguous(), "kn", P.contiguous(), "4kn", palette, group_size)

    @staticmethod
    def soft_bwd_elementwise(grad_W, P_aos, palette, group_size):
        """grad_W (K, N) bf16 (or fp32), P_aos (K, N, 4) fp16 -> [grad_logits, grad_palette]  (:662-683)"""
        return _Extension._bwd_from(grad_W.contiguous(), "kn", P_aos.contiguous(), "kn4", palette, group_size)

    @staticmethod
    def fused_lut_linear_soft_bwd_fused(grad_y, x, P, palette, group_size):
        """grad_W = x^T grad_y computed here (fp32, tensor cores), then the element-wise backward  (:338-366)"""
        gw = _ops.weight_grad(x.contiguous(), grad_y.contiguous(), "kn")
        return _Extension._bwd_from(gw, "kn", P.contiguous(), "4kn", palette, group_size)

    @staticmethod
    def fused_lut_linear_soft_bwd_fused_aos(grad_y, x, P_aos, palette, group_size):
        """Same with P in the (K, N, 4) layout  (:421-452)"""
        gw = _ops.weight_grad(x.contiguous(), grad_y.contiguous(), "kn")
        return _Extension._bwd_from(gw, "kn", P_aos.contiguous(), "kn4", palette, group_size)

    @staticmethod
    def fused_compute_P_W_batched(logits_list, palette_list, group_size, tau, step_seed):
        """One launch for all layers -> flat [P_aos_0, W_0, P_aos_1, W_1, ...]; layer i draws its noise with the seed
        step_seed ^ (i * 0x9E3779B9)  (:505-607; scripts/fused_lut_kernel.cu:2097-2158)"""
        if len(logits_list) != len(palette_list):
            raise RuntimeError("palette_list size must match logits_list size")
        items, flat = [], []
        for i, (lg, pal) in enumerate(zip(logits_list, palette_list)):
            _, K, N = lg.shape
            Pa = torch.empty(K, N, 4, dtype=torch.float16, device=lg.device)
            W = torch.empty(K, N, dtype=torch.bfloat16, device=lg.device)
            seed = (int(step_seed) ^ ((i * 0x9E3779B9) & 0xFFFFFFFF)) & 0xFFFFFFFF
            items.append(_soft_item(pal.detach(), lg.detach(), int(group_size), seed, P=(Pa, "kn4"), w_soft=(W, "kn")))
            flat += [Pa, W]
        if items:
            _ops.soft_weights(items, float(tau))
        return flat


def fused_compute_P_W_batched(student, tau: float, step_seed: int, group_size: int | None = None):
    """(P_aos, W_soft) of every soft PalettizedLinear under `student` in one launch, in named_modules() order
    (scripts/fused_lut_linear_cuda.py:1016-1077). Modules are recognised by their attributes (index_logits, palette,
    group_size, _use_cuda), so the reference's class and any module shaped like it both qualify."""
    layers = [m for _, m in student.named_modules()
              if type(m).__name__ == "PalettizedLinear" and getattr(m, "index_logits", None) is not None
              and getattr(m, "_use_cuda", False)]
    if not layers:
        return []
    if group_size is None:
        group_size = layers[0].group_size
    for i, m in enumerate(layers):
        if m.group_size != group_size:
            raise ValueError(f"All PalettizedLinears must share group_size for the batched compute_P_W kernel; layer {i} has "
                             f"group_size={m.group_size} vs expected {group_size}")
    flat = _Extension.fused_compute_P_W_batched([m.index_logits for m in layers], [m.palette for m in layers], int(group_size),
                                                float(tau), int(step_seed))
    return [(flat[i], flat[i + 1]) for i in range(0, len(flat), 2)]
