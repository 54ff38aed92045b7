"""Functional wrappers over the C ABI: one Python function per entry point of include/plz.h.

Tensors are torch CUDA tensors; outputs are allocated here with torch (the library itself never
allocates) and every call goes to the current torch stream.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

import plz_native as P


@dataclass
class PackedWeight:
    """W[n, k] = palette[(n // gs_n) * (K // gs_k) + k // gs_k][idx[n, k]] with idx packed 4 per byte along k."""
    packed: torch.Tensor   # uint8 [N, K // 4]
    palette: torch.Tensor  # bf16, (N // gs_n) * (K // gs_k) * 4 elements, contiguous
    N: int
    K: int
    gs_n: int
    gs_k: int

    def desc(self) -> P.Weight:
        return P.weight_desc(self.packed, self.palette, self.N, self.K, self.gs_n, self.gs_k)


def _pitch(K: int) -> int:
    return (K // 4 + 15) // 16 * 16


def empty_packed(N: int, K: int, device) -> torch.Tensor:
    buf = torch.empty(N, _pitch(K), dtype=torch.uint8, device=device)
    return buf[:, : K // 4] if _pitch(K) != K // 4 else buf


def pack_indices(idx: torch.Tensor, n_major: bool) -> torch.Tensor:
    """idx int8/uint8: [N, K] if n_major else (K, N) (the reference's runtime layout) -> packed uint8 [N, K//4]."""
    P._need_cuda(idx)
    assert idx.dtype in (torch.int8, torch.uint8) and idx.dim() == 2
    if n_major:
        N, K = idx.shape
        s_n, s_k = idx.stride(0), idx.stride(1)
    else:
        K, N = idx.shape
        s_k, s_n = idx.stride(0), idx.stride(1)
    out = empty_packed(N, K, idx.device)
    P.check(P.lib().plz_pack_indices(idx.data_ptr(), s_n, s_k, N, K, out.data_ptr(), out.stride(0), P.stream_ptr()),
            "plz_pack_indices")
    return out


def unpack_indices(packed: torch.Tensor, K: int, n_major: bool = True) -> torch.Tensor:
    N = packed.shape[0]
    out = torch.empty((N, K) if n_major else (K, N), dtype=torch.int8, device=packed.device)
    s_n, s_k = (K, 1) if n_major else (1, N)
    P.check(P.lib().plz_unpack_indices(packed.data_ptr(), packed.stride(0), N, K, out.data_ptr(), s_n, s_k,
                                       P.stream_ptr()), "plz_unpack_indices")
    return out


def dequantize(w: PackedWeight) -> torch.Tensor:
    out = torch.empty(w.N, w.K, dtype=torch.bfloat16, device=w.packed.device)
    d = w.desc()
    P.check(P.lib().plz_dequantize(C.byref(d), out.data_ptr(), w.K, 1, P.stream_ptr()), "plz_dequantize")
    return out


def _lora_args(lora, M, device):
    """lora = (A [r, K], B [N, r], scale) or None -> (descriptor pointer or None, workspace or None)."""
    if lora is None:
        return None, None, None
    a, b, scale = lora
    d = P.lora_desc(a, b, scale)
    ws = torch.empty(M, a.shape[0], dtype=torch.bfloat16, device=device)
    return d, C.byref(d), ws


def _mat(x: torch.Tensor, cols: int):
    P._need_cuda(x)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == cols and x.stride(1) == 1, \
        f"expected bf16 [M, {cols}] with unit column stride, got {tuple(x.shape)} {x.dtype}"
    return x


def hard_forward(w: PackedWeight, x: torch.Tensor, lora=None):
    """y = x W^T (+ LoRA).  Returns (y, t) where t = scale * x A^T (None without LoRA)."""
    _mat(x, w.K)
    M = x.shape[0]
    y = torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
    keep, lp, t = _lora_args(lora, M, x.device)
    d = w.desc()
    P.check(P.lib().plz_hard_fwd(C.byref(d), x.data_ptr(), x.stride(0), M, lp, t.data_ptr() if t is not None else None,
                                 y.data_ptr(), y.stride(0), P.stream_ptr()), "plz_hard_fwd")
    return y, t


def hard_forward_smallm(w: PackedWeight, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _mat(x, w.K)
    M = x.shape[0]
    y = out if out is not None else torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
    d = w.desc()
    P.check(P.lib().plz_hard_fwd_smallm(C.byref(d), x.data_ptr(), x.stride(0), M, y.data_ptr(), y.stride(0),
                                        P.stream_ptr()), "plz_hard_fwd_smallm")
    return y


def hard_forward_smallm_multi(ws, x: torch.Tensor, outs=None):
    """[x W_i^T for W_i in ws] in ONE launch (1..4 matrices sharing K and the palette grouping, M <= 16). outs: optional list of
    destinations (None entries are allocated); a destination may be a pitched view, e.g. one position of a key / value cache."""
    _mat(x, ws[0].K)
    M, n = x.shape[0], len(ws)
    ys = [outs[i] if outs is not None and outs[i] is not None else torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
          for i, w in enumerate(ws)]
    for y, w in zip(ys, ws):
        assert y.dtype == torch.bfloat16 and tuple(y.shape) == (M, w.N) and y.stride(1) == 1
    descs = [w.desc() for w in ws]
    wp = (C.POINTER(P.Weight) * n)(*[C.pointer(d) for d in descs])
    yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    ld = (C.c_int64 * n)(*[y.stride(0) for y in ys])
    P.check(P.lib().plz_hard_fwd_smallm_multi(wp, n, x.data_ptr(), x.stride(0), M, yp, ld, P.stream_ptr()),
            "plz_hard_fwd_smallm_multi")
    return ys


def soft_select(w: PackedWeight, logits: torch.Tensor, layout: str, noise=None, tau: float = 1.0, seed: int = 0,
                want_packed: bool = True, want_soft: bool = False):
    """Writes argmax indices into w.packed (if want_packed) and returns W_soft bf16 [N, K] (if want_soft)."""
    ld, nd = P.logits_desc(logits, layout), P.noise_desc(noise, layout, seed)
    w_soft = torch.empty(w.N, w.K, dtype=torch.bfloat16, device=logits.device) if want_soft else None
    d = w.desc()
    P.check(P.lib().plz_soft_select(C.byref(d), C.byref(ld), C.byref(nd), float(tau), int(want_packed),
                                    w_soft.data_ptr() if want_soft else None, w.K, 1, P.stream_ptr()), "plz_soft_select")
    return w_soft


def dense_forward(wd: torch.Tensor, x: torch.Tensor, lora=None):
    N, K = wd.shape
    _mat(x, K), _mat(wd, K)
    M = x.shape[0]
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    keep, lp, t = _lora_args(lora, M, x.device)
    P.check(P.lib().plz_dense_fwd(wd.data_ptr(), wd.stride(0), N, K, x.data_ptr(), x.stride(0), M, lp,
                                  t.data_ptr() if t is not None else None, y.data_ptr(), y.stride(0), P.stream_ptr()),
            "plz_dense_fwd")
    return y, t


def backward_dx(w: PackedWeight, dy: torch.Tensor, lora=None):
    """dX = dY W (+ LoRA).  Returns (dX, dt) with dt = scale * dY B."""
    _mat(dy, w.N)
    M = dy.shape[0]
    dx = torch.empty(M, w.K, dtype=torch.bfloat16, device=dy.device)
    keep, lp, dt = _lora_args(lora, M, dy.device)
    d = w.desc()
    P.check(P.lib().plz_bwd_dx(C.byref(d), dy.data_ptr(), dy.stride(0), M, lp, dt.data_ptr() if dt is not None else None,
                               dx.data_ptr(), dx.stride(0), P.stream_ptr()), "plz_bwd_dx")
    return dx, dt


def lora_dt(lora, dy: torch.Tensor) -> torch.Tensor:
    """dt = scale * dY B, bf16 [M, rank]."""
    a, b, scale = lora
    _mat(dy, b.shape[0])
    d = P.lora_desc(a, b, scale)
    dt = torch.empty(dy.shape[0], a.shape[0], dtype=torch.bfloat16, device=dy.device)
    P.check(P.lib().plz_lora_dt(C.byref(d), dy.data_ptr(), dy.stride(0), dy.shape[0], b.shape[0], dt.data_ptr(), P.stream_ptr()),
            "plz_lora_dt")
    return dt


def backward_dx_with_dt(w: PackedWeight, dy: torch.Tensor, lora, dt: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """dX = dY W + dt A with a precomputed dt. Rows are independent, so a caller may compute dX in row blocks (slices of
    dy, dt and `out`), e.g. to put other work between them."""
    _mat(dy, w.N)
    M = dy.shape[0]
    dx = out if out is not None else torch.empty(M, w.K, dtype=torch.bfloat16, device=dy.device)
    if out is not None:
        _mat(out, w.K)
        assert out.shape[0] == M
    ld = P.lora_desc(*lora)
    d = w.desc()
    P.check(P.lib().plz_bwd_dx_with_dt(C.byref(d), dy.data_ptr(), dy.stride(0), M, C.byref(ld), dt.data_ptr(), dx.data_ptr(),
                                       dx.stride(0), P.stream_ptr()), "plz_bwd_dx_with_dt")
    return dx


def dense_backward_dx(wd: torch.Tensor, dy: torch.Tensor, lora=None):
    N, K = wd.shape
    _mat(dy, N), _mat(wd, K)
    M = dy.shape[0]
    dx = torch.empty(M, K, dtype=torch.bfloat16, device=dy.device)
    keep, lp, dt = _lora_args(lora, M, dy.device)
    P.check(P.lib().plz_dense_bwd_dx(wd.data_ptr(), wd.stride(0), N, K, dy.data_ptr(), dy.stride(0), M, lp,
                                     dt.data_ptr() if dt is not None else None, dx.data_ptr(), dx.stride(0),
                                     P.stream_ptr()), "plz_dense_bwd_dx")
    return dx, dt


def backward_dw_soft(w: PackedWeight, x: torch.Tensor, dy: torch.Tensor, logits: torch.Tensor, layout: str, noise=None,
                     tau: float = 1.0, seed: int = 0, want_dlogits: bool = True, want_dpalette: bool = True, lora_ws=None):
    """Returns (dLogits with the dtype/shape of `logits`, dPalette fp32 [groups, 4]); with lora_ws = (t, dt), the workspaces
    left by the forward and by backward_dx, also (dA fp32 [r, K], dB fp32 [N, r]) computed in the same launch."""
    _mat(x, w.K), _mat(dy, w.N)
    M = x.shape[0]
    ld, nd = P.logits_desc(logits, layout), P.noise_desc(noise, layout, seed)
    dlog = torch.empty_like(logits) if want_dlogits else None
    if dlog is not None:
        assert dlog.stride() == logits.stride()
    dpal = torch.zeros(w.palette.numel() // 4, 4, dtype=torch.float32, device=x.device) if want_dpalette else None
    d = w.desc()
    if lora_ws is not None:
        t, dt = lora_ws
        r = t.shape[1]
        da = torch.zeros(r, w.K, dtype=torch.float32, device=x.device)
        db = torch.zeros(w.N, r, dtype=torch.float32, device=x.device)
        P.check(P.lib().plz_bwd_dw_soft_lora(C.byref(d), x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), M, C.byref(ld),
                                             C.byref(nd), float(tau), dlog.data_ptr() if dlog is not None else None,
                                             dpal.data_ptr() if dpal is not None else None, t.data_ptr(), dt.data_ptr(), r,
                                             da.data_ptr(), db.data_ptr(), P.stream_ptr()), "plz_bwd_dw_soft_lora")
        return dlog, dpal, da, db
    P.check(P.lib().plz_bwd_dw_soft(C.byref(d), x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), M, C.byref(ld),
                                    C.byref(nd), float(tau), dlog.data_ptr() if dlog is not None else None,
                                    dpal.data_ptr() if dpal is not None else None, P.stream_ptr()), "plz_bwd_dw_soft")
    return dlog, dpal


def backward_dw_soft_scatter(w: PackedWeight, x: torch.Tensor, dy: torch.Tensor, logits: torch.Tensor, stage_ptrs, world: int,
                             rank: int, noise=None, tau: float = 1.0, seed: int = 0, lora_ws=None, accumulate: bool = False,
                             outs=None):
    """Weight-gradient launch whose epilogue stores this rank's partial dLogits into the owners' staging buffers
    (`stage_ptrs`: the `world` device addresses, as mapped in this process, of the fp32 [world, N/world, K, 4] buffers; with
    accumulate=True of the zeroed fp32 [N/world, K, 4] accumulators that the partials are added to).
    Returns (dPalette, dA, dB) of THIS rank (fp32, not reduced; dA = dB = None without lora_ws = (t, dt)).
    outs = (dPalette, dA, dB): ZEROED fp32 tensors to accumulate into (e.g. views of one flat all-reduce bucket)."""
    _mat(x, w.K), _mat(dy, w.N)
    M = x.shape[0]
    ld, nd = P.logits_desc(logits, "nk4"), P.noise_desc(noise, "nk4", seed)
    dpal = outs[0] if outs is not None else torch.zeros(w.palette.numel() // 4, 4, dtype=torch.float32, device=x.device)
    table = (C.c_void_p * world)(*[int(p) for p in stage_ptrs])
    d = w.desc()
    t = dt = da = db = None
    r = 0
    if lora_ws is not None:
        t, dt = lora_ws
        r = t.shape[1]
        da = outs[1] if outs is not None else torch.zeros(r, w.K, dtype=torch.float32, device=x.device)
        db = outs[2] if outs is not None else torch.zeros(w.N, r, dtype=torch.float32, device=x.device)
    P.check(P.lib().plz_bwd_dw_soft_scatter(C.byref(d), x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), M, C.byref(ld),
                                            C.byref(nd), float(tau), table, world, rank, 1 if accumulate else 0, dpal.data_ptr(),
                                            t.data_ptr() if t is not None else None, dt.data_ptr() if dt is not None else None, r,
                                            da.data_ptr() if da is not None else None, db.data_ptr() if db is not None else None,
                                            P.stream_ptr()), "plz_bwd_dw_soft_scatter")
    return dpal, da, db


def reduce_slots(stage_ptr: int, world: int, out: torch.Tensor, scale: float = 1.0):
    """out (fp32, contiguous, the rank's shard) = scale * sum of the `world` slots of the staging buffer at `stage_ptr`."""
    assert out.dtype == torch.float32 and out.is_contiguous()
    P.check(P.lib().plz_reduce_slots(int(stage_ptr), world, out.numel(), out.data_ptr(), float(scale), P.stream_ptr()),
            "plz_reduce_slots")
    return out


def backward_dw_hard(w: PackedWeight, x: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    _mat(x, w.K), _mat(dy, w.N)
    dpal = torch.zeros(w.palette.numel() // 4, 4, dtype=torch.float32, device=x.device)
    d = w.desc()
    P.check(P.lib().plz_bwd_dw_hard(C.byref(d), x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), x.shape[0],
                                    dpal.data_ptr(), P.stream_ptr()), "plz_bwd_dw_hard")
    return dpal


def lora_backward(x: torch.Tensor, dy: torch.Tensor, t: torch.Tensor, dt: torch.Tensor):
    """dA fp32 [r, K], dB fp32 [N, r] from the workspaces left by the forward (t) and by backward_dx (dt)."""
    M, K = x.shape
    N = dy.shape[1]
    r = t.shape[1]
    da = torch.zeros(r, K, dtype=torch.float32, device=x.device)
    db = torch.zeros(N, r, dtype=torch.float32, device=x.device)
    P.check(P.lib().plz_lora_bwd(x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), t.data_ptr(), dt.data_ptr(),
                                 M, N, K, r, da.data_ptr(), db.data_ptr(), P.stream_ptr()), "plz_lora_bwd")
    return da, db


_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def adamw_step(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor, step: int, lr: float,
               betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0, grad_scale: float = 1.0, clamp=None,
               clamp_master: bool = False, param: torch.Tensor | None = None):
    """In-place fused fp32-master AdamW (+ optional clamp) on flat/contiguous tensors; writes `param` (model copy) if given."""
    P._need_cuda(master, m, v, grad, param)
    assert master.dtype == m.dtype == v.dtype == torch.float32 and master.is_contiguous() and grad.is_contiguous()
    assert grad.numel() == master.numel() and (param is None or (param.is_contiguous() and param.numel() == master.numel()))
    lo, hi = clamp if clamp is not None else (1.0, -1.0)
    P.check(P.lib().plz_adamw_step(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), _DT[grad.dtype], float(grad_scale),
                                   master.numel(), float(lr), float(betas[0]), float(betas[1]), float(eps), float(weight_decay),
                                   int(step), float(lo), float(hi), int(clamp_master), param.data_ptr() if param is not None else None,
                                   _DT[param.dtype] if param is not None else 0, P.stream_ptr()), "plz_adamw_step")


def distill_loss(s: torch.Tensor, t: torch.Tensor, w_cos: float = 0.5, w_mse: float = 0.5, want_grad: bool = True,
                 grad_dtype=torch.bfloat16, upstream: float = 1.0):
    """s, t bf16 [..., H].  Returns (stats fp32 [4] = loss, l_cos, l_mse, mean(t^2) on the device, dLoss/ds or None)."""
    H = s.shape[-1]
    s2, t2 = s.reshape(-1, H), t.reshape(-1, H)
    _mat(s2, H), _mat(t2, H)
    M = s2.shape[0]
    tot = float(w_cos) + float(w_mse)   # the reference normalises the two weights to sum 1 (normalize_weights)
    if tot > 0:
        w_cos, w_mse = w_cos / tot, w_mse / tot
    ws = torch.empty(4 + 4 * M, dtype=torch.float32, device=s.device)
    out4 = torch.empty(4, dtype=torch.float32, device=s.device)
    ds = torch.empty(M, H, dtype=grad_dtype, device=s.device) if want_grad else None
    P.check(P.lib().plz_distill_loss(s2.data_ptr(), s2.stride(0), t2.data_ptr(), t2.stride(0), M, H, float(w_cos), float(w_mse),
                                     float(upstream), ws.data_ptr(), out4.data_ptr(), ds.data_ptr() if ds is not None else None,
                                     H, _DT[grad_dtype], P.stream_ptr()), "plz_distill_loss")
    return out4, (ds.reshape(s.shape) if ds is not None else None)


def rms_rstd(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """fp32 [M]: 1 / sqrt(mean(x^2, -1) + eps)."""
    _mat(x, x.shape[1])
    out = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    P.check(P.lib().plz_rms_rstd(x.data_ptr(), x.stride(0), x.shape[0], x.shape[1], float(eps), out.data_ptr(), P.stream_ptr()),
            "plz_rms_rstd")
    return out


def hard_forward_norm(w: PackedWeight, x: torch.Tensor, rstd: torch.Tensor | None, norm_weight: torch.Tensor | None):
    """y = rmsnorm(x) W^T with the norm folded into the GEMM (rstd fp32 [M], norm_weight bf16 [K]; either may be None)."""
    _mat(x, w.K)
    M = x.shape[0]
    y = torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
    d = w.desc()
    P.check(P.lib().plz_hard_fwd_norm(C.byref(d), x.data_ptr(), x.stride(0), M, rstd.data_ptr() if rstd is not None else None,
                                      norm_weight.data_ptr() if norm_weight is not None else None, y.data_ptr(), y.stride(0),
                                      P.stream_ptr()), "plz_hard_fwd_norm")
    return y


def mlp_gate_up_forward(w_gate: PackedWeight, w_up: PackedWeight, x: torch.Tensor, rstd=None, norm_weight=None, keep: bool = False):
    """act = silu(h Wg^T) * (h Wu^T), h = rmsnorm(x) (optional), in one launch; bf16 [M, N].
    keep=True: returns (act, gate, up) with the two pre-activations written by the same launch (for swiglu_backward)."""
    _mat(x, w_gate.K)
    M = x.shape[0]
    act = torch.empty(M, w_gate.N, dtype=torch.bfloat16, device=x.device)
    dg, du = w_gate.desc(), w_up.desc()
    if keep:
        gate, up = torch.empty_like(act), torch.empty_like(act)
        P.check(P.lib().plz_mlp_gate_up_fwd_keep(C.byref(dg), C.byref(du), x.data_ptr(), x.stride(0), M,
                                                 rstd.data_ptr() if rstd is not None else None,
                                                 norm_weight.data_ptr() if norm_weight is not None else None, act.data_ptr(),
                                                 act.stride(0), gate.data_ptr(), up.data_ptr(), gate.stride(0), P.stream_ptr()),
                "plz_mlp_gate_up_fwd_keep")
        return act, gate, up
    P.check(P.lib().plz_mlp_gate_up_fwd(C.byref(dg), C.byref(du), x.data_ptr(), x.stride(0), M,
                                        rstd.data_ptr() if rstd is not None else None,
                                        norm_weight.data_ptr() if norm_weight is not None else None, act.data_ptr(), act.stride(0),
                                        P.stream_ptr()), "plz_mlp_gate_up_fwd")
    return act


def swiglu_backward(gate: torch.Tensor, up: torch.Tensor, dact: torch.Tensor):
    """(dGate, dUp) of act = silu(gate) * up; all bf16 [M, N]."""
    M, N = gate.shape
    _mat(gate, N), _mat(up, N), _mat(dact, N)
    dgate, dup = torch.empty_like(gate), torch.empty_like(up)
    P.check(P.lib().plz_swiglu_bwd(gate.data_ptr(), gate.stride(0), up.data_ptr(), up.stride(0), dact.data_ptr(), dact.stride(0), M, N,
                                   dgate.data_ptr(), dgate.stride(0), dup.data_ptr(), dup.stride(0), P.stream_ptr()), "plz_swiglu_bwd")
    return dgate, dup


def rmsnorm_backward(x: torch.Tensor, dh: torch.Tensor, rstd: torch.Tensor, norm_weight: torch.Tensor | None, want_dg: bool = True):
    """(dX bf16 [M, K], dG fp32 [K] or None) from dH, the gradient with respect to rmsnorm(x)."""
    M, K = x.shape
    _mat(x, K), _mat(dh, K)
    dx = torch.empty_like(x)
    dg = torch.zeros(K, dtype=torch.float32, device=x.device) if (want_dg and norm_weight is not None) else None
    P.check(P.lib().plz_rmsnorm_bwd(x.data_ptr(), x.stride(0), dh.data_ptr(), dh.stride(0), rstd.data_ptr(),
                                    norm_weight.data_ptr() if norm_weight is not None else None, M, K, dx.data_ptr(), dx.stride(0),
                                    dg.data_ptr() if dg is not None else None, P.stream_ptr()), "plz_rmsnorm_bwd")
    return dx, dg


def mlp_front_backward(w_gate: PackedWeight, w_up: PackedWeight, x: torch.Tensor, rstd, norm_weight, dact: torch.Tensor,
                       gate: torch.Tensor | None = None, up: torch.Tensor | None = None):
    """Backward of act = silu(h Wg^T) * (h Wu^T), h = rmsnorm(x): swiglu_backward -> two dX products -> rmsnorm_backward.
    gate / up: the pre-activations kept by mlp_gate_up_forward(keep=True); without them they are recomputed (two LUT
    GEMMs with the norm folded in).  Returns (dX, dG, dGate, dUp); dGate / dUp are what the weight-gradient launches
    of the two Linears take as dY (with h as their x)."""
    if gate is None or up is None:
        gate = hard_forward_norm(w_gate, x, rstd, norm_weight)
        up = hard_forward_norm(w_up, x, rstd, norm_weight)
    dgate, dup = swiglu_backward(gate, up, dact)
    dh = backward_dx(w_gate, dgate)[0]
    dh += backward_dx(w_up, dup)[0]
    if rstd is None:
        return dh, None, dgate, dup
    dx, dg = rmsnorm_backward(x, dh, rstd, norm_weight)
    return dx, dg, dgate, dup


def hard_forward_bias(w: PackedWeight, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """y = x W^T + bias, the bias (bf16 [N]) added in fp32 inside the GEMM epilogue."""
    _mat(x, w.K)
    M = x.shape[0]
    y = torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
    if bias is not None:
        P._need_cuda(bias)
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == w.N
    d = w.desc()
    P.check(P.lib().plz_hard_fwd_bias(C.byref(d), x.data_ptr(), x.stride(0), M, bias.data_ptr() if bias is not None else None,
                                      y.data_ptr(), y.stride(0), P.stream_ptr()), "plz_hard_fwd_bias")
    return y


def col_sum(dy: torch.Tensor) -> torch.Tensor:
    """fp32 [N]: sum over the rows of a bf16 [M, N] matrix (the bias gradient)."""
    _mat(dy, dy.shape[1])
    out = torch.zeros(dy.shape[1], dtype=torch.float32, device=dy.device)
    P.check(P.lib().plz_col_sum(dy.data_ptr(), dy.stride(0), dy.shape[0], dy.shape[1], out.data_ptr(), P.stream_ptr()), "plz_col_sum")
    return out


def _strides_nk(t: torch.Tensor, layout: str):
    """(s_n, s_k[, s_p]) of a tensor given as 'kn' (K, N), 'nk' [N, K], 'kn4' (K, N, 4), '4kn' (4, K, N) or 'nk4' [N, K, 4]."""
    st = t.stride()
    if layout == "kn":
        return st[1], st[0]
    if layout == "nk":
        return st[0], st[1]
    if layout == "kn4":
        return st[1], st[0], st[2]
    if layout == "4kn":
        return st[2], st[1], st[0]
    if layout == "nk4":
        return st[0], st[1], st[2]
    raise ValueError(f"unknown layout {layout}")


def soft_weights(items, tau: float, hard_from_noisy: bool = False):
    """One launch over several matrices. items: list of dicts with keys
      N, K, gs_n, gs_k, palette (bf16), logits (tensor), logits_layout ('4kn' | 'nk4'), noise (None | 'hash' | fp32 tensor in the
      logits' layout), seed, and the wanted outputs as (tensor, layout) pairs or None: P (fp16; '4kn' | 'kn4' | 'nk4'),
      w_soft / w_hard (bf16; 'kn' | 'nk')."""
    n = len(items)
    keep, wps, lps, nps, ops_ = [], [], [], [], []
    for it in items:
        wd = P.Weight(it["N"], it["K"], it["gs_n"], it["gs_k"], None, 0, it["palette"].data_ptr())
        ld = P.logits_desc(it["logits"], it["logits_layout"])
        nd = P.noise_desc(it.get("noise"), it["logits_layout"], it.get("seed", 0))
        so = P.SoftOut()
        if it.get("P") is not None:
            t, lay = it["P"]
            assert t.dtype == torch.float16
            so.P, (so.p_n, so.p_k, so.p_p) = t.data_ptr(), _strides_nk(t, lay)
        for key, fld in (("w_soft", "ws"), ("w_hard", "wh")):
            if it.get(key) is not None:
                t, lay = it[key]
                assert t.dtype == torch.bfloat16
                s_n, s_k = _strides_nk(t, lay)
                setattr(so, key, t.data_ptr()); setattr(so, fld + "_n", s_n); setattr(so, fld + "_k", s_k)
        keep += [wd, ld, nd, so]
        wps.append(C.pointer(wd)); lps.append(C.pointer(ld)); nps.append(C.pointer(nd)); ops_.append(C.pointer(so))
    P.check(P.lib().plz_soft_weights(n, (C.POINTER(P.Weight) * n)(*wps), (C.POINTER(P.Logits) * n)(*lps), (C.POINTER(P.Noise) * n)(*nps),
                                     float(tau), int(hard_from_noisy), (C.POINTER(P.SoftOut) * n)(*ops_), P.stream_ptr()),
            "plz_soft_weights")


def soft_bwd_elementwise(N, K, gs_n, gs_k, palette, dw, dw_layout, p, p_layout, dlogits, dlogits_layout, want_dpalette=True):
    """dLogits (written into `dlogits`, fp16 or fp32, may be None) and dPalette fp32 [groups, 4] from a materialised
    dW (fp32 or bf16) and P (fp16)."""
    wd = P.Weight(N, K, gs_n, gs_k, None, 0, palette.data_ptr())
    dw_n, dw_k = _strides_nk(dw, dw_layout)
    p_n, p_k, p_p = _strides_nk(p, p_layout)
    dl = P.logits_desc(dlogits, dlogits_layout) if dlogits is not None else None
    dpal = torch.zeros(palette.numel() // 4, 4, dtype=torch.float32, device=dw.device) if want_dpalette else None
    P.check(P.lib().plz_soft_bwd_elementwise(C.byref(wd), dw.data_ptr(), _DT[dw.dtype], dw_n, dw_k, p.data_ptr(), p_n, p_k, p_p,
                                             C.byref(dl) if dl is not None else None, dpal.data_ptr() if dpal is not None else None,
                                             P.stream_ptr()), "plz_soft_bwd_elementwise")
    return dpal


def weight_grad(x: torch.Tensor, dy: torch.Tensor, layout: str = "kn") -> torch.Tensor:
    """dW = x^T dY as an fp32 tensor: (K, N) for layout 'kn', [N, K] for 'nk'."""
    M, K = x.shape
    N = dy.shape[1]
    _mat(x, K), _mat(dy, N)
    dw = torch.zeros((K, N) if layout == "kn" else (N, K), dtype=torch.float32, device=x.device)
    s_n, s_k = _strides_nk(dw, layout)
    P.check(P.lib().plz_weight_grad(x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), M, N, K, dw.data_ptr(), s_n, s_k,
                                    P.stream_ptr()), "plz_weight_grad")
    return dw


def attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, B: int, S: int, n_heads: int, n_kv_heads: int,
                      head_dim: int = 128, scale: float | None = None):
    """Causal GQA attention. q bf16 [B*S, n_heads*head_dim], k / v bf16 [B*S, n_kv_heads*head_dim] (rows may be pitched: slices of
    one fused projection output are fine). Returns (o bf16 [B*S, n_heads*head_dim], lse fp32 [B, n_heads, S])."""
    _mat(q, n_heads * head_dim), _mat(k, n_kv_heads * head_dim), _mat(v, n_kv_heads * head_dim)
    assert q.shape[0] == B * S == k.shape[0] == v.shape[0]
    o = torch.empty(B * S, n_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, n_heads, S, dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else head_dim ** -0.5
    P.check(P.lib().plz_attn_fwd(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), B, S, n_heads, n_kv_heads,
                                 head_dim, sc, o.data_ptr(), o.stride(0), lse.data_ptr(), P.stream_ptr()), "plz_attn_fwd")
    return o, lse


def attention_backward(q, k, v, o, do, lse, B: int, S: int, n_heads: int, n_kv_heads: int, head_dim: int = 128, scale: float | None = None):
    """(dq, dk, dv) in the layouts of (q, k, v); dk / dv are summed over the query heads of each group."""
    _mat(do, n_heads * head_dim), _mat(o, n_heads * head_dim)
    assert o.stride(0) == do.stride(0)
    dq = torch.empty(B * S, n_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    dk = torch.empty(B * S, n_kv_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    dv = torch.empty_like(dk)
    assert dq.stride(0) == q.stride(0) and dk.stride(0) == k.stride(0) and dv.stride(0) == v.stride(0), \
        "gradients are written with the pitches of q / k / v: pass contiguous q, k, v"
    ws = torch.empty(B * n_heads * S, dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else head_dim ** -0.5
    P.check(P.lib().plz_attn_bwd(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), o.data_ptr(), do.data_ptr(),
                                 o.stride(0), lse.data_ptr(), B, S, n_heads, n_kv_heads, head_dim, sc, ws.data_ptr(), dq.data_ptr(),
                                 dk.data_ptr(), dv.data_ptr(), P.stream_ptr()), "plz_attn_bwd")
    return dq, dk, dv


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, T: int, n_heads: int, n_kv_heads: int,
                     head_dim: int = 128, scale: float | None = None) -> torch.Tensor:
    """Attention of one new token per sequence over the first T positions of the caches. q bf16 [B, n_heads * head_dim]; caches
    bf16 [B, T_max, n_kv_heads * head_dim] (position T - 1 holds the new token's key / value). Returns bf16 [B, n_heads * head_dim]."""
    _mat(q, n_heads * head_dim)
    B = q.shape[0]
    assert k_cache.dim() == 3 and k_cache.shape == v_cache.shape and k_cache.shape[0] == B and k_cache.stride() == v_cache.stride()
    assert k_cache.shape[2] == n_kv_heads * head_dim and k_cache.stride(2) == 1 and 0 < T <= k_cache.shape[1]
    out = torch.empty(B, n_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    nbytes = int(P.lib().plz_attn_decode_ws_bytes(B, T, n_heads, n_kv_heads))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    sc = float(scale) if scale is not None else head_dim ** -0.5
    P.check(P.lib().plz_attn_decode(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1),
                                    B, T, n_heads, n_kv_heads, head_dim, sc, out.data_ptr(), out.stride(0), ws.data_ptr(), nbytes,
                                    P.stream_ptr()), "plz_attn_decode")
    return out


def embed_gather(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """table[ids] for a bf16 [vocab, width] table and int64 ids (any shape); returns bf16 [ids.numel(), width]."""
    assert table.dtype == torch.bfloat16 and table.dim() == 2 and table.stride(1) == 1 and ids.dtype == torch.int64
    flat = ids.reshape(-1).contiguous()
    out = torch.empty(flat.numel(), table.shape[1], dtype=torch.bfloat16, device=table.device)
    P.check(P.lib().plz_embed_gather(table.data_ptr(), table.stride(0), flat.data_ptr(), flat.numel(), table.shape[1], table.shape[0],
                                     out.data_ptr(), out.stride(0), None, P.stream_ptr()), "plz_embed_gather")
    return out


def rmsnorm_forward(x: torch.Tensor, weight: torch.Tensor | None, eps: float = 1e-6):
    """(h bf16 [M, K] = rmsnorm(x) * weight, rstd fp32 [M])."""
    M, K = x.shape
    _mat(x, K)
    h = torch.empty(M, K, dtype=torch.bfloat16, device=x.device)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    P.check(P.lib().plz_rmsnorm_fwd(x.data_ptr(), x.stride(0), weight.data_ptr() if weight is not None else None, M, K, float(eps),
                                    h.data_ptr(), h.stride(0), rstd.data_ptr(), P.stream_ptr()), "plz_rmsnorm_fwd")
    return h, rstd


def add_rmsnorm_forward(x: torch.Tensor, addend: torch.Tensor, weight: torch.Tensor | None, eps: float = 1e-6, want_rstd: bool = False):
    """(s = x + addend, h = rmsnorm(s) * weight), both bf16 [M, K], in one pass; with want_rstd also rstd fp32 [M] (the
    backward of the norm needs it)."""
    M, K = x.shape
    _mat(x, K), _mat(addend, K)
    s = torch.empty(M, K, dtype=torch.bfloat16, device=x.device)
    h = torch.empty(M, K, dtype=torch.bfloat16, device=x.device)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device) if want_rstd else None
    P.check(P.lib().plz_add_rmsnorm_fwd(x.data_ptr(), x.stride(0), addend.data_ptr(), addend.stride(0), s.data_ptr(), s.stride(0),
                                        weight.data_ptr() if weight is not None else None, M, K, float(eps), h.data_ptr(), h.stride(0),
                                        rstd.data_ptr() if rstd is not None else None, P.stream_ptr()), "plz_add_rmsnorm_fwd")
    return (s, h, rstd) if want_rstd else (s, h)


def qknorm_rope_forward2(xq, wq, n_heads: int, xk, wk, n_kv_heads: int, cos, sin, S: int, eps: float = 1e-6, out_q=None, out_k=None):
    """qknorm_rope_forward of the q and the k projection of the same tokens in one launch: (q, k)."""
    _mat(xq, n_heads * 128), _mat(xk, n_kv_heads * 128)
    T = xq.shape[0]
    assert xk.shape[0] == T
    oq = out_q if out_q is not None else torch.empty(T, n_heads * 128, dtype=torch.bfloat16, device=xq.device)
    ok = out_k if out_k is not None else torch.empty(T, n_kv_heads * 128, dtype=torch.bfloat16, device=xq.device)
    for o, h in ((oq, n_heads), (ok, n_kv_heads)):
        assert o.dtype == torch.bfloat16 and tuple(o.shape) == (T, h * 128) and o.stride(1) == 1
    P.check(P.lib().plz_qknorm_rope_fwd2(xq.data_ptr(), xq.stride(0), wq.data_ptr() if wq is not None else None, n_heads, oq.data_ptr(), oq.stride(0),
                                         xk.data_ptr(), xk.stride(0), wk.data_ptr() if wk is not None else None, n_kv_heads, ok.data_ptr(),
                                         ok.stride(0), cos.data_ptr(), sin.data_ptr(), T, S, 128, float(eps), P.stream_ptr()),
            "plz_qknorm_rope_fwd2")
    return oq, ok


def rope_tables(S: int, head_dim: int = 128, theta: float = 1e6, device="cuda"):
    """(cos, sin) fp32 [S, head_dim / 2] of transformers' default rotary embedding: angle = position * theta^(-2i / head_dim)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return ang.cos().contiguous().to(device), ang.sin().contiguous().to(device)


def qknorm_rope_forward(x: torch.Tensor, weight: torch.Tensor | None, cos: torch.Tensor, sin: torch.Tensor, n_heads: int, S: int,
                        eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """Per-head RMSNorm (weight bf16 [128]) + rotary embedding of x bf16 [tokens, n_heads * 128] (rows may be pitched). Row i has
    position i % S in the cos / sin tables; a decode step passes S = 1 and the table rows of its position. out may be a pitched
    view (one position of a key cache)."""
    _mat(x, n_heads * 128)
    if out is None:
        out = torch.empty(x.shape[0], n_heads * 128, dtype=torch.bfloat16, device=x.device)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (x.shape[0], n_heads * 128) and out.stride(1) == 1
    P.check(P.lib().plz_qknorm_rope_fwd(x.data_ptr(), x.stride(0), weight.data_ptr() if weight is not None else None, cos.data_ptr(),
                                        sin.data_ptr(), x.shape[0], n_heads, S, 128, float(eps), out.data_ptr(), out.stride(0), P.stream_ptr()),
            "plz_qknorm_rope_fwd")
    return out


def qknorm_rope_backward(x: torch.Tensor, weight: torch.Tensor | None, cos: torch.Tensor, sin: torch.Tensor, dy: torch.Tensor, n_heads: int,
                         S: int, eps: float = 1e-6, want_dw: bool = True):
    """(dx bf16 in the shape of x, dw fp32 [128] or None) from dy, the gradient of qknorm_rope_forward's output."""
    _mat(x, n_heads * 128), _mat(dy, n_heads * 128)
    dx = torch.empty(x.shape[0], n_heads * 128, dtype=torch.bfloat16, device=x.device)
    dw = torch.zeros(128, dtype=torch.float32, device=x.device) if (want_dw and weight is not None) else None
    P.check(P.lib().plz_qknorm_rope_bwd(x.data_ptr(), x.stride(0), weight.data_ptr() if weight is not None else None, cos.data_ptr(),
                                        sin.data_ptr(), dy.data_ptr(), dy.stride(0), x.shape[0], n_heads, S, 128, float(eps), dx.data_ptr(),
                                        dx.stride(0), dw.data_ptr() if dw is not None else None, P.stream_ptr()), "plz_qknorm_rope_bwd")
    return dx, dw


def swiglu_forward(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    M, N = gate.shape
    _mat(gate, N), _mat(up, N)
    act = torch.empty(M, N, dtype=torch.bfloat16, device=gate.device)
    P.check(P.lib().plz_swiglu_fwd(gate.data_ptr(), gate.stride(0), up.data_ptr(), up.stride(0), M, N, act.data_ptr(), act.stride(0),
                                   P.stream_ptr()), "plz_swiglu_fwd")
    return act


def add(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """a + b (+ c) of bf16 [M, N] matrices in one pass (fp32 sum, one rounding)."""
    M, N = a.shape
    _mat(a, N), _mat(b, N)
    o = out if out is not None else torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    P.check(P.lib().plz_add(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), c.data_ptr() if c is not None else None,
                            c.stride(0) if c is not None else 0, M, N, o.data_ptr(), o.stride(0), P.stream_ptr()), "plz_add")
    return o


def backward_dw_hard_lora(w: PackedWeight, x: torch.Tensor, dy: torch.Tensor, t: torch.Tensor, dt: torch.Tensor):
    """(dPalette fp32 [groups, 4], dA fp32 [r, K], dB fp32 [N, r]) of a hard palettized Linear with LoRA, one launch."""
    _mat(x, w.K), _mat(dy, w.N)
    r = t.shape[1]
    dpal = torch.zeros(w.palette.numel() // 4, 4, dtype=torch.float32, device=x.device)
    da = torch.zeros(r, w.K, dtype=torch.float32, device=x.device)
    db = torch.zeros(w.N, r, dtype=torch.float32, device=x.device)
    d = w.desc()
    P.check(P.lib().plz_bwd_dw_hard_lora(C.byref(d), x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), x.shape[0], dpal.data_ptr(),
                                         t.data_ptr(), dt.data_ptr(), r, da.data_ptr(), db.data_ptr(), P.stream_ptr()), "plz_bwd_dw_hard_lora")
    return dpal, da, db
