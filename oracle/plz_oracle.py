"""CPU oracle for the PalettizedLinear hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU (numpy for the integer/byte work, torch fp32 for the arithmetic),
what the reference `pkhairkh/qwen-palettize` computes on this path.  It is the checker for the CUDA
kernels: only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may
import it.  The product never calls it and has no CPU fallback.

Parity status: PINNED.  oracle/pin_against_reference.py runs the reference's own PyTorch functions
(imported from the reference checkout) on seeded inputs, checks every function below against them and
writes the small golden vectors under tests/golden/ that tests/test_oracle.py replays without the
reference.  The known-answer vectors of scripts/verify_2bit_format.py:50-109 are asserted there too.

Two tensor layouts are covered by one addressing rule  W[n, k] = palette[n // gs_n, k // gs_k, idx[n, k]]:
  layout R (reference API):  indices (K, N) int8, palette (N/256, 4) bf16, logits (4, K, N) fp16,
                             y = x @ W_R with W_R[k, n]            -> gs_n = 256, gs_k = K
  layout B (native/bench):   indices [N, K] packed 4 per byte, palette [N, K/256, 4], logits fp32 [N, K, 4]
                                                                   -> gs_n = 1,   gs_k = 256
Everything below works on the "N-major" view W[n, k]; layout-R callers transpose at the edge
(see to_nk_* helpers).
"""
from __future__ import annotations

import numpy as np
import torch

# --------------------------------------------------------------------------------------------
# 2-bit packing  (reference: scripts/palettize_core.py:31-42 pack_idx2, :45-56 unpack;
#                 known answers scripts/verify_2bit_format.py:50-109)
# --------------------------------------------------------------------------------------------

def pack_rows(idx: np.ndarray) -> np.ndarray:
    """idx uint8 [N, K] in {0..3} -> packed uint8 [N, ceil(K/4)], element k in bits 2*(k%4).. of byte k//4."""
    idx = np.asarray(idx, dtype=np.uint8) & 3
    n, k = idx.shape
    kp = (k + 3) // 4 * 4
    if kp != k:
        idx = np.concatenate([idx, np.zeros((n, kp - k), np.uint8)], axis=1)
    q = idx.reshape(n, kp // 4, 4)
    return (q[..., 0] | (q[..., 1] << 2) | (q[..., 2] << 4) | (q[..., 3] << 6)).astype(np.uint8)


def unpack_rows(packed: np.ndarray, k: int) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    n = packed.shape[0]
    out = np.empty((n, packed.shape[1], 4), np.uint8)
    for j in range(4):
        out[..., j] = (packed >> (2 * j)) & 3
    return out.reshape(n, -1)[:, :k]


def pack_flat(idx_flat: np.ndarray) -> bytes:
    """The reference's on-disk packing of a flattened index array (pads the last byte with zeros)."""
    return pack_rows(np.asarray(idx_flat, np.uint8).reshape(1, -1)).tobytes()


# --------------------------------------------------------------------------------------------
# hard weights and forward
#   reference: W[k, n] = palette.flatten()[(n // gs) * 4 + indices[k, n]];  y = x @ W
#   (scripts/qwen_model.py:98-102, 183-192; scripts/bench_triton_kernels.py:123-132)
# --------------------------------------------------------------------------------------------

def dequantize(idx_nk: torch.Tensor, palette: torch.Tensor, gs_n: int, gs_k: int) -> torch.Tensor:
    """idx_nk integer [N, K]; palette bf16 [(N/gs_n) * (K/gs_k), 4] (or any shape with that many rows of 4)
    -> W bf16 [N, K] (pure gather, bit exact)."""
    n, k = idx_nk.shape
    pal = palette.reshape(-1, 4)
    gn = torch.arange(n) // gs_n
    gk = torch.arange(k) // gs_k
    g = gn[:, None] * (k // gs_k) + gk[None, :]
    return pal[g, idx_nk.long()]


def matmul_bf16(a: torch.Tensor, b_t: torch.Tensor) -> torch.Tensor:
    """a [M, R] bf16, b_t [J, R] bf16 -> (a @ b_t.T) with fp32 accumulation, rounded once to bf16."""
    return (a.float() @ b_t.float().t()).to(torch.bfloat16)


def hard_forward(x: torch.Tensor, w_nk: torch.Tensor) -> torch.Tensor:
    return matmul_bf16(x, w_nk)


# --------------------------------------------------------------------------------------------
# Gumbel noise
#   counter-based sampler: scripts/fused_lut_kernel.cu:1245-1256, scripts/triton_soft_forward.py:51-66
#   noise index of element (k, n, plane): (k * N + n) * 4 + plane  (scripts/fused_lut_kernel.cu:1296-1299)
# --------------------------------------------------------------------------------------------

def gumbel_hash_u24(seed: int, idx: np.ndarray) -> np.ndarray:
    """Integer part of the sampler: the 24-bit uniform numerator, bit exact (uint32 wrap-around)."""
    with np.errstate(over="ignore"):
        x = np.uint32(seed) ^ (idx.astype(np.uint32) * np.uint32(0x9E3779B9))
        x ^= x >> np.uint32(13)
        x = x * np.uint32(1103515245) + np.uint32(12345)
        x ^= x >> np.uint32(17)
        x = x * np.uint32(1103515245) + np.uint32(12345)
    return x & np.uint32(0xFFFFFF)


def gumbel_hash(seed: int, n_total: int, k_total: int) -> torch.Tensor:
    """fp32 noise tensor [N, K, 4] for the counter-based sampler."""
    k = np.arange(k_total, dtype=np.uint32)[None, :, None]
    n = np.arange(n_total, dtype=np.uint32)[:, None, None]
    p = np.arange(4, dtype=np.uint32)[None, None, :]
    with np.errstate(over="ignore"):
        idx = (k * np.uint32(n_total) + n) * np.uint32(4) + p
    u = gumbel_hash_u24(seed, idx).astype(np.float32) * np.float32(1.0 / 16777216.0)
    u = np.maximum(u, np.float32(1e-7))
    return torch.from_numpy(-np.log(-np.log(u))).float()


def gumbel_from_uniform(u: torch.Tensor) -> torch.Tensor:
    """-log(-log(U)) with U clamped to [1e-7, 1) as the reference does (scripts/fused_lut_kernel.cu:1254)."""
    u = u.float().clamp(min=1e-7)
    return -torch.log(-torch.log(u))


# --------------------------------------------------------------------------------------------
# soft weights  (scripts/bench_triton_kernels.py:65-86, scripts/test_triton_soft_forward.py:36-75,
#                scripts/triton_soft_forward.py:119-181)
# --------------------------------------------------------------------------------------------

def group_palette(palette: torch.Tensor, n: int, k: int, gs_n: int, gs_k: int) -> torch.Tensor:
    """fp32 palette entries per weight position: [N, K, 4]."""
    pal = palette.reshape(-1, 4).float()
    g = (torch.arange(n) // gs_n)[:, None] * (k // gs_k) + (torch.arange(k) // gs_k)[None, :]
    return pal[g]


def soft_weights(logits_nk4: torch.Tensor, noise_nk4: torch.Tensor | None, palette: torch.Tensor, tau: float,
                 gs_n: int, gs_k: int):
    """logits [N, K, 4] (fp16 or fp32 as stored), noise fp32 [N, K, 4] or None.
    Returns P fp32 [N, K, 4], W_soft fp32 [N, K], hard index int64 [N, K] (argmax of the PLAIN logits,
    first maximum wins), W_hard bf16 [N, K]."""
    n, k, _ = logits_nk4.shape
    lf = logits_nk4.float()
    z = lf if noise_nk4 is None else lf + noise_nk4.float()
    p = torch.softmax(z / tau, dim=-1)
    c = group_palette(palette, n, k, gs_n, gs_k)
    w_soft = (p * c).sum(-1)
    hard = torch.argmax(lf, dim=-1)  # torch.argmax returns the first maximal index
    w_hard = dequantize(hard, palette, gs_n, gs_k)
    return p, w_soft, hard, w_hard


# --------------------------------------------------------------------------------------------
# soft backward  (scripts/bench_triton_kernels.py:89-120, scripts/test_triton_soft_backward.py:45-117)
# --------------------------------------------------------------------------------------------

def soft_backward(x: torch.Tensor, dy: torch.Tensor, w_fwd_nk: torch.Tensor, p_nk4: torch.Tensor,
                  palette: torch.Tensor, gs_n: int, gs_k: int, dx_fp32: bool = False):
    """x bf16 [M, K], dy bf16 [M, N], w_fwd_nk bf16 [N, K] = the weight the forward multiplied by
    (W_hard under the straight-through estimator, W_soft otherwise).
    Returns dX bf16 [M, K] (fp32, before the rounding, with dx_fp32: a caller that adds the LoRA term rounds the sum),
    dLogits fp32 [N, K, 4] (no 1/tau factor), dPalette fp32 [groups, 4], dW fp32 [N, K]."""
    n, k = w_fwd_nk.shape
    dx = dy.float() @ w_fwd_nk.float()
    if not dx_fp32:
        dx = dx.to(torch.bfloat16)
    dw = dy.float().t() @ x.float()  # [N, K]
    c = group_palette(palette, n, k, gs_n, gs_k)
    w_soft = (p_nk4 * c).sum(-1)
    contrib = dw[..., None] * p_nk4
    dlogits = contrib * (c - w_soft[..., None])
    g = (torch.arange(n) // gs_n)[:, None] * (k // gs_k) + (torch.arange(k) // gs_k)[None, :]
    n_groups = (n // gs_n) * (k // gs_k)
    dpal = torch.zeros(n_groups, 4, dtype=torch.float32)
    dpal.index_add_(0, g.reshape(-1), contrib.reshape(-1, 4))
    return dx, dlogits, dpal, dw


def hard_backward(x: torch.Tensor, dy: torch.Tensor, idx_nk: torch.Tensor, palette: torch.Tensor, gs_n: int,
                  gs_k: int):
    """Autograd of the gather + matmul (scripts/qwen_model.py:183-192; scripts/fused_lut_kernel.cu:1102-1108):
    dX = dY W, dPalette[g, p] = sum of dW over the positions of group g that hold index p."""
    n, k = idx_nk.shape
    w = dequantize(idx_nk, palette, gs_n, gs_k)
    dx = (dy.float() @ w.float()).to(torch.bfloat16)
    dw = dy.float().t() @ x.float()
    g = (torch.arange(n) // gs_n)[:, None] * (k // gs_k) + (torch.arange(k) // gs_k)[None, :]
    n_groups = (n // gs_n) * (k // gs_k)
    dpal = torch.zeros(n_groups * 4, dtype=torch.float32)
    dpal.index_add_(0, (g * 4 + idx_nk.long()).reshape(-1), dw.reshape(-1))
    return dx, dpal.reshape(n_groups, 4)


# --------------------------------------------------------------------------------------------
# LoRA  (scripts/qwen_model.py:291-304): y = base(x) + ((x @ A_R) @ B^T) * scaling, A_R (K, r), B (N, r)
# Here A is passed as [r, K] (= A_R^T).
# --------------------------------------------------------------------------------------------

def lora_forward(x: torch.Tensor, a_rk: torch.Tensor, b_nr: torch.Tensor, scale: float) -> torch.Tensor:
    """fp32 value of the LoRA branch (the reference rounds to bf16 after each of its three ops; the
    difference is far inside the bf16 tolerance of the sum)."""
    return (x.float() @ a_rk.float().t()) @ b_nr.float().t() * scale


def lora_backward(x: torch.Tensor, dy: torch.Tensor, a_rk: torch.Tensor, b_nr: torch.Tensor, scale: float):
    """Returns dX contribution fp32 [M, K], dA fp32 [r, K], dB fp32 [N, r]."""
    xf, dyf, af, bf = x.float(), dy.float(), a_rk.float(), b_nr.float()
    t = xf @ af.t()                      # [M, r]
    dt = (dyf @ bf) * scale              # [M, r]
    return dt @ af, dt.t() @ xf, dyf.t() @ t * scale


# --------------------------------------------------------------------------------------------
# layout R <-> N-major view
# --------------------------------------------------------------------------------------------

def to_nk_indices(indices_kn: torch.Tensor) -> torch.Tensor:
    return indices_kn.t().contiguous()


def to_nk_logits(logits_4kn: torch.Tensor) -> torch.Tensor:
    """(4, K, N) -> [N, K, 4]"""
    return logits_4kn.permute(2, 1, 0).contiguous()


def from_nk_logits(t_nk4: torch.Tensor) -> torch.Tensor:
    """[N, K, 4] -> (4, K, N)"""
    return t_nk4.permute(2, 1, 0).contiguous()


# --------------------------------------------------------------------------------------------
# full reference step for one Linear (used by the parity tests and the CPU baseline)
# --------------------------------------------------------------------------------------------

def linear_step(x, dy, logits_nk4, noise_nk4, palette, tau, gs_n, gs_k, lora=None, ste=True):
    """Soft forward + full backward of one palettized Linear (+ LoRA).  lora = (A [r,K], B [N,r], scale).
    Returns dict(y, dx, dlogits, dpalette, da, db, hard)."""
    p, w_soft, hard, w_hard = soft_weights(logits_nk4, noise_nk4, palette, tau, gs_n, gs_k)
    w_fwd = w_hard if ste else w_soft.to(torch.bfloat16)
    yf = x.float() @ w_fwd.float().t()
    if lora is not None:
        yf = yf + lora_forward(x, *lora)
    out = {"y": yf.to(torch.bfloat16), "hard": hard, "w_fwd": w_fwd}
    if dy is not None:
        dxf, dlogits, dpal, _ = soft_backward(x, dy, w_fwd, p, palette, gs_n, gs_k, dx_fp32=True)
        if lora is not None:
            dxl, da, db = lora_backward(x, dy, *lora)
            dxf = dxf + dxl
            out["da"], out["db"] = da, db
        out["dx"] = dxf.to(torch.bfloat16)
        out["dlogits"], out["dpalette"] = dlogits, dpal
    return out


# --------------------------------------------------------------------------------------------
# comparison helpers (the tolerances of the parity contract live in the tests)
# --------------------------------------------------------------------------------------------

def max_rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a - b| / max |b|  (per tensor)."""
    a, b = a.double().flatten(), b.double().flatten()
    den = b.abs().max().item()
    return (a - b).abs().max().item() / (den if den > 0 else 1.0)


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    den = (a.norm() * b.norm()).item()
    return (a @ b).item() / den if den > 0 else 1.0


# --------------------------------------------------------------------------------------------
# the steps around the Linear in the distillation loop
# --------------------------------------------------------------------------------------------

def distill_loss(s: torch.Tensor, t: torch.Tensor, w_cos: float = 0.5, w_mse: float = 0.5):
    """compute_loss of the reference, type "1-cos+norm_mse" (scripts/train_qwen.py:229-249): fp32 math,
    per-token cosine with eps 1e-4, MSE normalised by mean(t^2) clamped at 1e-6.
    s, t [..., H].  Returns (loss, l_cos, l_mse, t_var) as python floats and dLoss/ds (fp32) by autograd."""
    sf = s.detach().float().clone().requires_grad_(True)
    tf = t.detach().float()
    h = sf.shape[-1]
    cos_per = torch.nn.functional.cosine_similarity(sf.reshape(-1, h), tf.reshape(-1, h), dim=-1, eps=1e-4)
    l_cos = (1 - cos_per).mean()
    t_var = (tf * tf).mean().clamp(min=1e-6)
    l_mse = ((sf - tf) ** 2).mean() / t_var
    tot = w_cos + w_mse
    loss = (w_cos / tot) * l_cos + (w_mse / tot) * l_mse
    loss.backward()
    return (loss.item(), l_cos.item(), l_mse.item(), t_var.item()), sf.grad


def adamw_reference(param, grads, lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, clamp=None, clamp_master=False,
                    grad_scale=1.0):
    """fp32-master AdamW as FP32MasterAdamW runs it (scripts/train_qwen.py:154-215: torch.optim.AdamW on an fp32 master,
    model copy rewritten after every step; betas/eps :600) followed by the clamp of the model copy (:1343-1348).
    param: initial model tensor (any float dtype); grads: list of per-step gradients.
    Returns (master fp32, model copy in param.dtype, m, v)."""
    master = param.detach().float().clone().requires_grad_(True)
    opt = torch.optim.AdamW([master], lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    model = param.detach().clone()
    for g in grads:
        master.grad = g.detach().float() * grad_scale
        opt.step()
        with torch.no_grad():
            if clamp is not None and clamp_master:
                master.clamp_(clamp[0], clamp[1])
            model.copy_(master)
            if clamp is not None:
                model.clamp_(clamp[0], clamp[1])
    st = opt.state[master]
    return master.detach(), model, st["exp_avg"], st["exp_avg_sq"]


# --------------------------------------------------------------------------------------------
# on-disk formats (scripts/palettize_core.py:31-48 writer, :159-178 readers)
# --------------------------------------------------------------------------------------------

def read_idx2(data: bytes, out_dim: int, in_dim: int) -> np.ndarray:
    """.idx2 payload -> uint8 indices (in_dim, out_dim): the flat array is in (K, N) row-major order."""
    n = out_dim * in_dim
    arr = np.frombuffer(data, dtype=np.uint8)
    flat = unpack_rows(arr[: (n + 3) // 4].reshape(1, -1), n)[0]
    return flat.reshape(in_dim, out_dim)


def read_lut_scalar(data: bytes) -> np.ndarray:
    return np.frombuffer(data, dtype=np.float16).astype(np.float32)


# --------------------------------------------------------------------------------------------
# decoder-layer ops around the Linears (no reference code: the reference calls transformers' Qwen3 modules,
# scripts/train_qwen.py:1259-1266; these follow Qwen3RMSNorm / Qwen3MLP of transformers 5.5)
# --------------------------------------------------------------------------------------------

def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float = 1e-6) -> torch.Tensor:
    """fp32 result of x * rsqrt(mean(x^2) + eps) * weight."""
    xf = x.float()
    h = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return h if weight is None else h * weight.float()


def mlp_gate_up(x: torch.Tensor, w_gate_nk: torch.Tensor, w_up_nk: torch.Tensor, norm_weight=None, eps: float = 1e-6,
                normalize: bool = True) -> torch.Tensor:
    """silu(h Wg^T) * (h Wu^T) in fp32, h = rmsnorm(x) if normalize else x."""
    h = rmsnorm(x, norm_weight, eps) if normalize else x.float()
    g = h @ w_gate_nk.float().t()
    u = h @ w_up_nk.float().t()
    return torch.nn.functional.silu(g) * u


def swiglu_backward(gate: torch.Tensor, up: torch.Tensor, dact: torch.Tensor):
    """fp32 (dGate, dUp) of act = silu(gate) * up. Autograd of transformers' Qwen3MLP activation (no reference kernel:
    the reference trains through the HuggingFace module, scripts/train_qwen.py:1259-1266)."""
    g, u, d = gate.float(), up.float(), dact.float()
    sg = torch.sigmoid(g)
    return d * u * sg * (1.0 + g * (1.0 - sg)), d * g * sg


def rmsnorm_backward(x: torch.Tensor, weight, dh: torch.Tensor, eps: float = 1e-6):
    """fp32 (dX, dWeight) of h = x * rsqrt(mean(x^2) + eps) * weight given dH (autograd of Qwen3RMSNorm)."""
    xf, d = x.float(), dh.float()
    K = xf.shape[-1]
    rs = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    gd = d if weight is None else d * weight.float()
    dx = rs * gd - xf * rs.pow(3) * (xf * gd).sum(-1, keepdim=True) / K
    dw = None if weight is None else (d * xf * rs).sum(0)
    return dx, dw
