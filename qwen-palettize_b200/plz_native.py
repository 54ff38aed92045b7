"""ctypes binding of libplz.so (C ABI in include/plz.h) for torch tensors.

torch is used for device memory and streams only; every computation happens in the library's
sm_100a kernels.  There is no fallback: if the library is missing or a call fails this raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libplz.so")
_lib = None


class Weight(C.Structure):
    _fields_ = [("N", C.c_int32), ("K", C.c_int32), ("gs_n", C.c_int32), ("gs_k", C.c_int32),
                ("packed", C.c_void_p), ("packed_pitch", C.c_int64), ("palette", C.c_void_p)]


class Lora(C.Structure):
    _fields_ = [("rank", C.c_int32), ("scale", C.c_float), ("A", C.c_void_p), ("lda", C.c_int64),
                ("B", C.c_void_p), ("ldb", C.c_int64)]


class Logits(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("s_n", C.c_int64), ("s_k", C.c_int64),
                ("s_p", C.c_int64)]


class SoftOut(C.Structure):
    _fields_ = [("P", C.c_void_p), ("p_n", C.c_int64), ("p_k", C.c_int64), ("p_p", C.c_int64),
                ("w_soft", C.c_void_p), ("ws_n", C.c_int64), ("ws_k", C.c_int64),
                ("w_hard", C.c_void_p), ("wh_n", C.c_int64), ("wh_k", C.c_int64)]


class Noise(C.Structure):
    _fields_ = [("mode", C.c_int32), ("seed", C.c_uint32), ("ptr", C.c_void_p), ("s_n", C.c_int64),
                ("s_k", C.c_int64), ("s_p", C.c_int64)]


_I32, _I64, _P, _F = C.c_int32, C.c_int64, C.c_void_p, C.c_float
_WP, _LP, _GP, _NP = C.POINTER(Weight), C.POINTER(Lora), C.POINTER(Logits), C.POINTER(Noise)

# name -> argtypes; every function returns int32 unless listed in _RESTYPES
SIGNATURES = {
    "plz_version": [],
    "plz_last_error": [],
    "plz_launch_count": [],
    "plz_device_status": [C.POINTER(C.c_uint32)],
    "plz_set_cta_limit": [_I32],
    "plz_set_pair_gemm": [_I32],
    "plz_pack_indices": [_P, _I64, _I64, _I32, _I32, _P, _I64, _P],
    "plz_unpack_indices": [_P, _I64, _I32, _I32, _P, _I64, _I64, _P],
    "plz_dequantize": [_WP, _P, _I64, _I64, _P],
    "plz_hard_fwd": [_WP, _P, _I64, _I32, _LP, _P, _P, _I64, _P],
    "plz_hard_fwd_lora_static": [_WP, _P, _I64, _I32, _LP, _P, _I64, _P],
    "plz_hard_fwd_smallm": [_WP, _P, _I64, _I32, _P, _I64, _P],
    "plz_hard_fwd_smallm_multi": [C.POINTER(_WP), _I32, _P, _I64, _I32, C.POINTER(C.c_void_p), C.POINTER(C.c_int64), _P],
    "plz_set_smallm_overlap": [_I32],
    "plz_soft_select": [_WP, _GP, _NP, _F, _I32, _P, _I64, _I64, _P],
    "plz_dense_fwd": [_P, _I64, _I32, _I32, _P, _I64, _I32, _LP, _P, _P, _I64, _P],
    "plz_bwd_dx": [_WP, _P, _I64, _I32, _LP, _P, _P, _I64, _P],
    "plz_lora_dt": [_LP, _P, _I64, _I32, _I32, _P, _P],
    "plz_bwd_dx_with_dt": [_WP, _P, _I64, _I32, _LP, _P, _P, _I64, _P],
    "plz_dense_bwd_dx": [_P, _I64, _I32, _I32, _P, _I64, _I32, _LP, _P, _P, _I64, _P],
    "plz_bwd_dw_soft": [_WP, _P, _I64, _P, _I64, _I32, _GP, _NP, _F, _P, _P, _P],
    "plz_bwd_dw_soft_lora": [_WP, _P, _I64, _P, _I64, _I32, _GP, _NP, _F, _P, _P, _P, _P, _I32, _P, _P, _P],
    "plz_bwd_dw_soft_scatter": [_WP, _P, _I64, _P, _I64, _I32, _GP, _NP, _F, C.POINTER(C.c_void_p), _I32, _I32, _I32, _P, _P, _P, _I32,
                                _P, _P, _P],
    "plz_peer_alloc": [_I64, C.POINTER(C.c_void_p), C.c_char_p],
    "plz_peer_open": [C.c_char_p, C.POINTER(C.c_void_p)],
    "plz_peer_copy": [_P, _P, _I64, _P],
    "plz_peer_zero": [_P, _I64, _P],
    "plz_peer_close": [_P],
    "plz_peer_free": [_P],
    "plz_reduce_slots": [_P, _I32, _I64, _P, _F, _P],
    "plz_bwd_dw_hard": [_WP, _P, _I64, _P, _I64, _I32, _P, _P],
    "plz_lora_bwd": [_P, _I64, _P, _I64, _P, _P, _I32, _I32, _I32, _I32, _P, _P, _P],
    "plz_rms_rstd": [_P, _I64, _I32, _I32, _F, _P, _P],
    "plz_swiglu_bwd": [_P, _I64, _P, _I64, _P, _I64, _I32, _I32, _P, _I64, _P, _I64, _P],
    "plz_rmsnorm_bwd": [_P, _I64, _P, _I64, _P, _P, _I32, _I32, _P, _I64, _P, _P],
    "plz_hard_fwd_norm": [_WP, _P, _I64, _I32, _P, _P, _P, _I64, _P],
    "plz_mlp_gate_up_fwd": [_WP, _WP, _P, _I64, _I32, _P, _P, _P, _I64, _P],
    "plz_mlp_gate_up_fwd_keep": [_WP, _WP, _P, _I64, _I32, _P, _P, _P, _I64, _P, _P, _I64, _P],
    "plz_adamw_step": [_P, _P, _P, _P, _I32, _F, _I64, _F, _F, _F, _F, _F, _I32, _F, _F, _I32, _P, _I32, _P],
    "plz_hard_fwd_bias": [_WP, _P, _I64, _I32, _P, _P, _I64, _P],
    "plz_col_sum": [_P, _I64, _I32, _I32, _P, _P],
    "plz_soft_weights": [_I32, C.POINTER(_WP), C.POINTER(_GP), C.POINTER(_NP), _F, _I32, C.POINTER(C.POINTER(SoftOut)), _P],
    "plz_soft_bwd_elementwise": [_WP, _P, _I32, _I64, _I64, _P, _I64, _I64, _I64, _GP, _P, _P],
    "plz_weight_grad": [_P, _I64, _P, _I64, _I32, _I32, _I32, _P, _I64, _I64, _P],
    "plz_attn_fwd": [_P, _I64, _P, _I64, _P, _I64, _I32, _I32, _I32, _I32, _I32, _F, _P, _I64, _P, _P],
    "plz_attn_bwd": [_P, _I64, _P, _I64, _P, _I64, _P, _P, _I64, _P, _I32, _I32, _I32, _I32, _I32, _F, _P, _P, _P, _P, _P],
    "plz_attn_decode_ws_bytes": [_I32, _I32, _I32, _I32],
    "plz_attn_decode": [_P, _I64, _P, _P, _I64, _I64, _I32, _I32, _I32, _I32, _I32, _F, _P, _I64, _P, _I64, _P],
    "plz_embed_gather": [_P, _I64, _P, _I64, _I32, _I64, _P, _I64, _P, _P],
    "plz_rmsnorm_fwd": [_P, _I64, _P, _I32, _I32, _F, _P, _I64, _P, _P],
    "plz_add_rmsnorm_fwd": [_P, _I64, _P, _I64, _P, _I64, _P, _I32, _I32, _F, _P, _I64, _P, _P],
    "plz_qknorm_rope_fwd2": [_P, _I64, _P, _I32, _P, _I64, _P, _I64, _P, _I32, _P, _I64, _P, _P, _I64, _I32, _I32, _F, _P],
    "plz_qknorm_rope_fwd": [_P, _I64, _P, _P, _P, _I64, _I32, _I32, _I32, _F, _P, _I64, _P],
    "plz_qknorm_rope_bwd": [_P, _I64, _P, _P, _P, _P, _I64, _I64, _I32, _I32, _I32, _F, _P, _I64, _P, _P],
    "plz_swiglu_fwd": [_P, _I64, _P, _I64, _I32, _I32, _P, _I64, _P],
    "plz_add": [_P, _I64, _P, _I64, _P, _I64, _I32, _I32, _P, _I64, _P],
    "plz_bwd_dw_hard_lora": [_WP, _P, _I64, _P, _I64, _I32, _P, _P, _P, _I32, _P, _P, _P],
    "plz_distill_loss": [_P, _I64, _P, _I64, _I32, _I32, _F, _F, _F, _P, _P, _P, _I64, _I32, _P],
}
_RESTYPES = {"plz_last_error": C.c_char_p, "plz_launch_count": C.c_uint64, "plz_attn_decode_ws_bytes": C.c_int64}


def lib():
    """Load libplz.so (built by build.py).  Raises if it is absent: there is no other code path."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"{_LIB_PATH} is missing: run `python {os.path.join(_HERE, 'build.py')}` first; "
                               "this package has no fallback implementation")
        _lib = C.CDLL(_LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, C.c_int32)
    return _lib


class PlzError(RuntimeError):
    pass


def check(rc: int, what: str):
    if rc != 0:
        raise PlzError(f"{what} failed with code {rc}: {lib().plz_last_error().decode()}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def device_status():
    """Synchronize and return the device status word (code, where, count); raises if a kernel gave up."""
    out = (C.c_uint32 * 4)()
    check(lib().plz_device_status(out), "plz_device_status")
    return tuple(out)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise PlzError("libplz works on CUDA tensors only (no CPU path exists)")


def weight_desc(packed: torch.Tensor, palette: torch.Tensor, N: int, K: int, gs_n: int, gs_k: int) -> Weight:
    _need_cuda(packed, palette)
    assert packed.dtype == torch.uint8 and packed.dim() == 2 and packed.stride(1) == 1
    assert palette.dtype == torch.bfloat16 and palette.is_contiguous()
    assert palette.numel() == (N // gs_n) * (K // gs_k) * 4, "palette size does not match the grouping"
    return Weight(N, K, gs_n, gs_k, packed.data_ptr(), packed.stride(0), palette.data_ptr())


def lora_desc(a_rk: torch.Tensor, b_nr: torch.Tensor, scale: float) -> Lora:
    _need_cuda(a_rk, b_nr)
    assert a_rk.dtype == torch.bfloat16 and b_nr.dtype == torch.bfloat16
    assert a_rk.stride(1) == 1 and b_nr.stride(1) == 1 and a_rk.shape[0] == b_nr.shape[1]
    return Lora(a_rk.shape[0], float(scale), a_rk.data_ptr(), a_rk.stride(0), b_nr.data_ptr(), b_nr.stride(0))


def logits_desc(t: torch.Tensor, layout: str) -> Logits:
    """layout 'nk4': tensor [N, K, 4]; layout '4kn': tensor (4, K, N)."""
    _need_cuda(t)
    dt = {torch.float32: 0, torch.float16: 1}[t.dtype]
    if layout == "nk4":
        return Logits(t.data_ptr(), dt, t.stride(0), t.stride(1), t.stride(2))
    return Logits(t.data_ptr(), dt, t.stride(2), t.stride(1), t.stride(0))


def noise_desc(noise, layout: str, seed: int = 0) -> Noise:
    """noise: None (no noise), a fp32 tensor in the given layout, or the string 'hash' (counter-based)."""
    if noise is None:
        return Noise(0, 0, None, 0, 0, 0)
    if isinstance(noise, str):
        return Noise(2, seed & 0xFFFFFFFF, None, 0, 0, 0)
    _need_cuda(noise)
    assert noise.dtype == torch.float32
    if layout == "nk4":
        return Noise(1, 0, noise.data_ptr(), noise.stride(0), noise.stride(1), noise.stride(2))
    return Noise(1, 0, noise.data_ptr(), noise.stride(2), noise.stride(1), noise.stride(0))
