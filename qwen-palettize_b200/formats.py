"""On-disk formats of the reference -> the native packed device layout (and back).

  .idx2        2-bit indices of a Linear, flattened in (in_dim, out_dim) = (K, N) row-major order, 4 per byte, element i in
               bits 2*(i%4).. of byte i//4 (writer: pack_idx2 / pack_indices_transposed_2bit, scripts/palettize_core.py:31-48;
               reader: load_indices, :167-172).  The device layout of this library packs along K instead ([N, K/4]), so a
               file is transposed once at load time by two device kernels (unpack to (K, N) int8, pack along K).
  .lut_scalar  fp16 palette entries, flat, 4 per group of 256 output columns (write_lut_scalar, scripts/palettize_pytorch.py:150-159;
               load_lut, scripts/palettize_core.py:175-178) -> bf16 (N/256, 4), the reference's runtime palette.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)

import plz_ops as ops  # noqa: E402


def load_idx2(path_or_bytes, out_dim: int, in_dim: int, device="cuda"):
    """Returns (packed uint8 [N, K/4] in the native layout, indices int8 (K, N) in the reference's runtime layout)."""
    data = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    N, K = out_dim, in_dim
    assert N % 4 == 0, "out_dim must be a multiple of 4 for a row-aligned .idx2"
    need = K * N // 4
    if len(data) < need:
        raise ValueError(f".idx2 payload has {len(data)} bytes, {need} needed for ({K}, {N})")
    file_rows = torch.from_numpy(np.frombuffer(data, dtype=np.uint8, count=need).copy()).reshape(K, N // 4).to(device)
    # the file is "packed rows" of a (K, N) matrix: unpack it as such, then pack along K
    idx_kn = ops.unpack_indices(file_rows, N, n_major=True)  # rows here are k, columns n -> int8 (K, N)
    packed = ops.pack_indices(idx_kn, n_major=False)
    return packed, idx_kn


def save_idx2(packed: torch.Tensor, in_dim: int) -> bytes:
    """Native packed [N, K/4] -> .idx2 payload (the inverse of load_idx2; extract_hard_indices + save_state path,
    scripts/train_qwen.py:828-847)."""
    idx_kn = ops.unpack_indices(packed, in_dim, n_major=False)      # (K, N) int8
    file_rows = ops.pack_indices(idx_kn, n_major=True)               # rows = k, packed along n
    return file_rows.contiguous().cpu().numpy().tobytes()


def load_lut_scalar(path_or_bytes, device="cuda") -> torch.Tensor:
    data = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    lut = torch.from_numpy(np.frombuffer(data, dtype=np.float16).copy())
    return lut.reshape(-1, 4).to(torch.bfloat16).to(device)
