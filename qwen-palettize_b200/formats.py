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


# --------------------------------------------------------------------------------------------------------------
# metadata.json, palettized directories and training checkpoints
# --------------------------------------------------------------------------------------------------------------
import hashlib  # noqa: E402
import json  # noqa: E402

BITWIDTH, GROUP_SIZE = 2, 256


def sanitize_name(name: str) -> str:
    """Tensor / module name -> file stem (sanitize_name, scripts/palettize_pytorch.py:20-22)."""
    return name.replace(".", "_").replace("/", "_").replace("[", "").replace("]", "")


def lut_scalar_bytes(palette: torch.Tensor) -> bytes:
    """Palette (groups, 4) -> .lut_scalar payload: flat fp16 (write_lut_scalar, scripts/palettize_pytorch.py:150-159)."""
    return palette.detach().reshape(-1).to(torch.float16).cpu().numpy().tobytes()


def tensor_meta(name: str, out_dim: int, in_dim: int, idx_payload: bytes, lut_payload: bytes, cos: float | None = None) -> dict:
    """One entry of metadata.json["tensors"], with the keys and values the reference writes
    (palettize_tensor_2bit, scripts/palettize_core.py:122-141)."""
    san = sanitize_name(name)
    m = {"var": name, "dense_shape": [out_dim, in_dim], "indices_shape": [out_dim, in_dim], "bitwidth": BITWIDTH,
         "groups": out_dim // GROUP_SIZE, "group_axis": 1, "group_size": GROUP_SIZE, "nibble_order": "LSB_FIRST",
         "indices_layout": "D0D1", "consumer_transpose_y": False, "index_file": f"{san}.idx2", "lut_file": f"{san}.lut_scalar",
         "sha256_idx": hashlib.sha256(idx_payload).hexdigest(), "sha256_lut": hashlib.sha256(lut_payload).hexdigest(),
         "packed_len_bytes": len(idx_payload), "idx_payload_offset_used": 0, "lut_payload_offset_used": 0}
    if cos is not None:
        m["_achieved_cos"] = cos
    return m


def write_metadata(path: str, tensor_metas, teacher_id: str = "qwen35-4b"):
    """metadata.json as write_metadata_json leaves it (scripts/palettize_core.py:144-153 on top of
    scripts/palettize_pytorch.py:162-181): {"tensors": {name: meta}, "default_group_size", "teacher_id", "bitwidth"}."""
    if isinstance(tensor_metas, dict):
        tensor_metas = list(tensor_metas.items())
    meta = {"tensors": {n: m for n, m in tensor_metas}, "default_group_size": GROUP_SIZE, "teacher_id": teacher_id, "bitwidth": BITWIDTH}
    with open(path, "w") as f:
        json.dump(meta, f, indent=2)


def read_metadata(path: str) -> dict:
    """Parse and validate a metadata.json: returns {tensor name: entry}. Accepts both the file the palettizer writes
    ("default_group_size") and the shipped palettized/superblock_0 one ("group_size", "quantization_type", ...).
    Only what this library can run is accepted: 2-bit, LSB-first, (K, N) flattening ("D0D1"), groups along out_dim."""
    with open(path) as f:
        meta = json.load(f)
    tensors = meta.get("tensors")
    if not isinstance(tensors, dict):
        raise ValueError(f"{path}: no 'tensors' table")
    if meta.get("bitwidth", BITWIDTH) != BITWIDTH:
        raise ValueError(f"{path}: bitwidth {meta.get('bitwidth')} (only 2-bit palettes are supported)")
    for name, t in tensors.items():
        for key in ("dense_shape", "index_file", "lut_file"):
            if key not in t:
                raise ValueError(f"{path}: tensor {name} lacks '{key}'")
        out_dim, in_dim = t["dense_shape"]
        gs = t.get("group_size", meta.get("group_size", meta.get("default_group_size", GROUP_SIZE)))
        if t.get("bitwidth", BITWIDTH) != BITWIDTH or t.get("nibble_order", "LSB_FIRST") != "LSB_FIRST" or \
           t.get("indices_layout", "D0D1") != "D0D1" or t.get("consumer_transpose_y", False):
            raise ValueError(f"{path}: tensor {name} uses an index format other than 2-bit LSB_FIRST D0D1")
        if out_dim % gs or t.get("groups", out_dim // gs) != out_dim // gs:
            raise ValueError(f"{path}: tensor {name}: {t.get('groups')} groups do not tile out_dim {out_dim} by {gs}")
        if "packed_len_bytes" in t and t["packed_len_bytes"] != (out_dim * in_dim + 3) // 4:
            raise ValueError(f"{path}: tensor {name}: packed_len_bytes {t['packed_len_bytes']} != out_dim*in_dim/4")
    return tensors


def verify_files(directory: str, entry: dict):
    """Read the two payloads of a metadata entry and check sizes and sha256. Returns (idx_payload, lut_payload)."""
    out_dim, in_dim = entry["dense_shape"]
    gs = entry.get("group_size", GROUP_SIZE)
    idx = open(os.path.join(directory, entry["index_file"]), "rb").read()[entry.get("idx_payload_offset_used", 0):]
    lut = open(os.path.join(directory, entry["lut_file"]), "rb").read()[entry.get("lut_payload_offset_used", 0):]
    if len(idx) != (out_dim * in_dim + 3) // 4:
        raise ValueError(f"{entry['index_file']}: {len(idx)} bytes, expected {(out_dim * in_dim + 3) // 4}")
    if len(lut) != (out_dim // gs) * 4 * 2:
        raise ValueError(f"{entry['lut_file']}: {len(lut)} bytes, expected {(out_dim // gs) * 8}")
    for payload, key in ((idx, "sha256_idx"), (lut, "sha256_lut")):
        if key in entry and hashlib.sha256(payload).hexdigest() != entry[key]:
            raise ValueError(f"{entry['var'] if 'var' in entry else entry['index_file']}: {key} mismatch")
    return idx, lut


def load_palettized_dir(directory: str, device="cuda", names=None, verify: bool = True):
    """{tensor name: (PackedWeight in the reference grouping gs_n = 256 / gs_k = K, indices int8 (K, N))} for the tensors of
    a palettized directory (metadata.json + one .idx2 / .lut_scalar pair per Linear), i.e. what
    PalettizedLinear is built from (scripts/qwen_model.py:769-794)."""
    out = {}
    for name, t in read_metadata(os.path.join(directory, "metadata.json")).items():
        if names is not None and name not in names:
            continue
        N, K = t["dense_shape"]
        if verify:
            idx, lut = verify_files(directory, t)
        else:
            idx = open(os.path.join(directory, t["index_file"]), "rb").read()
            lut = open(os.path.join(directory, t["lut_file"]), "rb").read()
        packed, idx_kn = load_idx2(idx, N, K, device)
        pal = load_lut_scalar(lut, device)
        out[name] = (ops.PackedWeight(packed, pal, N, K, t.get("group_size", GROUP_SIZE), K), idx_kn)
    return out


def save_checkpoint(out_dir: str, linears: dict, small_params: dict, sb_idx: int, step: int, cos: float, loss: float,
                    write_meta: bool = True):
    """Training checkpoint in the reference's format (save_state, scripts/train_qwen.py:813-864):
      <sanitized module name>.idx2 + .lut_scalar per palettized Linear, one <name with dots as underscores>.pt per other
      trainable parameter (LoRA factors, norms), and _resume.json {step, cos, loss, sb_idx}.
    linears: {module name: (packed uint8 [N, K/4] hard indices in the native layout -- after soft training the argmax of the
      logits, which plz_soft_select writes -- , palette (N/256, 4), K)}.
    Also writes a metadata.json with the sha256 of every payload (the reference's checkpoints carry none; its palettized
    directories do), so that a checkpoint can be read back with load_palettized_dir."""
    os.makedirs(out_dir, exist_ok=True)
    metas = []
    for name, (packed, palette, K) in linears.items():
        san = sanitize_name(name)
        idx_payload = save_idx2(packed, K)
        lut_payload = lut_scalar_bytes(palette)
        with open(os.path.join(out_dir, f"{san}.idx2"), "wb") as f:
            f.write(idx_payload)
        with open(os.path.join(out_dir, f"{san}.lut_scalar"), "wb") as f:
            f.write(lut_payload)
        metas.append((name, tensor_meta(name, packed.shape[0], K, idx_payload, lut_payload)))
    for name, p in small_params.items():
        torch.save(p.detach().cpu(), os.path.join(out_dir, name.replace(".", "_") + ".pt"))
    with open(os.path.join(out_dir, "_resume.json"), "w") as f:
        json.dump({"step": step, "cos": cos, "loss": loss, "sb_idx": sb_idx}, f)
    if write_meta:
        write_metadata(os.path.join(out_dir, "metadata.json"), metas)
    return len(metas), len(small_params)


def load_checkpoint(resume_dir: str, linear_shapes: dict, small_names, device="cuda"):
    """Inverse of save_checkpoint / reader of the reference's checkpoints (load_state, scripts/train_qwen.py:867-950).
    linear_shapes: {module name: (N, K)}. Returns (resume dict, {name: (packed, palette bf16, indices int8 (K, N))},
    {name: tensor}); files that are absent are skipped, as the reference does."""
    with open(os.path.join(resume_dir, "_resume.json")) as f:
        resume = json.load(f)
    lin, small = {}, {}
    for name, (N, K) in linear_shapes.items():
        san = sanitize_name(name)
        ip, lp = os.path.join(resume_dir, f"{san}.idx2"), os.path.join(resume_dir, f"{san}.lut_scalar")
        if not (os.path.exists(ip) and os.path.exists(lp)):
            continue
        packed, idx_kn = load_idx2(ip, N, K, device)
        lin[name] = (packed, load_lut_scalar(lp, device), idx_kn)
    for name in small_names:
        pp = os.path.join(resume_dir, name.replace(".", "_") + ".pt")
        if os.path.exists(pp):
            small[name] = torch.load(pp, map_location=device, weights_only=True)
    return resume, lin, small


def one_hot_logits(idx_kn: torch.Tensor, hi: float = 1.0, lo: float = -1.0) -> torch.Tensor:
    """fp16 (4, K, N) logits that restart soft training from loaded indices: `hi` on the stored index, `lo` elsewhere
    (+-1 on resume so that gradients flow, scripts/train_qwen.py:905-916; +-10 at first construction,
    scripts/qwen_model.py:135-143)."""
    K, N = idx_kn.shape
    lg = torch.full((4, K, N), lo, dtype=torch.float16, device=idx_kn.device)
    lg.scatter_(0, idx_kn.long().unsqueeze(0), hi)
    return lg
