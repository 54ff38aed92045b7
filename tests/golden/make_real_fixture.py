"""Build tests/golden/real_k_proj.npz from ONE pair of the reference's shipped palettized files, read with the reference's
own loaders.

    PLZ_REFERENCE_DIR=<reference checkout> python tests/golden/make_real_fixture.py

The pair is model.layers.3.self_attn.k_proj.weight of palettized/superblock_0 (out_dim 1024, in_dim 2560: the smallest
Linear of the set).  Stored: the two payloads as they are on disk, the tensor's metadata.json entry, and what the reference's
load_indices / load_lut (scripts/palettize_core.py:167-178) return for them -- the indices as the (K, N) uint8 matrix the
reference builds its module from, re-packed along K ([N, K/4], 4 per byte, LSB first) to keep the file small.
The reference is imported, never copied."""
import hashlib
import json
import os
import sys

import numpy as np

REF = os.environ.get("PLZ_REFERENCE_DIR")
if not REF or not os.path.isdir(REF):
    sys.exit("set PLZ_REFERENCE_DIR to a checkout of the reference repository (pkhairkh/qwen-palettize)")
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.dont_write_bytecode = True
sys.path.insert(0, os.path.join(REF, "scripts"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import plz_oracle as O  # noqa: E402
from palettize_core import load_indices, load_lut  # noqa: E402

NAME = "model.layers.3.self_attn.k_proj.weight"
d = os.path.join(REF, "palettized", "superblock_0")
meta = json.load(open(os.path.join(d, "metadata.json")))
entry = meta["tensors"][NAME]
out_dim, in_dim = entry["dense_shape"]
idx_bytes = open(os.path.join(d, entry["index_file"]), "rb").read()
lut_bytes = open(os.path.join(d, entry["lut_file"]), "rb").read()
assert hashlib.sha256(idx_bytes).hexdigest() == entry["sha256_idx"] and hashlib.sha256(lut_bytes).hexdigest() == entry["sha256_lut"]
idx_kn = load_indices(os.path.join(d, entry["index_file"]), out_dim, in_dim).numpy()      # (K, N) uint8, reference loader
lut = load_lut(os.path.join(d, entry["lut_file"])).numpy()                                # flat fp32, reference loader
assert idx_kn.shape == (in_dim, out_dim) and lut.size == out_dim // 256 * 4
top = {k: v for k, v in meta.items() if k != "tensors"}
np.savez_compressed(os.path.join(HERE, "real_k_proj.npz"),
                    idx2=np.frombuffer(idx_bytes, np.uint8), lut_scalar=np.frombuffer(lut_bytes, np.uint8),
                    entry=np.array(json.dumps(entry)), meta_top=np.array(json.dumps(top)), name=np.array(NAME),
                    ref_packed_nk=O.pack_rows(np.ascontiguousarray(idx_kn.T)), ref_lut=lut.astype(np.float32))
print("wrote", os.path.join(HERE, "real_k_proj.npz"), os.path.getsize(os.path.join(HERE, "real_k_proj.npz")), "bytes")
