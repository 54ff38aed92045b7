"""Host side of the on-disk formats: metadata.json schema, payload verification, file naming.  No GPU.
Where a reference checkout is available (PLZ_REFERENCE_DIR) all 25 shipped pairs of palettized/superblock_0 are parsed and
verified against the sha256 values of their metadata.json."""
import hashlib
import json
import os

import numpy as np
import pytest

REF = os.environ.get("PLZ_REFERENCE_DIR")
HAVE_REF = bool(REF) and os.path.isdir(os.path.join(REF or "", "palettized", "superblock_0"))
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def real():
    return np.load(os.path.join(ROOT, "tests", "golden", "real_k_proj.npz"))


def test_tensor_meta_has_the_reference_keys_and_values(real):
    import formats as F
    entry = json.loads(str(real["entry"]))
    name = str(real["name"])
    mine = F.tensor_meta(name, 1024, 2560, real["idx2"].tobytes(), real["lut_scalar"].tobytes(), cos=entry["_achieved_cos"])
    assert mine == entry                                 # same keys, same values, same sha256 of the same payloads
    assert F.sanitize_name(name) + ".idx2" == entry["index_file"]
    assert F.sanitize_name("a.b/c[3]") == "a_b_c3"


def test_metadata_round_trip_and_validation(tmp_path, real):
    import formats as F
    entry = json.loads(str(real["entry"]))
    name = str(real["name"])
    p = tmp_path / "metadata.json"
    F.write_metadata(str(p), [(name, entry)])
    raw = json.load(open(p))
    assert raw["default_group_size"] == 256 and raw["teacher_id"] == "qwen35-4b" and raw["bitwidth"] == 2
    assert F.read_metadata(str(p)) == {name: entry}
    # the shipped file's top-level keys are accepted as well
    top = json.loads(str(real["meta_top"]))
    json.dump(dict(top, tensors={name: entry}), open(p, "w"))
    assert list(F.read_metadata(str(p))) == [name]
    for key, bad in (("bitwidth", 4), ("nibble_order", "MSB_FIRST"), ("groups", 5), ("packed_len_bytes", 7)):
        json.dump({"tensors": {name: dict(entry, **{key: bad})}}, open(p, "w"))
        with pytest.raises(ValueError):
            F.read_metadata(str(p))
    json.dump({"tensors": {name: {k: v for k, v in entry.items() if k != "lut_file"}}}, open(p, "w"))
    with pytest.raises(ValueError):
        F.read_metadata(str(p))


def test_verify_files_detects_damage(tmp_path, real):
    import formats as F
    entry = json.loads(str(real["entry"]))
    idx, lut = real["idx2"].tobytes(), real["lut_scalar"].tobytes()
    open(tmp_path / entry["index_file"], "wb").write(idx)
    open(tmp_path / entry["lut_file"], "wb").write(lut)
    got = F.verify_files(str(tmp_path), entry)
    assert got == (idx, lut)
    flipped = bytearray(idx)
    flipped[1000] ^= 0x10
    open(tmp_path / entry["index_file"], "wb").write(bytes(flipped))
    with pytest.raises(ValueError, match="sha256_idx"):
        F.verify_files(str(tmp_path), entry)
    open(tmp_path / entry["index_file"], "wb").write(idx[:-4])
    with pytest.raises(ValueError, match="bytes"):
        F.verify_files(str(tmp_path), entry)


def test_fixture_matches_the_packing_rule(real):
    """The stored reference-loader output is what the packing rule gives from the payload: element i of the flattened
    (K, N) matrix in bits 2 * (i % 4) of byte i // 4 (known answers of scripts/verify_2bit_format.py:50-109)."""
    import plz_oracle as O
    N, K = 1024, 2560
    flat = O.unpack_rows(real["idx2"].reshape(1, -1), K * N)[0]           # CPU restatement of unpack_idx2
    idx_kn = flat.reshape(K, N)
    assert np.array_equal(O.pack_rows(np.ascontiguousarray(idx_kn.T)), real["ref_packed_nk"])
    assert np.array_equal(np.frombuffer(real["lut_scalar"].tobytes(), np.float16).astype(np.float32), real["ref_lut"])


@pytest.mark.skipif(not HAVE_REF, reason="needs a checkout of the reference (PLZ_REFERENCE_DIR)")
def test_all_shipped_pairs_parse_and_verify():
    import formats as F
    d = os.path.join(REF, "palettized", "superblock_0")
    tensors = F.read_metadata(os.path.join(d, "metadata.json"))
    assert len(tensors) == 25
    total = 0
    for name, t in tensors.items():
        idx, lut = F.verify_files(d, t)                   # sizes + sha256 of both payloads
        assert t["index_file"] == F.sanitize_name(name) + ".idx2"
        assert F.tensor_meta(name, *t["dense_shape"], idx, lut, cos=t.get("_achieved_cos")) == t
        total += len(idx)
    assert total == sum(t["packed_len_bytes"] for t in tensors.values())
