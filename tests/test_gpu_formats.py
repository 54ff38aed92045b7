"""Bit-exact checks of the integer work on the GPU: packing, unpacking, palette lookup, hard argmax."""
import numpy as np
import pytest
import torch

import plz_oracle as O
from helpers import check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K", [(8, 64), (40, 192), (256, 512), (1000, 2560)])
def test_pack_unpack_bit_exact(N, K):
    import plz_ops as ops
    g = torch.Generator().manual_seed(N * 7 + K)
    idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
    want = O.pack_rows(idx.numpy())
    got_n = ops.pack_indices(idx.cuda().view(torch.int8), n_major=True)
    got_r = ops.pack_indices(idx.t().contiguous().cuda().view(torch.int8), n_major=False)  # reference (K, N) layout
    assert np.array_equal(got_n.cpu().numpy(), want)
    assert np.array_equal(got_r.cpu().numpy(), want)
    back = ops.unpack_indices(got_n, K, n_major=True)
    assert torch.equal(back.cpu().view(torch.uint8), idx)
    back_r = ops.unpack_indices(got_n, K, n_major=False)
    assert torch.equal(back_r.cpu().view(torch.uint8), idx.t())
    check_status()


def test_pack_known_answers():
    import plz_ops as ops
    idx = torch.tensor([[0, 1, 2, 3] * 16, [3, 0, 1, 2] * 16], dtype=torch.int8).cuda()
    got = ops.pack_indices(idx, n_major=True).cpu().numpy()
    assert (got[0] == 0xE4).all() and (got[1] == 0x93).all()


@pytest.mark.parametrize("N,K,gs_n,gs_k", [(256, 256, 1, 256), (512, 1024, 256, 1024), (384, 512, 1, 64), (256, 2560, 128, 256)])
def test_dequantize_bit_exact(N, K, gs_n, gs_k):
    import plz_ops as ops
    g = torch.Generator().manual_seed(11)
    idx = torch.randint(0, 4, (N, K), generator=g, dtype=torch.uint8)
    pal = (torch.randn((N // gs_n) * (K // gs_k), 4, generator=g) * 0.02).to(torch.bfloat16)
    w = ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), pal.cuda(), N, K, gs_n, gs_k)
    got = ops.dequantize(w).cpu()
    want = O.dequantize(idx.long(), pal, gs_n, gs_k)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    check_status()


@pytest.mark.parametrize("layout,dtype", [("nk4", torch.float32), ("4kn", torch.float16), ("4kn", torch.float32)])
def test_hard_argmax_bit_exact_with_ties(layout, dtype):
    import plz_ops as ops
    N, K = 512, 320
    g = torch.Generator().manual_seed(5)
    lg = torch.randn(N, K, 4, generator=g).to(dtype)
    lg[:64, :, 1] = lg[:64, :, 0]      # ties: the lowest index must win
    lg[64:128, :, 3] = lg[64:128, :, 2]
    lg[128:160] = 0
    want = O.pack_rows(torch.argmax(lg.float(), -1).to(torch.uint8).numpy())
    dev = lg.cuda() if layout == "nk4" else O.from_nk_logits(lg).cuda()
    pal = torch.zeros(N * (K // 64), 4, dtype=torch.bfloat16).cuda()
    w = ops.PackedWeight(ops.empty_packed(N, K, "cuda"), pal, N, K, 1, 64)
    ops.soft_select(w, dev, layout, want_packed=True)
    assert np.array_equal(w.packed.cpu().numpy(), want)
    check_status()


def test_soft_weights_match_oracle():
    import plz_ops as ops
    N, K, tau = 256, 512, 0.8
    g = torch.Generator().manual_seed(9)
    lg = torch.randn(N, K, 4, generator=g)
    nz = O.gumbel_from_uniform(torch.rand(N, K, 4, generator=g))
    pal = (torch.randn(N, K // 256, 4, generator=g) * 0.02).sort(-1).values.to(torch.bfloat16)
    _, w_soft, _, _ = O.soft_weights(lg, nz, pal, tau, 1, 256)
    w = ops.PackedWeight(ops.empty_packed(N, K, "cuda"), pal.cuda(), N, K, 1, 256)
    got = ops.soft_select(w, lg.cuda(), "nk4", noise=nz.cuda(), tau=tau, want_packed=False, want_soft=True).cpu().float()
    assert (got - w_soft).abs().max() <= 2e-2 * w_soft.abs().max()   # one bf16 rounding of a |w| <= 0.1 value
    assert (got.min() >= pal.float().min()) and (got.max() <= pal.float().max())
    # counter-based noise: same integer stream as the oracle, float part to a few ulp
    got_h = ops.soft_select(w, lg.cuda(), "nk4", noise="hash", seed=123, tau=tau, want_packed=False, want_soft=True).cpu().float()
    _, w_soft_h, _, _ = O.soft_weights(lg, O.gumbel_hash(123, N, K), pal, tau, 1, 256)
    assert (got_h - w_soft_h).abs().max() <= 2e-2 * w_soft_h.abs().max()
    check_status()


def test_idx2_and_lut_files_load_into_the_native_layout(golden):
    import formats
    data = golden["idx2_bytes"].tobytes()
    packed, idx_kn = formats.load_idx2(data, 64, 96)
    want_kn = golden["idx2_kn"].astype(np.uint8)                 # (K=96, N=64) as the reference's reader returns it
    assert np.array_equal(idx_kn.cpu().numpy().astype(np.uint8), want_kn)
    assert np.array_equal(packed.cpu().numpy(), O.pack_rows(want_kn.T.copy()))
    assert formats.save_idx2(packed, 96) == data                 # round trip back to the file payload
    pal = formats.load_lut_scalar(golden["lut_bytes"].tobytes())
    assert pal.shape == (2, 4) and pal.dtype == torch.bfloat16
    assert torch.equal(pal.cpu(), torch.from_numpy(golden["lut_vals"]).to(torch.bfloat16).reshape(2, 4))
    check_status()


@pytest.fixture(scope="module")
def real():
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return np.load(os.path.join(root, "tests", "golden", "real_k_proj.npz"))


def test_real_shipped_pair_loads_bit_exact(tmp_path, real):
    """One .idx2 / .lut_scalar pair of the reference's palettized/superblock_0 (stored with what the reference's own
    load_indices / load_lut return for it): the device loader must reproduce both bit for bit, write the same bytes back,
    and the loaded weight must run."""
    import json
    import formats as F
    import plz_ops as ops
    N, K = 1024, 2560
    entry, name = json.loads(str(real["entry"])), str(real["name"])
    idx_payload, lut_payload = real["idx2"].tobytes(), real["lut_scalar"].tobytes()
    packed, idx_kn = F.load_idx2(idx_payload, N, K)
    assert np.array_equal(packed.cpu().numpy(), real["ref_packed_nk"])
    assert np.array_equal(O.pack_rows(idx_kn.t().contiguous().cpu().numpy().astype(np.uint8)), real["ref_packed_nk"])
    pal = F.load_lut_scalar(lut_payload)
    assert pal.shape == (N // 256, 4) and torch.equal(pal.cpu(), torch.from_numpy(real["ref_lut"]).to(torch.bfloat16).reshape(-1, 4))
    assert F.save_idx2(packed, K) == idx_payload
    # through the directory reader (metadata.json + sha256 verification)
    open(tmp_path / entry["index_file"], "wb").write(idx_payload)
    open(tmp_path / entry["lut_file"], "wb").write(lut_payload)
    F.write_metadata(str(tmp_path / "metadata.json"), [(name, entry)])
    loaded = F.load_palettized_dir(str(tmp_path))
    w, idx2 = loaded[name]
    assert torch.equal(w.packed, packed) and torch.equal(idx2, idx_kn) and (w.N, w.K, w.gs_n, w.gs_k) == (N, K, 256, K)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(200, K, generator=g).to(torch.bfloat16)
    y, _ = ops.hard_forward(w, x.cuda())
    check_status()
    idx_nk = torch.from_numpy(O.unpack_rows(real["ref_packed_nk"], K)).long()
    want = O.hard_forward(x, O.dequantize(idx_nk, pal.cpu(), 256, K))
    from helpers import assert_close
    assert_close(y, want, "y from the shipped k_proj weights")


def test_checkpoint_round_trip(tmp_path):
    """save_checkpoint writes the reference's checkpoint layout (.idx2 + .lut_scalar per Linear, .pt per small parameter,
    _resume.json); load_checkpoint and load_palettized_dir read it back bit for bit."""
    import json
    import os
    import formats as F
    import plz_ops as ops
    g = torch.Generator().manual_seed(3)
    shapes = {"layers.0.self_attn.q_proj.base": (512, 256), "layers.0.mlp.down_proj.base": (256, 768)}
    lin = {}
    for name, (N, K) in shapes.items():
        lg = torch.randn(N, K, 4, generator=g).cuda()
        pal = (torch.randn(N // 256, 4, generator=g) * 0.02).to(torch.bfloat16).cuda()
        w = ops.PackedWeight(ops.empty_packed(N, K, "cuda"), pal, N, K, 256, K)
        ops.soft_select(w, lg, "nk4", want_packed=True)               # hard indices = argmax of the trained logits
        lin[name] = (w.packed, pal, K)
    small = {"layers.0.self_attn.q_proj.lora_A": torch.randn(256, 16, generator=g).to(torch.bfloat16).cuda(),
             "layers.0.input_layernorm.weight": torch.randn(256, generator=g).to(torch.bfloat16).cuda()}
    n = F.save_checkpoint(str(tmp_path), lin, small, sb_idx=0, step=120, cos=0.93, loss=0.08)
    assert n == (2, 2)
    files = sorted(os.listdir(tmp_path))
    assert "layers_0_self_attn_q_proj_base.idx2" in files and "layers_0_self_attn_q_proj_lora_A.pt" in files
    assert json.load(open(tmp_path / "_resume.json")) == {"step": 120, "cos": 0.93, "loss": 0.08, "sb_idx": 0}
    resume, lin2, small2 = F.load_checkpoint(str(tmp_path), shapes, list(small) + ["not.saved"])
    assert resume["step"] == 120 and set(small2) == set(small)
    for name in shapes:
        packed, pal, idx_kn = lin2[name]
        assert torch.equal(packed, lin[name][0])
        assert torch.equal(pal, lin[name][1].to(torch.float16).to(torch.bfloat16))   # palettes travel as fp16
        lg = F.one_hot_logits(idx_kn)                                                # restart logits: +1 on the index, -1 elsewhere
        assert lg.shape == (4,) + tuple(idx_kn.shape) and torch.equal(lg.argmax(0).to(torch.int8), idx_kn)
        assert lg.float().sum(0).eq(-2).all()
    for k in small:
        assert torch.equal(small2[k], small[k])
    both = F.load_palettized_dir(str(tmp_path))                                      # the checkpoint also reads as a palettized dir
    assert set(both) == set(shapes) and torch.equal(both["layers.0.mlp.down_proj.base"][0].packed, lin["layers.0.mlp.down_proj.base"][0])
    check_status()
