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
