"""The CPU oracle against the golden vectors produced from the reference's own PyTorch code
(oracle/pin_against_reference.py) and against the reference's packing known answers."""
import numpy as np
import torch

import plz_oracle as O
from helpers import assert_close, bf16_from_bits


def test_packing_known_answers():
    # scripts/verify_2bit_format.py:50-109
    assert O.pack_flat(np.array([0, 1, 2, 3])) == b"\xE4"
    assert O.pack_flat(np.array([3, 0, 1, 2])) == b"\x93"
    assert O.pack_flat(np.array([1, 2, 3])) == b"\x39"
    rng = np.random.default_rng(0)
    idx = rng.integers(0, 4, (9, 100), dtype=np.uint8)
    assert np.array_equal(O.unpack_rows(O.pack_rows(idx), 100), idx)
    # equality with numpy's little-endian bit packing (the CoreML convention the reference checks)
    bits = np.unpackbits(idx.reshape(-1, 1), bitorder="little", axis=-1)[:, :2]
    assert O.pack_rows(idx).tobytes() == np.packbits(bits.flatten(), bitorder="little").tobytes()


def test_hash_sampler_integer_part(golden):
    u = O.gumbel_hash_u24(int(golden["hash_seed"]), np.arange(8, dtype=np.uint32))
    assert np.array_equal(u, golden["hash_u24"])
    # scalar restatement with python integers
    def scalar(seed, idx):
        m = 0xFFFFFFFF
        x = (seed ^ (idx * 0x9E3779B9)) & m
        x ^= x >> 13
        x = (x * 1103515245 + 12345) & m
        x ^= x >> 17
        x = (x * 1103515245 + 12345) & m
        return x & 0xFFFFFF
    assert [scalar(5, i) for i in range(8)] == [int(v) for v in u]
    g = O.gumbel_hash(5, 3, 4)
    assert g.shape == (3, 4, 4) and torch.isfinite(g).all()


def _load(golden):
    d = {k: golden[k] for k in golden.files}
    t = {}
    for k in ("x", "dy", "palette", "lora_a_kr", "lora_b_nr", "w_hard_kn", "y_hard", "y_mod", "dx_hard", "y_lora",
              "dx_lora", "da_kr", "db_nr", "w_ste_kn", "y_soft", "dx_soft"):
        t[k] = bf16_from_bits(d[k])
    for k in ("logits", "noise", "p_4kn", "dlogits_4kn", "dpal_soft", "dpal_hard"):
        t[k] = torch.from_numpy(d[k])
    t["indices"] = torch.from_numpy(d["indices"].astype(np.int64))
    t["argmax_kn"] = torch.from_numpy(d["argmax_kn"].astype(np.int64))
    meta = {k: d[k].item() for k in ("M", "K", "N", "GS", "R", "tau", "scale")}
    return t, meta


def test_hard_path_against_reference(golden):
    t, m = _load(golden)
    idx_nk = O.to_nk_indices(t["indices"])
    w = O.dequantize(idx_nk, t["palette"], m["GS"], m["K"])
    assert torch.equal(w.t(), t["w_hard_kn"])  # gather is bit exact
    y = O.hard_forward(t["x"], w)
    assert_close(y, t["y_hard"], "hard y vs torch_hard_forward")
    assert_close(y, t["y_mod"], "hard y vs PalettizedLinear fallback")
    dx, dpal = O.hard_backward(t["x"], t["dy"], idx_nk, t["palette"], m["GS"], m["K"])
    assert_close(dx, t["dx_hard"], "hard dX vs autograd")
    assert_close(dpal, t["dpal_hard"], "hard dPalette vs autograd (fp32 activations)")


def test_lora_against_reference(golden):
    t, m = _load(golden)
    w = O.dequantize(O.to_nk_indices(t["indices"]), t["palette"], m["GS"], m["K"])
    a_rk = t["lora_a_kr"].t().contiguous()
    y = (t["x"].float() @ w.float().t() + O.lora_forward(t["x"], a_rk, t["lora_b_nr"], m["scale"])).to(torch.bfloat16)
    assert_close(y, t["y_lora"], "LoRA y vs QwenLoRA")
    dxl, da, db = O.lora_backward(t["x"], t["dy"], a_rk, t["lora_b_nr"], m["scale"])
    assert_close((t["dy"].float() @ w.float() + dxl).to(torch.bfloat16), t["dx_lora"], "LoRA dX")
    # the reference accumulates these two in bf16: looser value bound, same direction
    assert_close(da.t(), t["da_kr"], "dA", rel=2e-2, cos=0.999)
    assert_close(db, t["db_nr"], "dB", rel=2e-2, cos=0.999)


def test_soft_path_against_reference(golden):
    t, m = _load(golden)
    lg, nz = O.to_nk_logits(t["logits"]), O.to_nk_logits(t["noise"])
    p, w_soft, hard, w_hard = O.soft_weights(lg, nz, t["palette"], m["tau"], m["GS"], m["K"])
    assert torch.equal(hard.t(), t["argmax_kn"])          # ties resolved to the lowest index
    assert torch.equal(w_hard.t(), t["w_ste_kn"])
    assert_close(O.from_nk_logits(p), t["p_4kn"], "P", rel=1e-6, cos=0.999999)
    assert (p.sum(-1) - 1).abs().max() < 1e-5
    assert_close(O.hard_forward(t["x"], w_hard), t["y_soft"], "soft (STE) y")
    dx, dlog, dpal, _ = O.soft_backward(t["x"], t["dy"], w_hard, p, t["palette"], m["GS"], m["K"])
    assert_close(dx, t["dx_soft"], "soft dX")
    assert_close(O.from_nk_logits(dlog), t["dlogits_4kn"].float(), "dLogits (reference output is fp16)", rel=2e-3)
    assert_close(dpal, t["dpal_soft"], "dPalette", rel=1e-5, cos=0.999999)


def test_soft_gradients_by_finite_difference():
    """dPalette and dLogits of the pure-soft path against central differences in fp64
    (the reference's own check of dPalette, scripts/test_palettized_v2.py:111-159).
    dLogits carries no 1/tau factor in the reference, so the numeric derivative is scaled by tau."""
    g = torch.Generator().manual_seed(3)
    M, N, K, tau = 5, 4, 64, 0.7
    x = torch.randn(M, K, generator=g, dtype=torch.float64)
    dy = torch.randn(M, N, generator=g, dtype=torch.float64)
    pal = torch.randn(N, 1, 4, generator=g, dtype=torch.float64) * 0.1
    lg = torch.randn(N, K, 4, generator=g, dtype=torch.float64)
    nz = torch.randn(N, K, 4, generator=g, dtype=torch.float64)

    def loss(pal_, lg_):
        p = torch.softmax((lg_ + nz) / tau, -1)
        w = (p * pal_.reshape(N, 1, 4)).sum(-1)
        return ((x @ w.t()) * dy).sum()

    p = torch.softmax((lg + nz) / tau, -1)
    dw = dy.t() @ x
    c = pal.reshape(N, 1, 4).expand(N, K, 4)
    w_soft = (p * c).sum(-1)
    dlog = dw[..., None] * p * (c - w_soft[..., None])
    dpal = (dw[..., None] * p).sum(1)
    eps = 1e-6
    for (n, q) in [(0, 0), (2, 3)]:
        e = torch.zeros_like(pal); e[n, 0, q] = eps
        num = (loss(pal + e, lg) - loss(pal - e, lg)) / (2 * eps)
        assert abs(num - dpal[n, q]) <= 1e-6 * max(1.0, abs(num))
    for (n, k, q) in [(1, 5, 2), (3, 63, 0)]:
        e = torch.zeros_like(lg); e[n, k, q] = eps
        num = (loss(pal, lg + e) - loss(pal, lg - e)) / (2 * eps)
        assert abs(num * tau - dlog[n, k, q]) <= 1e-5 * max(1.0, abs(num))


def test_loss_and_optimizer_against_reference(golden):
    """compute_loss and FP32MasterAdamW + clamp of the reference's training loop (scripts/train_qwen.py:154-249, 1343-1348)."""
    s, t = bf16_from_bits(golden["loss_s"]), bf16_from_bits(golden["loss_t"])
    (loss, l_cos, _, _), ds = O.distill_loss(s, t, 0.5, 0.5)
    assert abs(loss - float(golden["loss_vals"][0])) <= 1e-6 and abs(l_cos - float(golden["loss_vals"][1])) <= 1e-6
    assert_close(ds, torch.from_numpy(golden["loss_ds"]), "dLoss/ds", rel=1e-6, cos=0.999999)
    p0 = torch.from_numpy(golden["adam_p0"])
    grads = list(torch.from_numpy(golden["adam_grads"]))
    _, model, _, _ = O.adamw_reference(p0, grads, 0.05, clamp=(-2.0, 2.0), clamp_master=False)
    assert torch.equal(model, torch.from_numpy(golden["adam_model"]))


def test_disk_formats_against_reference(golden):
    """.idx2 / .lut_scalar payloads written by the reference's own writer (scripts/palettize_core.py:31-48)."""
    data = golden["idx2_bytes"].tobytes()
    assert np.array_equal(O.read_idx2(data, 64, 96), golden["idx2_kn"].astype(np.uint8))
    assert np.array_equal(O.read_lut_scalar(golden["lut_bytes"].tobytes()), golden["lut_vals"])
