"""The two single-Linear benchmark configurations at their FULL sizes (N = 9728, K = 2560; hard forward at M = 512, soft
forward + full backward at M = 16384).

The CPU oracle cannot run 16384 x 9728 x 2560 three times in a test, so the full-size step is checked through
  * the oracle on SAMPLES that need no approximation: all outputs that belong to 64 sampled weight rows (y columns,
    dLogits, dPalette, dB rows: full sum over the 16384 tokens), all outputs of 256 sampled tokens (y, dX rows: full sum
    over the 9728 weight rows), and dA in full;
  * size-independent properties: the packed hard indices equal argmax of the plain logits everywhere (bit exact), the
    parameter gradients are additive over a split of the tokens, and y / dX rows do not depend on which other rows are in
    the batch (bit exact).
"""
import numpy as np
import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu

N, K, RANK, TAU = 9728, 2560, 16, 1.0


def _dense_hard_weight(packed_gpu, palette_cpu):
    """bf16 [N, K] hard weight from the kernel's own packed indices (checked against argmax separately)."""
    idx = torch.from_numpy(O.unpack_rows(packed_gpu.cpu().numpy(), K)).long()
    return O.dequantize(idx, palette_cpu.reshape(-1, 4), 1, 256)


def test_config0_full_size_against_oracle():
    import plz_ops as ops
    import synth
    d = synth.make_linear_inputs(512, N, K, seed=0, soft=False, lora=False, with_dy=False)
    idx = d["idx"]
    w = ops.PackedWeight(torch.from_numpy(O.pack_rows(idx.numpy())).cuda(), d["palette"].reshape(-1, 4).cuda(), N, K, 1, 256)
    y, _ = ops.hard_forward(w, d["x"].cuda())
    check_status()
    want = O.hard_forward(d["x"], O.dequantize(idx.long(), d["palette"].reshape(-1, 4), 1, 256))
    assert_close(y, want, "config 0: y")


def test_config1_full_size_samples_and_properties():
    import palettized_linear as PL
    import synth
    M = 16384
    dev = torch.device("cuda", 0)
    d = synth.make_linear_inputs_cuda(M, N, K, seed=0, rank=RANK, device=dev)
    x, dy, logits, noise = d["x"], d["dy"], d["logits"], d["noise"]
    palette = d["palette"].reshape(-1, 4).contiguous()
    lora = (d["lora_a"], d["lora_b"], 1.0)
    out = PL.linear_step(x, dy, palette, logits, noise, TAU, lora=lora)
    check_status()

    # ---- hard indices: argmax of the plain logits, everywhere, bit exact
    hard = torch.argmax(logits, dim=-1).to(torch.uint8)
    want_packed = (hard[:, 0::4] | (hard[:, 1::4] << 2) | (hard[:, 2::4] << 4) | (hard[:, 3::4] << 6))
    assert torch.equal(out["packed"], want_packed), "packed hard indices must equal argmax(logits) bit for bit"
    del hard, want_packed

    # ---- 64 sampled weight rows, full token sum, against the oracle
    g = torch.Generator().manual_seed(1)
    rows = torch.randperm(N, generator=g)[:64].sort().values
    rg = rows.to(dev)
    xc, dyc = x.cpu(), dy.cpu()
    pal3 = d["palette"].cpu()  # [N, K/256, 4]
    sub = O.linear_step(xc, dyc[:, rows].contiguous(), logits[rg].cpu(), noise[rg].cpu(), pal3[rows].reshape(-1, 4), TAU, 1, 256,
                        lora=(d["lora_a"].cpu(), d["lora_b"][rg].cpu(), 1.0), ste=True)
    assert np.array_equal(out["packed"][rg].cpu().numpy(), O.pack_rows(sub["hard"].to(torch.uint8).numpy()))
    assert_close(out["y"][:, rg], sub["y"], "y columns of the sampled weight rows")
    assert_close(out["dlogits"][rg], sub["dlogits"], "dLogits of the sampled weight rows")
    n_kg = K // 256
    dpal = out["dpalette"].reshape(N, n_kg, 4)[rg]
    assert_close(dpal, sub["dpalette"].reshape(64, n_kg, 4), "dPalette of the sampled weight rows")
    assert_close(out["db"][rg], sub["db"], "dB of the sampled weight rows")

    # ---- 256 sampled tokens, full sum over the weight rows, against the oracle; dA in full
    toks = torch.randperm(M, generator=g)[:256].sort().values
    tg = toks.to(dev)
    w_hard = _dense_hard_weight(out["packed"], pal3).float()
    a_f, b_f = d["lora_a"].cpu().float(), d["lora_b"].cpu().float()
    xs, dys = xc[toks].float(), dyc[toks].float()
    t_s = (xs @ a_f.t()).to(torch.bfloat16).float()
    y_want = xs @ w_hard.t() + t_s @ b_f.t()
    dt_s = (dys @ b_f).to(torch.bfloat16).float()
    dx_want = dys @ w_hard + dt_s @ a_f
    assert_close(out["y"][tg], y_want, "y rows of the sampled tokens")
    assert_close(out["dx"][tg], dx_want, "dX rows of the sampled tokens")
    dt_full = (dyc.float() @ b_f).to(torch.bfloat16).float()
    assert_close(out["da"], dt_full.t() @ xc.float(), "dA")
    del w_hard, xc, dyc, dt_full

    # ---- properties: additivity of the parameter gradients over a split of the tokens; row independence of y and dX
    h = M // 2 + 128  # uneven split
    o1 = PL.linear_step(x[:h], dy[:h], palette, logits, noise, TAU, lora=lora)
    o2 = PL.linear_step(x[h:], dy[h:], palette, logits, noise, TAU, lora=lora)
    check_status()
    for k in ("dlogits", "dpalette", "da", "db"):
        assert_close(o1[k] + o2[k], out[k], f"{k}: sum over the two halves of the tokens", rel=1e-4)
    assert torch.equal(torch.cat([o1["y"], o2["y"]]), out["y"]), "y rows must not depend on the rest of the batch"
    assert torch.equal(torch.cat([o1["dx"], o2["dx"]]), out["dx"]), "dX rows must not depend on the rest of the batch"
