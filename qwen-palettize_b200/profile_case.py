"""Run one kernel of the hot path a few times on a small case, for `ncu` captures.

    python qwen-palettize_b200/profile_case.py --case fwd|dx|dw|dwscatter|smallm|smallm8|select|gateup [--M 4096] [--N 9728] [--K 2560] [--iters 3]

The shapes keep the full weight matrix of the benchmark Linear (so per-tile behaviour is the benchmark's) and cut
the token count; everything held on the device stays under 2 GB.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import plz_native  # noqa: E402
import plz_ops as ops  # noqa: E402
import synth  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["fwd", "dx", "dw", "dwscatter", "smallm", "smallm8", "select", "gateup"])
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--N", type=int, default=9728)
    ap.add_argument("--K", type=int, default=2560)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    d = synth.make_linear_inputs_cuda(a.M, a.N, a.K, seed=0)
    pal = d["palette"].reshape(-1, 4).contiguous()
    w = ops.PackedWeight(ops.pack_indices(d["idx"].view(torch.int8), n_major=True), pal, a.N, a.K, 1, 256)
    lora = (d["lora_a"], d["lora_b"], 1.0)
    t = dt = w2 = rstd = g = None
    stage = None
    if a.case == "dwscatter":
        # the data-parallel form of the dW launch as rank 0 of 2, both owners' staging buffers in this GPU's memory (ncu
        # profiles one process; the peer stores become local stores, everything else is the multi-GPU kernel)
        stage = torch.empty(2, a.N // 2, a.K, 4, dtype=torch.float32, device=d["x"].device)
    if a.case in ("dw", "dwscatter"):  # the workspaces the weight-gradient launch takes its dA / dB side items from
        t = ops.hard_forward(w, d["x"], lora)[1]
        dt = ops.lora_dt(lora, d["dy"])
    if a.case == "gateup":  # second matrix of the fused gate/up launch and the RMSNorm factors
        w2 = ops.PackedWeight(ops.pack_indices(((d["idx"].view(torch.uint8) + 1) & 3).view(torch.int8), n_major=True), pal, a.N, a.K, 1, 256)
        rstd = ops.rms_rstd(d["x"], 1e-6)
        g = torch.ones(a.K, dtype=torch.bfloat16, device=d["x"].device)
    for _ in range(a.iters):
        if a.case == "gateup":
            ops.mlp_gate_up_forward(w, w2, d["x"], rstd, g)
        elif a.case == "fwd":
            ops.hard_forward(w, d["x"], lora)
        elif a.case == "dx":
            ops.backward_dx(w, d["dy"], lora)
        elif a.case == "dwscatter":
            ops.backward_dw_soft_scatter(w, d["x"], d["dy"], d["logits"], [stage[0].data_ptr(), stage[1].data_ptr()], 2, 0,
                                         noise=d["noise"], tau=1.0, lora_ws=(t, dt))
        elif a.case == "dw":
            ops.backward_dw_soft(w, d["x"], d["dy"], d["logits"], "nk4", noise=d["noise"], tau=1.0, lora_ws=(t, dt))
        elif a.case == "smallm8":  # eight rows: the mma.sync kernel (up to 16 rows)
            ops.hard_forward_smallm(w, d["x"][:8].contiguous())
        elif a.case == "smallm":
            ops.hard_forward_smallm(w, d["x"][: min(a.M, 64)].contiguous())
        else:
            ops.soft_select(w, d["logits"], "nk4", noise=d["noise"], tau=1.0, want_packed=True)
    torch.cuda.synchronize()
    print("status", plz_native.device_status())


if __name__ == "__main__":
    main()
