"""Per-kernel measurements that complement bench.py (which times the whole training step of one Linear):

  smallm   hard forward at decode batch sizes M in {1, 8, 16, 64}: achieved GB/s on the packed weights
           (N*K/4 index bytes + palette bytes per launch) against the measured HBM copy bandwidth.
           The weights rotate over enough copies to exceed the 126 MB L2, so every launch reads HBM.
  config0  hard forward at M = 512 (BASELINE config 0): time and TFLOP/s of the tiled tcgen05 kernel.
  select   logits -> packed argmax indices: GB/s on the 16 bytes per weight it reads.
  swiglu / rmsnorm backward: GB/s on the bytes they read and write.

    python qwen-palettize_b200/bench_kernels.py [--iters 200]
Prints one JSON object per measurement.  Timing: CUDA events on the launching stream around `iters` back-to-back
launches after 10 warm-up launches.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import plz_native  # noqa: E402
import plz_ops as ops  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timed(fn_i, iters, warm=10, graph_batch=0):
    """ms per launch. graph_batch > 0: the launches are captured `graph_batch` at a time in a CUDA graph, so that the
    Python call overhead of this harness (about 20 us per call) does not hide a kernel that is shorter than that."""
    for i in range(warm):
        fn_i(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph_batch:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(graph_batch):
                fn_i(i)
        g.replay()
        torch.cuda.synchronize()
        reps = max(1, iters // graph_batch)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (reps * graph_batch)
    a.record()
    for i in range(iters):
        fn_i(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters  # ms


def make_weights(N, K, copies, dev):
    g = torch.Generator(device=dev).manual_seed(0)
    ws = []
    for _ in range(copies):
        idx = torch.randint(0, 4, (N, K), generator=g, device=dev, dtype=torch.uint8)
        pal = (torch.randn(N * (K // 256), 4, generator=g, device=dev) * 0.02).sort(-1).values.to(torch.bfloat16)
        ws.append(ops.PackedWeight(ops.pack_indices(idx.view(torch.int8), n_major=True), pal, N, K, 1, 256))
        del idx
    return ws


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tf, src = peaks()
    for (N, K) in [(9728, 2560), (2560, 9728), (4096, 2560)]:
        wbytes = N * K // 4 + N * (K // 256) * 8
        copies = max(2, (2 * 126 * 2 ** 20) // wbytes + 1)
        ws = make_weights(N, K, copies, dev)
        for M in (1, 8, 16, 64):
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            ys = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
            ms = timed(lambda i: ops.hard_forward_smallm(ws[i % copies], x, out=ys[i & 1]), a.iters, graph_batch=copies)
            gbs = wbytes / (ms * 1e-3) / 1e9
            print(json.dumps({"kernel": "lut_smallm_mma_kernel" if M <= 16 else "lut_gemv_kernel (tcgen05 swap-AB)", "case": "smallm", "M": M, "N": N, "K": K, "us": ms * 1e3,
                              "weight_bytes": wbytes, "GBps": gbs, "hbm_peak_GBps": hbm, "frac": gbs / hbm,
                              "peak_source": src, "weight_copies_rotated": copies, "timing": "CUDA graph of one launch per weight copy"}))
        if (N, K) == (9728, 2560):
            # gate_proj + up_proj share x: one launch streams both matrices (pairs of consecutive weight copies)
            for M in (1, 8, 16):
                x = torch.randn(M, K, device=dev).to(torch.bfloat16)
                pairs = copies // 2
                ms = timed(lambda i: ops.hard_forward_smallm_multi([ws[2 * (i % pairs)], ws[2 * (i % pairs) + 1]], x), a.iters,
                           graph_batch=pairs)
                gbs = 2 * wbytes / (ms * 1e-3) / 1e9
                print(json.dumps({"kernel": "lut_smallm_mma_kernel", "case": "smallm gate+up in one launch", "M": M, "N": [N, N], "K": K,
                                  "us": ms * 1e3, "weight_bytes": 2 * wbytes, "GBps": gbs, "hbm_peak_GBps": hbm, "frac": gbs / hbm,
                                  "peak_source": src, "timing": "CUDA graph of one launch per pair of weight copies"}))
            # launches allowed to start under the tail of the previous one (programmatic stream serialization)
            plz_native.lib().plz_set_smallm_overlap(1)
            for M in (1, 8):
                x = torch.randn(M, K, device=dev).to(torch.bfloat16)
                ms = timed(lambda i: ops.hard_forward_smallm(ws[i % copies], x, out=ys[i & 1][:M]), a.iters, graph_batch=copies)
                gbs = wbytes / (ms * 1e-3) / 1e9
                print(json.dumps({"kernel": "lut_smallm_mma_kernel", "case": "smallm, overlapped launches", "M": M, "N": N, "K": K,
                                  "us": ms * 1e3, "GBps": gbs, "frac": gbs / hbm}))
                pairs = copies // 2
                ms = timed(lambda i: ops.hard_forward_smallm_multi([ws[2 * (i % pairs)], ws[2 * (i % pairs) + 1]], x), a.iters,
                           graph_batch=pairs)
                gbs = 2 * wbytes / (ms * 1e-3) / 1e9
                print(json.dumps({"kernel": "lut_smallm_mma_kernel", "case": "smallm gate+up in one launch, overlapped launches", "M": M,
                                  "us": ms * 1e3, "GBps": gbs, "frac": gbs / hbm}))
            plz_native.lib().plz_set_smallm_overlap(0)
            # the kernels that served M <= 16 before the mma.sync one, for comparison
            plz_native.lib().plz_debug_set_smallm_variant(1)
            for M in (1, 8):
                x = torch.randn(M, K, device=dev).to(torch.bfloat16)
                ms = timed(lambda i: ops.hard_forward_smallm(ws[i % copies], x, out=ys[i & 1][:M]), a.iters, graph_batch=copies)
                print(json.dumps({"kernel": "lut_gemv_rows_kernel" if M <= 4 else "lut_gemv_kernel (tcgen05 swap-AB)", "case": "smallm, previous kernel",
                                  "M": M, "N": N, "K": K, "us": ms * 1e3, "GBps": wbytes / (ms * 1e-3) / 1e9}))
            plz_native.lib().plz_debug_set_smallm_variant(0)
            x = torch.randn(512, K, device=dev).to(torch.bfloat16)
            ms = timed(lambda i: ops.hard_forward(ws[i % copies], x), a.iters)
            fl = 2.0 * 512 * N * K
            print(json.dumps({"kernel": "lut_gemm_kernel<2,B_DECODE_K>", "case": "config0", "M": 512, "N": N, "K": K,
                              "us": ms * 1e3, "TFLOPs": fl / (ms * 1e-3) / 1e12, "tensor_peak_TFLOPs": tf,
                              "frac": fl / (ms * 1e-3) / 1e12 / tf, "peak_source": src}))
        del ws
    N, K = 9728, 2560
    logits = torch.randn(N, K, 4, device=dev)
    w = ops.PackedWeight(ops.empty_packed(N, K, dev), torch.zeros(N * (K // 256), 4, dtype=torch.bfloat16, device=dev), N, K, 1, 256)
    ms = timed(lambda i: ops.soft_select(w, logits, "nk4", want_packed=True), 50)
    rb = N * K * 16 + N * K // 4
    print(json.dumps({"kernel": "soft_select_kfast_kernel", "case": "select", "N": N, "K": K, "us": ms * 1e3, "bytes": rb,
                      "GBps": rb / (ms * 1e-3) / 1e9, "hbm_peak_GBps": hbm, "frac": rb / (ms * 1e-3) / 1e9 / hbm,
                      "peak_source": src}))
    # element-wise backward ops around the MLP Linears at the benchmark's token count (inputs larger than L2)
    M = 16384
    gate, up, dact = (torch.randn(M, N, device=dev).to(torch.bfloat16) for _ in range(3))
    ms = timed(lambda i: ops.swiglu_backward(gate, up, dact), 30)
    rb = 5 * M * N * 2
    print(json.dumps({"kernel": "swiglu_bwd_kernel", "case": "swiglu backward", "M": M, "N": N, "us": ms * 1e3, "bytes": rb,
                      "GBps": rb / (ms * 1e-3) / 1e9, "hbm_peak_GBps": hbm, "frac": rb / (ms * 1e-3) / 1e9 / hbm, "peak_source": src}))
    del gate, up, dact
    Mx = 65536  # 335 MB per tensor, so that x + dH exceed L2
    xx, dh = (torch.randn(Mx, K, device=dev).to(torch.bfloat16) for _ in range(2))
    nw = torch.ones(K, dtype=torch.bfloat16, device=dev)
    rstd = ops.rms_rstd(xx, 1e-6)
    ms = timed(lambda i: ops.rmsnorm_backward(xx, dh, rstd, nw), 30)
    rb = 3 * Mx * K * 2
    print(json.dumps({"kernel": "rmsnorm_bwd_kernel<5>", "case": "rmsnorm backward", "M": Mx, "K": K, "us": ms * 1e3, "bytes": rb,
                      "GBps": rb / (ms * 1e-3) / 1e9, "hbm_peak_GBps": hbm, "frac": rb / (ms * 1e-3) / 1e9 / hbm, "peak_source": src}))
    print(json.dumps({"status": list(plz_native.device_status())}))


if __name__ == "__main__":
    main()
