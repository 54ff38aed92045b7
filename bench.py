#!/usr/bin/env python
"""Benchmark of the PalettizedLinear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --case fwd|dx|dw|dwscatter|smallm|smallm8|select|gateup|layer8|decode1|decode8|decode64|prefill|layertrain [--M 4096]   one kernel, a few launches (ncu captures)
    python bench.py --kernels [--iters 200]                                              per-kernel table, one JSON line each

One step = soft forward (straight-through) + full backward of ONE palettized Linear with LoRA at the
Qwen-4B MLP shape: M = 32 x 512 = 16384 tokens per GPU, K = 2560, N = 9728, rank 16, tau = 1, explicit Gumbel
noise, i.e. y, dX, dPalette, dLogits, dA, dB.  With N > 1 GPUs every rank runs that step on its own 16384
tokens (weak scaling over the batch) and the parameter gradients are sum-all-reduced over NCCL inside the
timed region.  Prints ONE JSON line (rank 0).
"""
import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "qwen-palettize_b200")
sys.path.insert(0, PKG)

M_TOK, N_OUT, K_IN, RANK, TAU = 16384, 9728, 2560, 16, 1.0
METRIC = "fwd+bwd tokens/s, Qwen-4B-shaped PalettizedLinear (soft forward + full backward + LoRA r16)"
WORKLOAD = "configs[1]: one Linear N=9728 K=2560, M=32x512=16384 tokens per GPU, soft fwd (STE) + full bwd, LoRA r16, tau=1"
GEMM_FLOPS = 2.0 * M_TOK * N_OUT * K_IN  # one of the three products
COMM_SMS = 48  # SMs left free for NCCL during the dX product when the gradient exchange is in flight (N > 1); measured at N = 2: all-reduce 0.76 ms + dX 0.66 ms take 1.34 ms with no SMs free, 0.91 ms with 48 free


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops_burst": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


_SAMPLER_SRC = r"""
import sys, time
import pynvml as nv
nv.nvmlInit()
h = nv.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
print("max", nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM), flush=True)
while True:
    try:
        print(time.time(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
              nv.nvmlDeviceGetCurrentClocksEventReasons(h), flush=True)
    except Exception:
        pass
    time.sleep(0.002)
"""


class ClockSampler:
    """SM clock, power and throttle reasons read through NVML (read-only queries) every 2 ms by a helper process
    for the whole run; stop(t0, t1) keeps the samples taken inside the timed region [t0, t1] (time.time())."""

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self):
        import subprocess
        import tempfile
        try:
            fd, self.path = tempfile.mkstemp(suffix=".clk")
            os.close(fd)
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_SRC, str(self.gpu_index)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def ready(self, timeout=20.0):
        """Wait until the helper has produced its first sample."""
        t_end = time.time() + timeout
        while self.proc is not None and time.time() < t_end:
            try:
                if sum(1 for _ in open(self.path)) >= 3:
                    return
            except OSError:
                pass
            time.sleep(0.05)

    def stop(self, t0, t1):
        out = self.window(t0, t1)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            os.unlink(self.path)
            self.proc = None
        return out

    def window(self, t0, t1):
        """Summary of the samples taken in [t0, t1]; the helper keeps running."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        rows = []
        for line in open(self.path):
            f = line.split()
            try:
                if f[0] == "max":
                    out["sm_max_mhz"] = int(f[1])
                elif len(f) == 4 and t0 <= float(f[0]) <= t1:
                    rows.append((int(f[1]), float(f[2]), int(f[3])))
            except (ValueError, IndexError):
                continue
        if rows:
            bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                    "hw_power_brake_slowdown": 0x80}
            seen = 0
            for _, _, r in rows:
                seen |= r
            out.update(sm_mhz=statistics.median(r[0] for r in rows), samples=len(rows), sm_min_mhz=min(r[0] for r in rows),
                       power_w_max=max(r[1] for r in rows), reasons=sorted(k for k, v in bits.items() if seen & v))
        return out


def dist_setup(n_gpus):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL launches its kernels as 4-CTA clusters by default; a cluster needs its SMs free in ONE GPC, which the few
        # SMs the persistent dX kernel leaves (scattered over the GPCs) never offer, so the small collectives of the
        # exchange would wait for dX to end. Without clusters they run on whatever SMs are free.
        os.environ.setdefault("NCCL_CGA_CLUSTER_SIZE", "0")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def run_ours(args):
    import torch
    import torch.distributed as dist
    import dp
    import palettized_linear as PL
    import plz_native
    import plz_ops as ops
    import synth

    saved_stdout = os.dup(1)
    os.dup2(2, 1)  # anything a library prints (NCCL's version banner) goes to stderr; the JSON line gets stdout back
    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local if world > 1 else 0)
    plz_native.lib().plz_set_pair_gemm(args.pair_gemm)
    d = synth.make_linear_inputs_cuda(M_TOK, N_OUT, K_IN, seed=rank, rank=RANK, device=dev)
    # parameters are replicated: every rank uses rank 0's parameters, its own tokens
    if world > 1:
        for k in ("idx", "palette", "logits", "noise", "lora_a", "lora_b"):
            dist.broadcast(d[k], src=0)
    x, dy, logits, noise = d["x"], d["dy"], d["logits"], d["noise"]
    palette = d["palette"].reshape(-1, 4).contiguous()
    lora = (d["lora_a"], d["lora_b"], 1.0)
    packed = ops.empty_packed(N_OUT, K_IN, dev)
    w = ops.PackedWeight(packed, palette, N_OUT, K_IN, 1, 256)
    exch = dp.GradExchange()
    # N > 1: reduce-scatter of dLogits fused into the weight-gradient kernel over peer memory (--exchange allreduce
    # selects the plain NCCL all-reduce of the full gradient instead, for comparison)
    scatter = None
    if world > 1 and args.exchange in ("fused", "fused-add"):
        try:
            scatter = dp.LogitGradScatter(N_OUT, K_IN, dev, mode="slots" if args.exchange == "fused" else "add")
        except RuntimeError as e:  # raised on every rank together: peer mappings unavailable, use the NCCL exchange
            print(f"[bench] fused exchange unavailable ({e}); using the NCCL all-reduce", file=sys.stderr)
            scatter = None
    # the fused exchange gathers with the copy engines and needs no SM; the NCCL all-reduce does
    # fused slot mode: dX in two row blocks, the first (two rounds of 256-row tiles on 140 SMs) beside the small all-reduce
    split_rows = args.split_dx if (scatter is not None and scatter.mode == "slots") else 0
    dx_buf = torch.empty(M_TOK, K_IN, dtype=torch.bfloat16, device=dev) if split_rows > 0 else None
    comm_sms = args.comm_sms if args.comm_sms >= 0 else (COMM_SMS if scatter is None else (0 if scatter.mode == "slots" else 16))
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    phases = ["select", "fwd", "lora_dt", "dw", "dx"]
    if world > 1:
        # what the exchange adds to the compute stream: the small all-reduce + slot reduction (fused mode), and the wait for
        # whatever part of the exchange the dX product did not hide
        phases = phases[:4] + (["exch_sync", "exch_reduce"] if scatter is not None else []) + ["dx", "exch_wait"]
    ev = {p: [] for p in phases}
    # deferred exchange (fused slot mode): the whole exchange of a step runs on the side stream and is waited for only
    # right before the next step's weight-gradient kernel reuses the staging slots (and once more after the last step)
    deferred = bool(args.defer_exchange) and scatter is not None and scatter.mode == "slots" and split_rows == 0
    pending = [None]

    def drain():
        if deferred and pending[0] is not None:
            scatter.finish(pending[0])
            pending[0] = None

    def step(record):
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(7)] if record else None
        xm = [torch.cuda.Event(enable_timing=True) for _ in range(2)] if record else None
        dmark = torch.cuda.Event(enable_timing=True) if record else None
        if record: marks[0].record()
        ops.soft_select(w, logits, "nk4", noise=noise, tau=TAU, want_packed=True)
        if record: marks[1].record()
        y, t = ops.hard_forward(w, x, lora)                       # lora_down + LUT GEMM (+ LoRA block)
        if record: marks[2].record()
        dt = ops.lora_dt(lora, dy)                                # skinny product, timed with the dx phase below
        if record: marks[3].record()
        if scatter is not None:
            # dLogits partials go straight from the epilogue into the owner ranks' staging buffers (reduce-scatter fused
            # into the kernel); small all-reduce + slot reduction + all-gather then run beside the dX product
            if deferred and pending[0] is not None:
                # the previous step's exchange must be over on every rank before its staging slots are written again
                scatter.finish(pending[0])
                pending[0] = None
            if record and deferred: dmark.record()
            dpal, da, db = scatter.dw(w, x, dy, logits, noise, TAU, lora_ws=(t, dt))
            if record: marks[4].record()
            if deferred:
                h1 = scatter.start_beside([dpal, da, db])
                pending[0] = h1
                if record: xm[0].record(); xm[1].record()
            elif scatter.mode == "add":
                h1 = scatter.start([dpal, da, db])
                if record: xm[0].record(); xm[1].record()
            elif split_rows > 0:
                # the first rows of dX run while the small all-reduce (and the wait for the slowest rank's dW behind it)
                # happens on the side stream; then the slot reduction, then the rest of dX beside the all-gather
                h1 = scatter.sync_small_beside([dpal, da, db])
                plz_native.lib().plz_set_cta_limit(sm_count - 8)  # a few SMs for the small collective
                ops.backward_dx_with_dt(w, dy[:split_rows], lora, dt[:split_rows], out=dx_buf[:split_rows])
                plz_native.lib().plz_set_cta_limit(0)
                if record: xm[0].record()
                scatter.reduce_and_push()
                if record: xm[1].record()
            else:
                h1 = scatter.sync_small([dpal, da, db])
                if record: xm[0].record()
                scatter.reduce_and_push()
                if record: xm[1].record()
        else:
            dlog, dpal, da, db = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=TAU, lora_ws=(t, dt))
            if record: marks[4].record()
            h1 = exch.start([dlog, dpal, da, db])                 # all-reduce, overlaps the dX GEMM below (N > 1 only)
        if world > 1:
            plz_native.lib().plz_set_cta_limit(sm_count - comm_sms)  # leave SMs to NCCL while the exchange runs
        if scatter is not None and scatter.mode == "slots" and split_rows > 0:
            dx = ops.backward_dx_with_dt(w, dy[split_rows:], lora, dt[split_rows:], out=dx_buf[split_rows:])
            dx = dx_buf
        else:
            dx = ops.backward_dx_with_dt(w, dy, lora, dt)         # LUT GEMM (+ LoRA block)
        if world > 1:
            plz_native.lib().plz_set_cta_limit(0)
        if record: marks[5].record()
        if deferred:
            dlog = scatter.full          # complete after the finish() that precedes the next dw (or the drain below)
        elif scatter is not None:
            dlog = scatter.finish(h1)
        else:
            exch.finish(h1)
        if record: marks[6].record()
        if record:
            ev["select"].append((marks[0], marks[1])); ev["fwd"].append((marks[1], marks[2]))
            ev["lora_dt"].append((marks[2], marks[3])); ev["dw"].append((dmark if deferred else marks[3], marks[4]))
            if scatter is not None:
                ev["exch_sync"].append((marks[4], xm[0])); ev["exch_reduce"].append((xm[0], xm[1])); ev["dx"].append((xm[1], marks[5]))
            else:
                ev["dx"].append((marks[4], marks[5]))
            if world > 1:
                ev["exch_wait"].append((marks[3], dmark) if deferred else (marks[5], marks[6]))
        return y, dx, dlog, dpal, da, db

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local if world > 1 else 0)
    if rank == 0:
        sampler.start()
    # N > 1: correctness of the fused exchange on this very configuration, outside the timed region
    parity = None
    if world > 1 and scatter is not None and not args.no_parity:
        parity = exchange_parity(world, rank, dev, ops, dp, dist, torch, scatter, w, x, dy, logits, noise, lora)
        parity["sharded_optimizer"] = sharded_optimizer_parity(world, rank, dev, ops, dp, dist, torch, scatter.mode)
        parity["pass"] = bool(parity["pass"] and parity["sharded_optimizer"]["pass"])
    for _ in range(max(args.warmup, 3)):
        step(False)
    drain()
    barrier()
    plz_native.device_status()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if rank == 0:
        sampler.ready()
    barrier()
    wall0 = time.time()
    launches0 = plz_native.lib().plz_launch_count()
    t0.record()
    for _ in range(args.steps):
        step(True)
    drain()      # the last step's exchange ends inside the timed region
    t1.record()
    launches = plz_native.lib().plz_launch_count() - launches0
    barrier()
    wall1 = time.time()
    ms = t0.elapsed_time(t1)
    clocks = sampler.window(wall0, wall1) if rank == 0 else None
    plz_native.device_status()
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()

    # ---- sustained leg: the same step back to back for several seconds, so that the power cap and the clocks it sets
    # are part of a recorded number (the timed region above is a burst of a few tens of milliseconds)
    sustained = None
    if args.sustained_s > 0:
        n_chunk = max(10, int(0.25 / max(ms / args.steps * 1e-3, 1e-6)))   # about a quarter of a second per chunk
        barrier()
        s_wall0 = time.time()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        n_done = 0
        while True:
            for _ in range(n_chunk):
                step(False)
            drain()
            n_done += n_chunk
            torch.cuda.synchronize()
            stop = torch.tensor([1.0 if time.time() - s_wall0 >= args.sustained_s else 0.0], device=dev)
            if world > 1:
                dist.all_reduce(stop, op=dist.ReduceOp.MAX)   # all ranks leave together
            if stop.item() > 0:
                break
        s1.record()
        barrier()
        s_wall1 = time.time()
        s_ms = s0.elapsed_time(s1)
        if world > 1:
            tt = torch.tensor([s_ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            s_ms = tt.item()
        s_clk = sampler.window(s_wall0, s_wall1) if rank == 0 else None
        sustained = {"steps": n_done, "seconds": s_ms * 1e-3, "ms_per_step": s_ms / n_done, "tokens_per_s": M_TOK * world * n_done / (s_ms * 1e-3),
                     "tflops_per_gpu": 3 * GEMM_FLOPS * n_done / (s_ms * 1e-3) / 1e12, "clocks": s_clk}
    if rank == 0:
        sampler.stop(0, 0)
    phase_ms = {p: statistics.mean(a.elapsed_time(b) for a, b in ev[p]) for p in phases}

    # the two rank-16 products that ride in the fwd / dx phases, timed alone so that the big kernels' own
    # durations can be stated: t = x A^T is plz_dense_fwd with Wd = A, dt = dY B is plz_dense_bwd_dx with Wd = B
    def timed(fn, n=5):
        fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n
    skinny = {"fwd": timed(lambda: ops.dense_forward(d["lora_a"], x)), "dx": 0.0, "dw": 0.0}

    # ---- end to end: host buffers in, gradients out, through the public step call
    hx, hdy = x.cpu().pin_memory(), dy.cpu().pin_memory()
    bufs = [(torch.empty_like(x), torch.empty_like(dy)) for _ in range(2)]
    hout = [torch.empty(palette.numel(), dtype=torch.float32).pin_memory(), torch.empty(RANK * K_IN, dtype=torch.float32).pin_memory(),
            torch.empty(N_OUT * RANK, dtype=torch.float32).pin_memory()]
    copy_s = torch.cuda.Stream(device=dev)
    main_s = torch.cuda.current_stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]

    def upload(b):
        with torch.cuda.stream(copy_s):
            copy_s.wait_event(free[b])
            bufs[b][0].copy_(hx, non_blocking=True)
            bufs[b][1].copy_(hdy, non_blocking=True)
            ready[b].record(copy_s)

    def e2e_loop(n):
        for b in range(2):
            free[b].record(main_s)
        upload(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                upload(b ^ 1)
            main_s.wait_event(ready[b])
            out = PL.linear_step(bufs[b][0], bufs[b][1], palette, logits, noise, TAU, lora=lora, packed=packed, dp_scatter=scatter)
            free[b].record(main_s)
            if world > 1 and scatter is None:
                exch.finish(exch.start([out["dlogits"], out["dpalette"], out["da"], out["db"]]))
            hout[0].copy_(out["dpalette"].reshape(-1), non_blocking=True)
            hout[1].copy_(out["da"].reshape(-1), non_blocking=True)
            hout[2].copy_(out["db"].reshape(-1), non_blocking=True)

    h2d_bytes = hx.numel() * 2 + hdy.numel() * 2
    e2e_loop(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    copy_s.wait_event(e0)
    e2e_loop(args.steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = tt.item()
    plz_native.device_status()
    if scatter is not None:
        scatter.close()
    extras = None
    if world == 1 and not args.no_extra:
        del bufs, hx, hdy
        extras = extra_configs(torch, ops, plz_native, dev, peaks())
        plz_native.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if parity is not None and not parity["pass"]:
            sys.exit(3)
        return
    pk = peaks()
    tokens = M_TOK * world * args.steps
    gemm_phase = max(("fwd", "dw", "dx"), key=lambda p: phase_ms[p])
    kern_ms = {p: max(phase_ms[p] - skinny[p], 1e-6) for p in ("fwd", "dw", "dx")}
    achieved = GEMM_FLOPS / (kern_ms[gemm_phase] * 1e-3) / 1e12
    # the denominator follows the length of the timed region: a region of well under a second runs at boost clocks with no
    # power cap and is compared with the BURST cuBLAS figure; a seconds-long one with the sustained figure
    burst_region = (ms * 1e-3) < 1.0
    peak_val = pk["tflops_burst"] if burst_region else pk["tflops_sustained"]
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum): one ncu capture of each kernel at 4096
    # tokens (profiles/*.md) gave measured / algorithmic = 0.51 (fwd: most of y was still in L2 when the capture
    # ended) and 0.90 (dx). The dW launch measured 1413.7 MB there: 1195.4 MB of logits / noise / dLogits that do not
    # depend on the token count, plus x and dY streamed twice (once for dW, once more by the dA / dB side items in
    # the last round); the figure below scales that token-proportional part to the full 16384-token launch.
    alg = {"fwd": M_TOK * K_IN * 2 + N_OUT * K_IN // 4 + N_OUT * (K_IN // 256) * 8 + M_TOK * N_OUT * 2,
           "dx": M_TOK * N_OUT * 2 + N_OUT * K_IN // 4 + N_OUT * (K_IN // 256) * 8 + M_TOK * K_IN * 2,
           "dw": 3 * N_OUT * K_IN * 16 + M_TOK * (N_OUT + K_IN) * 2}
    xdy_small = 4096 * (N_OUT + K_IN) * 2
    traffic = {"fwd": 0.51 * alg["fwd"], "dx": 0.90 * alg["dx"],
               "dw": (1413.7e6 - 2 * xdy_small) + 2 * M_TOK * (N_OUT + K_IN) * 2}
    traffic_src = {"fwd": "profiles/lut_gemm_forward_M4096_N9728_K2560.md", "dx": "profiles/lut_gemm_dx_M4096_N9728_K2560.md",
                   "dw": "profiles/tn_gemm_soft_gradient_M4096_N9728_K2560.md"}
    line = {
        "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": M_TOK, "N": N_OUT, "K": K_IN, "lora_rank": RANK,
                   "parallelism": f"dp{world}", "split_dx_rows": split_rows, "exchange": ("none" if world == 1 else (f"reduce-scatter fused into the dW epilogue over peer memory ({scatter.mode}) + copy-engine all-gather" if scatter is not None else "NCCL all-reduce")), "l2": "inputs larger than L2 (x+dY 403 MB, logits+noise 797 MB per step)"},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": sum(h.numel() * 4 for h in hout), "ms_per_step": e2e_ms / args.steps,
                "d2h_note": "the parameter gradients that leave the step (dPalette, dA, dB) are read back; y, dX and dLogits stay on the "
                            "device, where the next layer's backward and the optimizer consume them"},
        "gpu_launches": int(launches),
        "gpu_launches_note": "kernels of libplz.so launched inside the timed region, counted by the library (plz_launch_count); "
                             "NCCL's own kernels at N > 1 are not included",
        "phases_ms": phase_ms,
        "tflops_step": 3 * GEMM_FLOPS * world / (ms / args.steps * 1e-3) / 1e12,
        "roofline": {"bound": "tensor", "kernel": ({"fwd": "lut_gemm_pair_kernel<B_DECODE_K> (cta_group::2)", "dw": "tn_gemm_kernel<EPI_SOFT,float,rows=k,pair> (cta_group::2; + dA, dB items)",
                                                     "dx": "lut_gemm_pair_kernel<B_DECODE_MN> (cta_group::2)"} if args.pair_gemm else
                                                    {"fwd": "lut_gemm_kernel<2,B_DECODE_K>", "dw": "tn_gemm_kernel<EPI_SOFT,float,rows=k> (+ dA, dB items)",
                                                     "dx": "lut_gemm_kernel<2,B_DECODE_MN>"})[gemm_phase],
                     "achieved": achieved, "peak": peak_val, "unit": "TFLOP/s", "frac": achieved / peak_val,
                     "peak_kind": ("burst" if burst_region else "sustained") + " cuBLAS bf16, " + pk["source"],
                     "timed_region_s": ms * 1e-3,
                     "frac_of_burst_peak": achieved / pk["tflops_burst"], "frac_of_sustained_peak": achieved / pk["tflops_sustained"],
                     "frac_of_nominal_2250": achieved / 2250.0,
                     "step_frac_of_burst_peak": 3 * GEMM_FLOPS / (ms / args.steps * 1e-3) / 1e12 / pk["tflops_burst"],
                     "traffic": traffic[gemm_phase],
                     "traffic_note": "ESTIMATE, not measured in this run: DRAM bytes of one ncu capture at 4096 tokens (" + traffic_src[gemm_phase] +
                                     "), its token-proportional part scaled to the 16384-token launch",
                     "algorithmic_bytes": alg[gemm_phase],
                     "kernel_ms": kern_ms, "skinny_lora_ms": skinny,
                     "per_kernel_tflops": {p: GEMM_FLOPS / (kern_ms[p] * 1e-3) / 1e12 for p in ("fwd", "dw", "dx")}},
    }
    if sustained is not None:
        sustained["frac_of_sustained_peak"] = sustained["tflops_per_gpu"] / pk["tflops_sustained"]
        clk = (sustained.get("clocks") or {}).get("sm_mhz")
        sustained["ms_x_mhz"] = sustained["ms_per_step"] * clk if clk else None
        line["sustained"] = sustained
    if parity is not None:
        line["parity"] = parity
    if extras is not None:
        line["extra_configs"] = extras
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(budget_s=20.0)
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["pass"]:
        sys.exit(3)



# ---------------------------------------------------------------------------------------------------------
# checks and extra measurements that ride in the same JSON line
# ---------------------------------------------------------------------------------------------------------
QWEN_LAYER = {"q": (4096, 2560), "k": (1024, 2560), "v": (1024, 2560), "o": (2560, 4096), "gate": (9728, 2560),
              "up": (9728, 2560), "down": (2560, 9728)}  # name -> (N = out features, K = in features)


def _rel(a, b):
    den = b.abs().max().item()
    return (a - b).abs().max().item() / (den if den > 0 else 1.0)


def exchange_parity(world, rank, dev, ops, dp, dist, torch, scatter, w, x, dy, logits, noise, lora):
    """N > 1, outside the timed region: one step of the fused exchange (dW kernel storing into the peers' staging memory ->
    small all-reduce -> slot reduction -> copy-engine gather) against the unfused kernel followed by NCCL all-reduces of the
    same gradients.  In slot mode at 2 ranks both sum a + b in the same order: bit-exact."""
    ops.soft_select(w, logits, "nk4", noise=noise, tau=TAU, want_packed=True)
    _, t = ops.hard_forward(w, x, lora)
    dt = ops.lora_dt(lora, dy)
    dlog, dpal, da, db = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=TAU, lora_ws=(t, dt))
    for g in (dlog, dpal, da, db):
        dist.all_reduce(g)
    dpal2, da2, db2 = scatter.dw(w, x, dy, logits, noise, TAU, lora_ws=(t, dt))
    full = scatter.finish(scatter.start([dpal2, da2, db2]))
    torch.cuda.synchronize()
    res = {"dlogits_max_rel": _rel(full, dlog), "bit_exact": bool(torch.equal(full, dlog)),
           "small_max_rel": max(_rel(a, b) for a, b in ((dpal2, dpal), (da2, da), (db2, db)))}
    del dlog, full
    ok = res["dlogits_max_rel"] <= 1e-5 and res["small_max_rel"] <= 1e-4
    if scatter.mode == "slots" and world == 2:
        ok = ok and res["bit_exact"]
    # every rank must agree (a rank that saw a mismatch makes the whole run fail)
    flag = torch.tensor([1.0 if ok else 0.0, res["dlogits_max_rel"], res["small_max_rel"], 1.0 if res["bit_exact"] else 0.0], device=dev)
    mn, mx = flag.clone(), flag.clone()
    dist.all_reduce(mn, op=dist.ReduceOp.MIN)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    return {"dlogits_max_rel": mx[1].item(), "small_max_rel": mx[2].item(), "bit_exact": bool(mn[3].item() == 1.0),
            "pass": bool(mn[0].item() == 1.0), "against": "unfused dW kernel + NCCL all-reduce, same inputs, full size",
            "mode": scatter.mode}


def sharded_optimizer_parity(world, rank, dev, ops, dp, dist, torch, mode):
    """N > 1: the sharded logits optimizer (each rank steps its own rows after the slot reduction, updated PARAMETER rows
    are gathered) against a replicated fused AdamW on the all-reduced gradient.  Small shape, three steps."""
    import synth
    M, N, K = 512, 2048, 1024
    base = synth.make_linear_inputs(M, N, K, seed=5, rank=16)
    mine = synth.make_linear_inputs(M, N, K, seed=50 + rank, rank=16)
    logits, noise = base["logits"].to(dev), base["noise"].to(dev)
    lora = (base["lora_a"].to(dev), base["lora_b"].to(dev), 1.0)
    w = ops.PackedWeight(ops.empty_packed(N, K, dev), base["palette"].reshape(-1, 4).to(dev), N, K, 1, 256)
    ops.soft_select(w, logits, "nk4", noise=noise, tau=1.0, want_packed=True)
    sc = dp.LogitGradScatter(N, K, dev, mode=mode, shard_optimizer=True)
    sc.param.copy_(logits)
    r0, r1 = sc.shard_rows()
    m_s = torch.zeros((r1 - r0) * K * 4, device=dev)
    v_s = torch.zeros_like(m_s)
    ref = logits.clone()
    ref_m, ref_v = torch.zeros(N * K * 4, device=dev), torch.zeros(N * K * 4, device=dev)
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-3)
    worst, moved = 0.0, 0.0
    x, dy = mine["x"].to(dev), mine["dy"].to(dev)
    for step in range(3):
        _, t = ops.hard_forward(w, x, lora)
        dt = ops.lora_dt(lora, dy)
        dlog = ops.backward_dw_soft(w, x, dy, ref, "nk4", noise=noise, tau=1.0)[0]
        dist.all_reduce(dlog)
        ops.adamw_step(ref.view(-1), ref_m, ref_v, dlog.view(-1), step + 1, **hp)
        small = sc.dw(w, x, dy, sc.param, noise, 1.0, lora_ws=(t, dt))
        h = sc.start(list(small), step_fn=lambda p_, g_: ops.adamw_step(p_.reshape(-1), m_s, v_s, g_.reshape(-1), step + 1, **hp))
        sc.finish(h)
        torch.cuda.synchronize()
        worst = max(worst, (sc.param - ref).abs().max().item())
        moved = max(moved, (ref - logits).abs().max().item())
    sc.close()
    flag = torch.tensor([worst, -moved], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    worst, moved = flag[0].item(), -flag[1].item()
    return {"param_max_abs_diff": worst, "param_moved": moved, "pass": bool(worst < 2e-5 and moved > 1e-3),
            "against": "replicated plz_adamw_step on the all-reduced gradient, 3 steps, N=2048 K=1024 M=512 per rank"}


def graph_timed(torch, fn_i, n_in_graph, reps):
    """ms per call of fn_i(i), i = 0 .. n_in_graph - 1 captured in ONE CUDA graph that is replayed `reps` times: the Python
    call overhead (about 20 us) stays out of kernels that are shorter than that."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(n_in_graph):
            fn_i(i)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_in_graph):
            fn_i(i)
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (reps * n_in_graph)


def make_weight(torch, ops, N, K, dev, gen):
    idx = torch.randint(0, 4, (N, K), generator=gen, device=dev, dtype=torch.uint8)
    pal = (torch.randn(N * (K // 256), 4, generator=gen, device=dev) * 0.02).sort(-1).values.to(torch.bfloat16)
    return ops.PackedWeight(ops.pack_indices(idx.view(torch.int8), n_major=True), pal, N, K, 1, 256)


def weight_bytes(N, K):
    return N * K // 4 + N * (K // 256) * 8


def layer_decode_runner(torch, ops, plz_native, dev, M, copies):
    """Hard forward of the seven Linears of one Qwen-4B decoder layer at M rows, as a decode step issues them: q/k/v in one
    launch (they share x), o, gate/up in one launch, down; `copies` independent layers so that a rotation over them
    exceeds L2.  Returns (fn(i) running layer i % copies, weight bytes per layer)."""
    gen = torch.Generator(device=dev).manual_seed(1)
    layers = []
    for _ in range(copies):
        layers.append({k: make_weight(torch, ops, n, kk, dev, gen) for k, (n, kk) in QWEN_LAYER.items()})
    xs = {2560: torch.randn(M, 2560, device=dev).to(torch.bfloat16), 4096: torch.randn(M, 4096, device=dev).to(torch.bfloat16),
          9728: torch.randn(M, 9728, device=dev).to(torch.bfloat16)}
    out_o = torch.empty(M, 2560, dtype=torch.bfloat16, device=dev)
    out_d = torch.empty(M, 2560, dtype=torch.bfloat16, device=dev)

    def run(i):
        L = layers[i % copies]
        if M <= 16:
            ops.hard_forward_smallm_multi([L["q"], L["k"], L["v"]], xs[2560])
            ops.hard_forward_smallm(L["o"], xs[4096], out=out_o)
            ops.hard_forward_smallm_multi([L["gate"], L["up"]], xs[2560])
            ops.hard_forward_smallm(L["down"], xs[9728], out=out_d)
        else:
            for k in ("q", "k", "v", "o", "gate", "up", "down"):
                ops.hard_forward_smallm(L[k], xs[QWEN_LAYER[k][1]])
    return run, sum(weight_bytes(n, k) for n, k in QWEN_LAYER.values())


def extra_configs(torch, ops, plz_native, dev, pk):
    """Measurements of the other single-GPU configurations, each with inputs or weights that exceed L2."""
    out = {}
    gen = torch.Generator(device=dev).manual_seed(0)
    N, K = N_OUT, K_IN
    wb = weight_bytes(N, K)
    copies = (2 * 126 * 2 ** 20) // wb + 2
    ws = [make_weight(torch, ops, N, K, dev, gen) for _ in range(copies)]
    # config 0: hard forward at M = 512 through the tiled tcgen05 kernel, weights rotated
    x512 = torch.randn(512, K, device=dev).to(torch.bfloat16)
    ys = [torch.empty(512, N, dtype=torch.bfloat16, device=dev)]
    ms = graph_timed(torch, lambda i: ops.hard_forward(ws[i % copies], x512), copies, 10)
    fl = 2.0 * 512 * N * K
    out["config0_hard_fwd_M512"] = {"us": ms * 1e3, "tflops": fl / (ms * 1e-3) / 1e12, "frac_of_burst_peak": fl / (ms * 1e-3) / 1e12 / pk["tflops_burst"],
                                    "kernel": "lut_gemm_kernel<B_DECODE_K>", "weights_rotated": copies}
    # small-M decode, one 9728 x 2560 Linear per launch
    sm = {}
    for M in (1, 8, 64):
        xm = torch.randn(M, K, device=dev).to(torch.bfloat16)
        yy = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        ms = graph_timed(torch, lambda i: ops.hard_forward_smallm(ws[i % copies], xm, out=yy[i & 1]), copies, 10)
        gbs = wb / (ms * 1e-3) / 1e9
        sm[f"M{M}"] = {"us": ms * 1e3, "GBps": gbs, "frac_of_hbm": gbs / pk["hbm_gbs"]}
    out["smallm_one_linear_9728x2560"] = dict(sm, weight_bytes=wb, weights_rotated=copies, timing="CUDA graph, one launch per weight copy")
    del ws, ys
    # small-M decode over the seven Linears of a layer (4 launches per layer, launches allowed to overlap)
    layer = {}
    lcopies = 10
    plz_native.lib().plz_set_smallm_overlap(1)
    try:
        for M in (1, 8):
            run, lbytes = layer_decode_runner(torch, ops, plz_native, dev, M, lcopies)
            ms = graph_timed(torch, run, lcopies, 10)
            gbs = lbytes / (ms * 1e-3) / 1e9
            layer[f"M{M}"] = {"us_per_layer": ms * 1e3, "GBps": gbs, "frac_of_hbm": gbs / pk["hbm_gbs"]}
            del run
    finally:
        plz_native.lib().plz_set_smallm_overlap(0)
    out["smallm_layer_7_linears"] = dict(layer, weight_bytes_per_layer=lbytes, layers_rotated=lcopies,
                                         launches_per_layer=4, timing="CUDA graph of 10 layers, programmatic dependent launches")
    # config 2: four Qwen3-style decoder layers (hidden 2560, 32 / 8 heads of 128, intermediate 9728, rank-16 LoRA on all seven
    # hard-palettized Linears), forward + backward at batch 32 x seq 512, every op a kernel of this library
    import decoder_layer as DL
    cfg = DL.LayerConfig()
    Bc, Sc, n_layers = 32, 512, 4
    layers = [DL.random_layer(cfg, dev, seed=10 + i) for i in range(n_layers)]
    gl = torch.Generator(device=dev).manual_seed(3)
    xl = torch.randn(Bc * Sc, cfg.hidden, generator=gl, device=dev).to(torch.bfloat16)
    dyl = torch.randn(Bc * Sc, cfg.hidden, generator=gl, device=dev).to(torch.bfloat16)
    cos, sin = ops.rope_tables(Sc, cfg.head_dim, cfg.rope_theta, dev)
    n0 = plz_native.lib().plz_launch_count()
    DL.stack_forward_backward(cfg, layers, xl, dyl, Bc, Sc, cos, sin)
    launches = plz_native.lib().plz_launch_count() - n0
    for _ in range(2):
        DL.stack_forward_backward(cfg, layers, xl, dyl, Bc, Sc, cos, sin)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(5):
        DL.stack_forward_backward(cfg, layers, xl, dyl, Bc, Sc, cos, sin)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 5
    lin_fl = 3 * 2.0 * Bc * Sc * sum(n * k for n, k in cfg.shapes().values())
    att_fl = 7 * 2.0 * Bc * cfg.n_heads * Sc * Sc * cfg.head_dim / 2       # 2 forward + 5 backward GEMMs, causal half
    out["config2_stack_4_layers_B32_S512"] = {
        "ms": ms, "tokens_per_s": Bc * Sc / (ms * 1e-3), "tflops": n_layers * (lin_fl + att_fl) / (ms * 1e-3) / 1e12,
        "frac_of_burst_peak": n_layers * (lin_fl + att_fl) / (ms * 1e-3) / 1e12 / pk["tflops_burst"], "kernel_launches": int(launches),
        "what": "4 decoder layers forward + backward (activations kept, hand-written backward): RMSNorm, q/k/v/o/gate/up/down hard LUT GEMMs "
                "with LoRA, q/k norm + RoPE, causal GQA attention on tcgen05, SwiGLU, residuals; gradients of palettes, LoRA factors and norm weights"}
    del layers, xl, dyl
    torch.cuda.empty_cache()
    # config 4, one GPU, super-block sized: a distillation step over 4 layers in SOFT mode (index logits trained, counter-based
    # Gumbel noise) against a dense bf16 teacher of the same 4 layers on a second stream, loss, backward, fused AdamW
    import distill_step as DS
    sb = DS.Superblock(DL.LayerConfig(), 4, dev, seed=20, max_positions=512)
    xs = torch.randn(Bc * Sc, 2560, device=dev).to(torch.bfloat16)
    n0 = plz_native.lib().plz_launch_count()
    sb.step(xs, Bc, Sc)
    launches = plz_native.lib().plz_launch_count() - n0
    sb.step(xs, Bc, Sc)
    torch.cuda.synchronize()
    a.record()
    for _ in range(3):
        stats = sb.step(xs, Bc, Sc)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 3
    out["config4_superblock_distill_step_B32_S512"] = {
        "ms": ms, "tokens_per_s": Bc * Sc / (ms * 1e-3), "kernel_launches": int(launches), "loss": float(stats[0].item()),
        "what": "one optimizer step on 16384 tokens: dense bf16 teacher forward of 4 layers (side stream) + student forward in soft mode "
                "(logits -> packed argmax per Linear, LUT GEMMs + LoRA) + cos/MSE loss + backward with dLogits, dPalette, dA, dB from the "
                "weight-gradient epilogues + fused fp32-master AdamW on index logits (403.6 M weights x 4 logits), palettes, LoRA, norms"}
    sb.close()
    del sb, xs
    torch.cuda.empty_cache()
    # config 3: the full 36-layer model (vocab 151936, tied embeddings), every Linear hard-palettized, inference only:
    # prefill of 8 x 2048 tokens, then one decode step at batch 1 / 8 / 64 against a 2048-token bf16 key / value cache
    import decode_model as DM
    mcfg = DM.ModelConfig()
    model = DM.PalettizedQwen.random(mcfg, dev, seed=4, max_positions=2304)
    gm = torch.Generator(device=dev).manual_seed(5)
    c3 = {"what": "36 layers, hidden 2560, 32 / 8 heads of 128, intermediate 9728, vocab 151936 tied; random-init; all seven Linears per "
                  "layer 2-bit palettized, no LoRA", "layer_weight_bytes": model.weight_bytes(), "embedding_bytes": model.embed.numel() * 2}
    Bp, Sp = 8, 2048
    ids = torch.randint(0, mcfg.vocab, (Bp, Sp), generator=gm, device=dev)
    cache = model.new_cache(Bp, Sp)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for it in range(3):
        cache.length = 0
        torch.cuda.synchronize()
        a.record()
        model.prefill(ids, cache)
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    ms = min(times[1:])
    lin_fl = 2.0 * Bp * Sp * (sum(n * k for n, k in mcfg.shapes().values()) * mcfg.n_layers)
    att_fl = mcfg.n_layers * 2 * 2.0 * Bp * mcfg.n_heads * Sp * Sp * mcfg.head_dim / 2
    c3["prefill_B8_S2048"] = {"ms": ms, "tokens_per_s": Bp * Sp / (ms * 1e-3), "tflops": (lin_fl + att_fl) / (ms * 1e-3) / 1e12,
                              "frac_of_burst_peak": (lin_fl + att_fl) / (ms * 1e-3) / 1e12 / pk["tflops_burst"]}
    del cache, ids
    torch.cuda.empty_cache()
    T0 = 2048
    for Bd in (1, 8, 64):
        cache = model.new_cache(Bd, T0 + 1)
        cache.k.normal_(generator=gm)
        cache.v.normal_(generator=gm)
        cache.length = T0
        step_ids = torch.randint(0, mcfg.vocab, (Bd,), generator=gm, device=dev)
        n0 = plz_native.lib().plz_launch_count()
        graph, _ = model.decode_graph(step_ids, cache, T0)
        launches = (plz_native.lib().plz_launch_count() - n0) // 2
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        a.record()
        for _ in range(10):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 10
        kv_bytes = 2 * mcfg.n_layers * Bd * (T0 + 1) * mcfg.n_kv_heads * mcfg.head_dim * 2
        total = model.weight_bytes() + model.embed.numel() * 2 + kv_bytes
        c3[f"decode_B{Bd}_T2048"] = {"ms_per_step": ms, "tokens_per_s": Bd / (ms * 1e-3), "kv_cache_bytes": kv_bytes, "kernel_launches": int(launches),
                                     "GBps": total / (ms * 1e-3) / 1e9, "frac_of_hbm": total / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                                     "timing": "CUDA graph of one whole step (embedding, 36 layers, final norm, logits), replayed"}
        del graph, cache
        torch.cuda.empty_cache()
    out["config3_inference_36_layers"] = c3
    del model
    torch.cuda.empty_cache()
    # the reference API (layout R: fp16 planar logits (4, K, N), one palette per 256 output columns) through torch autograd
    import fused_lut_linear_cuda as F
    g2 = torch.Generator(device=dev).manual_seed(2)
    xr = torch.randn(M_TOK, K, generator=g2, device=dev).to(torch.bfloat16).requires_grad_(True)
    dyr = torch.randn(M_TOK, N, generator=g2, device=dev).to(torch.bfloat16)
    pal = (torch.randn(N // 256, 4, generator=g2, device=dev) * 0.02).sort(-1).values.to(torch.bfloat16).requires_grad_(True)
    lg = torch.randn(4, K, N, generator=g2, device=dev).to(torch.float16).requires_grad_(True)

    def ref_step():
        xr.grad = pal.grad = lg.grad = None
        F.fused_lut_linear_soft(xr, pal, lg, None, 256, TAU).backward(dyr)
    for _ in range(3):
        ref_step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(10):
        ref_step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 10
    out["reference_api_layout_R_step"] = {"ms": ms, "tokens_per_s": M_TOK / (ms * 1e-3), "tflops": 3 * GEMM_FLOPS / (ms * 1e-3) / 1e12,
                                          "what": "fused_lut_linear_soft forward + backward through torch autograd, M=16384, no LoRA, counter-based noise"}
    return out


def run_case(a):
    """One kernel of the hot path, a few launches, on a small case: the full 9728 x 2560 weight matrix of the benchmark Linear
    (so per-tile behaviour is the benchmark's) with the token count cut to --M; under 2 GB on the device.  For ncu."""
    import torch
    import plz_native
    import plz_ops as ops
    import synth
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    if a.case in ("layer1", "layer8"):
        M = 1 if a.case == "layer1" else 8
        plz_native.lib().plz_set_smallm_overlap(1)
        run, _ = layer_decode_runner(torch, ops, plz_native, dev, M, 10)
        for i in range(max(a.iters, 1) * 10):
            run(i)
        torch.cuda.synchronize()
        print("status", plz_native.device_status())
        return
    if a.case == "layertrain":
        # one full-size decoder layer, forward + backward, at batch 8 x seq 512 (a quarter of the config-2 batch)
        import decoder_layer as DL
        cfg = DL.LayerConfig()
        P_ = DL.random_layer(cfg, dev, seed=10)
        g = torch.Generator(device=dev).manual_seed(3)
        Bc, Sc = 8, 512
        xl = torch.randn(Bc * Sc, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
        dyl = torch.randn(Bc * Sc, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
        cos, sin = ops.rope_tables(Sc, cfg.head_dim, cfg.rope_theta, dev)
        for _ in range(max(a.iters, 1)):
            DL.stack_forward_backward(cfg, [P_], xl, dyl, Bc, Sc, cos, sin)
        torch.cuda.synchronize()
        print("status", plz_native.device_status())
        return
    if a.case in ("decode1", "decode8", "decode64", "prefill"):
        # two full-size layers of the 36-layer model (vocab cut to 32768 rows) so that a capture stays small: one decode step at
        # batch 1 / 8 / 64 against a 2048-token cache, or a prefill of 2 x 1024 tokens
        import decode_model as DM
        mcfg = DM.ModelConfig(n_layers=2, vocab=32768)
        model = DM.PalettizedQwen.random(mcfg, dev, seed=4, max_positions=2304)
        gm = torch.Generator(device=dev).manual_seed(5)
        if a.case == "prefill":
            ids = torch.randint(0, mcfg.vocab, (2, 1024), generator=gm, device=dev)
            cache = model.new_cache(2, 1024)
            for _ in range(max(a.iters, 1)):
                cache.length = 0
                model.prefill(ids, cache)
        else:
            Bd = int(a.case[6:])
            cache = model.new_cache(Bd, 2049)
            cache.k.normal_(generator=gm)
            cache.v.normal_(generator=gm)
            ids = torch.randint(0, mcfg.vocab, (Bd,), generator=gm, device=dev)
            for _ in range(max(a.iters, 1)):
                model.decode_logits(ids, cache, 2048)
        torch.cuda.synchronize()
        print("status", plz_native.device_status())
        return
    d = synth.make_linear_inputs_cuda(a.M, a.N, a.K, seed=0)
    pal = d["palette"].reshape(-1, 4).contiguous()
    w = ops.PackedWeight(ops.pack_indices(d["idx"].view(torch.int8), n_major=True), pal, a.N, a.K, 1, 256)
    lora = (d["lora_a"], d["lora_b"], 1.0)
    t = dt = w2 = rstd = g = stage = None
    if a.case == "dwscatter":
        # the data-parallel form of the dW launch as rank 0 of 2, both owners' staging buffers in this GPU's memory (ncu
        # profiles one process; the peer stores become local stores, everything else is the multi-GPU kernel)
        stage = torch.empty(2, a.N // 2, a.K, 4, dtype=torch.float32, device=dev)
    if a.case in ("dw", "dwscatter"):  # the workspaces the weight-gradient launch takes its dA / dB side items from
        t = ops.hard_forward(w, d["x"], lora)[1]
        dt = ops.lora_dt(lora, d["dy"])
    if a.case == "gateup":  # second matrix of the fused gate/up launch and the RMSNorm factors
        w2 = ops.PackedWeight(ops.pack_indices(((d["idx"].view(torch.uint8) + 1) & 3).view(torch.int8), n_major=True), pal, a.N, a.K, 1, 256)
        rstd = ops.rms_rstd(d["x"], 1e-6)
        g = torch.ones(a.K, dtype=torch.bfloat16, device=dev)
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
        elif a.case == "select":
            ops.soft_select(w, d["logits"], "nk4", noise=d["noise"], tau=1.0, want_packed=True)
        else:
            raise SystemExit(f"unknown --case {a.case}")
    torch.cuda.synchronize()
    print("status", plz_native.device_status())


def run_distill(args):
    """--workload distill: the super-block distillation step (distill_step.Superblock: 4 layers of the Qwen-4B shape, dense
    teacher, soft student, loss, backward, optimizer) on N GPUs, 16384 tokens per rank (weak scaling). At N > 1 the
    index-logit gradients go through the reduce-scatter fused into the weight-gradient kernels with the sharded AdamW
    (--exchange allreduce: plain NCCL all-reduce of every gradient and a replicated AdamW, for comparison), and before timing
    the two exchanges are compared on a small super-block (same inputs, 2 steps, parameters must agree)."""
    import torch
    import torch.distributed as dist
    import decoder_layer as DL
    import distill_step as DS
    import plz_native
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local if world > 1 else 0)
    fused = args.exchange != "allreduce"
    parity = None
    if world > 1 and fused and not args.no_parity:
        cfg_s = DL.LayerConfig(hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, intermediate=512)
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        xs = torch.randn(256, cfg_s.hidden, generator=g, device=dev).to(torch.bfloat16)
        res = []
        for f in (True, False):
            sb = DS.Superblock(cfg_s, 2, dev, seed=7, fused_exchange=f, max_positions=256)
            for _ in range(2):
                sb.step(xs, 1, 256)
            torch.cuda.synchronize()
            L = sb.student[0]["down"]
            res.append((L.logits.clone(), L.w.palette.float().clone(), L.lora_b.float().clone(), sb.norms[1].post_ln.float().clone()))
            sb.close()
        worst = max((a - b).abs().max().item() for a, b in zip(*res))
        t = torch.tensor([worst], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        parity = {"param_max_abs_diff_fused_vs_allreduce": t.item(), "pass": bool(t.item() < 2e-3),
                  "what": "2 layers (hidden 256), 2 steps: logits, palette, LoRA B, norm weight after the fused exchange + sharded AdamW "
                          "against all-reduce + replicated AdamW"}
    cfg = DL.LayerConfig()
    Bc, Sc, n_layers = 32, 512, 4
    sb = DS.Superblock(cfg, n_layers, dev, seed=20, fused_exchange=fused, max_positions=Sc)
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(Bc * Sc, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        sb.step(x, Bc, Sc)
    barrier()
    plz_native.device_status()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = plz_native.lib().plz_launch_count()
    t0.record()
    for _ in range(args.steps):
        stats = sb.step(x, Bc, Sc)
    t1.record()
    launches = plz_native.lib().plz_launch_count() - n0
    barrier()
    ms = t0.elapsed_time(t1)
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()
    plz_native.device_status()
    line = {"metric": "distillation-step tokens/s, 4-layer super-block of the Qwen-4B shape", "value": Bc * Sc * world * args.steps / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "super-block distillation step: dense bf16 teacher + soft palettized student (LoRA r16), 4 layers, "
                                   "batch 32 x seq 512 per GPU, loss, backward, AdamW on logits / palettes / LoRA / norms",
                       "exchange": "none" if world == 1 else ("fused reduce-scatter in the weight-gradient kernels + sharded logits AdamW"
                                                             if fused else "NCCL all-reduce + replicated AdamW"), "parallelism": f"dp{world}"},
            "gpu_launches": int(launches), "loss": float(stats[0].item()), "parity": parity}
    sb.close()
    if rank == 0:
        os.dup2(saved_stdout, 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["pass"]:
        raise SystemExit(3)


def run_kernel_table(a):
    """Per-kernel measurements beside the step benchmark, one JSON line each: small-M decode at M in {1, 8, 16, 64} for three
    Linear shapes (weights rotated over more than 2 x L2 of copies, launches inside a CUDA graph), gate + up in one launch,
    overlapped launches, the layer of seven Linears, config 0, soft_select and the element-wise backward kernels."""
    import torch
    import plz_native
    import plz_ops as ops
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pk = peaks()
    hbm = pk["hbm_gbs"]
    iters = a.iters if a.iters > 3 else 200
    gen = torch.Generator(device=dev).manual_seed(0)
    for (N, K) in [(9728, 2560), (2560, 9728), (4096, 2560)]:
        wb = weight_bytes(N, K)
        copies = (2 * 126 * 2 ** 20) // wb + 2
        ws = [make_weight(torch, ops, N, K, dev, gen) for _ in range(copies)]
        reps = max(1, iters // copies)
        for M in (1, 8, 16, 64):
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            ys = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
            ms = graph_timed(torch, lambda i: ops.hard_forward_smallm(ws[i % copies], x, out=ys[i & 1]), copies, reps)
            print(json.dumps({"case": "smallm", "M": M, "N": N, "K": K, "us": ms * 1e3, "weight_bytes": wb, "GBps": wb / (ms * 1e-3) / 1e9,
                              "frac_of_hbm": wb / (ms * 1e-3) / 1e9 / hbm, "weights_rotated": copies}), flush=True)
        if (N, K) == (9728, 2560):
            pairs = copies // 2
            for overlap in (0, 1):
                plz_native.lib().plz_set_smallm_overlap(overlap)
                for M in (1, 8, 16):
                    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
                    ms = graph_timed(torch, lambda i: ops.hard_forward_smallm_multi([ws[2 * (i % pairs)], ws[2 * (i % pairs) + 1]], x), pairs,
                                     max(1, iters // pairs))
                    print(json.dumps({"case": "smallm gate+up in one launch", "overlapped_launches": overlap, "M": M, "us": ms * 1e3,
                                      "GBps": 2 * wb / (ms * 1e-3) / 1e9, "frac_of_hbm": 2 * wb / (ms * 1e-3) / 1e9 / hbm}), flush=True)
            plz_native.lib().plz_set_smallm_overlap(0)
            x = torch.randn(512, K, device=dev).to(torch.bfloat16)
            ms = graph_timed(torch, lambda i: ops.hard_forward(ws[i % copies], x), copies, reps)
            fl = 2.0 * 512 * N * K
            print(json.dumps({"case": "config0", "M": 512, "N": N, "K": K, "us": ms * 1e3, "TFLOPs": fl / (ms * 1e-3) / 1e12,
                              "frac_of_burst_peak": fl / (ms * 1e-3) / 1e12 / pk["tflops_burst"]}), flush=True)
        del ws
    for overlap in (0, 1):
        plz_native.lib().plz_set_smallm_overlap(overlap)
        for M in (1, 8, 16):
            run, lbytes = layer_decode_runner(torch, ops, plz_native, dev, M, 10)
            ms = graph_timed(torch, run, 10, max(1, iters // 10))
            print(json.dumps({"case": "smallm layer (7 Linears, 4 launches)", "overlapped_launches": overlap, "M": M, "us_per_layer": ms * 1e3,
                              "GBps": lbytes / (ms * 1e-3) / 1e9, "frac_of_hbm": lbytes / (ms * 1e-3) / 1e9 / hbm}), flush=True)
            del run
    plz_native.lib().plz_set_smallm_overlap(0)
    N, K = N_OUT, K_IN

    def plain(fn, n):
        fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n
    logits = torch.randn(N, K, 4, device=dev)
    w = ops.PackedWeight(ops.empty_packed(N, K, dev), torch.zeros(N * (K // 256), 4, dtype=torch.bfloat16, device=dev), N, K, 1, 256)
    ms = plain(lambda: ops.soft_select(w, logits, "nk4", want_packed=True), 50)
    rb = N * K * 16 + N * K // 4
    print(json.dumps({"case": "select", "us": ms * 1e3, "bytes": rb, "GBps": rb / (ms * 1e-3) / 1e9, "frac_of_hbm": rb / (ms * 1e-3) / 1e9 / hbm}), flush=True)
    del logits
    M = M_TOK
    gate, up, dact = (torch.randn(M, N, device=dev).to(torch.bfloat16) for _ in range(3))
    ms = plain(lambda: ops.swiglu_backward(gate, up, dact), 30)
    rb = 5 * M * N * 2
    print(json.dumps({"case": "swiglu backward", "us": ms * 1e3, "bytes": rb, "GBps": rb / (ms * 1e-3) / 1e9, "frac_of_hbm": rb / (ms * 1e-3) / 1e9 / hbm}), flush=True)
    del gate, up, dact
    Mx = 65536  # 335 MB per tensor, so that x + dH exceed L2
    xx, dh = (torch.randn(Mx, K, device=dev).to(torch.bfloat16) for _ in range(2))
    nw = torch.ones(K, dtype=torch.bfloat16, device=dev)
    rstd = ops.rms_rstd(xx, 1e-6)
    ms = plain(lambda: ops.rmsnorm_backward(xx, dh, rstd, nw), 30)
    rb = 3 * Mx * K * 2
    print(json.dumps({"case": "rmsnorm backward", "us": ms * 1e3, "bytes": rb, "GBps": rb / (ms * 1e-3) / 1e9, "frac_of_hbm": rb / (ms * 1e-3) / 1e9 / hbm}), flush=True)
    print(json.dumps({"status": list(plz_native.device_status())}), flush=True)


_CPU_INPUTS = {}


def cpu_step_sampled(m_s, n_s, threads):
    """One step of the CPU checker (the restatement of the reference's PyTorch path) on a sample of the workload:
    m_s tokens, the first n_s of the 9728 output rows, full K.  Returns seconds."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import plz_oracle as O
    import synth
    torch.set_num_threads(threads)
    key = (m_s, n_s)
    if key not in _CPU_INPUTS:
        _CPU_INPUTS.clear()
        _CPU_INPUTS[key] = synth.make_linear_inputs(m_s, n_s, K_IN, seed=0, rank=RANK)
    d = _CPU_INPUTS[key]
    t0 = time.perf_counter()
    O.linear_step(d["x"], d["dy"], d["logits"], d["noise"], d["palette"], TAU, 1, 256, lora=(d["lora_a"], d["lora_b"], 1.0), ste=True)
    return time.perf_counter() - t0


def cpu_sample_plan(budget_s, threads):
    """Pick (m_s, n_s) so that one CPU step takes about budget_s seconds; every cost of the step is proportional
    to the number of output rows, so a row sample is scaled back by N / n_s."""
    m_s, n_s = 2048, 608
    t = cpu_step_sampled(m_s, n_s, threads)            # calibration (also warms the thread pool)
    scale = max(1.0, min(budget_s / max(t, 1e-3), (M_TOK / m_s) * (N_OUT / n_s)))
    while scale >= 2.0 and m_s < M_TOK:
        m_s *= 2; scale /= 2.0
    while scale >= 2.0 and n_s * 2 <= N_OUT:
        n_s *= 2; scale /= 2.0
    return m_s, n_s


def cpu_baseline(budget_s=20.0):
    import torch
    threads = os.cpu_count() or 1
    m_s, n_s = cpu_sample_plan(budget_s, threads)
    t = cpu_step_sampled(m_s, n_s, threads)
    full_t = t * (N_OUT / n_s)                          # seconds for m_s tokens through the full Linear
    return {"value": m_s / full_t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{m_s} of {M_TOK} tokens x {n_s} of {N_OUT} output rows (time scaled by {N_OUT / n_s:.2f}), one step, "
                      f"{t:.2f} s measured; oracle/plz_oracle.py = restatement of the reference's PyTorch CPU path"}


def run_reference(args):
    """The reference's CPU implementation of the path (its PyTorch functions, restated in oracle/plz_oracle.py and
    pinned against them) on this box's host cores, same metric and config.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    threads = os.cpu_count() or 1
    total_steps = args.steps + args.warmup
    m_s, n_s = cpu_sample_plan(max(2.0, 150.0 / max(total_steps, 1)), threads)
    for _ in range(args.warmup):
        cpu_step_sampled(m_s, n_s, threads)
    ts = [cpu_step_sampled(m_s, n_s, threads) for _ in range(args.steps)]
    t = sum(ts) / len(ts)
    full_t = t * (N_OUT / n_s)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    val = m_s / full_t
    sample = f"{m_s} of {M_TOK} tokens x {n_s} of {N_OUT} output rows per step (time scaled by {N_OUT / n_s:.2f})"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": M_TOK / val * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": M_TOK, "N": N_OUT, "K": K_IN, "lora_rank": RANK, "parallelism": "cpu"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="N = 1: skip the extra_configs measurements (config 0, small-M decode, reference-API step)")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the correctness check of the fused exchange that runs before the timed region")
    ap.add_argument("--sustained-s", type=float, default=3.0, help="length of the sustained leg in seconds (0 = off)")
    ap.add_argument("--pair-gemm", type=int, default=1, help="0: keep the large products on the one-CTA-per-tile kernels (comparison)")
    ap.add_argument("--workload", default="linear", choices=["linear", "distill"],
                    help="linear (default): the benchmark step of one Linear; distill: the super-block distillation step (its own JSON line)")
    ap.add_argument("--case", default=None, help="run ONE kernel of the hot path a few times on a small case and exit (for ncu captures)")
    ap.add_argument("--kernels", action="store_true", help="per-kernel table: one JSON line per measurement")
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--N", type=int, default=N_OUT)
    ap.add_argument("--K", type=int, default=K_IN)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--defer-exchange", type=int, default=0, help="N > 1, fused slot mode: 1 = the whole exchange of a step runs on the side stream and is "
                    "waited for right before the next step's weight-gradient kernel (0, the default = waited for at the end of its own step; "
                    "deferring measured slower at 2 and 8 GPUs: the all-gather then competes with the HBM-bound select pass)")
    ap.add_argument("--split-dx", type=int, default=0, help="N > 1, fused slot mode: rows of dX computed beside the small all-reduce (0 = off; with it the exch_sync phase "
                         "contains that first block of dX)")
    ap.add_argument("--comm-sms", type=int, default=-1, help="N > 1: SMs the dX kernel leaves to the exchange (default: built-in)")
    ap.add_argument("--exchange", default="fused", choices=["fused", "fused-add", "allreduce"],
                    help="N > 1: dLogits reduce-scatter fused into the weight-gradient kernel (default) or a plain NCCL all-reduce")
    args = ap.parse_args()
    if args.workload == "distill":
        run_distill(args)
    elif args.case:
        run_case(args)
    elif args.kernels:
        run_kernel_table(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
