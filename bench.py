#!/usr/bin/env python
"""Benchmark of the PalettizedLinear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

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
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
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
        os.unlink(self.path)
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

    def step(record):
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(7)] if record else None
        xm = [torch.cuda.Event(enable_timing=True) for _ in range(2)] if record else None
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
            dpal, da, db = scatter.dw(w, x, dy, logits, noise, TAU, lora_ws=(t, dt))
            if record: marks[4].record()
            if scatter.mode == "add":
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
        if scatter is not None:
            dlog = scatter.finish(h1)
        else:
            exch.finish(h1)
        if record: marks[6].record()
        if record:
            ev["select"].append((marks[0], marks[1])); ev["fwd"].append((marks[1], marks[2]))
            ev["lora_dt"].append((marks[2], marks[3])); ev["dw"].append((marks[3], marks[4]))
            if scatter is not None:
                ev["exch_sync"].append((marks[4], xm[0])); ev["exch_reduce"].append((xm[0], xm[1])); ev["dx"].append((xm[1], marks[5]))
            else:
                ev["dx"].append((marks[4], marks[5]))
            if world > 1:
                ev["exch_wait"].append((marks[5], marks[6]))
        return y, dx, dlog, dpal, da, db

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local if world > 1 else 0)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(False)
    barrier()
    plz_native.device_status()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if rank == 0:
        sampler.ready()
    barrier()
    wall0 = time.time()
    t0.record()
    for _ in range(args.steps):
        step(True)
    t1.record()
    barrier()
    wall1 = time.time()
    ms = t0.elapsed_time(t1)
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    plz_native.device_status()
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()
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

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    tokens = M_TOK * world * args.steps
    gemm_phase = max(("fwd", "dw", "dx"), key=lambda p: phase_ms[p])
    kern_ms = {p: max(phase_ms[p] - skinny[p], 1e-6) for p in ("fwd", "dw", "dx")}
    achieved = GEMM_FLOPS / (kern_ms[gemm_phase] * 1e-3) / 1e12
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum): one ncu capture of each kernel at 4096
    # tokens (profiles/*.md) gave measured / algorithmic = 0.51 (fwd: most of y was still in L2 when the capture
    # ended) and 0.87 (dx). The dW launch measured 1391.8 MB there: 1195.4 MB of logits / noise / dLogits that do not
    # depend on the token count, plus x and dY streamed twice (once for dW, once more by the dA / dB side items in
    # the last round); the figure below scales that token-proportional part to the full 16384-token launch.
    alg = {"fwd": M_TOK * K_IN * 2 + N_OUT * K_IN // 4 + N_OUT * (K_IN // 256) * 8 + M_TOK * N_OUT * 2,
           "dx": M_TOK * N_OUT * 2 + N_OUT * K_IN // 4 + N_OUT * (K_IN // 256) * 8 + M_TOK * K_IN * 2,
           "dw": 3 * N_OUT * K_IN * 16 + M_TOK * (N_OUT + K_IN) * 2}
    xdy_small = 4096 * (N_OUT + K_IN) * 2
    traffic = {"fwd": 0.51 * alg["fwd"], "dx": 0.87 * alg["dx"],
               "dw": (1391.8e6 - 2 * xdy_small) + 2 * M_TOK * (N_OUT + K_IN) * 2}
    line = {
        "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": M_TOK, "N": N_OUT, "K": K_IN, "lora_rank": RANK,
                   "parallelism": f"dp{world}", "split_dx_rows": split_rows, "exchange": ("none" if world == 1 else (f"reduce-scatter fused into the dW epilogue over peer memory ({scatter.mode}) + copy-engine all-gather" if scatter is not None else "NCCL all-reduce")), "l2": "inputs larger than L2 (x+dY 403 MB, logits+noise 797 MB per step)"},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": hx.numel() * 2 + hdy.numel() * 2,
                "d2h_bytes_per_step": sum(h.numel() * 4 for h in hout), "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": (7 if scatter is not None else 6) * args.steps,
        "phases_ms": phase_ms,
        "tflops_step": 3 * GEMM_FLOPS * world / (ms / args.steps * 1e-3) / 1e12,
        "roofline": {"bound": "tensor", "kernel": {"fwd": "lut_gemm_kernel<2,B_DECODE_K>", "dw": "tn_gemm_kernel<EPI_SOFT,float,true> (+ dA, dB items)",
                                                    "dx": "lut_gemm_kernel<2,B_DECODE_MN>"}[gemm_phase],
                     "achieved": achieved, "peak": pk["tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / pk["tflops_sustained"],
                     "traffic": traffic[gemm_phase], "traffic_note": "ncu small-case ratio x algorithmic bytes of the full launch", "algorithmic_bytes": alg[gemm_phase], "peak_source": pk["source"] + " (sustained cuBLAS bf16)",
                     "kernel_ms": kern_ms, "skinny_lora_ms": skinny,
                     "per_kernel_tflops": {p: GEMM_FLOPS / (kern_ms[p] * 1e-3) / 1e12 for p in ("fwd", "dw", "dx")}},
    }
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(budget_s=20.0)
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    ap.add_argument("--split-dx", type=int, default=0, help="N > 1, fused slot mode: rows of dX computed beside the small all-reduce (0 = off; with it the exch_sync phase "
                         "contains that first block of dX)")
    ap.add_argument("--comm-sms", type=int, default=-1, help="N > 1: SMs the dX kernel leaves to the exchange (default: built-in)")
    ap.add_argument("--exchange", default="fused", choices=["fused", "fused-add", "allreduce"],
                    help="N > 1: dLogits reduce-scatter fused into the weight-gradient kernel (default) or a plain NCCL all-reduce")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
