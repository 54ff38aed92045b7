"""The weight-gradient kernel with the reduce-scatter of dLogits fused into its epilogue.

One GPU: the ranks are emulated as consecutive launches of one process, each with its own token shard and its own rank
number, all staging buffers in this GPU's memory (the launches do not wait on one another).  The reduced shards must be
bit-identical to the rank-ordered sum of the unfused kernel's per-rank dLogits, and match the CPU oracle run on the whole
batch.  Two GPUs (skipped on a one-GPU machine): the real thing, two processes under torchrun, staging buffers mapped
through CUDA IPC, against an NCCL all-reduce of the unfused gradients.
"""
import os
import subprocess
import sys

import pytest
import torch

import plz_oracle as O
from helpers import assert_close, check_status

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_inputs(world, M, N, K):
    import synth
    base = synth.make_linear_inputs(M, N, K, seed=11, rank=16)
    shards = []
    for r in range(world):
        s = synth.make_linear_inputs(M, N, K, seed=100 + r, rank=16)
        shards.append((s["x"], s["dy"]))
    return base, shards


@pytest.mark.parametrize("world,M,N,K", [(2, 256, 512, 512), (4, 200, 1024, 256), (8, 128, 1024, 768), (5, 96, 960, 768)])
def test_emulated_ranks_bit_exact_and_oracle(world, M, N, K):
    import plz_ops as ops
    base, shards = _rank_inputs(world, M, N, K)
    dev = torch.device("cuda", 0)
    logits, noise = base["logits"].to(dev), base["noise"].to(dev)
    palette = base["palette"].reshape(-1, 4).to(dev)
    lora = (base["lora_a"].to(dev), base["lora_b"].to(dev), base["lora_scale"])
    w = ops.PackedWeight(ops.empty_packed(N, K, dev), palette, N, K, 1, 256)
    ops.soft_select(w, logits, "nk4", noise=noise, tau=1.0, want_packed=True)
    rows = N // world
    stage = torch.full((world, world, rows, K, 4), float("nan"), dtype=torch.float32, device=dev)  # [owner][source]
    ptrs = [stage[o].data_ptr() for o in range(world)]
    unfused, small = [], []
    for r, (x, dy) in enumerate(shards):
        x, dy = x.to(dev), dy.to(dev)
        _, t = ops.hard_forward(w, x, lora)
        dt = ops.lora_dt(lora, dy)
        dlog, dpal, da, db = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=1.0, lora_ws=(t, dt))
        unfused.append(dlog)
        got = ops.backward_dw_soft_scatter(w, x, dy, logits, ptrs, world, r, noise=noise, tau=1.0, lora_ws=(t, dt))
        for g, u, name in zip(got, (dpal, da, db), ("dPalette", "dA", "dB")):
            assert_close(g, u, f"{name} of rank {r}", rel=1e-5)
        small.append(got)
    check_status()
    assert torch.isfinite(stage).all(), "every slot of every staging buffer must have been written"
    full = torch.empty(N, K, 4, dtype=torch.float32, device=dev)
    for o in range(world):
        ops.reduce_slots(ptrs[o], world, full[o * rows:(o + 1) * rows])
    want = unfused[0].clone()
    for u in unfused[1:]:
        want += u
    assert torch.equal(full, want), "fused reduce-scatter must equal the rank-ordered sum of the unfused partials bit for bit"
    # and the whole-batch gradient of the CPU oracle
    xs = torch.cat([s[0] for s in shards]); dys = torch.cat([s[1] for s in shards])
    ref = O.linear_step(xs, dys, base["logits"], base["noise"], base["palette"], 1.0, 1, 256,
                        lora=(base["lora_a"], base["lora_b"], base["lora_scale"]), ste=True)
    assert_close(full, ref["dlogits"], "reduced dLogits")
    assert_close(sum(s[0] for s in small), ref["dpalette"], "reduced dPalette")
    assert_close(sum(s[1] for s in small), ref["da"], "reduced dA")
    assert_close(sum(s[2] for s in small), ref["db"], "reduced dB")


def test_emulated_ranks_accumulate_mode():
    """accumulate = 1: partials are added into one zeroed accumulator per owner; equal to the sum up to fp32 addition order."""
    import plz_ops as ops
    world, M, N, K = 4, 200, 1024, 512
    base, shards = _rank_inputs(world, M, N, K)
    dev = torch.device("cuda", 0)
    logits, noise = base["logits"].to(dev), base["noise"].to(dev)
    w = ops.PackedWeight(ops.empty_packed(N, K, dev), base["palette"].reshape(-1, 4).to(dev), N, K, 1, 256)
    ops.soft_select(w, logits, "nk4", noise=noise, tau=1.0, want_packed=True)
    acc = torch.zeros(N, K, 4, dtype=torch.float32, device=dev)  # the owners' accumulators, back to back
    rows = N // world
    ptrs = [acc[o * rows:(o + 1) * rows].data_ptr() for o in range(world)]
    want = torch.zeros_like(acc)
    for r, (x, dy) in enumerate(shards):
        x, dy = x.to(dev), dy.to(dev)
        want += ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=1.0)[0]
        ops.backward_dw_soft_scatter(w, x, dy, logits, ptrs, world, r, noise=noise, tau=1.0, accumulate=True)
    check_status()
    assert_close(acc, want, "accumulated dLogits", rel=1e-6)


def test_scale_and_argument_checks():
    import ctypes as C
    import plz_native as P
    import plz_ops as ops
    dev = torch.device("cuda", 0)
    st = torch.arange(3 * 64, dtype=torch.float32, device=dev).reshape(3, 64)
    out = torch.empty(64, dtype=torch.float32, device=dev)
    ops.reduce_slots(st.data_ptr(), 3, out, scale=0.5)
    assert torch.equal(out, st.sum(0) * 0.5)
    with pytest.raises(P.PlzError):
        ops.reduce_slots(st.data_ptr(), 9, out)
    # world = 3 does not divide N = 512
    d = ops.PackedWeight(ops.empty_packed(512, 256, dev), torch.zeros(512, 4, dtype=torch.bfloat16, device=dev), 512, 256, 1, 256)
    x = torch.zeros(128, 256, dtype=torch.bfloat16, device=dev); dy = torch.zeros(128, 512, dtype=torch.bfloat16, device=dev)
    lg = torch.zeros(512, 256, 4, device=dev)
    with pytest.raises(P.PlzError):
        ops.backward_dw_soft_scatter(d, x, dy, lg, [st.data_ptr()] * 3, 3, 0)
    with pytest.raises(P.PlzError):
        ops.backward_dw_soft_scatter(d, x, dy, lg, [st.data_ptr(), 0], 2, 0)
    check_status()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["slots", "add", "slots-opt", "add-opt"])
def test_two_ranks_over_peer_memory(mode):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(ROOT, "tests", "scatter_worker.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "SCATTER_OK" in r.stdout


def test_peer_memory_helpers_single_process():
    """plz_peer_alloc gives zeroed device memory and a 64-byte handle; plz_peer_copy / plz_peer_zero are asynchronous on the
    given stream; plz_peer_free releases it. (Mapping a handle needs a second process: covered by the two-rank test.)"""
    import ctypes as C
    import plz_native as P
    from dp import _DeviceArray
    n = 1 << 16
    ptr, handle = C.c_void_p(), C.create_string_buffer(64)
    P.check(P.lib().plz_peer_alloc(n * 4, C.byref(ptr), handle), "plz_peer_alloc")
    try:
        assert any(handle.raw), "handle must be filled"
        t = torch.as_tensor(_DeviceArray(ptr.value, (n,)), device="cuda:0")
        assert t.data_ptr() == ptr.value and float(t.abs().sum()) == 0.0
        src = torch.arange(n, dtype=torch.float32, device="cuda:0")
        P.check(P.lib().plz_peer_copy(ptr.value, src.data_ptr(), n * 4, P.stream_ptr()), "plz_peer_copy")
        assert torch.equal(t, src)
        P.check(P.lib().plz_peer_zero(ptr.value + 4 * 16, (n - 16) * 4, P.stream_ptr()), "plz_peer_zero")
        assert torch.equal(t[:16], src[:16]) and float(t[16:].abs().sum()) == 0.0
        assert P.lib().plz_peer_copy(None, src.data_ptr(), 16, P.stream_ptr()) != 0
        assert P.lib().plz_peer_alloc(0, C.byref(ptr), handle) != 0
        del t
    finally:
        torch.cuda.synchronize()
        P.check(P.lib().plz_peer_free(ptr.value), "plz_peer_free")


def test_single_rank_falls_through():
    """Without a process group the exchange object maps nothing and dw() is the plain single-rank launch."""
    import dp
    import plz_ops as ops
    base, shards = _rank_inputs(1, 128, 256, 256)
    dev = torch.device("cuda", 0)
    logits, noise = base["logits"].to(dev), base["noise"].to(dev)
    w = ops.PackedWeight(ops.empty_packed(256, 256, dev), base["palette"].reshape(-1, 4).to(dev), 256, 256, 1, 256)
    ops.soft_select(w, logits, "nk4", noise=noise, tau=1.0, want_packed=True)
    x, dy = shards[0][0].to(dev), shards[0][1].to(dev)
    sc = dp.LogitGradScatter(256, 256, dev)
    assert sc.world == 1 and sc.full is None
    dpal, da, db = sc.dw(w, x, dy, logits, noise, 1.0)
    h = sc.start([dpal, da, db])
    full = sc.finish(h)
    want, wpal = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=1.0)
    check_status()
    assert torch.equal(full, want) and da is None and db is None
    assert_close(dpal, wpal, "dPalette", rel=1e-5)
    sc.close()
