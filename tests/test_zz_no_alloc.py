"""The allocation-free LoRA forward (plz_hard_fwd_lora_static) against the workspace-taking entry point.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
The entry point exists for hosts that give an operator only its inputs and outputs -- the host owns the device
memory pool and forbids driver allocations inside an operator -- so the [M, rank] LoRA intermediate lives in a
fixed array inside the library instead of a caller workspace.  Two calls in a row with different batches check
that nothing depends on what the previous call left in that shared array."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(M, seed, r=16, dev=0, watch_memory=False):
    import plz_native as P
    import plz_ops as ops
    import synth
    N, K = 512, 512
    d = synth.make_linear_inputs(M, N, K, seed=seed, rank=r, soft=False, with_dy=False)
    with torch.cuda.device(dev):
        x = d["x"].cuda()
        w = ops.PackedWeight(ops.pack_indices(d["idx"].cuda().view(torch.int8), n_major=True),
                             d["palette"].reshape(-1, 4).cuda(), N, K, 1, 256)
        a, b = d["lora_a"].cuda(), d["lora_b"].cuda()
        y_ref, _ = ops.hard_forward(w, x, (a, b, 2.0))            # existing entry point, caller-owned workspace
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        wd, ld = w.desc(), P.lora_desc(a, b, 2.0)
        torch.cuda.synchronize()
        free0, used0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = P.lib().plz_hard_fwd_lora_static(C.byref(wd), x.data_ptr(), x.stride(0), M, C.byref(ld), y.data_ptr(),
                                              y.stride(0), P.stream_ptr())
        P.check(rc, "plz_hard_fwd_lora_static")
        assert P.device_status()[0] == 0                           # synchronizes
        if watch_memory:
            # neither the driver's free-memory figure (cudaMemGetInfo) nor torch's allocator moved across the call
            assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == used0
    return y, y_ref


def test_static_scratch_matches_workspace_entry_point_twice():
    from helpers import assert_close
    y1, r1 = _call_pair(300, seed=1)      # first call on this device: looks up the scratch address
    assert_close(y1, r1, "first call")
    y2, r2 = _call_pair(130, seed=2, watch_memory=True)   # smaller batch: rows 130.. of the scratch still hold call 1's data
    assert_close(y2, r2, "second call")
    assert torch.equal(y1, r1) and torch.equal(y2, r2)   # same kernels, same inputs: identical bits


def test_static_scratch_at_its_largest_size():
    """Exactly M * rank = 262144 elements (4096 rows at rank 64) is accepted and correct."""
    y, r = _call_pair(4096, seed=3, r=64, watch_memory=True)
    assert torch.equal(y, r)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_static_scratch_on_a_second_device():
    """Every device has its own copy of the array and its own cached address."""
    y0, r0 = _call_pair(200, seed=4, dev=0)
    y1, r1 = _call_pair(200, seed=4, dev=1)
    assert torch.equal(y0, r0) and torch.equal(y1, r1) and torch.equal(y0.cpu(), y1.cpu())


def test_static_scratch_rejects_oversized_calls():
    import plz_native as P
    import plz_ops as ops
    N, K = 256, 256
    w = ops.PackedWeight(torch.zeros(N, K // 4, dtype=torch.uint8, device="cuda"),
                         torch.zeros(N, 4, dtype=torch.bfloat16, device="cuda"), N, K, 1, 256)
    a = torch.zeros(64, K, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(N, 64, dtype=torch.bfloat16, device="cuda")
    M = 4097                                                   # 4097 * 64 > 262144 elements
    x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
    y = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    wd, ld = w.desc(), P.lora_desc(a, b, 1.0)
    rc = P.lib().plz_hard_fwd_lora_static(C.byref(wd), x.data_ptr(), K, M, C.byref(ld), y.data_ptr(), N, P.stream_ptr())
    assert rc == 8 and b"exceeds the built-in scratch" in P.lib().plz_last_error()
    torch.cuda.synchronize()
    assert (y == 7.0).all()                                    # refused calls launch nothing
