"""One rank of the multi-GPU check of the fused reduce-scatter (launched by torchrun from test_gpu_scatter.py, or by hand:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node=N --master-addr 127.0.0.1 tests/scatter_worker.py [slots|add]).
Each rank runs several steps of dW (stores into the peers' staging buffers) -> small all-reduce -> reduce_slots -> all-gather
and compares the result with an NCCL all-reduce of the unfused kernel's dLogits."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "qwen-palettize_b200"))


def main():
    import dp
    import plz_native
    import plz_ops as ops
    import synth
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    M, N, K = 512, 2048, 1024
    base = synth.make_linear_inputs(M, N, K, seed=5, rank=16)   # same parameters on every rank
    mine = synth.make_linear_inputs(M, N, K, seed=50 + rank, rank=16)  # own tokens
    logits, noise = base["logits"].to(dev), base["noise"].to(dev)
    palette = base["palette"].reshape(-1, 4).to(dev)
    lora = (base["lora_a"].to(dev), base["lora_b"].to(dev), base["lora_scale"])
    w = ops.PackedWeight(ops.empty_packed(N, K, dev), palette, N, K, 1, 256)
    ops.soft_select(w, logits, "nk4", noise=noise, tau=1.0, want_packed=True)
    mode = sys.argv[1] if len(sys.argv) > 1 else "slots"
    if mode.endswith("-opt"):
        ok = sharded_optimizer_check(mode.split("-")[0], dp, ops, w, mine, logits, noise, lora, N, K, dev, rank, world)
        finish(ok, plz_native, dist, dev, rank)
        return
    sc = dp.LogitGradScatter(N, K, dev, mode=mode)
    ok = True
    for step in range(4):
        x = (mine["x"] * (1.0 + 0.25 * step)).to(torch.bfloat16).to(dev)
        dy = mine["dy"].to(dev)
        _, t = ops.hard_forward(w, x, lora)
        dt = ops.lora_dt(lora, dy)
        dlog, dpal, da, db = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=1.0, lora_ws=(t, dt))
        for g in (dlog, dpal, da, db):
            dist.all_reduce(g)
        dpal2, da2, db2 = sc.dw(w, x, dy, logits, noise, 1.0, lora_ws=(t, dt))
        h = sc.start([dpal2, da2, db2])
        full = sc.finish(h)
        torch.cuda.synchronize()
        scale = dlog.abs().max().item()
        err = (full - dlog).abs().max().item() / scale
        exact = bool(torch.equal(full, dlog))
        small = max(((a - b).abs().max() / b.abs().max()).item() for a, b in ((dpal2, dpal), (da2, da), (db2, db)))
        print(f"rank {rank} step {step}: dLogits rel err {err:.2e} bit-exact {exact}; small grads rel err {small:.2e}", flush=True)
        ok = ok and err < 1e-5 and small < 1e-4 and (exact or world > 2 or mode == "add")
    sc.close()
    finish(ok, plz_native, dist, dev, rank)


def finish(ok, plz_native, dist, dev, rank):
    st = plz_native.device_status()
    ok = ok and st[0] == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    if flag.item() != 1:
        sys.exit(1)
    if rank == 0:
        print("SCATTER_OK", flush=True)


def sharded_optimizer_check(mode, dp, ops, w, mine, logits, noise, lora, N, K, dev, rank, world):
    """Each rank runs AdamW on its own rows only (state of 1 / world of the size) and the updated parameter rows are
    gathered; the result must follow a replicated AdamW on the all-reduced gradient of the unfused kernel."""
    sc = dp.LogitGradScatter(N, K, dev, mode=mode, shard_optimizer=True)
    sc.param.copy_(logits)
    r0, r1 = sc.shard_rows()
    m_s = torch.zeros((r1 - r0) * K * 4, device=dev)
    v_s = torch.zeros_like(m_s)
    ref = logits.clone()
    ref_m, ref_v = torch.zeros(N * K * 4, device=dev), torch.zeros(N * K * 4, device=dev)
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-3)
    ok = True
    for step in range(4):
        x = (mine["x"] * (1.0 + 0.25 * step)).to(torch.bfloat16).to(dev)
        dy = mine["dy"].to(dev)
        _, t = ops.hard_forward(w, x, lora)
        dt = ops.lora_dt(lora, dy)
        dlog = ops.backward_dw_soft(w, x, dy, ref, "nk4", noise=noise, tau=1.0)[0]
        dist.all_reduce(dlog)
        ops.adamw_step(ref.view(-1), ref_m, ref_v, dlog.view(-1), step + 1, **hp)
        small = sc.dw(w, x, dy, sc.param, noise, 1.0, lora_ws=(t, dt))
        h = sc.start(list(small), step_fn=lambda p, g: ops.adamw_step(p.reshape(-1), m_s, v_s, g.reshape(-1), step + 1, **hp))
        sc.finish(h)
        torch.cuda.synchronize()
        err = (sc.param - ref).abs().max().item()
        moved = (ref - logits).abs().max().item()
        print(f"rank {rank} step {step}: sharded-optimizer parameter max abs diff {err:.2e} (moved {moved:.2e})", flush=True)
        ok = ok and err < 2e-5 and moved > 1e-3
    sc.close()
    return ok


if __name__ == "__main__":
    main()
