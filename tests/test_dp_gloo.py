"""The data-parallel exchange on CPU ranks (gloo, world_size 2): sharding covers the batch once, and the
all-reduced gradients equal the single-rank gradients of the whole batch."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rows_partition():
    sys.path.insert(0, os.path.join(ROOT, "qwen-palettize_b200"))
    import dp
    for n, w in [(16384, 8), (10, 3), (5, 8), (0, 2)]:
        spans = [dp.shard_rows(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, ret):
    sys.path.insert(0, os.path.join(ROOT, "qwen-palettize_b200"))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dp
    import plz_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(0)            # same parameters and the same global batch on every rank
    M, N, K, r = 96, 64, 256, 16
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    lg = torch.randn(N, K, 4, generator=g)
    nz = torch.randn(N, K, 4, generator=g)
    pal = (torch.randn(N, 1, 4, generator=g) * 0.02).to(torch.bfloat16)
    lora = ((torch.randn(r, K, generator=g) * 0.05).to(torch.bfloat16), (torch.randn(N, r, generator=g) * 0.05).to(torch.bfloat16), 2.0)
    b, e = dp.shard_rows(M, rank, world)
    loc = O.linear_step(x[b:e], dy[b:e], lg, nz, pal, 1.0, 1, 256, lora=lora)
    grads = [loc["dlogits"].clone(), loc["dpalette"].clone(), loc["da"].clone(), loc["db"].clone()]
    ex = dp.GradExchange(big_bytes=1 << 16)          # dlogits goes alone, the rest share one bucket
    ex.finish(ex.start(grads))
    full = O.linear_step(x, dy, lg, nz, pal, 1.0, 1, 256, lora=lora)
    ok = True
    for got, key in zip(grads, ("dlogits", "dpalette", "da", "db")):
        ok = ok and O.max_rel_err(got, full[key]) < 1e-5
    # y and dX are row-local: the shard's rows equal the corresponding rows of the full batch
    ok = ok and torch.equal(loc["y"], full["y"][b:e]) and torch.equal(loc["dx"], full["dx"][b:e])
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_exchange_equals_single_rank():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_scatter_refuses_a_second_dw_before_finish():
    """The staging slots and the gathered buffer of a step are in use until finish(): a second dw() before it must raise
    (checked on the state alone: no device, no peer memory)."""
    import pytest
    sys.path.insert(0, os.path.join(ROOT, "qwen-palettize_b200"))
    import dp
    sc = dp.LogitGradScatter.__new__(dp.LogitGradScatter)
    sc.world, sc._pending = 2, True
    with pytest.raises(RuntimeError, match="has not been finished"):
        sc.dw(None, None, None, None, None, 1.0)
    sc._pending, sc.full, sc.device = False, "g", None
    assert sc.finish(None) == "g" and sc._pending is False


def _worker_empty_shard(rank, world, port, ret):
    """5 tokens on 8... here 1 token on 2 ranks: rank 1 owns no rows and must still take part in the exchange with zeros."""
    sys.path.insert(0, os.path.join(ROOT, "qwen-palettize_b200"))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dp
    import plz_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(1)
    M, N, K = 1, 16, 256
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    lg = torch.randn(N, K, 4, generator=g)
    nz = torch.randn(N, K, 4, generator=g)
    pal = (torch.randn(N, 1, 4, generator=g) * 0.02).to(torch.bfloat16)
    b, e = dp.shard_rows(M, rank, world)
    if e > b:
        loc = O.linear_step(x[b:e], dy[b:e], lg, nz, pal, 1.0, 1, 256)
        grads = [loc["dlogits"].clone(), loc["dpalette"].clone()]
    else:
        grads = [torch.zeros(N, K, 4), torch.zeros(N, 4)]
    ex = dp.GradExchange(big_bytes=1 << 12)
    ex.finish(ex.start(grads))
    full = O.linear_step(x, dy, lg, nz, pal, 1.0, 1, 256)
    ret[rank] = bool(O.max_rel_err(grads[0], full["dlogits"]) < 1e-6 and O.max_rel_err(grads[1], full["dpalette"]) < 1e-6)
    dist.destroy_process_group()


def test_exchange_with_an_empty_shard():
    world = 2
    port = 31500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker_empty_shard, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
