"""Data parallelism over the token axis for the palettized Linear: one process per GPU, parameters
replicated, the batch split across ranks, and ONE exchange step per Linear -- a sum all-reduce of the
parameter gradients (index logits, palettes, LoRA factors), which are all sums over tokens.  y and dX are
row-local and never cross ranks.  The reference is single-GPU (no torch.distributed anywhere), so this has no
counterpart there; correctness is "P ranks on P shards == 1 rank on the whole batch".

The exchange is issued on a side stream right after the weight-gradient kernel, so that it overlaps the dX
GEMM that follows on the compute stream.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, rank: int, world: int):
    """Contiguous, balanced [begin, end) range of token rows owned by `rank`."""
    base, rem = divmod(n_rows, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class GradExchange:
    """Sum-all-reduce a fixed set of gradient tensors across the process group.

    Small tensors (palette, LoRA) are flattened into one fp32 bucket so that they cost one collective; tensors
    of at least `big_bytes` (the logit gradients) are reduced in place, one collective each.  Collectives are
    issued in the order the tensors were given, identically on every rank."""

    def __init__(self, group=None, big_bytes: int = 8 << 20, average: bool = False):
        self.group = group
        self.big_bytes = big_bytes
        self.average = average
        self._stream = None

    def world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def _comm_stream(self, device):
        if device.type != "cuda":
            return None
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=device)
        return self._stream

    def start(self, tensors):
        """Begin the exchange; returns a handle for finish().  Gradients must not be touched in between."""
        tensors = [t for t in tensors if t is not None]
        if self.world() == 1 or not tensors:
            return ([], tensors, None, None)
        device = tensors[0].device
        small = [t for t in tensors if t.numel() * t.element_size() < self.big_bytes]
        big = [t for t in tensors if t.numel() * t.element_size() >= self.big_bytes]
        stream = self._comm_stream(device)
        works = []
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream(device))
            ctx = torch.cuda.stream(stream)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx:
            bucket = None
            if small:
                n = sum(t.numel() for t in small)
                bucket = torch.empty(n, dtype=torch.float32, device=device)  # one per exchange in flight
                o = 0
                for t in small:
                    bucket[o:o + t.numel()].copy_(t.reshape(-1))
                    o += t.numel()
                works.append(dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            for t in big:
                works.append(dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        return (works, tensors, (small, bucket), stream)

    def finish(self, handle):
        works, tensors, small_pack, stream = handle
        if not works:
            return tensors
        for w in works:
            w.wait()
        small, bucket = small_pack
        ctx = torch.cuda.stream(stream) if stream is not None else None
        if ctx is not None:
            ctx.__enter__()
        try:
            if bucket is not None:
                o = 0
                for t in small:
                    t.copy_(bucket[o:o + t.numel()].reshape(t.shape))
                    o += t.numel()
            if self.average:
                inv = 1.0 / self.world()
                for t in tensors:
                    t.mul_(inv)
        finally:
            if ctx is not None:
                ctx.__exit__(None, None, None)
        if stream is not None:
            torch.cuda.current_stream(tensors[0].device).wait_stream(stream)
        return tensors
