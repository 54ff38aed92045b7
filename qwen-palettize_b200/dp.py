"""Data parallelism over the token axis for the palettized Linear: one process per GPU, parameters
replicated, the batch split across ranks, and ONE exchange step per Linear -- a sum all-reduce of the
parameter gradients (index logits, palettes, LoRA factors), which are all sums over tokens.  y and dX are
row-local and never cross ranks.  The reference is single-GPU (no torch.distributed anywhere), so this has no
counterpart there; correctness is "P ranks on P shards == 1 rank on the whole batch".

Two exchanges: GradExchange, a plain NCCL all-reduce issued on a side stream right after the weight-gradient kernel so
that it overlaps the dX GEMM that follows on the compute stream; and LogitGradScatter, where the weight-gradient
kernel itself stores its dLogits partials into the owner ranks' memory (reduce-scatter fused into the kernel) and the
reduced shards, or the parameter rows updated from them, are gathered by the copy engines.
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


class _DeviceArray:
    """Adapter that lets torch view library-allocated device memory (no copy) through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


class LogitGradScatter:
    """Exchange of the index-logit gradient between data-parallel ranks, built around the weight-gradient kernel:

      1. reduce-scatter inside the kernel: every rank owns N / world weight rows and a peer-visible staging buffer
         fp32 [world, N/world, K, 4].  The epilogue of rank s stores its partial dLogits for row n straight into slot s of
         the owner's buffer -- plain coalesced stores over NVLink, tile by tile while the tensor cores work on the next
         tile.  The partial gradient (398 MB at N x K = 9728 x 2560) is never written locally nor read back by a collective.
      2. a sum all-reduce of the small gradients (dPalette, dA, dB) on the compute stream: it is needed anyway and it is the
         point after which every rank's stores have landed.
      3. reduce_slots: the owner sums its `world` slots in rank order (deterministic) into its rows of `self.full`.
      4. all-gather by the copy engines on a side stream: each rank pushes its reduced shard into the peers' `full`
         buffers (world - 1 asynchronous peer copies, staggered so that every round is a permutation of the ranks), then
         a one-element all-reduce marks "all pushes done".  It uses no SM, so the dX product that runs beside it keeps
         the whole GPU.

    Hazards: a rank can only pass the all-reduce of step 2 after every rank has launched it, i.e. after every rank has
    finished consuming the previous step's `full` and staging slots, so the stores and pushes of a step never overtake
    the readers of the step before.

    mode 'add' replaces the slots and step 3 by vector reductions (red.add.v4.f32, executed by the owner's L2) into one
    shard-sized accumulator per rank: steps 2 and 4 then run entirely on the side stream and nothing of the exchange sits
    on the compute stream, at the price of a run-to-run varying order of the `world` additions per element.

    shard_optimizer=True keeps the parameter itself (`self.param`, fp32 [N, K, 4]) in peer-visible memory; start(small,
    step_fn=...) then runs step_fn(param_rows, grad_rows) on this rank's rows right after the reduction and gathers the
    updated PARAMETER rows instead of the gradient (optimizer state and work of 1 / world of the size per rank).

    Every rank starts the column sweep of its weight-gradient kernel at a different owner (a rotation by rank * tiles /
    world, applied by the launcher), so that at any moment the ranks store into different GPUs.

    With world == 1 nothing is mapped and `dw` falls through to the single-rank entry point."""

    def __init__(self, N: int, K: int, device, group=None, average: bool = False, mode: str = "slots",
                 shard_optimizer: bool = False):
        import ctypes as C
        import plz_native as P
        if mode not in ("slots", "add"):
            raise ValueError("mode must be 'slots' or 'add'")
        if mode == "add" and average:
            raise ValueError("mode 'add' returns sums: fold 1/world into the optimizer's gradient scale instead")
        self.N, self.K, self.group, self.device, self.mode = N, K, group, device, mode
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.scale = 1.0 / self.world if average else 1.0
        self.full = None
        self.ptrs, self.full_ptrs, self.param_ptrs, self._own, self._opened = [], [], [], [], []
        self.param = None          # shard_optimizer: the peer-visible fp32 [N, K, 4] parameter (index logits)
        self.shard_optimizer = shard_optimizer
        if self.world == 1:
            return
        if N % self.world:
            raise ValueError(f"N={N} must be a multiple of the number of ranks ({self.world})")
        self._stream = torch.cuda.Stream(device=device)
        self._done = torch.zeros(1, dtype=torch.float32, device=device)
        # Every rank reaches every collective below whatever fails locally, and all ranks raise together: a rank that
        # raised alone would leave the others waiting in the next collective.
        mine, err = [], None
        try:
            # staging: `world` slots of a shard each, or one shard-sized accumulator; then the gathered gradient
            sizes = [N * K * 16 if mode == "slots" else N * K * 16 // self.world, N * K * 16]
            if shard_optimizer:
                sizes.append(N * K * 16)  # the parameter itself, so that updated rows can be pushed straight into it
            for nbytes in sizes:
                own, handle = C.c_void_p(), C.create_string_buffer(64)
                P.check(P.lib().plz_peer_alloc(nbytes, C.byref(own), handle), "plz_peer_alloc")
                self._own.append(own.value)
                mine.append(handle.raw)
        except Exception as e:  # noqa: BLE001
            err = repr(e)
        handles = [None] * self.world
        dist.all_gather_object(handles, (mine, err), group=group)
        errs = [f"rank {r}: {h[1]}" for r, h in enumerate(handles) if h[1]]
        if not errs:
            try:
                for r, (hs, _) in enumerate(handles):
                    pair = []
                    for j, h in enumerate(hs):
                        if r == self.rank:
                            pair.append(self._own[j])
                            continue
                        p = C.c_void_p()
                        P.check(P.lib().plz_peer_open(C.create_string_buffer(h, 64), C.byref(p)), "plz_peer_open")
                        self._opened.append(p.value)
                        pair.append(p.value)
                    self.ptrs.append(pair[0])
                    self.full_ptrs.append(pair[1])
                    if shard_optimizer:
                        self.param_ptrs.append(pair[2])
            except Exception as e:  # noqa: BLE001
                err = repr(e)
            opened = [None] * self.world
            dist.all_gather_object(opened, err, group=group)
            errs = [f"rank {r}: {e}" for r, e in enumerate(opened) if e]
        if errs:
            self._release()
            raise RuntimeError("peer staging memory could not be set up on every rank: " + "; ".join(errs))
        self.full = torch.as_tensor(_DeviceArray(self._own[1], (N, K, 4)), device=device)
        if shard_optimizer:
            self.param = torch.as_tensor(_DeviceArray(self._own[2], (N, K, 4)), device=device)

    def shard_rows(self):
        """[begin, end) of the weight rows this rank owns (reduces, and with shard_optimizer updates)."""
        rows = self.N // self.world
        return self.rank * rows, (self.rank + 1) * rows

    def dw(self, w, x, dy, logits, noise, tau, seed=0, lora_ws=None):
        """Weight-gradient launch; returns this rank's (dPalette, dA, dB). The dLogits partials are in flight to their owners."""
        if self.world > 1 and getattr(self, "_pending", False):
            # the staging slots / accumulator and `full` of the previous step are still being reduced and gathered
            raise RuntimeError("LogitGradScatter.dw(): the previous step's exchange has not been finished; call "
                               "start(...) and finish(handle) before the next dw()")
        import plz_ops as ops
        if self.world == 1:
            r = ops.backward_dw_soft(w, x, dy, logits, "nk4", noise=noise, tau=tau, seed=seed, lora_ws=lora_ws)
            self.full = r[0]
            return (r[1], r[2], r[3]) if lora_ws is not None else (r[1], None, None)
        self._pending = True
        # the small gradients are produced as views of ONE flat buffer, which sync_small all-reduces in place: no packing
        n_pal = w.palette.numel()
        r = lora_ws[0].shape[1] if lora_ws is not None else 0
        flat = torch.zeros(n_pal + r * w.K + w.N * r, dtype=torch.float32, device=x.device)
        outs = (flat[:n_pal].view(-1, 4), flat[n_pal:n_pal + r * w.K].view(r, w.K), flat[n_pal + r * w.K:].view(w.N, r))
        res = ops.backward_dw_soft_scatter(w, x, dy, logits, self.ptrs, self.world, self.rank, noise=noise, tau=tau, seed=seed,
                                           lora_ws=lora_ws, accumulate=self.mode == "add", outs=outs)
        self._flat = (flat, [t for t in res if t is not None])
        return res

    def start(self, small, step_fn=None):
        """Steps 2-4 above. `small` (dPalette, dA, dB ...) are sum-all-reduced in place on the current stream; the pushes
        of the reduced shard run on the side stream. Returns a handle for finish()."""
        if self.world == 1:
            return None
        if step_fn is not None and self.param is None:
            raise ValueError("step_fn needs shard_optimizer=True (the parameter must live in peer-visible memory)")
        if self.mode == "add":
            return self._start_add(small, step_fn)
        handle = self.sync_small(small)
        self.reduce_and_push(step_fn)
        return handle

    def start_beside(self, small, step_fn=None):
        """Slot mode with NOTHING of the exchange on the compute stream: the small all-reduce (and with it the wait for the
        slowest rank's weight-gradient kernel), the slot reduction, the pushes and the completion all-reduce are all queued
        on the side stream. The caller goes on with work that does not need the gradients (the dX product, the next layer's
        or the next step's forward) and calls finish() before it reads `full` / `small` and before the next dw(), which
        reuses the staging slots: finish() returns only after every rank has reduced its slots (completion all-reduce).
        The side-stream kernels take SMs only between or beside the compute stream's kernels, so the time they need is
        not hidden, but the skew between the ranks is."""
        if self.world == 1:
            return None
        if self.mode == "add":
            return self._start_add(small, step_fn)
        if step_fn is not None and self.param is None:
            raise ValueError("step_fn needs shard_optimizer=True (the parameter must live in peer-visible memory)")
        cur = torch.cuda.current_stream(self.device)
        self._stream.wait_stream(cur)
        with torch.cuda.stream(self._stream):
            handle = self.sync_small(small)
            self.reduce_and_push(step_fn)      # its "current stream" is the side stream here
        return handle

    def _start_add(self, small, step_fn=None):
        """mode 'add': the owner's accumulator already holds the sum once every rank's kernel has finished, so the whole
        exchange runs on the side stream beside dX: small all-reduce (= all kernels finished) -> copy-engine pushes of the
        accumulator into every rank's `full` (this rank's included) -> accumulator zeroed for the next step -> completion
        all-reduce.  A peer's next additions come after it has passed this step's completion all-reduce, hence after the
        zeroing here."""
        import plz_native as P
        cur = torch.cuda.current_stream(self.device)
        self._stream.wait_stream(cur)
        rows = self.N // self.world
        shard_bytes = rows * self.K * 16
        off = self.rank * shard_bytes
        with torch.cuda.stream(self._stream):
            handle = self.sync_small(small)
            sp = self._stream.cuda_stream
            if step_fn is not None:
                # sharded optimizer: update this rank's parameter rows from its accumulator, gather the PARAMETER
                acc = torch.as_tensor(_DeviceArray(self._own[0], (rows, self.K, 4)), device=self.device)
                step_fn(self.param[self.rank * rows:(self.rank + 1) * rows], acc)
                for j in range(1, self.world):
                    dst = (self.rank + j) % self.world
                    P.check(P.lib().plz_peer_copy(self.param_ptrs[dst] + off, self._own[2] + off, shard_bytes, sp), "plz_peer_copy")
            else:
                for j in range(self.world):
                    dst = (self.rank + j) % self.world
                    P.check(P.lib().plz_peer_copy(self.full_ptrs[dst] + off, self._own[0], shard_bytes, sp), "plz_peer_copy")
            P.check(P.lib().plz_peer_zero(self._own[0], shard_bytes, sp), "plz_peer_zero")
            dist.all_reduce(self._done, group=self.group)
        return handle

    def sync_small_beside(self, small):
        """Step 2 on the side stream: the caller puts independent work (part of the dX product) on the compute stream
        meanwhile, so that neither the collective nor the wait for the slowest rank's kernel is exposed;
        reduce_and_push() then waits for it."""
        cur = torch.cuda.current_stream(self.device)
        self._stream.wait_stream(cur)
        with torch.cuda.stream(self._stream):
            handle = self.sync_small(small)
            self._sync_event = torch.cuda.Event()
            self._sync_event.record(self._stream)
        return handle

    def sync_small(self, small):
        """Step 2: sum-all-reduce `small` in place on the current stream (all ranks' staging stores are complete after it)."""
        small = [t for t in small if t is not None]
        flat = getattr(self, "_flat", None)
        if flat is not None and len(flat[1]) == len(small) and all(a is b for a, b in zip(flat[1], small)):
            # exactly the views handed out by dw(): reduce the flat buffer they live in
            self._flat = None
            dist.all_reduce(flat[0], op=dist.ReduceOp.SUM, group=self.group)
            if self.scale != 1.0:
                flat[0].mul_(self.scale)
            return (small, flat[0])
        n = sum(t.numel() for t in small)
        bucket = torch.empty(max(n, 1), dtype=torch.float32, device=self.device)
        o = 0
        for t in small:
            bucket[o:o + t.numel()].copy_(t.reshape(-1))
            o += t.numel()
        dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=self.group)
        o = 0
        for t in small:
            t.copy_(bucket[o:o + t.numel()].reshape(t.shape))
            if self.scale != 1.0:
                t.mul_(self.scale)
            o += t.numel()
        return (small, bucket)

    def reduce_and_push(self, step_fn=None):
        """Steps 3 and 4: reduce this rank's slots on the current stream, push the shard to the peers on the side stream.
        step_fn(param_rows, grad_rows) (shard_optimizer): the optimizer step of this rank's rows runs right after the
        reduction, and the updated PARAMETER rows are gathered instead of the gradient: same bytes on the wire, 1 / world
        of the optimizer state and work per rank, and `self.full` holds only this rank's rows of the gradient."""
        import plz_native as P
        import plz_ops as ops
        ev = getattr(self, "_sync_event", None)
        if ev is not None:  # step 2 ran on the side stream (sync_small_beside)
            torch.cuda.current_stream(self.device).wait_event(ev)
            self._sync_event = None
        rows = self.N // self.world
        shard = self.full[self.rank * rows:(self.rank + 1) * rows]
        ops.reduce_slots(self.ptrs[self.rank], self.world, shard, self.scale)
        src_base, dst_ptrs = self._own[1], self.full_ptrs
        if step_fn is not None:
            step_fn(self.param[self.rank * rows:(self.rank + 1) * rows], shard)
            src_base, dst_ptrs = self._own[2], self.param_ptrs
        cur = torch.cuda.current_stream(self.device)
        self._stream.wait_stream(cur)
        shard_bytes = rows * self.K * 16
        off = self.rank * shard_bytes
        with torch.cuda.stream(self._stream):
            for j in range(1, self.world):
                dst = (self.rank + j) % self.world
                P.check(P.lib().plz_peer_copy(dst_ptrs[dst] + off, src_base + off, shard_bytes, self._stream.cuda_stream),
                        "plz_peer_copy")
            dist.all_reduce(self._done, group=self.group)  # leaves only when every rank has issued and finished its pushes

    def finish(self, handle):
        """The compute stream waits for the pushes; afterwards `self.full` holds the reduced dLogits on every rank."""
        if handle is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._stream)
        self._pending = False
        return self.full

    def _release(self):
        import plz_native as P
        self.full = None
        self.param = None
        for p in self._opened:
            P.lib().plz_peer_close(p)
        self._opened = []
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)  # nobody frees while a peer still has the memory mapped
        for p in self._own:
            P.lib().plz_peer_free(p)
        self._own = []

    def close(self):
        if self.world > 1 and self._own:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # nobody unmaps while a peer may still store
            self._release()
