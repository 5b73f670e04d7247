"""Multi-GPU execution of one query: contiguous shards, one process per GPU, NCCL for the exchange step.

The reference runs LINQ queries on device 0 only (src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:188)
and has a generic data-parallel splitter that the LINQ path never calls
(src/Core/DotCompute.Core/Execution/ParallelExecutionStrategy.cs:167-218); NCCL is an enum label without a binding
(src/Core/DotCompute.Core/Execution/Types/CommunicationBackend.cs:12-19). Here the element range is cut into
contiguous shards, each rank runs the fused kernel on its shard, and only the 128-byte record crosses NVLink:

  reductions, by default  connect_peers(): a one-warp kernel on a side stream stores each GPU's partial into every
                          peer's memory over NVLink, waits (bounded) for theirs and folds them in rank order; it runs
                          beside the next query's reduce kernel, so the exchange is off the critical path
  reductions, NCCL route  Sum / Average / Count: the record tensor goes straight into all_reduce(SUM) on the same
                          stream; Min / Max: records are all-gathered and folded in rank order (NaN bookkeeping
                          needs an OR, which NCCL has no reduction for)
  ToArray                 each rank compacts its shard; all_gather of the survivor counts gives every rank its
                          offset in the global result, which is the shards' outputs concatenated in rank order -
                          identical to the single-GPU stable order

`torch.distributed` is plumbing only (process group, NCCL/gloo calls); the records and their combination are
ours. The combine functions take plain tensors, so they are exercised on CPU with the gloo backend.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import errors, native as N
from .accelerator import CudaAccelerator, UnifiedBuffer, dcb_type
from .linq import CompiledPipeline

_INT_SMALL = (N.T_I8, N.T_U8, N.T_I16, N.T_U16, N.T_I32, N.T_U32, N.T_BOOL)


def _stream_handle(stream) -> int:
    """cudaStream_t of a torch stream as an integer the C ABI accepts. Torch reports its default stream as 0, which the
    ABI reads as "the context's own stream", so the legacy default stream is passed by its CUDA handle value
    (cudaStreamLegacy == 1)."""
    return stream.cuda_stream or 1


def shard_bounds(n: int, world: int, rank: int, elem_size: int = 4) -> tuple[int, int]:
    """[start, stop) of rank's contiguous shard of n elements. Every shard but the last has ceil(n/world) elements
    rounded up to a multiple of 16 bytes, so each shard base stays 128-bit aligned for the vector kernels."""
    if world <= 0 or not (0 <= rank < world):
        raise errors.ArgumentException("bad world / rank")
    if n < 0:
        raise errors.ArgumentException("n must not be negative")
    per = -(-n // world)
    align = max(1, 16 // max(elem_size, 1))
    per = -(-per // align) * align
    start = min(n, rank * per)
    stop = min(n, start + per)
    return start, stop


def fold_records(records: np.ndarray, out_type: int) -> np.ndarray:
    """Fold per-rank records (shape [world, 16] int64) in rank order into one record. Exact: integer sums are carried
    in 128 bits, floating sums are added in rank order (deterministic for a given world size)."""
    recs = np.asarray(records, dtype=np.int64).reshape(-1, N.SLOT_NSLOTS)
    out = recs[0].copy()
    f = out.view(np.float64)
    if int(recs[0][N.SLOT_FLAGS]) & N.RES_PREFIX_RANGE:
        # checked integer Sum: append the ranks' (total, smallest, largest running sum) in rank order
        def wide(r, lo_slot):
            return (int(r[lo_slot + 1]) << 64) + (int(r[lo_slot]) & (2**64 - 1))

        def put(slot, v):
            out[slot] = np.array(v & (2**64 - 1), dtype=np.uint64).view(np.int64)
            out[slot + 1] = np.int64(v >> 64)

        s = lo = hi = 0
        flags = 0
        for r in recs:
            rs = wide(r, N.SLOT_ISUM_LO)
            lo = min(lo, s + wide(r, N.SLOT_PREFIX_MIN_LO))
            hi = max(hi, s + wide(r, N.SLOT_PREFIX_MAX_LO))
            s += rs
            flags |= int(r[N.SLOT_FLAGS])
        bits = 31 if out_type == N.T_I32 else 63
        over = lo < -(2**bits) or hi > 2**bits - 1
        put(N.SLOT_ISUM_LO, s)
        put(N.SLOT_PREFIX_MIN_LO, lo)
        put(N.SLOT_PREFIX_MAX_LO, hi)
        out[N.SLOT_FLAGS] = (flags & ~N.RES_OVERFLOW) | (N.RES_OVERFLOW if over else 0)
        return out
    isum = (int(recs[0][N.SLOT_ISUM_HI]) << 64) + (int(recs[0][N.SLOT_ISUM_LO]) & (2**64 - 1))
    unsigned = out_type == N.T_U64
    for r in recs[1:]:
        rf = r.view(np.float64)
        f[N.SLOT_FSUM] += rf[N.SLOT_FSUM]
        isum += (int(r[N.SLOT_ISUM_HI]) << 64) + (int(r[N.SLOT_ISUM_LO]) & (2**64 - 1))
        out[N.SLOT_COUNT] += r[N.SLOT_COUNT]
        f[N.SLOT_FMIN] = min(f[N.SLOT_FMIN], rf[N.SLOT_FMIN])
        f[N.SLOT_FMAX] = max(f[N.SLOT_FMAX], rf[N.SLOT_FMAX])
        if unsigned:
            a, b = int(out[N.SLOT_IMIN]) & (2**64 - 1), int(r[N.SLOT_IMIN]) & (2**64 - 1)
            out[N.SLOT_IMIN] = np.array(min(a, b), dtype=np.uint64).view(np.int64)
            a, b = int(out[N.SLOT_IMAX]) & (2**64 - 1), int(r[N.SLOT_IMAX]) & (2**64 - 1)
            out[N.SLOT_IMAX] = np.array(max(a, b), dtype=np.uint64).view(np.int64)
        else:
            out[N.SLOT_IMIN] = min(out[N.SLOT_IMIN], r[N.SLOT_IMIN])
            out[N.SLOT_IMAX] = max(out[N.SLOT_IMAX], r[N.SLOT_IMAX])
        out[N.SLOT_FLAGS] |= r[N.SLOT_FLAGS]
    lo = isum & (2**64 - 1)
    hi = (isum >> 64)
    out[N.SLOT_ISUM_LO] = np.array(lo, dtype=np.uint64).view(np.int64)
    out[N.SLOT_ISUM_HI] = np.int64(max(min(hi, 2**63 - 1), -2**63))
    f[N.SLOT_COUNT_F] = float(out[N.SLOT_COUNT])
    return out


def combine_record(rec, terminal: int, out_type: int, group=None):
    """Combine the 16-slot int64 record tensor `rec` across ranks, in place, with the cheapest exact collective.
    `rec` lives where the process group works (CUDA for nccl, CPU for gloo). Returns the tensor."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return rec
    fp = out_type in (N.T_F32, N.T_F64)
    if terminal in (N.OP_SUM, N.OP_AVERAGE) and fp:
        dist.all_reduce(rec.view(torch.float64)[N.SLOT_FSUM: N.SLOT_COUNT_F + 1], op=dist.ReduceOp.SUM, group=group)
        if terminal == N.OP_AVERAGE:
            dist.all_reduce(rec[N.SLOT_COUNT: N.SLOT_COUNT + 1], op=dist.ReduceOp.SUM, group=group)
        return rec
    if (terminal == N.OP_AVERAGE or out_type != N.T_I32) and terminal in (N.OP_SUM, N.OP_AVERAGE) and out_type in _INT_SMALL:
        # per-rank sums of <= 32-bit elements stay far inside int64, so a plain int64 SUM is exact
        dist.all_reduce(rec[N.SLOT_ISUM_LO: N.SLOT_COUNT + 1], op=dist.ReduceOp.SUM, group=group)
        rec[N.SLOT_ISUM_HI] = torch.where(rec[N.SLOT_ISUM_LO] < 0, -1, 0)
        return rec
    if terminal in (N.OP_COUNT, N.OP_TOARRAY):
        dist.all_reduce(rec[N.SLOT_COUNT: N.SLOT_COUNT + 1], op=dist.ReduceOp.SUM, group=group)
        return rec
    # Min / Max, and Sum over int / long (checked: the running sum's range must be appended in rank order): gather every
    # rank's record and fold exactly in rank order.
    world = dist.get_world_size(group)
    gathered = torch.empty((world, N.SLOT_NSLOTS), dtype=torch.int64, device=rec.device)
    dist.all_gather_into_tensor(gathered, rec.reshape(1, -1), group=group) if rec.is_cuda else \
        dist.all_gather(list(gathered.unbind(0)), rec, group=group)
    folded = fold_records(gathered.cpu().numpy(), out_type)
    rec.copy_(torch.from_numpy(folded).to(rec.device))
    return rec


def gather_counts(local_count: int, device=None, group=None):
    """all_gather of per-shard survivor counts -> (counts per rank, this rank's offset, total)."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [int(local_count)], 0, int(local_count)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    mine = torch.tensor([int(local_count)], dtype=torch.int64, device=device)
    allc = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allc, mine, group=group)
    counts = [int(c.item()) for c in allc]
    return counts, sum(counts[:rank]), sum(counts)


def finalize_record(rec_host: np.ndarray, terminal: int, out_type: int) -> N.Result:
    """dcb_record_finalize on a host copy of a (combined) record; raises the System.Linq exceptions."""
    rec = np.ascontiguousarray(rec_host, dtype=np.int64)
    res = N.Result()
    N.check(N.lib().dcb_record_finalize(terminal, out_type, rec.ctypes.data_as(C.c_void_p), C.byref(res)))
    return res


def connect_peers(acc: CudaAccelerator, group=None) -> bool:
    """Set up the fused combine: every rank creates its exchange area, the CUDA IPC handles are all-gathered, and each
    rank maps its peers' areas (dcb_peer_connect). From then on every reduction run on `acc` exchanges its partial with
    the other GPUs inside the reduce kernel (NVLink peer stores) and its record holds the global result; no collective is
    launched per query. Returns False (and leaves the NCCL path in place) when there is a single rank."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return False
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if world > 8:
        raise errors.NotSupportedException("the fused combine serves up to 8 GPUs of one node")
    handle = (C.c_ubyte * 64)()
    N.check(N.lib().dcb_peer_area_create(acc.handle, handle, 64), acc.handle)
    mine = torch.tensor(list(handle), dtype=torch.uint8, device=f"cuda:{acc.DeviceId}")
    allh = torch.empty(world * 64, dtype=torch.uint8, device=mine.device)
    dist.all_gather_into_tensor(allh, mine, group=group)
    table = np.ascontiguousarray(allh.cpu().numpy())
    N.check(N.lib().dcb_peer_connect(acc.handle, world, rank, table.ctypes.data_as(C.c_void_p), 64), acc.handle)
    dist.barrier(group)          # every rank has mapped every area before the first exchange
    acc._peers_connected = True
    return True


def disconnect_peers(acc: CudaAccelerator) -> None:
    N.check(N.lib().dcb_peer_disconnect(acc.handle), acc.handle)
    acc._peers_connected = False


class ShardedQuery:
    """One rank's part of a sharded query. `local` is this rank's shard (a device UnifiedBuffer), `ops` the
    (kind, lambda) list without the terminal."""

    RING = 8     # records in flight: a reduction may be enqueued before the exchange of the one RING steps earlier ended

    def __init__(self, accelerator: CudaAccelerator, local: UnifiedBuffer, ops=(), local_second: UnifiedBuffer | None = None,
                 group=None, force_jit: bool = False):
        self.acc = accelerator
        self.local = local
        self.second = local_second
        self.ops = tuple(ops)
        self.group = group
        self.force_jit = force_jit
        self._pipes = {}
        self._ring = None
        self._step = 0
        self._side = None
        self._kernel_done = None
        self._exchange_done = None

    @property
    def fused(self) -> bool:
        return bool(getattr(self.acc, "_peers_connected", False))

    def pipeline(self, terminal: int) -> CompiledPipeline:
        if terminal not in self._pipes:
            t1 = dcb_type(self.second.dtype) if self.second is not None else N.T_NONE
            self._pipes[terminal] = CompiledPipeline(self.acc, dcb_type(self.local.dtype), t1,
                                                     self.ops + ((terminal, None),), self.force_jit)
        return self._pipes[terminal]

    def _setup(self):
        import torch
        if self._ring is None:
            dev = f"cuda:{self.acc.DeviceId}"
            self._ring = [torch.zeros(N.SLOT_NSLOTS, dtype=torch.int64, device=dev) for _ in range(self.RING)]
            self._kernel_done = [torch.cuda.Event() for _ in range(self.RING)]
            self._exchange_done = [None] * self.RING
            self._side = torch.cuda.Stream(device=dev)

    def record_tensor(self):
        self._setup()
        return self._ring[0]

    def launch_local(self, terminal: int, stream, rec) -> None:
        """Only the fused kernel over this rank's shard, on `stream` (a torch stream); its 128-byte record goes to `rec`."""
        pipe = self.pipeline(terminal)
        n = self.local.Length if self.second is None else min(self.local.Length, self.second.Length)
        in1 = C.c_void_p(self.second.GetDeviceMemory()) if self.second is not None else None
        N.check(N.lib().dcb_pipeline_run_async(pipe.handle, C.c_void_p(self.local.GetDeviceMemory()), in1, n, None, 0,
                                               C.c_void_p(rec.data_ptr()), None, C.c_void_p(_stream_handle(stream))), self.acc.handle)

    def exchange(self, terminal: int, stream, rec, slot: int):
        """Enqueue the combination of `rec` across ranks. Fused: a one-warp kernel on the side stream, gated by an event on
        `stream`; returns the event that marks the record complete. NCCL: collectives on `stream`; returns None."""
        import torch
        pipe = self.pipeline(terminal)
        if not self.fused:
            with torch.cuda.stream(stream):
                combine_record(rec, terminal, pipe.info.out_type, self.group)
            return None
        self._kernel_done[slot].record(stream)
        self._side.wait_event(self._kernel_done[slot])
        N.check(N.lib().dcb_peer_exchange_async(self.acc.handle, C.c_void_p(rec.data_ptr()), pipe.info.out_type,
                                                C.c_void_p(_stream_handle(self._side))), self.acc.handle)
        done = self._exchange_done[slot] or torch.cuda.Event()
        done.record(self._side)
        self._exchange_done[slot] = done
        return done

    def enqueue_reduce(self, terminal: int, stream):
        """Kernel on `stream`, then the exchange step. No host synchronisation. Returns (record tensor, event or None): the
        record holds the global result once the event has completed (fused), or once `stream` reaches this point (NCCL)."""
        self._setup()
        slot = self._step % self.RING
        self._step += 1
        rec = self._ring[slot]
        if self._exchange_done[slot] is not None:
            stream.wait_event(self._exchange_done[slot])     # the record's previous use must be over before it is rewritten
        self.launch_local(terminal, stream, rec)
        return rec, self.exchange(terminal, stream, rec, slot)

    def reduce(self, terminal: int):
        """Run a reduction over all shards and return its scalar (same value on every rank)."""
        import torch
        stream = torch.cuda.current_stream()
        rec, done = self.enqueue_reduce(terminal, stream)
        if done is not None:
            done.synchronize()
        else:
            stream.synchronize()
        pipe = self.pipeline(terminal)
        res = finalize_record(rec.cpu().numpy(), terminal, pipe.info.out_type)
        return pipe.scalar(res)

    def Sum(self):
        return self.reduce(N.OP_SUM)

    def Average(self):
        return self.reduce(N.OP_AVERAGE)

    def Min(self):
        p = self.pipeline(N.OP_MIN)
        return p.out_dtype.type(self.reduce(N.OP_MIN))

    def Max(self):
        p = self.pipeline(N.OP_MAX)
        return p.out_dtype.type(self.reduce(N.OP_MAX))

    def Count(self):
        return self.reduce(N.OP_COUNT)

    def compact_local(self, out: UnifiedBuffer, stream_ptr: int = 0):
        """Enqueue this rank's compaction into `out`; returns the record tensor whose COUNT slot holds the local count."""
        pipe = self.pipeline(N.OP_TOARRAY)
        rec = self.record_tensor()
        n = self.local.Length if self.second is None else min(self.local.Length, self.second.Length)
        in1 = C.c_void_p(self.second.GetDeviceMemory()) if self.second is not None else None
        N.check(N.lib().dcb_pipeline_run_async(pipe.handle, C.c_void_p(self.local.GetDeviceMemory()), in1, n,
                                               C.c_void_p(out.GetDeviceMemory()), out.Length, C.c_void_p(rec.data_ptr()), None,
                                               C.c_void_p(stream_ptr)), self.acc.handle)
        return rec

    def enqueue_compact(self, out: UnifiedBuffer, stream, rec=None):
        """Compaction of this rank's shard into `out` on `stream` (a torch stream), then the exchange of the survivor counts.
        Fused route: the one-warp peer-store kernel on the same stream leaves, in the record, the global total
        (SLOT_COUNT), this rank's own count (SLOT_LOCAL_COUNT) and the number of survivors on lower ranks (SLOT_OFFSET),
        with no collective and no host round trip. Returns the record tensor; it is complete when `stream` gets there."""
        pipe = self.pipeline(N.OP_TOARRAY)
        if rec is None:
            rec = self.record_tensor()
        n = self.local.Length if self.second is None else min(self.local.Length, self.second.Length)
        in1 = C.c_void_p(self.second.GetDeviceMemory()) if self.second is not None else None
        sh = C.c_void_p(_stream_handle(stream))
        N.check(N.lib().dcb_pipeline_run_async(pipe.handle, C.c_void_p(self.local.GetDeviceMemory()), in1, n,
                                               C.c_void_p(out.GetDeviceMemory()), out.Length, C.c_void_p(rec.data_ptr()), None, sh),
                self.acc.handle)
        if self.fused:
            N.check(N.lib().dcb_peer_exchange_async(self.acc.handle, C.c_void_p(rec.data_ptr()), pipe.info.out_type, sh), self.acc.handle)
        return rec

    def ToArray(self):
        """Compacts the local shard. Returns (local survivors as a host array, this rank's offset in the global
        result, global survivor count). Concatenating the local arrays in rank order gives the single-GPU result."""
        import torch
        pipe = self.pipeline(N.OP_TOARRAY)
        n = self.local.Length if self.second is None else min(self.local.Length, self.second.Length)
        out = self.acc.Memory.AllocateAsync(max(n, 1), pipe.out_dtype)
        try:
            stream = torch.cuda.current_stream()
            if pipe.has_filter:
                rec = self.enqueue_compact(out, stream)
                host = rec.cpu().numpy()
                finalize_record(host, N.OP_TOARRAY, pipe.info.out_type)
                if self.fused:
                    local_count, offset, total = int(host[N.SLOT_LOCAL_COUNT]), int(host[N.SLOT_OFFSET]), int(host[N.SLOT_COUNT])
                    arr = out.CopyToAsync(count=local_count) if local_count else np.empty(0, pipe.out_dtype)
                    return arr, offset, total
                local_count = int(host[N.SLOT_COUNT])
            else:
                in1 = C.c_void_p(self.second.GetDeviceMemory()) if self.second is not None else None
                N.check(N.lib().dcb_pipeline_run_async(pipe.handle, C.c_void_p(self.local.GetDeviceMemory()), in1, n,
                                                       C.c_void_p(out.GetDeviceMemory()), n, None, None,
                                                       C.c_void_p(_stream_handle(stream))), self.acc.handle)
                stream.synchronize()
                local_count = n
            counts, offset, total = gather_counts(local_count, device=f"cuda:{self.acc.DeviceId}", group=self.group)
            arr = out.CopyToAsync(count=local_count) if local_count else np.empty(0, pipe.out_dtype)
            return arr, offset, total
        finally:
            out.Dispose()
