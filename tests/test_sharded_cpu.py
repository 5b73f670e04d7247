"""Host logic of the multi-GPU path, without a GPU: shard bounds, record folding, and the collectives run as two gloo
ranks on CPU. Each rank fabricates the record its kernel would have written from the CPU oracle's partial over its
shard; the combined, finalized result must equal the oracle over the whole array."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dotcompute_b200 import native as N
from dotcompute_b200.sharded import combine_record, finalize_record, fold_records, gather_counts, shard_bounds

F = np.float32


@pytest.mark.parametrize("n,world,esz", [(0, 1, 4), (1, 2, 4), (10, 4, 4), (1 << 30, 8, 4), (1000003, 8, 4), (1000003, 3, 8), (17, 8, 1)])
def test_shard_bounds_partition_the_range(n, world, esz):
    prev = 0
    for r in range(world):
        a, b = shard_bounds(n, world, r, esz)
        assert a == prev and a <= b <= n
        assert (a * esz) % 16 == 0 or a == n             # every shard starts 16-byte aligned
        prev = b
    assert prev == n


def _record_for(x, terminal):
    """The record a rank's kernel leaves for Where(x>0.5f).Select(x*x+3f).<terminal> over its shard (oracle partials)."""
    v = x[x > F(0.5)]
    v = v * v + F(3)
    rec = np.zeros(16, dtype=np.int64)
    f = rec.view(np.float64)
    f[N.SLOT_FSUM] = np.cumsum(v.astype(np.float64))[-1] if v.size else 0.0
    rec[N.SLOT_COUNT] = v.size
    f[N.SLOT_COUNT_F] = float(v.size)
    f[N.SLOT_FMIN] = v.min() if v.size else np.inf
    f[N.SLOT_FMAX] = v.max() if v.size else -np.inf
    rec[N.SLOT_FLAGS] = 16 if v.size else 0
    return rec


def _int_record(k):
    rec = np.zeros(16, dtype=np.int64)
    s = int(k.astype(object).sum()) if k.size else 0
    rec[N.SLOT_ISUM_LO] = np.array(s & (2**64 - 1), dtype=np.uint64).view(np.int64)
    rec[N.SLOT_ISUM_HI] = s >> 64
    rec[N.SLOT_COUNT] = k.size
    rec[N.SLOT_IMIN] = k.min() if k.size else np.iinfo(np.int64).max
    rec[N.SLOT_IMAX] = k.max() if k.size else np.iinfo(np.int64).min
    return rec


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = np.random.Generator(np.random.PCG64(31)).random(n, dtype=F)
        a, b = shard_bounds(n, world, rank, 4)
        out = {}
        for name, term in (("sum", N.OP_SUM), ("avg", N.OP_AVERAGE), ("count", N.OP_COUNT), ("min", N.OP_MIN), ("max", N.OP_MAX)):
            rec = torch.from_numpy(_record_for(x[a:b], term).copy())
            combine_record(rec, term, N.T_F32)
            res = finalize_record(rec.numpy(), term, N.T_F32)
            out[name] = res.count if term == N.OP_COUNT else res.f64
        k = np.random.Generator(np.random.PCG64(8)).integers(-2**62, 2**62, n, dtype=np.int64)
        rec = torch.from_numpy(_int_record(k[a:b]).copy())
        combine_record(rec, N.OP_SUM, N.T_I64)              # 64-bit sums take the gather-and-fold route (128-bit exact)
        try:
            out["isum"] = finalize_record(rec.numpy(), N.OP_SUM, N.T_I64).i64
        except Exception as e:                              # overflow is a legitimate outcome here
            out["isum"] = type(e).__name__
        k32 = np.random.Generator(np.random.PCG64(8)).integers(-1000, 1001, n, dtype=np.int32)
        rec = torch.from_numpy(_int_record(k32[a:b].astype(np.int64)).copy())
        combine_record(rec, N.OP_SUM, N.T_I32)              # 32-bit sums take the plain all-reduce
        out["isum32"] = finalize_record(rec.numpy(), N.OP_SUM, N.T_I32).i64
        local_count = int((x[a:b] > F(0.5)).sum())
        counts, offset, total = gather_counts(local_count)
        out["counts"], out["offset"], out["total"] = counts, offset, total
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_combine_across_gloo_ranks(world):
    n = 200_003
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = np.random.Generator(np.random.PCG64(31)).random(n, dtype=F)
    v = x[x > F(0.5)]
    v = v * v + F(3)
    raw = float(np.cumsum(v.astype(np.float64))[-1])
    k = np.random.Generator(np.random.PCG64(8)).integers(-2**62, 2**62, n, dtype=np.int64)
    isum = int(k.astype(object).sum())
    k32 = np.random.Generator(np.random.PCG64(8)).integers(-1000, 1001, n, dtype=np.int32)
    bounds = [shard_bounds(n, world, r, 4) for r in range(world)]
    counts = [int((x[a:b] > F(0.5)).sum()) for a, b in bounds]
    for r in range(world):
        out = results[r]
        assert abs(out["sum"] - raw) <= 1e-5 * raw and out["sum"] == float(F(raw)) or abs(out["sum"] - float(F(raw))) <= abs(float(np.spacing(F(raw))))
        assert abs(out["avg"] - raw / v.size) <= 1e-5 * raw / v.size
        assert out["count"] == v.size
        assert out["min"] == float(v.min()) and out["max"] == float(v.max())
        assert out["isum"] == (isum if -2**63 <= isum < 2**63 else "OverflowException")
        assert out["isum32"] == int(k32.astype(np.int64).sum())
        assert out["counts"] == counts and out["offset"] == sum(counts[:r]) and out["total"] == sum(counts)


def test_fold_records_is_exact_and_ordered():
    recs = np.stack([_int_record(np.array([2**62, 2**62], dtype=np.int64)), _int_record(np.array([2**62, -5], dtype=np.int64))])
    out = fold_records(recs, N.T_I64)
    total = 3 * 2**62 - 5
    assert (int(out[N.SLOT_ISUM_HI]) << 64) + (int(out[N.SLOT_ISUM_LO]) & (2**64 - 1)) == total
    assert out[N.SLOT_COUNT] == 4 and out[N.SLOT_IMIN] == -5 and out[N.SLOT_IMAX] == 2**62
    u = np.zeros((2, 16), dtype=np.int64)
    u[0][N.SLOT_IMIN] = np.array(2**63 + 5, dtype=np.uint64).view(np.int64)
    u[0][N.SLOT_IMAX] = np.array(2**63 + 5, dtype=np.uint64).view(np.int64)
    u[1][N.SLOT_IMIN] = 7
    u[1][N.SLOT_IMAX] = 7
    out = fold_records(u, N.T_U64)
    assert out[N.SLOT_IMIN] == 7 and int(out[N.SLOT_IMAX]) & (2**64 - 1) == 2**63 + 5     # unsigned order


def _prefix_record(k, bits):
    """What the checked Sum kernel leaves for one shard: total, smallest and largest running sum (empty prefix included)."""
    rec = np.zeros(16, dtype=np.int64)
    pref = [0]
    for v in k.tolist():
        pref.append(pref[-1] + int(v))

    def put(slot, v):
        rec[slot] = np.array(v & (2**64 - 1), dtype=np.uint64).view(np.int64)
        rec[slot + 1] = v >> 64
    put(N.SLOT_ISUM_LO, pref[-1])
    put(N.SLOT_PREFIX_MIN_LO, min(pref))
    put(N.SLOT_PREFIX_MAX_LO, max(pref))
    over = min(pref) < -(2**bits) or max(pref) > 2**bits - 1
    rec[N.SLOT_FLAGS] = N.RES_PREFIX_RANGE | (N.RES_OVERFLOW if over else 0)
    return rec


@pytest.mark.parametrize("dtype,t,bits", [(np.int32, N.T_I32, 31), (np.int64, N.T_I64, 63)])
def test_fold_records_appends_running_sum_ranges_in_rank_order(dtype, t, bits):
    top = 2**bits - 1
    shards_ok = [np.array([top - 10, -3], dtype=dtype), np.array([13, -top], dtype=dtype), np.array([5], dtype=dtype)]
    out = fold_records(np.stack([_prefix_record(s, bits) for s in shards_ok]), t)
    assert not int(out[N.SLOT_FLAGS]) & N.RES_OVERFLOW            # touches the maximum exactly, never above
    assert finalize_record(out, N.OP_SUM, t).i64 == 5
    assert (int(out[N.SLOT_PREFIX_MAX_HI]) << 64) + (int(out[N.SLOT_PREFIX_MAX_LO]) & (2**64 - 1)) == top
    # the same shards in another order cross the limit in the middle although every shard alone, and the total, are inside
    shards_bad = [shards_ok[0], np.array([14, -top - 1], dtype=dtype), shards_ok[2]]
    assert all(not int(_prefix_record(s, bits)[N.SLOT_FLAGS]) & N.RES_OVERFLOW for s in shards_bad)
    out = fold_records(np.stack([_prefix_record(s, bits) for s in shards_bad]), t)
    assert int(out[N.SLOT_FLAGS]) & N.RES_OVERFLOW
    with pytest.raises(Exception) as e:
        finalize_record(out, N.OP_SUM, t)
    assert type(e.value).__name__ == "OverflowException"
