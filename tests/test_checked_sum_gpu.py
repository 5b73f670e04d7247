"""Sum over int / long is checked the way Enumerable.Sum is (System.Linq adds in a checked context, element by element in
source order): the call fails as soon as a *running* sum leaves the element type's range, even when the total is back
inside. The ordered kernel is compared with the oracle (oracle/linq_oracle.py Enumerable.Sum) on sequences whose running
sum crosses the limit inside one lane's elements, between lanes, warps and blocks, in the host path's chunks, behind a
Where, and on sequences that stay just inside."""
import numpy as np
import pytest

from dotcompute_b200 import AsComputeQueryable, OverflowException
from dotcompute_b200 import native as N
from oracle.linq_oracle import Enumerable

pytestmark = pytest.mark.gpu

I32_MAX, I32_MIN = 2**31 - 1, -(2**31)
I64_MAX, I64_MIN = 2**63 - 1, -(2**63)


def both(x, acc, *ops):
    """(value or 'overflow') from the oracle and from the GPU path for x[.Where][.Select].Sum(). The GPU path runs twice,
    from the host array (chunked staging) and from a device buffer (one launch), and must agree with itself."""
    def run(q, which):
        for op in ops:
            q = getattr(q, op[0])(op[which])     # (operator, C# lambda for the GPU path, numpy callable for the oracle)
        try:
            return q.Sum()
        except (OverflowError, OverflowException):
            return "overflow"
    o = run(Enumerable(x), 2)
    g = run(AsComputeQueryable(x, acc), 1)
    buf = acc.Memory.AllocateAndCopyAsync(x) if x.size else None
    if buf is not None:
        g2 = run(AsComputeQueryable(buf, acc), 1)
        buf.Dispose()
        assert g2 == g, ("host path and device path differ", g, g2)
    return o, g


def test_small_sequences_int(acc):
    cases = [
        [I32_MAX, 1, -5],            # prefix leaves the range, total does not
        [I32_MAX, -5, 1],            # same elements, another order: stays inside
        [I32_MIN, -1, 7],
        [I32_MIN, 7, -1],
        [I32_MAX], [I32_MIN], [], [0],
        [2**30, 2**30 - 1, 1, -1],   # reaches the maximum exactly, then one more
        [2**30, 2**30 - 1, -1, 1],   # touches the maximum only
        [-(2**30), -(2**30), -1, 1], # one below the minimum
        [-(2**30), -(2**30), 1, -1], # touches the minimum only
    ]
    for c in cases:
        x = np.array(c, dtype=np.int32)
        o, g = both(x, acc)
        assert o == g, (c, o, g)


def test_small_sequences_long(acc):
    cases = [
        [I64_MAX, 1, -5], [I64_MAX, -5, 1], [I64_MIN, -1, 7], [I64_MIN, 7, -1], [I64_MAX], [I64_MIN],
        [2**62, 2**62 - 1, 1, -1], [2**62, 2**62 - 1, -1, 1], [-(2**62), -(2**62), -1, 1], [-(2**62), -(2**62), 1, -1],
        [2**62, 2**62, -(2**62), -(2**62)],
    ]
    for c in cases:
        x = np.array(c, dtype=np.int64)
        o, g = both(x, acc)
        assert o == g, (c, o, g)


@pytest.mark.parametrize("n", [1000, 4096 + 3, 1 << 16, (1 << 20) + 5, (1 << 24) + 1])
@pytest.mark.parametrize("where", [False, True])
def test_spike_positions_int(acc, n, where):
    """A flat sequence with one +spike/-spike pair: whether the running sum crosses the limit depends only on which comes
    first. The pair is placed next to each other, across lanes, warps and far apart, at seeded positions."""
    rng = np.random.Generator(np.random.PCG64(n + where))
    base = rng.integers(-3, 4, n, dtype=np.int32)
    ops = (("Where", "x => x != 2", lambda v: v != 2),) if where else ()
    for gap in (1, 5, 70, 513, 4099, n // 2):
        if gap >= n:
            continue
        for _ in range(2):
            i = int(rng.integers(0, n - gap))
            j = i + gap
            for first_up in (True, False):
                x = base.copy()
                x[i], x[j] = (I32_MAX - 100, -(I32_MAX - 100)) if first_up else (-(I32_MAX - 100), I32_MAX - 100)
                o, g = both(x, acc, *ops)
                assert o == g, (n, gap, i, first_up, o, g)


def test_just_inside_and_just_outside(acc):
    """Running sum climbs to exactly int.MaxValue (allowed), or one above (throws), far into a long sequence."""
    n = (1 << 22) + 17
    x = np.zeros(n, dtype=np.int32)
    x[::4096] = 1                     # 1025 ones
    ones = int(x.sum())
    k = 3_000_001
    x[k] = I32_MAX - int(x[:k].sum())     # running sum == int.MaxValue right here
    x[k + 1] = -(I32_MAX // 2)            # and falls back at once
    o, g = both(x, acc)
    assert o == g and o != "overflow"
    y = x.copy(); y[k - 1] = 1            # one more before: crosses
    o, g = both(y, acc)
    assert o == g == "overflow"
    assert ones > 1000


def test_random_walk_long(acc):
    rng = np.random.Generator(np.random.PCG64(77))
    n = (1 << 20) + 3
    x = rng.integers(-(2**40), 2**40, n, dtype=np.int64)
    o, g = both(x, acc)
    assert o == g and o != "overflow"
    x[1000] = I64_MAX - 2**50
    x[900_000] = -(I64_MAX - 2**50)
    o, g = both(x, acc)
    assert o == g     # whether it crosses depends on the walk in between: the oracle decides


def test_select_then_sum_and_zip(acc):
    rng = np.random.Generator(np.random.PCG64(5))
    n = 300_000
    a = rng.integers(0, 40000, n, dtype=np.int32)
    o, g = both(a, acc, ("Select", "x => x * 3", lambda v: v * np.int32(3)))
    assert o == g
    small = a[:15000]
    o, g = both(small, acc, ("Select", "x => x * 3", lambda v: v * np.int32(3)))
    assert o == g and o != "overflow"
    b = rng.integers(-5, 6, n, dtype=np.int32)
    got = AsComputeQueryable(a, acc).Zip(b, "(x, y) => x * y").Sum()
    assert got == int(np.sum(a.astype(np.int64) * b.astype(np.int64)))


def test_host_chunks_keep_source_order(acc):
    """The host path cuts the input into chunks; the range of the running sum is appended chunk by chunk."""
    n = (1 << 24) + 11                    # several staging chunks
    x = np.zeros(n, dtype=np.int32)
    x[5] = I32_MAX - 3
    x[n - 7] = -(I32_MAX - 3)
    o, g = both(x, acc)
    assert o == g == 0
    x[n // 2] = 4                         # in a middle chunk: crosses there
    o, g = both(x, acc)
    assert o == g == "overflow"
    x[n // 2] = 3                         # touches the limit only
    o, g = both(x, acc)
    assert o == g == 3


def test_record_carries_the_range(acc):
    """The 128-byte record of an asynchronous run holds the total and the smallest / largest running sum."""
    import ctypes as C
    import torch
    x = np.array([5, -9, 20, -1, 0, 0, -3], dtype=np.int32)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    pipe = AsComputeQueryable(buf, acc)._compile(N.OP_SUM)
    rec = torch.zeros(N.SLOT_NSLOTS, dtype=torch.int64, device="cuda")
    N.check(N.lib().dcb_pipeline_run_async(pipe.handle, C.c_void_p(buf.GetDeviceMemory()), None, x.size, None, 0,
                                           C.c_void_p(rec.data_ptr()), None, None), acc.handle)
    acc.Synchronize()
    r = rec.cpu().numpy()
    assert int(r[N.SLOT_FLAGS]) & N.RES_PREFIX_RANGE
    assert int(r[N.SLOT_ISUM_LO]) == 12 and int(r[N.SLOT_ISUM_HI]) == 0
    assert (int(r[N.SLOT_PREFIX_MIN_LO]), int(r[N.SLOT_PREFIX_MIN_HI])) == (-4, -1)
    assert (int(r[N.SLOT_PREFIX_MAX_LO]), int(r[N.SLOT_PREFIX_MAX_HI])) == (16, 0)
    buf.Dispose()


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
@pytest.mark.parametrize("skip", [0, 1, 2, 3, 4, 5, 8])
def test_slices_that_start_anywhere(acc, dtype, skip):
    """A device slice may start at any element: 32-byte, 16-byte or element alignment each take another load path."""
    rng = np.random.Generator(np.random.PCG64(100 + skip))
    n = 200_003
    x = rng.integers(-50, 51, n, dtype=dtype)
    top = np.iinfo(dtype).max
    x[skip + 7] = top - 1000
    x[n - 9] = -(top - 1000)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    part = buf.Slice(skip, n - skip)
    want = Enumerable(x[skip:])
    try:
        expect = want.Sum()
    except OverflowError:
        expect = "overflow"
    try:
        got = AsComputeQueryable(part, acc).Sum()
    except OverflowException:
        got = "overflow"
    assert got == expect
    buf.Dispose()


@pytest.mark.parametrize("dtype,bits", [(np.int32, 31), (np.int64, 63)])
def test_exchange_appends_ranges_in_rank_order(built_library, dtype, bits):
    """The exchange kernel's fold for a checked Sum, on one GPU: a world of two in which the other rank's record is written
    into this rank's exchange area by the host before the launch (nothing on the GPU waits for anything that is not there
    yet). Rank 0 holds [top-10, -3]; the fabricated rank 1 once stays inside when appended and once crosses the limit,
    although its own range and the global total are inside both times."""
    import ctypes as C
    from dotcompute_b200 import CudaAccelerator
    top = 2**bits - 1

    def record_of(values):
        pref = [0]
        for v in values:
            pref.append(pref[-1] + v)
        return pref[-1], min(pref), max(pref)

    def words(v):
        return [v & (2**64 - 1), (v >> 64) & (2**64 - 1)]

    for other, crosses in (([13, -top], False), ([14, -top - 1 + 10], True)):
        acc2 = CudaAccelerator(0)
        try:
            area, nbytes = C.c_void_p(), C.c_size_t()
            N.check(N.lib().dcb_peer_area_ptr(acc2.handle, C.byref(area), C.byref(nbytes)), acc2.handle)
            scratch = acc2.Memory.AllocateAsync(nbytes.value, np.uint8)
            scratch.FillAsync(0)
            areas = (C.c_void_p * 2)(area.value, scratch.GetDeviceMemory())
            N.check(N.lib().dcb_peer_connect_local(acc2.handle, 2, 0, areas), acc2.handle)
            s, lo, hi = record_of(other)
            assert -(2**bits) <= lo and hi <= top
            # PeerSlot = {fsum, isum_lo, isum_hi, count, mn_bits, mx_bits, flags, stamp}; a checked Sum carries the range in
            # mn_bits / fsum (smallest, low / high word) and mx_bits / count (largest); first exchange: stamp 1, ring row 1
            slot = np.array([words(lo)[1], words(s)[0], words(s)[1], words(hi)[1], words(lo)[0], words(hi)[0],
                             N.RES_PREFIX_RANGE | ((1 << 34) if bits == 31 else 0), 1], dtype=np.uint64)
            mine = acc2.Memory.WrapDevicePointer(area.value, nbytes.value // 8, np.uint64)
            mine.CopyFromAsync(slot, offset=(1 * 8 + 1) * 8)
            acc2.Synchronize()
            x = np.array([top - 10, -3], dtype=dtype)
            q = AsComputeQueryable(acc2.Memory.AllocateAndCopyAsync(x))
            if crosses:
                with pytest.raises(OverflowException):
                    q.Sum()
            else:
                assert q.Sum() == top - 13 + s
            N.check(N.lib().dcb_peer_disconnect(acc2.handle), acc2.handle)
            scratch.Dispose()
        finally:
            acc2.Dispose()
