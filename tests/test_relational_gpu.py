"""GPU parity of OrderBy, GroupBy-with-aggregate and Join against the sequential oracle (System.Linq / the reference's CPU
generator semantics, CpuKernelGenerator.cs:475-723), on sizes from one element to several radix tiles and blocks."""
import numpy as np
import pytest

from dotcompute_b200 import AsComputeQueryable
from oracle.linq_oracle import Enumerable

pytestmark = pytest.mark.gpu
F = np.float32


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


@pytest.mark.parametrize("n", [0, 1, 2, 33, 4095, 4096, 4097, 100_003, 3_000_001])
@pytest.mark.parametrize("dtype", [np.float32, np.int32, np.int64, np.float64, np.uint8, np.int16])
def test_orderby_natural_keys(acc, n, dtype):
    r = rng(n + 7)
    if np.dtype(dtype).kind == "f":
        x = (r.standard_normal(n) * 1000).astype(dtype)
        if n > 40:
            x[5] = np.nan; x[17] = -0.0; x[18] = 0.0; x[19] = np.inf; x[20] = -np.inf
    else:
        info = np.iinfo(dtype)
        x = r.integers(info.min, info.max, n, dtype=dtype, endpoint=True)
    got = AsComputeQueryable(x, acc).OrderBy().ToArray()
    want = Enumerable(x).OrderBy().ToArray()
    assert got.dtype == x.dtype and np.array_equal(got.view(np.uint8), want.view(np.uint8))
    gd = AsComputeQueryable(x, acc).OrderByDescending().ToArray()
    wd = Enumerable(x).OrderByDescending().ToArray()
    assert np.array_equal(gd.view(np.uint8), wd.view(np.uint8))


def test_orderby_key_selector_is_stable_and_composes(acc):
    """Few distinct keys, many ties: the elements of one key must come out in source order (Enumerable.OrderBy is stable);
    the sorted sequence feeds further fused operators; a device buffer works as the source."""
    n = 1_000_003
    x = rng(3).integers(0, 1_000_000, n, dtype=np.int32)
    got = AsComputeQueryable(x, acc).OrderBy("v => v % 7").ToArray()
    want = x[np.argsort(x % 7, kind="stable")]
    assert np.array_equal(got, want)
    got = AsComputeQueryable(x, acc).OrderByDescending("v => v % 7").ToArray()
    assert np.array_equal(got, x[np.argsort(-(x % 7), kind="stable")])
    buf = acc.Memory.AllocateAndCopyAsync(x)
    q = AsComputeQueryable(buf, acc).Where("v => v % 2 == 0").OrderBy("v => -v").Select("v => v + 1").Take(1000)
    ev = x[x % 2 == 0]
    assert np.array_equal(q.ToArray(), (ev[np.argsort(-ev, kind="stable")] + 1)[:1000])
    f = rng(4).random(300_000, dtype=F)
    assert np.array_equal(AsComputeQueryable(f, acc).OrderBy("v => MathF.Floor(v * 10f)").ToArray(), f[np.argsort(np.floor(f * F(10)), kind="stable")])
    buf.Dispose()


@pytest.mark.parametrize("n,groups", [(1, 1), (1000, 7), (4097, 4097), (500_000, 1000), (2_000_003, 13)])
@pytest.mark.parametrize("spread", [1, 100_003])
def test_groupby_aggregates(acc, n, groups, spread):
    """spread = 1: keys 0..groups-1 differ in their low bits only and index a table directly; spread = 100003 scatters them
    over the whole int range, which takes the sort-based path. Same groups, same order of first occurrence either way."""
    r = rng(n + groups)
    x = r.integers(0, 1_000_000, n, dtype=np.int32)
    key_py = lambda v: (v % groups) * np.int32(spread)               # noqa: E731
    key_cs = f"v => (v % {groups}) * {spread}"
    g = AsComputeQueryable(x, acc).GroupBy(key_cs)
    e = Enumerable(x)
    wk, wc = e.GroupAggregate(key_py, "Count")
    assert np.array_equal(g.Keys(), wk) and np.array_equal(g.Count(), np.asarray(wc, dtype=np.int32))
    for agg in ("Sum", "Min", "Max"):
        _k, w = e.GroupAggregate(key_py, agg)
        with np.errstate(over="ignore"):
            want = np.asarray(w, dtype=np.int64).astype(np.int32)     # integer sums wrap in the reference's generated code
        assert np.array_equal(getattr(g, agg)(), want), agg
    _k, w = e.GroupAggregate(key_py, "Average")
    assert np.allclose(g.Average(), np.asarray(w), rtol=1e-12)
    # floating values, a value selector, a floating key
    f = r.standard_normal(n).astype(F)
    gf = AsComputeQueryable(f, acc).GroupBy("v => MathF.Floor(v)")
    wk, ws = Enumerable(f).GroupAggregate(lambda v: np.floor(v), "Sum", lambda v: v * F(2))
    assert np.array_equal(gf.Keys(), wk)
    tol = 1e-5 * float(np.abs(f.astype(np.float64) * 2).sum()) + 1e-6
    assert np.all(np.abs(gf.Sum("v => v * 2f").astype(np.float64) - np.asarray(ws)) <= tol)
    _k, wm = Enumerable(f).GroupAggregate(lambda v: np.floor(v), "Max")
    assert np.array_equal(gf.Max(), np.asarray(wm, dtype=F))


@pytest.mark.parametrize("n_outer,n_inner,keys", [(1, 1, 1), (1000, 10, 10), (5000, 5000, 50_000), (300_000, 70_000, 100_000), (50_000, 1_000, 7)])
def test_join_inner_semi_anti(acc, n_outer, n_inner, keys):
    r = rng(n_outer + keys)
    outer = r.integers(0, keys * 10, n_outer, dtype=np.int64)
    inner = r.integers(0, keys * 10, n_inner, dtype=np.int64)
    ok_cs, ok_py = f"o => o % {keys}", (lambda v: v % keys)
    ik_cs, ik_py = f"i => (i * 3L) % {keys}", (lambda v: (v * 3) % keys)
    got = AsComputeQueryable(outer, acc).Join(inner, ok_cs, ik_cs, "(o, i) => o * 1000L + i").ToArray()
    want = Enumerable(outer).Join(inner, ok_py, ik_py, lambda o, i: o * 1000 + i).ToArray()
    assert got.dtype == np.int64 and np.array_equal(got, want)
    has = np.isin(ok_py(outer), ik_py(inner))
    assert np.array_equal(AsComputeQueryable(outer, acc).SemiJoin(inner, ok_cs, ik_cs).ToArray(), outer[has])
    assert np.array_equal(AsComputeQueryable(outer, acc).AntiJoin(inner, ok_cs, ik_cs).ToArray(), outer[~has])
    assert AsComputeQueryable(outer, acc).Join(inner[:0], ok_cs, ik_cs, "(o, i) => o + i").ToArray().size == 0


def test_sort_is_a_permutation_at_scale(acc):
    """2^26 float keys: sortedness and the multiset of values (checksum of checksums) instead of an element-wise oracle."""
    n = 1 << 26
    x = rng(11).random(n, dtype=F)
    got = AsComputeQueryable(x, acc).OrderBy().ToArray()
    assert got.size == n and bool(np.all(got[1:] >= got[:-1]))
    assert got.view(np.uint32).astype(np.uint64).sum() == x.view(np.uint32).astype(np.uint64).sum()
    assert np.bitwise_xor.reduce(got.view(np.uint32)) == np.bitwise_xor.reduce(x.view(np.uint32))
    assert got[0] == x.min() and got[-1] == x.max()


def test_sort_by_key_carries_values_of_another_type(acc):
    """dcb_sort_by_key through the C ABI: float values ordered by separate integer keys with many ties (stable), both
    directions; values wider than 4 bytes and an output that aliases the input are refused."""
    import ctypes as C
    from dotcompute_b200 import native as N
    r = rng(91)
    for n in (1, 4096, 4097, 777_777):
        keys = r.integers(-50, 50, n, dtype=np.int64)
        vals = r.standard_normal(n).astype(F)
        dk, dv = acc.Memory.AllocateAndCopyAsync(keys), acc.Memory.AllocateAndCopyAsync(vals)
        out = acc.Memory.AllocateAsync(n, F)
        for desc in (0, 1):
            N.check(N.lib().dcb_sort_by_key(acc.handle, N.T_I64, C.c_void_p(dk.GetDeviceMemory()), n, desc, 4,
                                            C.c_void_p(dv.GetDeviceMemory()), C.c_void_p(out.GetDeviceMemory()), None), acc.handle)
            acc.Synchronize()
            order = np.argsort(-keys if desc else keys, kind="stable")
            assert np.array_equal(out.CopyToAsync().view(np.uint32), vals[order].view(np.uint32))
        assert N.lib().dcb_sort_by_key(acc.handle, N.T_I64, C.c_void_p(dk.GetDeviceMemory()), n, 0, 8,
                                       C.c_void_p(dk.GetDeviceMemory()), C.c_void_p(out.GetDeviceMemory()), None) == 302   # DCB_ERR_NOT_SUPPORTED
        assert N.lib().dcb_sort_by_key(acc.handle, N.T_I64, C.c_void_p(dk.GetDeviceMemory()), n, 0, 4,
                                       C.c_void_p(dv.GetDeviceMemory()), C.c_void_p(dv.GetDeviceMemory()), None) == 301   # DCB_ERR_INVALID_ARGUMENT
        dk.Dispose(); dv.Dispose(); out.Dispose()


@pytest.mark.parametrize("n", [0, 1, 255, 4096, 4097, 1_000_003, (1 << 24) + 5])
@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
def test_scan_running_sum(acc, n, dtype):
    """Running sums over one element to thousands of tiles: integers bit-exact (they wrap in their own width), floats
    within 1e-5 * sum|x| of the sequential fp64 running sum (and normally equal to it after the rounding)."""
    r = rng(n * 3 + 1)
    if np.dtype(dtype).kind == "i":
        info = np.iinfo(dtype)
        x = r.integers(info.min // 2, info.max // 2, n, dtype=dtype)      # wraps many times over
    else:
        x = (r.standard_normal(n) * 10).astype(dtype)
    for inclusive in (True, False):
        got = AsComputeQueryable(x, acc).Scan(inclusive).ToArray()
        want = Enumerable(x).Scan(inclusive).ToArray()
        assert got.dtype == x.dtype and got.shape == want.shape
        if np.dtype(dtype).kind == "i":
            assert np.array_equal(got, want)
        elif n:
            tol = (1e-5 if dtype == np.float32 else 1e-12) * float(np.abs(x.astype(np.float64)).sum())
            assert float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)))) <= tol
    if n:   # composes with the fused operators on both sides
        got = AsComputeQueryable(x, acc).Where("v => v > 0").Select("v => v + v").Scan().Take(100).ToArray()
        pos = x[x > 0]
        want = Enumerable(pos + pos).Scan().ToArray()[:100]
        if np.dtype(dtype).kind == "i":
            assert np.array_equal(got, want)
        else:
            assert np.allclose(got, want, rtol=1e-5, atol=1e-3)


def test_sort_skips_passes_but_not_order(acc):
    """Keys that share whole digits (all equal; equal but for one byte in the middle; 64-bit keys that differ in the top
    byte only): the passes that would move nothing are skipped, the result is the same stable order."""
    n = 300_001
    r = rng(12)
    x = r.integers(0, 1_000_000, n, dtype=np.int32)
    assert np.array_equal(AsComputeQueryable(x, acc).OrderBy("v => 0").ToArray(), x)                       # no pass at all
    assert np.array_equal(AsComputeQueryable(x, acc).OrderByDescending("v => 5").ToArray(), x)
    mid = ((x & 0xFF) << 8) | 0x40000001                                                                  # only bits 8..15 differ
    assert np.array_equal(AsComputeQueryable(x, acc).OrderBy("v => ((v & 0xFF) << 8) | 0x40000001").ToArray(), x[np.argsort(mid, kind="stable")])
    k64 = (r.integers(0, 7, n, dtype=np.int64) << 56) + 12345
    got = AsComputeQueryable(k64, acc).OrderBy().ToArray()
    assert np.array_equal(got, np.sort(k64, kind="stable"))
    f = np.full(n, 2.5, dtype=F); f[::1000] = np.nan
    assert np.array_equal(AsComputeQueryable(f, acc).OrderBy().ToArray().view(np.uint32), Enumerable(f).OrderBy().ToArray().view(np.uint32))
