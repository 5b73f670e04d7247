"""The benchmark configurations at their full sizes (2^20 map, 2^24 reductions, 2^26 fused filter-map, 2^28 Zip dot product and
int64 filter), and the host path over several staging chunks. Every case is compared with the sequential CPU oracle directly
(it finishes these sizes in about a second each)."""
import numpy as np
import pytest

from dotcompute_b200 import AsComputeQueryable

pytestmark = pytest.mark.gpu
F = np.float32


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def test_config3_full_size(acc, c_oracle):
    x = rng(11).random(1 << 26, dtype=F)
    for thr, txt in ((0.5, "0.5f"), (0.99, "0.99f"), (0.01, "0.01f")):
        q = AsComputeQueryable(x, acc).Where(f"x => x > {txt}").Select("x => x * x + 3f")
        got = q.ToArray()                                    # host path: 8 staging chunks chained on the device
        want = c_oracle.where_gt_select_sq_add(x, thr, 3.0)
        assert got.size == want.size and np.array_equal(got.view(np.uint32), want.view(np.uint32))
        s = q.Sum()
        want_s, raw, cnt = c_oracle.where_gt_select_sq_add_sum(x, thr, 3.0)
        assert s == want_s and abs(float(s) - raw) <= 1e-5 * raw and q.Count() == cnt
    # the same from a device-resident buffer (one launch, no chunking)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    try:
        q = AsComputeQueryable(buf).Where("x => x > 0.5f").Select("x => x * x + 3f")
        assert np.array_equal(q.ToArray(), c_oracle.where_gt_select_sq_add(x, 0.5, 3.0))
        assert np.array_equal(q.Take(1000).ToArray(), c_oracle.where_gt_select_sq_add(x, 0.5, 3.0)[:1000])
    finally:
        buf.Dispose()


def test_config4_zip_dot_full_size(acc, c_oracle):
    n = 1 << 28
    a = rng(21).standard_normal(n, dtype=F)
    b = rng(22).standard_normal(n, dtype=F)
    got = AsComputeQueryable(a, acc).Zip(b, "(x, y) => x * y").Sum()
    want, raw, sum_abs = c_oracle.zip_mul_sum(a, b)
    assert abs(float(got) - raw) <= 1e-5 * sum_abs and got == want


def test_config4_int64_where_full_size(acc, c_oracle):
    n = 1 << 28
    k = rng(23).integers(-2**63, 2**63 - 1, n, dtype=np.int64, endpoint=True)
    got = AsComputeQueryable(k, acc).Where("k => (k & 0xF) == 3").ToArray()
    want = c_oracle.where_mask_eq_i64(k, 0xF, 3)
    assert got.size == want.size and np.array_equal(got, want)


def test_config1_and_2_full_size(acc, c_oracle):
    x = rng(42).random(1 << 20, dtype=F)
    assert np.array_equal(AsComputeQueryable(x, acc).Select("x => x * 2f + 1f").ToArray(), c_oracle.select_mul_add(x, 2.0, 1.0))
    y = rng(7).standard_normal(1 << 24, dtype=F)
    q = AsComputeQueryable(y, acc)
    assert q.Sum() == c_oracle.sum_f32(y)[0] and q.Min() == c_oracle.min_f32(y) and q.Max() == c_oracle.max_f32(y)
    assert q.Average() == c_oracle.average_f32(y)
    k = rng(8).integers(-1000, 1001, 1 << 24, dtype=np.int32)
    assert AsComputeQueryable(k, acc).Sum() == c_oracle.sum_i32(k) and AsComputeQueryable(k, acc).Min() == c_oracle.min_i32(k)


def test_host_path_over_several_chunks(acc, c_oracle):
    """Ragged size just over two 32 MiB staging chunks: compaction offsets chain from chunk to chunk on the device, plain
    maps come back chunk by chunk, reductions fold per-chunk records in order."""
    n = (2 << 23) + 12_345
    x = rng(5).random(n, dtype=F)
    q = AsComputeQueryable(x, acc)
    assert np.array_equal(q.Where("x => x > 0.3f").Select("x => x * x + 3f").ToArray(), c_oracle.where_gt_select_sq_add(x, 0.3, 3.0))
    assert np.array_equal(q.Select("x => x * 2f + 1f").ToArray(), c_oracle.select_mul_add(x, 2.0, 1.0))
    assert q.Where("x => x > 0.3f").Select("x => x * x + 3f").Sum() == c_oracle.where_gt_select_sq_add_sum(x, 0.3, 3.0)[0]
    assert q.Min() == x.min() and q.Max() == x.max() and q.Count("x => x > 0.3f") == int((x > F(0.3)).sum())
    assert q.Where("x => x > 0.3f").Take(77).ToArray().tolist() == x[x > F(0.3)][:77].tolist()
    assert q.Cast("double").Sum() == float(np.cumsum(x.astype(np.float64))[-1])
