"""GPU parity of the pipelined (persistent, bulk-copy fed) compaction kernel: the same queries with the kernel switched
on and off must return the same arrays, and both must equal the oracle, bit for bit. The switch is the environment
variable the library reads at every launch.
"""
import numpy as np
import pytest

from dotcompute_b200 import AsComputeQueryable, native as N
from oracle.linq_oracle import Enumerable

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


@pytest.fixture
def pipe(acc):
    def switch(on: bool):
        acc.SetOption(N.OPT_COMPACT_KERNEL, 0 if on else 1)      # 0 = the streamed kernel, 1 = one tile per block
    yield switch
    acc.SetOption(N.OPT_COMPACT_KERNEL, 0)


def both(pipe, make_query):
    pipe(False)
    a = make_query().ToArray()
    pipe(True)
    b = make_query().ToArray()
    assert a.dtype == b.dtype and np.array_equal(a, b)
    return b


@pytest.mark.parametrize("n", [0, 1, 31, 4095, 4096, 4097, 8191, 65_537, 1_000_003, (1 << 23) + 17])
def test_f32_where_select_sizes(acc, pipe, n):
    x = rng(n + 1).random(n, dtype=np.float32)
    got = both(pipe, lambda: AsComputeQueryable(x, acc).Where("x => x > 0.5f").Select("x => x * x + 3f"))
    want = np.asarray(Enumerable(x).Where(lambda v: v > np.float32(0.5)).Select(lambda v: np.float32(np.float32(v * v) + np.float32(3))).ToArray(),
                      dtype=np.float32) if n <= 70_000 else (x[x > 0.5] * x[x > 0.5] + np.float32(3)).astype(np.float32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("keep", [0.0, 0.01, 0.99, 1.0])
def test_selectivities(acc, pipe, keep):
    x = rng(3).random(3_000_000, dtype=np.float32)
    thr = np.float32(1.0 - keep)
    got = both(pipe, lambda: AsComputeQueryable(x, acc).Where(f"x => x >= {float(thr)!r}f"))
    assert np.array_equal(got, x[x >= thr])


@pytest.mark.parametrize("dtype", [np.int64, np.int32, np.uint8, np.int16, np.float64])
def test_element_types(acc, pipe, dtype):
    r = rng(9)
    n = 2_500_001
    x = (r.standard_normal(n) * 100).astype(dtype) if np.dtype(dtype).kind == "f" else r.integers(0, 120, n).astype(dtype)
    lam = "x => x > 50.0" if dtype == np.float64 else "x => x > 50"
    got = both(pipe, lambda: AsComputeQueryable(x, acc).Where(lam))
    assert np.array_equal(got, x[x > 50])


def test_zip_then_where(acc, pipe):
    r = rng(10)
    a = r.standard_normal(1_234_567, dtype=np.float32)
    b = r.standard_normal(1_234_567, dtype=np.float32)
    got = both(pipe, lambda: AsComputeQueryable(a, acc).Zip(b, "(p, q) => p * q").Where("v => v > 0f"))
    w = a * b
    assert np.array_equal(got, w[w > 0])


def test_device_buffers_many_launches_and_take(acc, pipe):
    """Device-resident input, the same pipeline launched repeatedly (the tile and finished-block counters must be back
    at zero after every launch), and a capped output (Take) that ends up truncated."""
    x = rng(12).random(5_000_000, dtype=np.float32)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    want = x[x > 0.25]
    pipe(True)
    for _ in range(5):
        got = AsComputeQueryable(buf, acc).Where("x => x > 0.25f").ToArray()
        assert np.array_equal(got, want)
    assert np.array_equal(AsComputeQueryable(buf, acc).Where("x => x > 0.25f").Take(1000).ToArray(), want[:1000])
    assert AsComputeQueryable(buf, acc).Count("x => x > 0.25f") == want.size


def test_host_chunks_chain_offsets(acc, pipe):
    """A host array larger than one staging chunk: every chunk's launch starts at the previous chunk's survivor count."""
    x = rng(13).integers(-2**62, 2**62, 9_000_000, dtype=np.int64)     # 72 MB: three chunks
    got = both(pipe, lambda: AsComputeQueryable(x, acc).Where("k => (k & 0xF) == 3"))
    assert np.array_equal(got, x[(x & 0xF) == 3])


def test_three_compactions_at_once_on_one_gpu(built_library):
    """Three contexts (three streams) compact at the same time from three host threads. Each launch asks for as many
    persistent blocks as fit the GPU alone, so together they cannot all be resident: the kernels must make progress
    without that assumption (a tile waits only for tiles of blocks that are already running), with no wait running out."""
    import threading

    from dotcompute_b200 import CudaAccelerator
    accs = [CudaAccelerator(0) for _ in range(3)]
    r = rng(17)
    xs = [r.random(24_000_000, dtype=np.float32) for _ in accs]
    bufs = [a.Memory.AllocateAndCopyAsync(x) for a, x in zip(accs, xs)]
    wants = [x[x > 0.5] * x[x > 0.5] + np.float32(3) for x in xs]
    ok = [True] * len(accs)
    errors = []

    def work(i):
        try:
            for _ in range(6):
                got = AsComputeQueryable(bufs[i], accs[i]).Where("x => x > 0.5f").Select("x => x * x + 3f").ToArray()
                ok[i] &= bool(np.array_equal(got, wants[i]))
        except Exception as e:   # surfaced below: an exception in a thread must fail the test
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(accs))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert ok == [True, True, True]
