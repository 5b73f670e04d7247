"""GPU tests of what surrounds the kernels: the look-back time-out path (driven from the host, no fault), one compiled
pipeline used from two threads at once, the bound on the compiled-pipeline cache, and the streamed compaction kernel on
inputs that do not start at a 16-byte boundary.
"""
import ctypes as C
import threading

import numpy as np
import pytest

from dotcompute_b200 import AsComputeQueryable, CudaAccelerator, CudaErrorClass, CudaException, native as N
from dotcompute_b200.accelerator import dcb_type
from dotcompute_b200.linq import CompiledPipeline

pytestmark = pytest.mark.gpu
F = np.float32


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


@pytest.mark.parametrize("kernel", [1, 0], ids=["one-tile-per-block", "streamed"])
def test_lookback_wait_runs_out_and_reports_timeout(built_library, kernel):
    """Failure detection without a GPU fault: the host tells the kernel to keep the survivor count of its first tile to
    itself (a flag that nothing sets), so every bounded look-back wait for it runs out; the launch ends by itself with
    the time-out flag in its record, the blocking call returns DCB_ERR_TIMEOUT (transient, retryable), and the same
    context then computes the right answer again."""
    acc = CudaAccelerator(0)
    try:
        x = rng(41).random(1 << 22, dtype=F)
        buf = acc.Memory.AllocateAndCopyAsync(x)
        want = x[x > 0.5] * x[x > 0.5] + F(3)
        acc.SetOption(N.OPT_COMPACT_KERNEL, kernel)
        q = lambda: AsComputeQueryable(buf, acc).Where("x => x > 0.5f").Select("x => x * x + 3f").ToArray()   # noqa: E731
        assert np.array_equal(q(), want)
        acc.SetSpinLimit(64)                                          # a few tens of microseconds of polling per wait
        acc.SetOption(N.OPT_WITHHOLD_FIRST_COUNT, 1)
        with pytest.raises(CudaException) as e:
            q()
        assert e.value.status == 102 and e.value.Classification == CudaErrorClass.Transient and e.value.IsRetryable
        acc.SetOption(N.OPT_WITHHOLD_FIRST_COUNT, 0)
        acc.SetSpinLimit(1 << 22)
        for _ in range(3):
            assert np.array_equal(q(), want)                          # retry succeeds: scratch and counters were left clean
        buf.Dispose()
    finally:
        acc.Dispose()


def test_one_pipeline_from_two_threads_on_two_streams(acc):
    """Two host threads run the same cached pipelines on one context, each on a stream of its own, 50 times: the
    blocking call (shared record, serialised inside the library) and the asynchronous call (own record, own scratch per
    stream, so the launches really overlap). Every result must equal the single-threaded one."""
    import torch
    x = rng(51).random(6_000_000, dtype=F)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    keep = x > 0.5
    want_arr = x[keep] * x[keep] + F(3)
    ops = ((N.OP_WHERE, "x => x > 0.5f"), (N.OP_SELECT, "x => x * x + 3f"))
    p_sum = CompiledPipeline(acc, dcb_type(F), 0, ops + ((N.OP_SUM, None),))
    p_arr = CompiledPipeline(acc, dcb_type(F), 0, ops + ((N.OP_TOARRAY, None),))
    r0 = N.Result()
    N.check(N.lib().dcb_pipeline_run(p_sum.handle, C.c_void_p(buf.GetDeviceMemory()), None, x.size, None, 0, C.byref(r0), None), acc.handle)
    want_sum = r0.f64
    errors = []

    def work(tid):
        try:
            stream = torch.cuda.Stream()
            sh = C.c_void_p(stream.cuda_stream)
            out = acc.Memory.AllocateAsync(x.size, F)
            rec_s = torch.zeros(16, dtype=torch.int64, device="cuda")
            rec_a = torch.zeros(16, dtype=torch.int64, device="cuda")
            torch.cuda.synchronize()
            for it in range(50):
                r = N.Result()
                N.check(N.lib().dcb_pipeline_run(p_sum.handle, C.c_void_p(buf.GetDeviceMemory()), None, x.size, None, 0, C.byref(r), sh), acc.handle)
                assert r.f64 == want_sum, (tid, it, r.f64, want_sum)
                N.check(N.lib().dcb_pipeline_run_async(p_sum.handle, C.c_void_p(buf.GetDeviceMemory()), None, x.size, None, 0,
                                                       C.c_void_p(rec_s.data_ptr()), None, sh), acc.handle)
                N.check(N.lib().dcb_pipeline_run_async(p_arr.handle, C.c_void_p(buf.GetDeviceMemory()), None, x.size,
                                                       C.c_void_p(out.GetDeviceMemory()), x.size, C.c_void_p(rec_a.data_ptr()), None, sh), acc.handle)
                stream.synchronize()
                hs, ha = rec_s.cpu().numpy(), rec_a.cpu().numpy()
                assert hs.view(np.float64)[N.SLOT_FSUM] == np.float64(rec_fsum[0]), (tid, it)
                assert int(ha[N.SLOT_COUNT]) == want_arr.size and int(ha[N.SLOT_FLAGS]) == 0, (tid, it, ha[:12])
                if it % 10 == 0:
                    assert np.array_equal(out.CopyToAsync(count=want_arr.size), want_arr), (tid, it)
            out.Dispose()
        except Exception as exc:                                      # an exception in a thread must fail the test
            errors.append(exc)

    # the fp64 partial the kernel leaves for this input (deterministic for a given launch shape)
    import torch as _t
    rec = _t.zeros(16, dtype=_t.int64, device="cuda")
    N.check(N.lib().dcb_pipeline_run_async(p_sum.handle, C.c_void_p(buf.GetDeviceMemory()), None, x.size, None, 0,
                                           C.c_void_p(rec.data_ptr()), None, None), acc.handle)
    acc.Synchronize()
    rec_fsum = rec.cpu().numpy().view(np.float64)[N.SLOT_FSUM: N.SLOT_FSUM + 1].copy()
    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    buf.Dispose()


def test_cache_is_bounded_and_evicted_queries_recompile(built_library):
    """With room for four compiled pipelines, eight distinct lambdas leave four in the cache, the memory of the evicted
    ones comes back, and an evicted query, asked for again, is rebuilt and still right."""
    import torch
    acc = CudaAccelerator(0)
    try:
        acc.SetOption(N.OPT_CACHE_MAX_ENTRIES, 4)
        x = rng(61).random(300_000, dtype=F)
        buf = acc.Memory.AllocateAndCopyAsync(x)

        def run(i):
            lam = f"x => x * {i + 2}f + 1f"
            got = AsComputeQueryable(buf, acc).Where("x => x > 0.25f").Select(lam).Sum()
            w = x[x > 0.25] * F(i + 2) + F(1)
            assert abs(float(got) - float(w.astype(np.float64).sum())) <= 1e-5 * float(np.abs(w).astype(np.float64).sum())

        for i in range(4):
            run(i)
        import gc
        gc.collect()                                                  # the Python pipeline objects give their references back
        assert acc.GetOption(N.OPT_CACHE_ENTRIES) == 4
        acc.Synchronize()
        free_with_four = torch.cuda.mem_get_info()[0]
        for i in range(4, 8):
            run(i)
            gc.collect()
        assert acc.GetOption(N.OPT_CACHE_ENTRIES) == 4                # four went out as four came in
        acc.Synchronize()
        free_after_eight = torch.cuda.mem_get_info()[0]
        assert free_after_eight >= free_with_four - (1 << 20), (free_with_four, free_after_eight)   # no growth per distinct lambda
        run(0)                                                        # evicted long ago: compiled again, same answer
        gc.collect()
        assert acc.GetOption(N.OPT_CACHE_ENTRIES) == 4
        buf.Dispose()
    finally:
        acc.Dispose()


@pytest.mark.parametrize("off", [1, 2, 3, 5])
def test_streamed_kernel_on_unaligned_slices(acc, off):
    """A slice that starts off a 16-byte boundary still runs the streamed kernel (its bulk copies start at the boundary
    below, the elements before the slice are masked out); the result equals the one-tile-per-block kernel's and numpy's.
    Lengths chosen so that the first and the last tile are both ragged, and so that there is only one tile."""
    x = rng(70 + off).random(3_000_000, dtype=F)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    k = rng(80 + off).integers(-2**62, 2**62, 1_000_000, dtype=np.int64)
    kbuf = acc.Memory.AllocateAndCopyAsync(k)
    try:
        for length in (x.size - off - 7, 4096 - off, 100, 1):
            view = buf.Slice(off, length)
            xs = x[off: off + length]
            want = xs[xs > 0.5] * xs[xs > 0.5] + F(3)
            got = {}
            for kernel in (0, 1):
                acc.SetOption(N.OPT_COMPACT_KERNEL, kernel)
                got[kernel] = AsComputeQueryable(view).Where("x => x > 0.5f").Select("x => x * x + 3f").ToArray()
            assert np.array_equal(got[0], want) and np.array_equal(got[1], want)
        acc.SetOption(N.OPT_COMPACT_KERNEL, 0)
        kv = kbuf.Slice(off % 2 + 1, k.size - 11)                      # 8-byte elements: one element past the boundary
        ks = k[off % 2 + 1: off % 2 + 1 + k.size - 11]
        assert np.array_equal(AsComputeQueryable(kv).Where("k => (k & 0xF) == 3").ToArray(), ks[(ks & 0xF) == 3])
        # Zip: both inputs displaced alike run the streamed kernel; displaced differently they fall back. Same answer.
        a, b = buf.Slice(off, 1_000_000), buf.Slice(off + 4, 1_000_000)
        c = buf.Slice(off + 1, 1_000_000)
        xa, xb, xc = x[off: off + 1_000_000], x[off + 4: off + 4 + 1_000_000], x[off + 1: off + 1 + 1_000_000]
        got = AsComputeQueryable(a).Zip(b, "(p, q) => p - q").Where("v => v > 0f").ToArray()
        w = xa - xb
        assert np.array_equal(got, w[w > 0])
        got = AsComputeQueryable(a).Zip(c, "(p, q) => p - q").Where("v => v > 0f").ToArray()
        w = xa - xc
        assert np.array_equal(got, w[w > 0])
    finally:
        acc.SetOption(N.OPT_COMPACT_KERNEL, 0)
        buf.Dispose()
        kbuf.Dispose()


def test_host_arrays_larger_than_the_staging_ring(built_library):
    """Host arrays of five staging chunks (the ring holds three input and two output chunks): map, compaction, reduction
    and Zip give the right answer, and the device memory the context took for all of it stays below 256 MiB (352 MiB with
    a second input) however large the arrays are."""
    import torch
    torch.cuda.init()
    acc = CudaAccelerator(0)
    try:
        n = 5 * (8 << 20) + 12_345
        x = rng(91).random(n, dtype=F)
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        got = AsComputeQueryable(x, acc).Select("x => x * 2f + 1f").ToArray()
        assert np.array_equal(got, x * F(2) + F(1))
        got = AsComputeQueryable(x, acc).Where("x => x > 0.5f").Select("x => x * x + 3f").ToArray()
        keep = x > 0.5
        assert np.array_equal(got, x[keep] * x[keep] + F(3))
        s = AsComputeQueryable(x, acc).Where("x => x > 0.5f").Select("x => x * x + 3f").Sum()
        w = (x[keep] * x[keep] + F(3)).astype(np.float64)
        assert abs(float(s) - float(w.sum())) <= 1e-5 * float(w.sum())
        assert AsComputeQueryable(x, acc).Count("x => x > 0.5f") == int(keep.sum())
        taken = AsComputeQueryable(x, acc).Where("x => x > 0.5f").Take(10_000_000).ToArray()      # capped output: stops copying, keeps counting
        assert np.array_equal(taken, x[keep][:10_000_000])
        acc.Synchronize()
        used_one_input = free0 - torch.cuda.mem_get_info()[0]
        assert used_one_input <= (256 << 20), used_one_input
        y = rng(92).random(n - 1000, dtype=F)
        got = AsComputeQueryable(x, acc).Zip(y, "(a, b) => a - b").Where("v => v > 0f").ToArray()
        d = x[: n - 1000] - y
        assert np.array_equal(got, d[d > 0])
        acc.Synchronize()
        assert free0 - torch.cuda.mem_get_info()[0] <= (352 << 20)
        k = rng(93).integers(-2**62, 2**62, n // 2, dtype=np.int64)
        assert np.array_equal(AsComputeQueryable(k, acc).Where("k => (k & 0xF) == 3").ToArray(), k[(k & 0xF) == 3])
        assert AsComputeQueryable(np.empty(0, F), acc).Where("x => x > 0.5f").ToArray().size == 0
    finally:
        acc.Dispose()


def test_overlapped_launches_give_the_same_results(built_library):
    """DCB_OPT_OVERLAP_LAUNCHES: back-to-back reductions on one stream, each allowed to start while the one before it is
    still finishing (scratch and record are touched only after the grid-dependency wait). 60 queries of three kinds over
    static inputs, every record equal to the one the same query leaves without the option."""
    import torch
    acc = CudaAccelerator(0)
    try:
        x = rng(95).random(9_000_001, dtype=F)
        buf = acc.Memory.AllocateAndCopyAsync(x)
        ops = ((N.OP_WHERE, "x => x > 0.5f"), (N.OP_SELECT, "x => x * x + 3f"))
        pipes = [CompiledPipeline(acc, dcb_type(F), 0, ops + ((t, None),)) for t in (N.OP_SUM, N.OP_MAX, N.OP_COUNT)]
        recs = torch.zeros((60, 16), dtype=torch.int64, device="cuda")

        def run_all():
            recs.zero_()
            torch.cuda.synchronize()
            for i in range(60):
                p = pipes[i % 3]
                N.check(N.lib().dcb_pipeline_run_async(p.handle, C.c_void_p(buf.GetDeviceMemory()), None, x.size - (i % 7), None, 0,
                                                       C.c_void_p(recs[i].data_ptr()), None, None), acc.handle)
            acc.Synchronize()
            return recs.cpu().numpy()[:, :10].copy()

        plain = run_all()
        acc.SetOption(N.OPT_OVERLAP_LAUNCHES, 1)
        assert acc.GetOption(N.OPT_OVERLAP_LAUNCHES) == 1
        for _ in range(3):
            assert np.array_equal(run_all(), plain)
        buf.Dispose()
    finally:
        acc.Dispose()
