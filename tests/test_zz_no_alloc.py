"""dcb_compact_noalloc: the compaction entry point for callers that are not allowed to allocate device memory (for
instance a host whose own buffer pool owns all of HBM). Collected last on purpose, so that a run stopping at the first
failure has already run everything else.

The new entry point is called through the C ABI twice in a row on different inputs and must give, bit for bit, what the
ordinary entry point (dcb_pipeline_run) gives for the same query; the second call sees the scratch left by the first.
"""
import ctypes as C

import numpy as np
import pytest

from dotcompute_b200 import native as N

pytestmark = pytest.mark.gpu


def _desc(ops, t0):
    arr = (N.Op * len(ops))()
    keep = []
    for i, (kind, lam) in enumerate(ops):
        arr[i].kind = kind
        if lam is not None:
            keep.append(lam.encode())
            arr[i].lambda_ = keep[-1]
    return N.PipelineDesc(t0, N.T_NONE, len(ops), arr, 0), (arr, keep)


def test_noalloc_matches_ordinary_entry_point_twice(acc):
    L = N.lib()
    ops = [(N.OP_WHERE, "x => x > 0.5f"), (N.OP_SELECT, "x => x * x + 3f"), (N.OP_TOARRAY, None)]
    desc, keep = _desc(ops, N.T_F32)
    pipe = C.c_void_p()
    N.check(L.dcb_pipeline_compile(acc.handle, C.byref(desc), C.byref(pipe)), acc.handle)
    rec = acc.Memory.AllocateAsync(16, np.int64)            # the caller's record; the test may allocate, the call may not
    import torch
    try:
        # The first call on a device is the set-up call: it looks up the device address of the fixed scratch, which makes
        # the driver load that part of the library image if it has not yet. From then on free device memory must not move.
        tiny = acc.Memory.AllocateAndCopyAsync(np.array([0.25, 0.75, 0.9, 0.1], dtype=np.float32))
        tiny_out = acc.Memory.AllocateAsync(4, np.float32)
        N.check(L.dcb_compact_noalloc(acc.DeviceId, C.byref(desc), C.c_void_p(tiny.GetDeviceMemory()), None, 4,
                                      C.c_void_p(tiny_out.GetDeviceMemory()), 4, C.c_void_p(rec.GetDeviceMemory()), None))
        torch.cuda.synchronize(acc.DeviceId)
        assert int(rec.ToArray()[N.SLOT_COUNT]) == 2
        assert tiny_out.CopyToAsync(count=2).tolist() == [np.float32(0.75) * np.float32(0.75) + np.float32(3), np.float32(0.9) * np.float32(0.9) + np.float32(3)]
        tiny.Dispose(); tiny_out.Dispose()
        for seed, n in ((1, 300_001), (2, 1_234_567)):
            x = np.random.Generator(np.random.PCG64(seed)).random(n, dtype=np.float32)
            d_in = acc.Memory.AllocateAndCopyAsync(x)
            d_ref = acc.Memory.AllocateAsync(n, np.float32)
            d_new = acc.Memory.AllocateAsync(n, np.float32)
            try:
                res = N.Result()
                N.check(L.dcb_pipeline_run(pipe, C.c_void_p(d_in.GetDeviceMemory()), None, n, C.c_void_p(d_ref.GetDeviceMemory()), n,
                                           C.byref(res), None), acc.handle)
                torch.cuda.synchronize(acc.DeviceId)
                before = acc.Memory.Statistics["AllocationCount"]
                free_before = torch.cuda.mem_get_info(acc.DeviceId)[0]
                N.check(L.dcb_compact_noalloc(acc.DeviceId, C.byref(desc), C.c_void_p(d_in.GetDeviceMemory()), None, n,
                                              C.c_void_p(d_new.GetDeviceMemory()), n, C.c_void_p(rec.GetDeviceMemory()), None))
                N.check(L.dcb_stream_sync(acc.handle, None), acc.handle)
                torch.cuda.synchronize(acc.DeviceId)        # the call ran on the default stream
                assert acc.Memory.Statistics["AllocationCount"] == before
                assert torch.cuda.mem_get_info(acc.DeviceId)[0] == free_before   # the driver handed out no memory either
                count = int(rec.ToArray()[N.SLOT_COUNT])
                assert count == res.count
                want = d_ref.CopyToAsync(count=count)
                got = d_new.CopyToAsync(count=count)
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32))     # bit exact, same order
            finally:
                d_in.Dispose(); d_ref.Dispose(); d_new.Dispose()
    finally:
        rec.Dispose()


def test_noalloc_rejects_what_it_cannot_hold(acc):
    L = N.lib()
    ops = [(N.OP_WHERE, "x => x > 0.5f"), (N.OP_SELECT, "x => x * x + 3f"), (N.OP_TOARRAY, None)]
    desc, keep = _desc(ops, N.T_F32)
    too_many = 8192 * 65536 + 1
    dummy = acc.Memory.AllocateAsync(64, np.float32)
    try:
        p = C.c_void_p(dummy.GetDeviceMemory())
        st = L.dcb_compact_noalloc(acc.DeviceId, C.byref(desc), p, None, too_many, p, too_many, p, None)
        assert st == 301 and "tiles" in N.last_error(None)
        # a query outside the precompiled table would need NVRTC, which allocates
        desc2, keep2 = _desc([(N.OP_WHERE, "x => x > 0.123f"), (N.OP_TOARRAY, None)], N.T_F32)
        st = L.dcb_compact_noalloc(acc.DeviceId, C.byref(desc2), p, None, 16, p, 16, p, None)
        assert st == 302
    finally:
        dummy.Dispose()
