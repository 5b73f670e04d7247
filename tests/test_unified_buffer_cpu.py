"""IUnifiedMemoryBuffer<T> members of UnifiedBuffer (host views, dirty tracking, Map, Slice, AsType, buffer-to-buffer copy)
against a stand-in for the native layer: "device memory" is plain host memory and the four copy entry points are
memmoves, so the bookkeeping above the C ABI is checked without a GPU. The real copies are covered by the GPU tests.
"""
import ctypes as C

import numpy as np
import pytest

from dotcompute_b200 import ArgumentException, BufferState, MapMode, UnifiedBuffer, accelerator, native as N


class FakeLib:
    """dcb_h2d/d2h/d2d/fill/buf_slice/devptr/free over host memory; a buffer handle is the address of its bytes."""

    def __init__(self):
        self.blocks = []
        self.h2d = self.d2h = 0

    def alloc(self, nbytes):
        blk = C.create_string_buffer(max(nbytes, 1))
        self.blocks.append(blk)
        return C.c_void_p(C.addressof(blk))

    @staticmethod
    def _addr(h):
        return h.value if isinstance(h, C.c_void_p) else int(h)

    def dcb_h2d_async(self, ctx, dst, off, host, nbytes, stream):
        self.h2d += 1
        C.memmove(self._addr(dst) + off, self._addr(host), nbytes)
        return 0

    def dcb_d2h_async(self, ctx, host, src, off, nbytes, stream):
        self.d2h += 1
        C.memmove(self._addr(host), self._addr(src) + off, nbytes)
        return 0

    def dcb_d2d_async(self, ctx, dst, doff, src, soff, nbytes, stream):
        C.memmove(self._addr(dst) + doff, self._addr(src) + soff, nbytes)
        return 0

    def dcb_fill_async(self, ctx, dst, off, pattern, pbytes, count, stream):
        for i in range(count):
            C.memmove(self._addr(dst) + off + i * pbytes, self._addr(pattern), pbytes)
        return 0

    def dcb_buf_slice(self, ctx, parent, off, nbytes, out):
        out._obj.value = self._addr(parent) + off
        return 0

    def dcb_devptr(self, h):
        return self._addr(h)

    def dcb_free(self, ctx, h):
        return 0


class FakeAcc:
    handle = C.c_void_p(1)
    _h = C.c_void_p(1)
    _disposed = False

    def Synchronize(self):
        pass


@pytest.fixture
def fake(monkeypatch):
    lib = FakeLib()
    monkeypatch.setattr(N, "lib", lambda: lib)
    monkeypatch.setattr(N, "check", lambda status, ctx=None: None if status == 0 else (_ for _ in ()).throw(RuntimeError(status)))
    return lib


def make(fake, data):
    data = np.ascontiguousarray(data)
    buf = UnifiedBuffer(FakeAcc(), fake.alloc(data.nbytes), data.size, data.dtype)
    buf.CopyFromAsync(data)
    return buf


def test_host_views_and_dirty_tracking(fake):
    buf = make(fake, np.arange(8, dtype=np.float32))
    assert buf.Length == buf.ElementCount == 8 and buf.SizeInBytes == 32 and buf.IsOnDevice and not buf.IsOnHost
    ro = buf.AsReadOnlySpan()
    assert ro.tolist() == list(range(8)) and not ro.flags.writeable and buf.IsOnHost and not buf.IsDirty
    span = buf.AsSpan()                      # writable: the host copy is the newer one from here on
    span[0] = 100
    assert buf.State is BufferState.HostDirty and buf.IsDirty
    uploads = fake.h2d
    ptr = buf.GetDeviceMemory()              # a kernel is about to read it: the change goes up first
    assert fake.h2d == uploads + 1 and buf.State is BufferState.Synchronized
    assert np.frombuffer((C.c_char * 32).from_address(ptr), dtype=np.float32)[0] == 100
    # a kernel writes the device copy behind the object's back: the next host view reads the device again
    np.frombuffer((C.c_char * 32).from_address(ptr), dtype=np.float32)[1] = -5
    assert buf.AsReadOnlySpan()[1] == -5
    buf.MarkDeviceDirty()
    assert buf.IsDirty
    buf.Synchronize()
    assert buf.State is BufferState.Synchronized


def test_pending_host_changes_survive_a_partial_copy(fake):
    buf = make(fake, np.zeros(6, dtype=np.int32))
    buf.AsSpan()[5] = 9                      # not uploaded yet
    buf.CopyFromAsync(np.array([1, 2], dtype=np.int32), offset=1)
    assert buf.ToArray().tolist() == [0, 1, 2, 0, 0, 9]


def test_map_modes(fake):
    buf = make(fake, np.arange(10, dtype=np.int64))
    with buf.Map(MapMode.Read) as m:
        assert m.Span.tolist() == list(range(10))
        m.Span[0] = 77                       # a read mapping is not written back
    assert buf.ToArray()[0] == 0
    with buf.MapRange(2, 3, MapMode.ReadWrite) as m:
        assert m.Span.tolist() == [2, 3, 4] and m.Length == 3
        m.Span[:] = [20, 30, 40]
    assert buf.ToArray().tolist() == [0, 1, 20, 30, 40, 5, 6, 7, 8, 9]
    m = buf.Map(MapMode.Write)
    m.Span[:] = 1
    m.Dispose()
    m.Dispose()                              # idempotent
    assert buf.ToArray().tolist() == [1] * 10
    with pytest.raises(ArgumentException):
        buf.MapRange(8, 5)


def test_slice_astype_fill_and_buffer_to_buffer_copy(fake):
    buf = make(fake, np.arange(16, dtype=np.int32))
    sl = buf.Slice(4, 8)
    assert sl.ToArray().tolist() == list(range(4, 12))
    sl.FillAsync(7, 0, 2)
    assert buf.ToArray()[4:6].tolist() == [7, 7]
    as_bytes = buf.AsType(np.uint8)
    assert as_bytes.Length == 64 and as_bytes.ToArray()[0] == 0
    with pytest.raises(ArgumentException):
        buf.Slice(0, 3).AsType(np.int64)     # 12 bytes are not a whole number of 8-byte elements
    dst = make(fake, np.zeros(16, dtype=np.int32))
    buf.CopyToAsync(dst)                     # IUnifiedMemoryBuffer<T> overload
    assert dst.ToArray().tolist() == buf.ToArray().tolist()
    buf.CopyToBufferAsync(dst, sourceOffset=0, destinationOffset=8, count=4)
    assert dst.ToArray()[8:12].tolist() == buf.ToArray()[0:4].tolist()
    with pytest.raises(ArgumentException):
        buf.CopyToBufferAsync(dst, 10, 10, 10)
    with pytest.raises(ArgumentException):
        buf.CopyToBufferAsync(make(fake, np.zeros(16, dtype=np.float32)))
