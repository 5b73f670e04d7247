"""CudaAccelerator and its memory manager: the host-side mirror of the reference's backend objects.

`CudaAccelerator` stands where `new CudaAccelerator(deviceId: 0)` stands in
src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:184-194; `CudaMemoryManager` and `UnifiedBuffer`
keep the member names of src/Backends/DotCompute.Backends.CUDA/Memory/CudaMemoryManager.cs:140-292 and
src/Core/DotCompute.Abstractions/Interfaces/IUnifiedMemoryBuffer.cs:13-261. All work is done by libdcb200.so.
"""
from __future__ import annotations

import ctypes as C
import enum
import threading

import numpy as np

from . import errors, native as N

_DTYPE_TO_T = {
    np.dtype(np.int8): N.T_I8, np.dtype(np.uint8): N.T_U8, np.dtype(np.int16): N.T_I16, np.dtype(np.uint16): N.T_U16,
    np.dtype(np.int32): N.T_I32, np.dtype(np.uint32): N.T_U32, np.dtype(np.int64): N.T_I64, np.dtype(np.uint64): N.T_U64,
    np.dtype(np.float32): N.T_F32, np.dtype(np.float64): N.T_F64, np.dtype(np.bool_): N.T_BOOL,
}
_T_TO_DTYPE = {v: k for k, v in _DTYPE_TO_T.items()}


def dcb_type(dtype) -> int:
    dt = np.dtype(dtype)
    if dt not in _DTYPE_TO_T:
        raise errors.NotSupportedException(f"Type {dt} is not supported for CUDA kernel generation.")
    return _DTYPE_TO_T[dt]


def np_dtype(t: int) -> np.dtype:
    return _T_TO_DTYPE[t]


class BufferState(enum.Enum):
    """Residency states of IUnifiedMemoryBuffer.State."""
    Uninitialized = 0
    HostOnly = 1
    DeviceOnly = 2
    Synchronized = 3
    HostDirty = 4
    DeviceDirty = 5
    Disposed = 6


class MapMode(enum.Enum):
    """Access modes of IUnifiedMemoryBuffer<T>.Map (src/Core/DotCompute.Abstractions/Memory/MapMode.cs:9-30)."""
    Read = 0
    Write = 1
    ReadWrite = 2


class MappedMemory:
    """What Map / MapRange return: a host view (`Span`, a numpy array) of a range of the buffer. Disposing it (or
    leaving the `with` block) writes the view back to the device unless it was mapped for reading only."""

    def __init__(self, buffer: "UnifiedBuffer", offset: int, length: int, mode: MapMode):
        self._buffer, self._offset, self.Mode = buffer, offset, mode
        self.Span = np.empty(length, dtype=buffer.dtype) if mode is MapMode.Write else buffer.CopyToAsync(None, offset, length)
        self.Length = length
        self._open = True

    def Dispose(self) -> None:
        if self._open:
            self._open = False
            if self.Mode is not MapMode.Read:
                self._buffer.CopyFromAsync(self.Span, self._offset)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.Dispose()
        return False


class CudaAccelerator:
    """One GPU: context, stream, compiled-pipeline cache."""

    _default = None
    _lock = threading.Lock()

    def __init__(self, deviceId: int = 0):
        self._h = C.c_void_p()
        N.check(N.lib().dcb_init(int(deviceId), C.byref(self._h)))
        self.DeviceId = int(deviceId)
        self.Memory = CudaMemoryManager(self)
        self._disposed = False
        name = C.create_string_buffer(256)
        sm, mem, maj, mnr = C.c_int32(), C.c_int64(), C.c_int32(), C.c_int32()
        N.check(N.lib().dcb_device_info(self._h, name, 256, C.byref(sm), C.byref(mem), C.byref(maj), C.byref(mnr)), self._h)
        self.Name = name.value.decode()
        self.MultiProcessorCount = sm.value
        self.TotalMemory = mem.value
        self.ComputeCapability = (maj.value, mnr.value)

    @classmethod
    def Default(cls) -> "CudaAccelerator":
        """Process-wide accelerator on the device torchrun assigned (LOCAL_RANK), else device 0."""
        import os
        with cls._lock:
            if cls._default is None or cls._default._disposed:
                cls._default = cls(int(os.environ.get("LOCAL_RANK", "0")))
            return cls._default

    @property
    def handle(self):
        if self._disposed:
            raise errors.ObjectDisposedException("CudaAccelerator")
        return self._h

    def SetStream(self, cuda_stream: int | None) -> None:
        """Enqueue on an existing cudaStream_t (for instance torch's current stream); None restores the own stream."""
        N.check(N.lib().dcb_set_stream(self.handle, C.c_void_p(cuda_stream or 0)), self._h)

    def Synchronize(self) -> None:
        N.check(N.lib().dcb_stream_sync(self.handle, None), self._h)

    def SetOption(self, option: int, value: int) -> None:
        """A per-context switch of the native library (native.OPT_*): which compaction kernel runs, the compiled-pipeline
        cache bound, the host-driven time-out test switch."""
        N.check(N.lib().dcb_set_option(self.handle, int(option), int(value)), self._h)

    def GetOption(self, option: int) -> int:
        v = C.c_int64()
        N.check(N.lib().dcb_get_option(self.handle, int(option), C.byref(v)), self._h)
        return int(v.value)

    def SetSpinLimit(self, max_polls: int) -> None:
        N.check(N.lib().dcb_set_spin_limit(self.handle, int(max_polls)), self._h)

    @property
    def LaunchCount(self) -> int:
        v = C.c_int64()
        N.check(N.lib().dcb_launch_count(self.handle, C.byref(v)), self._h)
        return v.value

    def Dispose(self) -> None:
        if not self._disposed:
            self._disposed = True
            N.lib().dcb_shutdown(self._h)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.Dispose()


class PinnedArray:
    """Page-locked host memory viewed as a numpy array (CudaPinnedMemoryAllocator)."""

    def __init__(self, acc: CudaAccelerator, length: int, dtype):
        self._acc = acc
        self.dtype = np.dtype(dtype)
        self.Length = int(length)
        self._ptr = C.c_void_p()
        nbytes = max(self.Length * self.dtype.itemsize, 1)
        N.check(N.lib().dcb_host_alloc_pinned(acc.handle, nbytes, C.byref(self._ptr)), acc.handle)
        raw = (C.c_char * nbytes).from_address(self._ptr.value)
        self.array = np.frombuffer(raw, dtype=self.dtype, count=self.Length)

    @property
    def ptr(self) -> int:
        return self._ptr.value

    def Dispose(self) -> None:
        if self._ptr:
            self.array = None
            N.lib().dcb_host_free_pinned(self._acc.handle, self._ptr)
            self._ptr = C.c_void_p()


class UnifiedBuffer:
    """Device-resident typed buffer: the IUnifiedMemoryBuffer<T> of this engine."""

    def __init__(self, acc: CudaAccelerator, handle, length: int, dtype, parent=None):
        self._acc = acc
        self._h = handle
        self.Length = int(length)
        self.dtype = np.dtype(dtype)
        self._parent = parent       # keeps the owner of a slice alive
        self.State = BufferState.DeviceOnly
        self.IsDisposed = False
        self._host = None           # host copy behind AsSpan / AsMemory; the device copy is the home of the data

    # -- properties of the interface
    @property
    def SizeInBytes(self) -> int:
        return self.Length * self.dtype.itemsize

    @property
    def Accelerator(self) -> CudaAccelerator:
        return self._acc

    @property
    def IsOnDevice(self) -> bool:
        return not self.IsDisposed

    @property
    def IsOnHost(self) -> bool:
        return self._host is not None and self.State in (BufferState.Synchronized, BufferState.HostDirty)

    @property
    def IsDirty(self) -> bool:
        return self.State in (BufferState.HostDirty, BufferState.DeviceDirty)

    @property
    def ElementCount(self) -> int:
        return self.Length

    @property
    def handle(self):
        if self.IsDisposed:
            raise errors.ObjectDisposedException("UnifiedBuffer")
        return self._h

    def GetDeviceMemory(self) -> int:
        self.EnsureOnDevice()
        return N.lib().dcb_devptr(self.handle) or 0

    # -- host views. The device copy is the home; the host copy exists from the first AsSpan / EnsureOnHost on. Kernels
    #    write the device copy without telling this object, so the host copy is trusted only while it is the newer one
    #    (HostDirty): every other EnsureOnHost reads the device again.
    def EnsureOnHost(self) -> None:
        if self.State is not BufferState.HostDirty or self._host is None:
            self._host = self.CopyToAsync(self._host if self._host is not None else None)
            self.State = BufferState.Synchronized

    EnsureOnHostAsync = EnsureOnHost

    def AsReadOnlySpan(self) -> np.ndarray:
        self.EnsureOnHost()
        view = self._host.view()
        view.flags.writeable = False
        return view

    AsReadOnlyMemory = AsReadOnlySpan

    def AsSpan(self) -> np.ndarray:
        """Writable host view. What is written becomes visible to the device at the next EnsureOnDevice / Synchronize /
        GetDeviceMemory: the buffer counts as changed on the host from here on."""
        self.EnsureOnHost()
        self.State = BufferState.HostDirty
        return self._host

    AsMemory = AsSpan

    def MarkHostDirty(self) -> None:
        if self._host is None:
            raise errors.InvalidOperationException("the buffer has no host copy to mark")
        self.State = BufferState.HostDirty

    def MarkDeviceDirty(self) -> None:
        self.State = BufferState.DeviceDirty

    def Synchronize(self) -> None:
        if self.State is BufferState.HostDirty:
            self.EnsureOnDevice()
        elif self._host is not None:
            self.EnsureOnHost()

    SynchronizeAsync = Synchronize

    def Map(self, mode: MapMode = MapMode.ReadWrite) -> MappedMemory:
        return self.MapRange(0, self.Length, mode)

    MapAsync = Map

    def MapRange(self, offset: int, length: int, mode: MapMode = MapMode.ReadWrite) -> MappedMemory:
        if offset < 0 or length < 0 or offset + length > self.Length:
            raise errors.ArgumentException("range outside the buffer")
        self.EnsureOnDevice()
        return MappedMemory(self, offset, length, mode)

    # -- transfers
    def CopyFromAsync(self, source: np.ndarray, offset: int = 0) -> None:
        if source is None:
            raise errors.ArgumentNullException("source")
        if self.State is BufferState.HostDirty and self._host is not None and source is not self._host:
            self.EnsureOnDevice()     # changes made through AsSpan reach the device before this copy lands on top
        src = np.ascontiguousarray(source, dtype=self.dtype)
        if offset < 0 or offset + src.size > self.Length:
            raise errors.ArgumentException("source does not fit the buffer at this offset")
        N.check(N.lib().dcb_h2d_async(self._acc.handle, self.handle, offset * self.dtype.itemsize,
                                      src.ctypes.data_as(C.c_void_p), src.nbytes, None), self._acc.handle)
        self._acc.Synchronize()   # `src` may be a temporary
        self.State = BufferState.Synchronized

    def CopyToAsync(self, destination: np.ndarray | None = None, offset: int = 0, count: int | None = None) -> np.ndarray:
        if isinstance(destination, UnifiedBuffer):
            return self.CopyToBufferAsync(destination, offset, 0, count)
        if self.State is BufferState.HostDirty and self._host is not None:
            self.EnsureOnDevice()
        n = self.Length - offset if count is None else int(count)
        if offset < 0 or n < 0 or offset + n > self.Length:
            raise errors.ArgumentException("range outside the buffer")
        if destination is None:
            destination = np.empty(n, dtype=self.dtype)
        if destination.dtype != self.dtype or destination.size < n or not destination.flags.c_contiguous:
            raise errors.ArgumentException("destination must be a contiguous array of the buffer's element type")
        N.check(N.lib().dcb_d2h_async(self._acc.handle, destination.ctypes.data_as(C.c_void_p), self.handle,
                                      offset * self.dtype.itemsize, n * self.dtype.itemsize, None), self._acc.handle)
        self._acc.Synchronize()
        return destination

    def ToArray(self) -> np.ndarray:
        return self.CopyToAsync()

    def FillAsync(self, value, offset: int = 0, count: int | None = None) -> None:
        n = self.Length - offset if count is None else int(count)
        pat = np.array([value], dtype=self.dtype)
        N.check(N.lib().dcb_fill_async(self._acc.handle, self.handle, offset * self.dtype.itemsize,
                                       pat.ctypes.data_as(C.c_void_p), self.dtype.itemsize, n, None), self._acc.handle)
        self._acc.Synchronize()

    # -- views (zero copy)
    def Slice(self, offset: int, length: int) -> "UnifiedBuffer":
        if offset < 0 or length < 0 or offset + length > self.Length:
            raise errors.ArgumentException("slice outside the buffer")
        h = C.c_void_p()
        N.check(N.lib().dcb_buf_slice(self._acc.handle, self.handle, offset * self.dtype.itemsize,
                                      length * self.dtype.itemsize, C.byref(h)), self._acc.handle)
        return UnifiedBuffer(self._acc, h, length, self.dtype, parent=self)

    def AsType(self, dtype) -> "UnifiedBuffer":
        dt = np.dtype(dtype)
        if self.SizeInBytes % dt.itemsize:
            raise errors.ArgumentException("buffer size is not a multiple of the new element size")
        h = C.c_void_p()
        N.check(N.lib().dcb_buf_slice(self._acc.handle, self.handle, 0, self.SizeInBytes, C.byref(h)), self._acc.handle)
        return UnifiedBuffer(self._acc, h, self.SizeInBytes // dt.itemsize, dt, parent=self)

    def EnsureOnDevice(self) -> None:
        _ = self.handle
        if self.State is BufferState.HostDirty and self._host is not None:
            host = self._host
            self.CopyFromAsync(host)          # sets Synchronized

    EnsureOnDeviceAsync = EnsureOnDevice

    def CopyToBufferAsync(self, destination: "UnifiedBuffer", sourceOffset: int = 0, destinationOffset: int = 0,
                          count: int | None = None) -> None:
        """CopyToAsync(IUnifiedMemoryBuffer<T> destination[, sourceOffset, destinationOffset, count]): device to device."""
        if destination is None:
            raise errors.ArgumentNullException("destination")
        n = self.Length - sourceOffset if count is None else int(count)
        if destination.dtype != self.dtype:
            raise errors.ArgumentException("destination has another element type")
        if sourceOffset < 0 or destinationOffset < 0 or n < 0 or sourceOffset + n > self.Length or destinationOffset + n > destination.Length:
            raise errors.ArgumentException("range outside a buffer")
        self.EnsureOnDevice()
        isz = self.dtype.itemsize
        N.check(N.lib().dcb_d2d_async(self._acc.handle, destination.handle, destinationOffset * isz, self.handle,
                                      sourceOffset * isz, n * isz, None), self._acc.handle)
        self._acc.Synchronize()
        destination.State = BufferState.DeviceDirty if destination._host is not None else BufferState.DeviceOnly

    def Dispose(self) -> None:
        if not self.IsDisposed:
            self.IsDisposed = True
            self.State = BufferState.Disposed
            if not self._acc._disposed:
                N.lib().dcb_free(self._acc._h, self._h)

    def __del__(self):
        # IDisposable with a finalizer: a buffer nobody disposed is given back when it is collected (views keep their owner
        # alive through _parent, so an owner is never collected before its slices).
        try:
            self.Dispose()
        except Exception:
            pass

    def __len__(self):
        return self.Length


class CudaMemoryManager:
    """AllocateAsync / AllocateAndCopyAsync / FreeAsync over the device's stream-ordered pool."""

    def __init__(self, acc: CudaAccelerator):
        self._acc = acc

    def AllocateAsync(self, length: int, dtype) -> UnifiedBuffer:
        if length < 0:
            raise errors.ArgumentException("length must not be negative")
        dt = np.dtype(dtype)
        dcb_type(dt)
        h = C.c_void_p()
        N.check(N.lib().dcb_alloc(self._acc.handle, int(length) * dt.itemsize, C.byref(h)), self._acc.handle)
        return UnifiedBuffer(self._acc, h, length, dt)

    def AllocateAndCopyAsync(self, source: np.ndarray) -> UnifiedBuffer:
        if source is None:
            raise errors.ArgumentNullException("source")
        src = np.ascontiguousarray(source)
        buf = self.AllocateAsync(src.size, src.dtype)
        if src.size:
            buf.CopyFromAsync(src)
        return buf

    def WrapDevicePointer(self, device_ptr: int, length: int, dtype) -> UnifiedBuffer:
        """Adopt memory owned by someone else (for instance a torch tensor's data_ptr()) without copying."""
        dt = np.dtype(dtype)
        h = C.c_void_p()
        N.check(N.lib().dcb_buf_wrap(self._acc.handle, C.c_void_p(device_ptr), int(length) * dt.itemsize, C.byref(h)), self._acc.handle)
        return UnifiedBuffer(self._acc, h, length, dt)

    def AllocatePinned(self, length: int, dtype) -> PinnedArray:
        return PinnedArray(self._acc, length, dtype)

    def FreeAsync(self, buffer: UnifiedBuffer) -> None:
        buffer.Dispose()

    @property
    def Statistics(self) -> dict:
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        N.check(N.lib().dcb_memory_stats(self._acc.handle, C.byref(a), C.byref(b), C.byref(c)), self._acc.handle)
        return {"CurrentAllocatedMemory": a.value, "PeakMemoryUsage": b.value, "AllocationCount": c.value}
