"""IComputeOrchestrator for `[Kernel]` methods: registry, argument marshalling, launch derivation, execution on the GPU.

Mirrors src/Core/DotCompute.Abstractions/Interfaces/IComputeOrchestrator.cs:12-105 as implemented by
KernelExecutionService (src/Runtime/DotCompute.Runtime/Services/KernelExecutionService.cs:196-443) and the registry the
`[Kernel]` source generator emits (src/Runtime/DotCompute.Generators/Kernel/Generation/KernelRegistrationEmitter.cs:56-192).
The generator runs inside the C# compiler in the reference; here `KernelRegistry.Register` takes the C# source text of
the method and the native library translates it to CUDA C (dcb_translate_kernel_method), NVRTC builds it for sm_100a
(dcb_kernel_compile) and dcb_kernel_launch runs it. There is no CPU invoker: a kernel either runs on the GPU or the
call raises.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass, field

import numpy as np

from . import errors, native as N
from .accelerator import CudaAccelerator, UnifiedBuffer

_CTYPES = {"sbyte": C.c_int8, "byte": C.c_uint8, "short": C.c_int16, "ushort": C.c_uint16, "int": C.c_int32, "uint": C.c_uint32,
           "long": C.c_int64, "ulong": C.c_uint64, "float": C.c_float, "double": C.c_double, "bool": C.c_bool}
_NP = {"sbyte": np.int8, "byte": np.uint8, "short": np.int16, "ushort": np.uint16, "int": np.int32, "uint": np.uint32,
       "long": np.int64, "ulong": np.uint64, "float": np.float32, "double": np.float64, "bool": np.bool_}


@dataclass
class KernelParam:
    Name: str
    IsBuffer: bool
    IsReadOnly: bool
    ElementType: str


@dataclass
class KernelRegistrationInfo:
    """One entry of the generated registry (KernelExecutionService_Simplified.cs:525-594)."""
    Name: str
    FullyQualifiedName: str
    CudaSource: str
    CudaEntryPoint: str
    CudaNeedsLength: bool
    Dimensions: int
    Parameters: list = field(default_factory=list)
    SupportedBackends: tuple = ("CUDA",)


def translate_kernel_method(csharp_method: str) -> KernelRegistrationInfo:
    """C# `[Kernel]` method text -> registry entry with its CUDA C source. Needs no GPU."""
    if csharp_method is None:
        raise errors.ArgumentNullException("csharp_method")
    need = C.c_size_t()
    meta = C.create_string_buffer(8192)
    err = C.create_string_buffer(512)
    src = csharp_method.encode()
    st = N.lib().dcb_translate_kernel_method(src, None, 0, C.byref(need), meta, len(meta), err, len(err))
    if st:
        raise errors.from_status(st, err.value.decode(), N.lib().dcb_status_name(st).decode())
    out = C.create_string_buffer(need.value)
    N.lib().dcb_translate_kernel_method(src, out, need.value, None, None, 0, err, len(err))
    m = json.loads(meta.value.decode())
    params = [KernelParam(p["name"], p["is_buffer"], p["is_readonly"], p["element_type"]) for p in m["params"]]
    return KernelRegistrationInfo(m["name"], m["name"], out.value.decode(), m["name"], m["needs_length"], m["dimensions"], params)


class KernelRegistry:
    """DotCompute.Generated.KernelRegistry: name -> registration."""

    def __init__(self):
        self._kernels: dict[str, KernelRegistrationInfo] = {}

    def Register(self, csharp_method: str, fully_qualified_name: str | None = None) -> KernelRegistrationInfo:
        reg = translate_kernel_method(csharp_method)
        if fully_qualified_name:
            reg.FullyQualifiedName = fully_qualified_name
            self._kernels[fully_qualified_name] = reg
        self._kernels[reg.Name] = reg
        return reg

    def RegisterCuda(self, name: str, cuda_source: str, parameters: list, needs_length: bool = False, dimensions: int = 1):
        """Register hand-written CUDA C (entry point = name, must be extern "C")."""
        reg = KernelRegistrationInfo(name, name, cuda_source, name, needs_length, dimensions, list(parameters))
        self._kernels[name] = reg
        return reg

    def TryResolve(self, name: str):
        return self._kernels.get(name)

    def GetAllKernels(self):
        return list({id(v): v for v in self._kernels.values()}.values())

    @property
    def Keys(self):
        return sorted(self._kernels)


class ComputeOrchestrator:
    """IComputeOrchestrator over one CudaAccelerator."""

    def __init__(self, accelerator: CudaAccelerator | None = None, registry: KernelRegistry | None = None):
        self._acc = accelerator
        self.Registry = registry or KernelRegistry()
        self._compiled: dict[str, C.c_void_p] = {}
        self._disposed = False

    # ---- accelerator selection (single backend: CUDA on this GPU)
    def GetOptimalAcceleratorAsync(self, kernelName: str | None = None) -> CudaAccelerator:
        if self._acc is None:
            self._acc = CudaAccelerator.Default()
        return self._acc

    def GetSupportedAcceleratorsAsync(self, kernelName: str):
        self._resolve(kernelName)
        return [self.GetOptimalAcceleratorAsync()]

    def GetDeviceInfo(self) -> dict:
        a = self.GetOptimalAcceleratorAsync()
        return {"Name": a.Name, "DeviceType": "CUDA", "MultiProcessorCount": a.MultiProcessorCount,
                "TotalMemory": a.TotalMemory, "ComputeCapability": a.ComputeCapability}

    # ---- registry helpers
    def _resolve(self, kernelName: str) -> KernelRegistrationInfo:
        if kernelName is None:
            raise errors.ArgumentNullException("kernelName")
        reg = self.Registry.TryResolve(kernelName)
        if reg is None:
            raise errors.ArgumentException(f"Kernel '{kernelName}' is not registered. Registered kernels: [{', '.join(self.Registry.Keys)}].")
        return reg

    def ValidateKernelArgsAsync(self, kernelName: str, *args) -> bool:
        reg = self.Registry.TryResolve(kernelName)
        if reg is None or args is None or len(args) != len(reg.Parameters):
            return False
        for p, a in zip(reg.Parameters, args):
            is_buf = isinstance(a, (np.ndarray, UnifiedBuffer))
            if p.IsBuffer != is_buf:
                return False
            if is_buf and np.dtype(a.dtype) != np.dtype(_NP[p.ElementType]):
                return False
        return True

    def PrecompileKernelAsync(self, kernelName: str, accelerator: CudaAccelerator | None = None) -> None:
        self._compile(self._resolve(kernelName), accelerator or self.GetOptimalAcceleratorAsync())

    def _compile(self, reg: KernelRegistrationInfo, acc: CudaAccelerator):
        key = f"{acc.DeviceId}:{reg.FullyQualifiedName}"
        if key not in self._compiled:
            h = C.c_void_p()
            N.check(N.lib().dcb_kernel_compile(acc.handle, reg.CudaSource.encode(), reg.CudaEntryPoint.encode(), C.byref(h)), acc.handle)
            self._compiled[key] = h
        return self._compiled[key]

    # ---- launch derivation (KernelExecutionService.cs:342-406)
    @staticmethod
    def DeriveWorkSize(reg: KernelRegistrationInfo, args) -> int:
        for p, a in zip(reg.Parameters, args):
            if p.IsBuffer and not p.IsReadOnly and isinstance(a, (np.ndarray, UnifiedBuffer)):
                return int(a.size if isinstance(a, np.ndarray) else a.Length)
        sizes = [int(a.size if isinstance(a, np.ndarray) else a.Length) for a in args if isinstance(a, (np.ndarray, UnifiedBuffer))]
        return max(sizes) if sizes else 0

    @staticmethod
    def DeriveLaunch(reg: KernelRegistrationInfo, args, totalWork: int):
        d = min(max(reg.Dimensions, 1), 3)
        ceil = lambda e, b: max(1, (int(e) + b - 1) // b)
        if d == 1:
            return (ceil(totalWork, 256), 1, 1), (256, 1, 1)
        extents = [int(a) for a in reversed(args) if isinstance(a, (int, np.integer)) and not isinstance(a, bool)][:d]
        x = extents[0] if len(extents) > 0 else max(1, totalWork)
        y = extents[1] if len(extents) > 1 else 1
        z = extents[2] if len(extents) > 2 else 1
        bx, by, bz = (16, 16, 1) if d == 2 else (8, 8, 4)
        return (ceil(x, bx), ceil(y, by), ceil(z, bz)), (bx, by, bz)

    # ---- execution
    def ExecuteAsync(self, kernelName: str, *args, accelerator: CudaAccelerator | None = None, preferredBackend: str | None = None):
        """Run a registered kernel. Host arrays are copied to the device, writable ones copied back; returns the first
        writable buffer argument (what ExecuteAsync<T> hands back for an array T).

        `preferredBackend` is the second overload of the reference (KernelExecutionService.cs:230-246): a wish, not a
        demand. This engine has CUDA devices only, so "CUDA" / "GPU" select them and any other name falls back to the
        optimal accelerator, as the reference does when no device of the wished type exists."""
        if self._disposed:
            raise errors.ObjectDisposedException("ComputeOrchestrator")
        if preferredBackend is not None and not isinstance(preferredBackend, str):
            raise errors.ArgumentException("preferredBackend must be a backend name")
        reg = self._resolve(kernelName)
        if not self.ValidateKernelArgsAsync(kernelName, *args):
            raise errors.ArgumentException(
                f"Kernel argument validation failed for kernel '{kernelName}' (received {len(args)} arguments). "
                "Verify argument count, types, and ordering match the kernel signature.")
        acc = accelerator or self.GetOptimalAcceleratorAsync()
        kernel = self._compile(reg, acc)
        total = self.DeriveWorkSize(reg, args)
        temporaries, copy_backs, holders, ptrs = [], [], [], []
        try:
            for p, a in zip(reg.Parameters, args):
                if p.IsBuffer:
                    if isinstance(a, UnifiedBuffer):
                        dev = a
                    else:
                        host = np.ascontiguousarray(a)
                        dev = acc.Memory.AllocateAndCopyAsync(host) if host.size else acc.Memory.AllocateAsync(1, host.dtype)
                        temporaries.append(dev)
                        if not p.IsReadOnly:
                            copy_backs.append((dev, a))
                    holders.append(C.c_void_p(dev.GetDeviceMemory()))
                else:
                    holders.append(_CTYPES[p.ElementType](a))
                ptrs.append(C.cast(C.byref(holders[-1]), C.c_void_p))
            if reg.CudaNeedsLength:
                holders.append(C.c_uint32(total))
                ptrs.append(C.cast(C.byref(holders[-1]), C.c_void_p))
            grid, block = self.DeriveLaunch(reg, args, total)
            if total > 0:
                argv = (C.c_void_p * len(ptrs))(*ptrs)
                g = (C.c_uint32 * 3)(*grid)
                b = (C.c_uint32 * 3)(*block)
                N.check(N.lib().dcb_kernel_launch(kernel, g, b, 0, argv, None), acc.handle)
                acc.Synchronize()
            for dev, host in copy_backs:
                if host.size:
                    dev.CopyToAsync(host.reshape(-1) if host.flags.c_contiguous else None)
        finally:
            for t in temporaries:
                t.Dispose()
        for p, a in zip(reg.Parameters, args):
            if p.IsBuffer and not p.IsReadOnly:
                return a
        return None

    def ExecuteWithBuffersAsync(self, kernelName: str, buffers, *scalarArgs):
        return self.ExecuteAsync(kernelName, *list(buffers), *scalarArgs)

    def ExecuteKernelAsync(self, kernelName: str, args, accelerator: CudaAccelerator | None = None):
        return self.ExecuteAsync(kernelName, *args, accelerator=accelerator)

    def Dispose(self) -> None:
        if not self._disposed:
            self._disposed = True
            for h in self._compiled.values():
                N.lib().dcb_kernel_destroy(h)
            self._compiled.clear()
