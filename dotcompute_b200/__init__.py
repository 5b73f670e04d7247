"""dotcompute_b200 — B200-native engine for DotCompute's data-parallel LINQ hot path.

Host-side mirror of the reference's surface (AsComputeQueryable, ComputeSelect/ComputeWhere, ToComputeArray,
IUnifiedMemoryBuffer, IComputeOrchestrator) over the C ABI of libdcb200.so. Every query runs as hand-written
sm_100a CUDA; there is no CPU or PyTorch path behind these names.
"""
from .errors import (ArgumentException, ArgumentNullException, CudaErrorClass, CudaException, DivideByZeroException,
                     DotComputeException, InvalidOperationException, NotSupportedException, ObjectDisposedException, OverflowException)
from .accelerator import (BufferState, CudaAccelerator, CudaMemoryManager, MapMode, MappedMemory, PinnedArray,
                          UnifiedBuffer)
from .orchestrator import ComputeOrchestrator, KernelParam, KernelRegistrationInfo, KernelRegistry, translate_kernel_method
from .linq import (AsComputeQueryable, CompiledPipeline, ComputeLinqProvider, ComputeQueryable, Grouping, ToComputeArray,
                   generate_source, translate_lambda)

__all__ = [
    "ArgumentException", "ArgumentNullException", "CudaErrorClass", "CudaException", "DivideByZeroException", "DotComputeException",
    "InvalidOperationException", "NotSupportedException", "ObjectDisposedException", "OverflowException",
    "BufferState", "CudaAccelerator", "CudaMemoryManager", "MapMode", "MappedMemory", "PinnedArray", "UnifiedBuffer",
    "AsComputeQueryable", "CompiledPipeline", "ComputeLinqProvider", "ComputeQueryable", "Grouping", "ToComputeArray",
    "generate_source", "translate_lambda",
    "ComputeOrchestrator", "KernelParam", "KernelRegistrationInfo", "KernelRegistry", "translate_kernel_method",
]
