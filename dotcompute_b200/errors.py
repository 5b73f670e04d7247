"""Exceptions the managed side of DotCompute throws, by the same names.

The C ABI returns status codes; this module maps them onto the exception types the reference's callers catch:
ArgumentNullException / ArgumentException for bad arguments
(src/Runtime/DotCompute.Runtime/Services/KernelExecutionService.cs:203-264), NotSupportedException for
untranslatable queries (src/Extensions/DotCompute.Linq/Compilation/ExpressionTreeVisitor.cs:90-95),
InvalidOperationException / OverflowException from System.Linq's Min/Max/Average/Sum, ObjectDisposedException,
and CudaException with its classification properties
(src/Backends/DotCompute.Backends.CUDA/Types/Native/CudaRuntime.cs:1057-1066,
src/Backends/DotCompute.Backends.CUDA/ErrorHandling/CudaErrorClassification.cs:17-46).
"""
from __future__ import annotations

import enum


class CudaErrorClass(enum.IntEnum):
    NONE = 0
    Transient = 1
    Resource = 2
    Programmer = 3
    Fatal = 4
    Query = 5


class DotComputeException(Exception):
    status = 0
    status_name = ""


class ArgumentException(DotComputeException, ValueError):
    pass


class ArgumentNullException(ArgumentException):
    def __init__(self, param_name: str, message: str | None = None):
        super().__init__(message or f"Value cannot be null. (Parameter '{param_name}')")
        self.ParamName = param_name


class NotSupportedException(DotComputeException):
    pass


class InvalidOperationException(DotComputeException):
    pass


class OverflowException(DotComputeException, ArithmeticError):
    pass


class DivideByZeroException(DotComputeException, ZeroDivisionError):
    """An integer / or % inside a lambda met a zero divisor (System.DivideByZeroException)."""


class ObjectDisposedException(InvalidOperationException):
    pass


class CudaException(DotComputeException):
    def __init__(self, message: str, status: int):
        super().__init__(message)
        self.status = status
        self.Classification = CudaErrorClass(min(status // 100, 5)) if status else CudaErrorClass.NONE

    @property
    def IsRetryable(self) -> bool:
        return self.Classification == CudaErrorClass.Transient

    @property
    def IsResourceError(self) -> bool:
        return self.Classification == CudaErrorClass.Resource

    @property
    def IsFatal(self) -> bool:
        return self.Classification == CudaErrorClass.Fatal

    @property
    def IsRecoverable(self) -> bool:
        return self.Classification in (CudaErrorClass.Transient, CudaErrorClass.Resource)


_BY_STATUS = {
    301: ArgumentException,
    302: NotSupportedException,
    304: ObjectDisposedException,
    501: InvalidOperationException,
    502: OverflowException,
    503: DivideByZeroException,
}


def from_status(status: int, message: str, name: str = "") -> DotComputeException:
    cls = _BY_STATUS.get(status)
    text = f"{message} [{name or status}]"
    if cls is None:
        exc = CudaException(text, status)
    else:
        exc = cls(text)
    exc.status = status
    exc.status_name = name
    return exc
