"""The LINQ provider surface: AsComputeQueryable / ComputeSelect / ComputeWhere / ToComputeArray and the
standard operators, executed as ONE fused sm_100a kernel per query.

Mirrors src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:19-68 (extension methods) and :105-443
(ComputeQueryProvider). The reference walks a C# expression tree; with no C# compiler in this build the lambdas
arrive as C# text ("x => x * x + 3f") and are typed and translated by the native library. What the reference
evaluates for these queries is System.Linq over the same lambdas (ComputeQueryableExtensions.cs:240-267, 344-352,
628-633); the results here follow those semantics: Where keeps order, Sum(float) accumulates in double, integer Sum
is checked, Min/Max/Average of nothing throw.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import errors, native as N
from .accelerator import CudaAccelerator, PinnedArray, UnifiedBuffer, dcb_type, np_dtype

_TERMINAL_NAMES = {N.OP_TOARRAY: "ToArray", N.OP_SUM: "Sum", N.OP_MIN: "Min", N.OP_MAX: "Max",
                   N.OP_AVERAGE: "Average", N.OP_COUNT: "Count"}


class CompiledPipeline:
    """A compiled query shape (operators + lambdas + element types), reusable over any data of those types."""

    def __init__(self, acc: CudaAccelerator, elem_type0: int, elem_type1: int, ops, force_jit: bool = False):
        self.acc = acc
        self._keep = []
        arr = (N.Op * len(ops))()
        for i, (kind, lam) in enumerate(ops):
            arr[i].kind = kind
            if lam is not None:
                b = lam.encode("utf-8")
                self._keep.append(b)
                arr[i].lambda_ = b
        desc = N.PipelineDesc(elem_type0, elem_type1, len(ops), arr, N.PIPE_FORCE_JIT if force_jit else 0)
        self._h = C.c_void_p()
        N.check(N.lib().dcb_pipeline_compile(acc.handle, C.byref(desc), C.byref(self._h)), acc.handle)
        info = N.PipelineInfo()
        N.check(N.lib().dcb_pipeline_info_get(self._h, C.byref(info)), acc.handle)
        self.info = info
        self.terminal = info.terminal
        self.out_dtype = np_dtype(info.out_type)
        self.result_dtype = np_dtype(info.result_type)
        self.has_filter = bool(info.has_filter)
        self.precompiled = bool(info.precompiled)

    @property
    def handle(self):
        return self._h

    def Dispose(self) -> None:
        """Give the reference back (the native cache keeps the compiled kernels until it needs the room)."""
        h, self._h = self._h, None
        if h is not None and h.value and not getattr(self.acc, "_disposed", True):
            N.lib().dcb_pipeline_destroy(h)

    def __del__(self):
        try:
            self.Dispose()
        except Exception:       # interpreter shutdown: the library may already be gone
            pass

    @property
    def Source(self) -> str:
        need = C.c_size_t()
        N.check(N.lib().dcb_pipeline_source(self._h, None, 0, C.byref(need)), self.acc.handle)
        buf = C.create_string_buffer(need.value)
        N.check(N.lib().dcb_pipeline_source(self._h, buf, need.value, None), self.acc.handle)
        return buf.value.decode()

    def scalar(self, res: N.Result):
        """The value a reduction returns, in the type System.Linq would return."""
        t = self.info.result_type
        if self.terminal == N.OP_COUNT:
            return int(res.count)
        if t == N.T_F32:
            return np.float32(res.f64)
        if t == N.T_F64:
            return float(res.f64)
        if t == N.T_U64:
            return int(res.u64)
        if t == N.T_BOOL:
            return bool(res.i64)
        return int(res.i64)

    def finalize(self, host_record: np.ndarray):
        """Apply the terminal's semantics to a 16-slot record (for instance one combined across GPUs)."""
        rec = np.ascontiguousarray(host_record).view(np.uint8)
        assert rec.nbytes == N.DEVICE_RESULT_BYTES
        res = N.Result()
        N.check(N.lib().dcb_result_finalize(self._h, rec.ctypes.data_as(C.c_void_p), C.byref(res)), self.acc.handle)
        return res


def generate_source(elem_type0, ops, elem_type1=None) -> str:
    """CUDA source the generator emits for a query; needs no GPU (used to test the generator anywhere)."""
    arr = (N.Op * len(ops))()
    keep = []
    for i, (kind, lam) in enumerate(ops):
        arr[i].kind = kind
        if lam is not None:
            keep.append(lam.encode())
            arr[i].lambda_ = keep[-1]
    desc = N.PipelineDesc(dcb_type(elem_type0), dcb_type(elem_type1) if elem_type1 is not None else 0, len(ops), arr, 0)
    need = C.c_size_t()
    err = C.create_string_buffer(512)
    st = N.lib().dcb_pipeline_generate_source(C.byref(desc), None, 0, C.byref(need), err, 512)
    if st:
        raise errors.from_status(st, err.value.decode(), N.lib().dcb_status_name(st).decode())
    buf = C.create_string_buffer(need.value)
    N.lib().dcb_pipeline_generate_source(C.byref(desc), buf, need.value, None, err, 512)
    return buf.value.decode()


def translate_lambda(lambda_text: str, *param_dtypes):
    """(CUDA expression, result dtype) of one C# lambda; needs no GPU."""
    types = (C.c_int32 * len(param_dtypes))(*[dcb_type(d) for d in param_dtypes])
    out = C.create_string_buffer(8192)
    err = C.create_string_buffer(512)
    rt = C.c_int32()
    st = N.lib().dcb_translate_lambda(lambda_text.encode(), types, len(param_dtypes), out, 8192, C.byref(rt), err, 512)
    if st:
        raise errors.from_status(st, err.value.decode(), N.lib().dcb_status_name(st).decode())
    return out.value.decode(), np_dtype(rt.value)


def _split_lambda(text: str):
    head, sep, body = text.partition("=>")
    if not sep:
        raise errors.NotSupportedException(f"not a lambda: {text!r}")
    return head.strip(), body.strip()


class ComputeQueryable:
    """IQueryable<T> bound to the compute provider. Operators only record themselves; a terminal runs the query."""

    def __init__(self, source, accelerator: CudaAccelerator | None = None, ops=(), second=None, force_jit=False, take=None):
        if source is None:
            raise errors.ArgumentNullException("source")
        self._source = source
        self._second = second
        self._ops = tuple(ops)
        self._acc = accelerator
        self._force_jit = force_jit
        self._take = take            # Take(k) after Select/Where: only the first k results are materialised

    # ------------------------------------------------------------------ plumbing
    @property
    def Accelerator(self) -> CudaAccelerator:
        if self._acc is None:
            src = self._source
            self._acc = src.Accelerator if isinstance(src, UnifiedBuffer) else CudaAccelerator.Default()
        return self._acc

    @staticmethod
    def _dtype_of(src) -> np.dtype:
        if isinstance(src, (UnifiedBuffer, PinnedArray)):
            return src.dtype
        return np.asarray(src).dtype

    @staticmethod
    def _len_of(src) -> int:
        if isinstance(src, (UnifiedBuffer, PinnedArray)):
            return src.Length
        return int(np.asarray(src).size)

    def _with(self, kind, lam, second=None):
        if self._take is not None:
            raise errors.NotSupportedException("operators after Take are not fused; materialise with ToArray first")
        return ComputeQueryable(self._source, self._acc, self._ops + ((kind, lam),), second if second is not None else self._second,
                                self._force_jit)

    def _compile(self, terminal: int) -> CompiledPipeline:
        t0 = dcb_type(self._dtype_of(self._source))
        t1 = dcb_type(self._dtype_of(self._second)) if self._second is not None else N.T_NONE
        ops = self._ops + ((terminal, None),)
        return CompiledPipeline(self.Accelerator, t0, t1, ops, self._force_jit)

    def _length(self) -> int:
        n = self._len_of(self._source)
        if self._second is not None:
            n = min(n, self._len_of(self._second))   # Zip stops at the shorter sequence
        return n

    @staticmethod
    def _host_ptr(src, n):
        if isinstance(src, PinnedArray):
            return src.array, C.c_void_p(src.ptr)
        a = np.ascontiguousarray(src).reshape(-1)
        return a, a.ctypes.data_as(C.c_void_p)

    def _run(self, terminal: int):
        """Run the query; returns (pipeline, Result, output array or None)."""
        if self._take is not None and terminal != N.OP_TOARRAY:
            raise errors.NotSupportedException("a reduction after Take is not fused; materialise with ToArray first")
        pipe = self._compile(terminal)
        acc = self.Accelerator
        n = self._length()
        res = N.Result()
        on_device = isinstance(self._source, UnifiedBuffer)
        if self._second is not None and isinstance(self._second, UnifiedBuffer) != on_device:
            raise errors.ArgumentException("both Zip inputs must live on the same side (host arrays or device buffers)")
        to_array = terminal == N.OP_TOARRAY
        out = None
        cap = n if self._take is None or not to_array else min(n, self._take)   # Take(k): the kernel stops writing at k
        if on_device:
            in0 = C.c_void_p(self._source.GetDeviceMemory())
            in1 = C.c_void_p(self._second.GetDeviceMemory()) if self._second is not None else None
            if to_array:
                dbuf = acc.Memory.AllocateAsync(max(cap, 1), pipe.out_dtype)
                try:
                    flags = N.RUN_TAKE if (self._take is not None and pipe.has_filter) else 0   # Take(k): stop scanning once k are known
                    N.check(N.lib().dcb_pipeline_run_ex(pipe.handle, in0, in1, n if pipe.has_filter else cap, C.c_void_p(dbuf.GetDeviceMemory()), cap,
                                                        flags, C.byref(res), None), acc.handle)
                    got = min(int(res.count), cap)
                    out = dbuf.CopyToAsync(count=got) if got else np.empty(0, pipe.out_dtype)
                finally:
                    dbuf.Dispose()
            else:
                N.check(N.lib().dcb_pipeline_run(pipe.handle, in0, in1, n, None, 0, C.byref(res), None), acc.handle)
        else:
            a0, p0 = self._host_ptr(self._source, n)
            a1, p1 = (None, None)
            if self._second is not None:
                a1, p1 = self._host_ptr(self._second, n)
            if to_array:
                out = np.empty(cap, dtype=pipe.out_dtype)
                flags = N.RUN_TAKE if (self._take is not None and pipe.has_filter) else 0
                N.check(N.lib().dcb_pipeline_run_host_ex(pipe.handle, p0, p1, n if pipe.has_filter else cap, out.ctypes.data_as(C.c_void_p), cap,
                                                         flags, C.byref(res)), acc.handle)
                got = min(int(res.count), cap)
                out = out[:got]
                if out.base is not None and got < cap:
                    out = out.copy()
            else:
                N.check(N.lib().dcb_pipeline_run_host(pipe.handle, p0, p1, n, None, 0, C.byref(res)), acc.handle)
            del a0, a1
        self.LastResult = res
        return pipe, res, out

    # ------------------------------------------------------------------ operators (deferred)
    def Select(self, selector: str) -> "ComputeQueryable":
        if selector is None:
            raise errors.ArgumentNullException("selector")
        return self._with(N.OP_SELECT, selector)

    def Where(self, predicate: str) -> "ComputeQueryable":
        if predicate is None:
            raise errors.ArgumentNullException("predicate")
        return self._with(N.OP_WHERE, predicate)

    def Zip(self, second, resultSelector: str) -> "ComputeQueryable":
        if second is None:
            raise errors.ArgumentNullException("second")
        if resultSelector is None:
            raise errors.ArgumentNullException("resultSelector")
        if self._ops:
            raise errors.NotSupportedException("Zip must be applied to the source sequence, before Select/Where")
        if isinstance(second, ComputeQueryable):
            if second._ops:
                raise errors.NotSupportedException("the second Zip operand must be a plain source")
            second = second._source
        return self._with(N.OP_ZIP, resultSelector, second=second)

    ComputeSelect = Select
    ComputeWhere = Where

    def Cast(self, type_name: str) -> "ComputeQueryable":
        """Cast<T>(): element-wise conversion to the C# type named (`"long"`, `"float"`, ...), a Select in the visitor's
        vocabulary (src/Extensions/DotCompute.Linq/Compilation/ExpressionTreeVisitor.cs:234-272)."""
        if type_name is None:
            raise errors.ArgumentNullException("type_name")
        return self.Select(f"x => ({type_name})x")

    def _has_where(self) -> bool:
        return any(kind == N.OP_WHERE for kind, _ in self._ops)

    def _sliced(self, offset: int, length: int) -> "ComputeQueryable":
        """The same Select / Zip chain over elements [offset, offset + length) of the source(s). Only valid while no Where
        precedes: a map sends element i of the source to element i of the result."""
        second = _slice(self._second, offset, length) if self._second is not None else None
        return ComputeQueryable(_slice(self._source, offset, length), self._acc, self._ops, second, self._force_jit)

    def _materialized(self) -> "ComputeQueryable":
        """Runs the query so far and continues over its result (for operators that need positions in a filtered sequence)."""
        return ComputeQueryable(self.ToArray(), self._acc, (), None, self._force_jit)

    def _index_of(self, terminal: int) -> int:
        """FirstIndex / LastIndex: position in the source of the first / last element that passes every Where (-1: none)."""
        if self._take is not None:
            raise errors.NotSupportedException("an index query after Take is not fused; materialise with ToArray first")
        if self._length() == 0:
            return -1
        _pipe, res, _ = self._run(terminal)
        return int(res.i64)

    def Skip(self, count: int) -> "ComputeQueryable":
        q = self._materialized() if (self._has_where() or self._take is not None) else self
        n = q._length()
        k = min(max(int(count), 0), n)
        return q._sliced(k, n - k)

    def TakeWhile(self, predicate: str) -> "ComputeQueryable":
        """Elements up to (not including) the first one that fails `predicate`. One fused pass finds that position (a Min over
        the indices of failing elements, DCB_OP_FIRST_INDEX); what follows runs over the source cut there. The reference's
        visitor lists the operator (ExpressionTreeVisitor.cs:248-249, 263-265); its scan kernel is single-block
        (CudaKernelGenerator.cs:499-576)."""
        if predicate is None:
            raise errors.ArgumentNullException("predicate")
        q = self._materialized() if (self._has_where() or self._take is not None) else self
        head, body = _split_lambda(predicate)
        stop = q.Where(f"{head} => !({body})")._index_of(N.OP_FIRST_INDEX)
        return q if stop < 0 else q._sliced(0, stop)

    def SkipWhile(self, predicate: str) -> "ComputeQueryable":
        """Elements from the first one that fails `predicate` on (that one included)."""
        if predicate is None:
            raise errors.ArgumentNullException("predicate")
        q = self._materialized() if (self._has_where() or self._take is not None) else self
        head, body = _split_lambda(predicate)
        n = q._length()
        start = q.Where(f"{head} => !({body})")._index_of(N.OP_FIRST_INDEX)
        return q._sliced(n, 0) if start < 0 else q._sliced(start, n - start)

    def Take(self, count: int):
        n = self._length()
        k = min(max(int(count), 0), n)
        if self._ops:
            # The first k results in source order: the compaction kernel keeps order and simply stops writing at k.
            return ComputeQueryable(self._source, self._acc, self._ops, self._second, self._force_jit,
                                    take=k if self._take is None else min(k, self._take))
        return ComputeQueryable(_slice(self._source, 0, k), self._acc, (), None, self._force_jit)

    # ------------------------------------------------------------------ OrderBy / GroupBy / Join (device-resident)
    def ToBuffer(self) -> UnifiedBuffer:
        """The query's result as a device buffer (the caller disposes it). A device source without operators is returned as
        a view of itself; everything else runs the fused kernel into a fresh buffer, with no trip through the host for
        device sources."""
        acc = self.Accelerator
        if not self._ops and self._take is None:
            src = self._source
            if isinstance(src, UnifiedBuffer):
                return src.Slice(0, src.Length)
            host = src.array if isinstance(src, PinnedArray) else np.ascontiguousarray(np.asarray(src).reshape(-1))
            return acc.Memory.AllocateAndCopyAsync(host)
        if not isinstance(self._source, UnifiedBuffer):
            return acc.Memory.AllocateAndCopyAsync(self.ToArray())
        pipe = self._compile(N.OP_TOARRAY)
        n = self._length()
        cap = n if self._take is None else min(n, self._take)
        dbuf = acc.Memory.AllocateAsync(max(cap, 1), pipe.out_dtype)
        res = N.Result()
        in1 = C.c_void_p(self._second.GetDeviceMemory()) if self._second is not None else None
        flags = N.RUN_TAKE if (self._take is not None and pipe.has_filter) else 0
        N.check(N.lib().dcb_pipeline_run_ex(pipe.handle, C.c_void_p(self._source.GetDeviceMemory()), in1, n if pipe.has_filter else cap,
                                            C.c_void_p(dbuf.GetDeviceMemory()), cap, flags, C.byref(res), None), acc.handle)
        got = min(int(res.count), cap)
        out = dbuf.Slice(0, got)
        out._owner = dbuf                      # keeps the allocation alive as long as the view
        return out

    def _keys_of(self, values: UnifiedBuffer, selector: str | None) -> UnifiedBuffer:
        if selector is None:
            return values.Slice(0, values.Length)
        return ComputeQueryable(values, self._acc, ((N.OP_SELECT, selector),), None, self._force_jit).ToBuffer()

    def _order(self, key_selector: str | None, descending: bool) -> "ComputeQueryable":
        acc = self.Accelerator
        values = self.ToBuffer()
        n = values.Length
        if n <= 1:
            return ComputeQueryable(values, acc, (), None, self._force_jit)
        keys = self._keys_of(values, key_selector)
        out = acc.Memory.AllocateAsync(n, values.dtype)
        if values.dtype.itemsize == 4:
            # 4-byte elements travel beside their keys through the sort: no gather afterwards
            N.check(N.lib().dcb_sort_by_key(acc.handle, dcb_type(keys.dtype), C.c_void_p(keys.GetDeviceMemory()), n, 1 if descending else 0, 4,
                                            C.c_void_p(values.GetDeviceMemory()), C.c_void_p(out.GetDeviceMemory()), None), acc.handle)
            acc.Synchronize()
            keys.Dispose()
            return ComputeQueryable(out, acc, (), None, self._force_jit)
        idx = acc.Memory.AllocateAsync(n, np.uint32)
        N.check(N.lib().dcb_sort_indices(acc.handle, dcb_type(keys.dtype), C.c_void_p(keys.GetDeviceMemory()), n, 1 if descending else 0,
                                         C.c_void_p(idx.GetDeviceMemory()), None), acc.handle)
        N.check(N.lib().dcb_gather(acc.handle, values.dtype.itemsize, C.c_void_p(values.GetDeviceMemory()), C.c_void_p(idx.GetDeviceMemory()), n,
                                   C.c_void_p(out.GetDeviceMemory()), None), acc.handle)
        acc.Synchronize()
        idx.Dispose(); keys.Dispose()
        return ComputeQueryable(out, acc, (), None, self._force_jit)

    def Scan(self, inclusive: bool = True) -> "ComputeQueryable":
        """Running sum of the sequence (after its fused Select / Where): element i is the sum of elements 0..i (or 0..i-1 with
        inclusive=False). The reference's visitor has the operation type (ExpressionTreeVisitor.cs:248-249) and a generator
        for one block of 256 elements (CudaKernelGenerator.cs:499-576); this one takes any length. int / long add in their
        own width and wrap, as that kernel's arithmetic does; float / double add in fp64, each output rounded once."""
        acc = self.Accelerator
        values = self.ToBuffer()
        n = values.Length
        if values.dtype not in (np.dtype(np.int32), np.dtype(np.int64), np.dtype(np.float32), np.dtype(np.float64)):
            raise errors.NotSupportedException("Scan is defined for int, long, float and double (project with Select first)")
        out = acc.Memory.AllocateAsync(max(n, 1), values.dtype).Slice(0, n) if n == 0 else acc.Memory.AllocateAsync(n, values.dtype)
        if n:
            N.check(N.lib().dcb_prefix_sum(acc.handle, dcb_type(values.dtype), C.c_void_p(values.GetDeviceMemory()), n, 1 if inclusive else 0,
                                           C.c_void_p(out.GetDeviceMemory()), None), acc.handle)
            acc.Synchronize()
        return ComputeQueryable(out, acc, (), None, self._force_jit)

    def OrderBy(self, keySelector: str | None = None) -> "ComputeQueryable":
        """Stable ascending sort by `keySelector` (the elements themselves if None): a multi-block radix sort on the device.
        The reference's generator emits a single-block bitonic sort (CudaKernelGenerator.cs:613-751, OrderByKernelGenerator.cs:108);
        its CPU path is Array.Sort(keys, values) (CpuKernelGenerator.cs:475-527). Ties keep source order, as Enumerable.OrderBy."""
        return self._order(keySelector, False)

    def OrderByDescending(self, keySelector: str | None = None) -> "ComputeQueryable":
        return self._order(keySelector, True)

    def GroupBy(self, keySelector: str | None = None) -> "Grouping":
        """GroupBy followed by an aggregate (Count / Sum / Min / Max / Average), one result per key in order of first occurrence -
        the order a Dictionary enumerates in, which is what the reference's CPU path produces (CpuKernelGenerator.cs:544-659;
        GPU generator CudaKernelGenerator.cs:753-825, GroupByKernelGenerator.cs:152)."""
        return Grouping(self, keySelector)

    def _join(self, inner, outerKeySelector, innerKeySelector, kind: int):
        acc = self.Accelerator
        if inner is None:
            raise errors.ArgumentNullException("inner")
        inner_q = inner if isinstance(inner, ComputeQueryable) else ComputeQueryable(inner, acc, (), None, self._force_jit)
        ov, iv = self.ToBuffer(), inner_q.ToBuffer()
        ok, ik = self._keys_of(ov, outerKeySelector), self._keys_of(iv, innerKeySelector)
        if ok.dtype != ik.dtype:
            raise errors.ArgumentException(f"join keys have different types: {ok.dtype} and {ik.dtype}")
        pairs = C.c_int64()
        args = (acc.handle, dcb_type(ok.dtype), C.c_void_p(ok.GetDeviceMemory()), ov.Length, C.c_void_p(ik.GetDeviceMemory()), iv.Length, kind)
        N.check(N.lib().dcb_join_indices(*args, 0, None, None, C.byref(pairs), None), acc.handle)
        m = int(pairs.value)
        oi = acc.Memory.AllocateAsync(max(m, 1), np.uint32)
        ii = acc.Memory.AllocateAsync(max(m, 1), np.uint32)
        if m:
            N.check(N.lib().dcb_join_indices(*args, m, C.c_void_p(oi.GetDeviceMemory()), C.c_void_p(ii.GetDeviceMemory()), C.byref(pairs), None), acc.handle)
        go = acc.Memory.AllocateAsync(max(m, 1), ov.dtype)
        gi = acc.Memory.AllocateAsync(max(m, 1), iv.dtype)
        if m:
            N.check(N.lib().dcb_gather(acc.handle, ov.dtype.itemsize, C.c_void_p(ov.GetDeviceMemory()), C.c_void_p(oi.GetDeviceMemory()), m,
                                       C.c_void_p(go.GetDeviceMemory()), None), acc.handle)
            if kind == N.JOIN_INNER:
                N.check(N.lib().dcb_gather(acc.handle, iv.dtype.itemsize, C.c_void_p(iv.GetDeviceMemory()), C.c_void_p(ii.GetDeviceMemory()), m,
                                           C.c_void_p(gi.GetDeviceMemory()), None), acc.handle)
        acc.Synchronize()
        for b in (ok, ik, oi, ii):
            b.Dispose()
        return go.Slice(0, m), gi.Slice(0, m), go, gi

    def Join(self, inner, outerKeySelector: str | None, innerKeySelector: str | None, resultSelector: str) -> "ComputeQueryable":
        """Inner equi-join: resultSelector(outer, inner) for every pair with equal keys, ordered by outer element, then inner
        element (the order of Enumerable.Join). The inner keys are sorted once (stable radix sort), every outer key finds its
        run by binary search, and the pairs are written in order; the result selector is a fused Zip over the gathered pairs.
        The reference's generator builds a fixed-size hash table (JoinKernelGenerator.cs:140-239, CudaKernelGenerator.cs:827-900)."""
        if resultSelector is None:
            raise errors.ArgumentNullException("resultSelector")
        o, i, keep_o, keep_i = self._join(inner, outerKeySelector, innerKeySelector, N.JOIN_INNER)
        q = ComputeQueryable(o, self.Accelerator, ((N.OP_ZIP, resultSelector),), i, self._force_jit)
        q._keep = (keep_o, keep_i)
        return q

    def SemiJoin(self, inner, outerKeySelector: str | None = None, innerKeySelector: str | None = None) -> "ComputeQueryable":
        """Outer elements that have at least one match among the inner keys, in source order (JoinType.Semi, JoinKernelGenerator.cs:71-74)."""
        o, _i, keep_o, _ki = self._join(inner, outerKeySelector, innerKeySelector, N.JOIN_SEMI)
        q = ComputeQueryable(o, self.Accelerator, (), None, self._force_jit)
        q._keep = keep_o
        return q

    def AntiJoin(self, inner, outerKeySelector: str | None = None, innerKeySelector: str | None = None) -> "ComputeQueryable":
        """Outer elements without a match (JoinType.Anti, JoinKernelGenerator.cs:75-77)."""
        o, _i, keep_o, _ki = self._join(inner, outerKeySelector, innerKeySelector, N.JOIN_ANTI)
        q = ComputeQueryable(o, self.Accelerator, (), None, self._force_jit)
        q._keep = keep_o
        return q

    # ------------------------------------------------------------------ terminals
    def ToArray(self) -> np.ndarray:
        if not self._ops:   # AsComputeQueryable().ToArray(): round trip of the source
            src = self._source
            if isinstance(src, UnifiedBuffer):
                return src.ToArray()
            return np.array(src.array if isinstance(src, PinnedArray) else src, copy=True).reshape(-1)
        _, _, out = self._run(N.OP_TOARRAY)
        return out

    ToComputeArray = ToArray

    def ToList(self) -> list:
        return self.ToArray().tolist()

    def __iter__(self):
        return iter(self.ToArray())

    def Sum(self, selector: str | None = None):
        q = self.Select(selector) if selector is not None else self
        pipe, res, _ = q._run(N.OP_SUM)
        return pipe.scalar(res)

    def Average(self, selector: str | None = None):
        q = self.Select(selector) if selector is not None else self
        pipe, res, _ = q._run(N.OP_AVERAGE)
        return pipe.scalar(res)

    def Min(self, selector: str | None = None):
        q = self.Select(selector) if selector is not None else self
        pipe, res, _ = q._run(N.OP_MIN)
        return pipe.out_dtype.type(pipe.scalar(res))

    def Max(self, selector: str | None = None):
        q = self.Select(selector) if selector is not None else self
        pipe, res, _ = q._run(N.OP_MAX)
        return pipe.out_dtype.type(pipe.scalar(res))

    def Count(self, predicate: str | None = None) -> int:
        q = self.Where(predicate) if predicate is not None else self
        if not q._ops:
            return q._length()
        pipe, res, _ = q._run(N.OP_COUNT)
        return int(res.count)

    LongCount = Count

    def Any(self, predicate: str | None = None) -> bool:
        return self.Count(predicate) > 0

    def First(self, predicate: str | None = None):
        """First element (that satisfies `predicate`); InvalidOperationException if there is none, as in System.Linq."""
        q = self.Where(predicate) if predicate is not None else self
        got = q.Take(1).ToArray()
        if got.size == 0:
            raise errors.InvalidOperationException("Sequence contains no " + ("matching element" if predicate else "elements"))
        return got[0]

    def FirstOrDefault(self, predicate: str | None = None):
        q = self.Where(predicate) if predicate is not None else self
        got = q.Take(1).ToArray()
        return got[0] if got.size else got.dtype.type(0)

    def _last(self, predicate, default: bool):
        q = self.Where(predicate) if predicate is not None else self
        if q._take is not None:
            q = q._materialized()
        idx = q._index_of(N.OP_LAST_INDEX) if q._has_where() else q._length() - 1
        maps = ComputeQueryable(q._source, q._acc, tuple(op for op in q._ops if op[0] != N.OP_WHERE), q._second, q._force_jit)
        if idx < 0:
            if default:
                return maps._compile(N.OP_TOARRAY).out_dtype.type(0)
            raise errors.InvalidOperationException("Sequence contains no " + ("matching element" if predicate else "elements"))
        return maps._sliced(idx, 1).ToArray()[0]          # the Selects of the chain applied to that one element

    def Last(self, predicate: str | None = None):
        """Last element (that satisfies `predicate`): one fused pass finds its position (a Max over the indices of surviving
        elements, DCB_OP_LAST_INDEX), then the chain's Selects run on that single element."""
        return self._last(predicate, False)

    def LastOrDefault(self, predicate: str | None = None):
        return self._last(predicate, True)

    def ElementAt(self, index: int):
        if index < 0:
            raise errors.ArgumentException("index must not be negative")
        got = self.Take(index + 1).ToArray()
        if got.size <= index:
            raise errors.ArgumentException("index is past the end of the sequence")
        return got[index]

    def Contains(self, value) -> bool:
        """Contains(value): an equality Where plus Count. The literal is printed in the element type's C# spelling."""
        dt = self._dtype_of(self._source) if not self._ops else None
        if dt is None:
            dt = self._compile(N.OP_TOARRAY).out_dtype
        lit = _literal(value, dt)
        return self.Count(f"x => x == {lit}") > 0

    def All(self, predicate: str) -> bool:
        if predicate is None:
            raise errors.ArgumentNullException("predicate")
        head, body = _split_lambda(predicate)
        return self.Count(f"{head} => !({body})") == 0


class Grouping:
    """`source.GroupBy(keySelector)` waiting for its aggregate. Every aggregate returns one numpy array with an entry per
    distinct key, in order of the key's first occurrence; `Keys()` gives the keys in the same order."""

    def __init__(self, query: ComputeQueryable, key_selector: str | None):
        self._q, self._sel = query, key_selector

    def _run(self, agg: int, value_selector: str | None):
        q = self._q
        acc = q.Accelerator
        values = q.ToBuffer()
        n = values.Length
        keys = q._keys_of(values, self._sel)
        vals = q._keys_of(values, value_selector)
        empty = (np.empty(0, keys.dtype), np.empty(0, np.int64), np.empty(0, np.float64), np.empty(0, np.int64), vals.dtype)
        if n == 0:
            return empty
        cap = min(n, 1 << 20)
        while True:
            first = acc.Memory.AllocateAsync(cap, np.uint32)
            counts = acc.Memory.AllocateAsync(cap, np.int64)
            f64 = acc.Memory.AllocateAsync(cap, np.float64)
            i64 = acc.Memory.AllocateAsync(cap, np.int64)
            groups = C.c_int64()
            st = N.lib().dcb_group_aggregate(acc.handle, dcb_type(keys.dtype), C.c_void_p(keys.GetDeviceMemory()), dcb_type(vals.dtype),
                                             C.c_void_p(vals.GetDeviceMemory()), n, agg, cap, C.c_void_p(first.GetDeviceMemory()),
                                             C.c_void_p(counts.GetDeviceMemory()), C.c_void_p(f64.GetDeviceMemory()),
                                             C.c_void_p(i64.GetDeviceMemory()), C.byref(groups), None)
            g = int(groups.value)
            if st == 202 and g > cap:               # more groups than guessed: once more with room for all of them
                for b in (first, counts, f64, i64):
                    b.Dispose()
                cap = g
                continue
            N.check(st, acc.handle)
            break
        acc.Synchronize()
        gk = acc.Memory.AllocateAsync(max(g, 1), keys.dtype)
        N.check(N.lib().dcb_gather(acc.handle, keys.dtype.itemsize, C.c_void_p(keys.GetDeviceMemory()), C.c_void_p(first.GetDeviceMemory()), g,
                                   C.c_void_p(gk.GetDeviceMemory()), None), acc.handle)
        out = (gk.CopyToAsync(count=g), counts.CopyToAsync(count=g), f64.CopyToAsync(count=g), i64.CopyToAsync(count=g), vals.dtype)
        for b in (first, counts, f64, i64, gk, keys, vals):
            b.Dispose()
        return out

    def Keys(self) -> np.ndarray:
        return self._run(N.AGG_COUNT, None)[0]

    def Count(self) -> np.ndarray:
        return self._run(N.AGG_COUNT, None)[1].astype(np.int32)

    def _typed(self, agg, selector):
        _k, _c, f, i, dt = self._run(agg, selector)
        if dt.kind == "f":
            return f.astype(dt)
        with np.errstate(over="ignore"):
            return i.astype(dt)                      # integer sums wrap, as the unchecked C# accumulation does

    def Sum(self, valueSelector: str | None = None) -> np.ndarray:
        return self._typed(N.AGG_SUM, valueSelector)

    def Min(self, valueSelector: str | None = None) -> np.ndarray:
        return self._typed(N.AGG_MIN, valueSelector)

    def Max(self, valueSelector: str | None = None) -> np.ndarray:
        return self._typed(N.AGG_MAX, valueSelector)

    def Average(self, valueSelector: str | None = None) -> np.ndarray:
        return self._run(N.AGG_AVERAGE, valueSelector)[2]

    def ToDictionary(self, aggregate: str = "Count", valueSelector: str | None = None) -> dict:
        keys = self.Keys()
        vals = getattr(self, aggregate)() if aggregate == "Count" else getattr(self, aggregate)(valueSelector)
        return dict(zip(keys.tolist(), vals.tolist()))


def _literal(value, dtype) -> str:
    """C# literal of `value` in the type of `dtype` (for queries built from values, such as Contains)."""
    dt = np.dtype(dtype)
    if dt == np.float32:
        return repr(float(np.float32(value))) + "f" if np.isfinite(value) else ("float.NaN" if np.isnan(value) else ("float.PositiveInfinity" if value > 0 else "float.NegativeInfinity"))
    if dt == np.float64:
        return repr(float(value)) + "d" if np.isfinite(value) else ("double.NaN" if np.isnan(value) else ("double.PositiveInfinity" if value > 0 else "double.NegativeInfinity"))
    if dt == np.bool_:
        return "true" if value else "false"
    v = int(value)
    suffix = {np.dtype(np.uint32): "u", np.dtype(np.int64): "L", np.dtype(np.uint64): "UL"}.get(dt, "")
    if v < 0:
        return f"(-{-v}{suffix})" if v != -2**63 else "long.MinValue"
    return f"{v}{suffix}"


def _slice(src, offset, length):
    if isinstance(src, UnifiedBuffer):
        return src.Slice(offset, length)
    a = src.array if isinstance(src, PinnedArray) else np.asarray(src).reshape(-1)
    return a[offset: offset + length]


def AsComputeQueryable(source, accelerator: CudaAccelerator | None = None, force_jit: bool = False) -> ComputeQueryable:
    """`source.AsQueryable().AsComputeQueryable()`: source is a host array, a PinnedArray or a device UnifiedBuffer."""
    if source is None:
        raise errors.ArgumentNullException("source")
    if isinstance(source, ComputeQueryable):
        return source
    return ComputeQueryable(source, accelerator, force_jit=force_jit)


def ToComputeArray(source) -> np.ndarray:
    """ToComputeArray on a non-compute source is a plain ToArray (ComputeQueryableExtensions.cs:34-41)."""
    if source is None:
        raise errors.ArgumentNullException("source")
    if isinstance(source, ComputeQueryable):
        return source.ToArray()
    return np.array(source, copy=True).reshape(-1)


class ComputeLinqProvider:
    """IComputeLinqProvider (src/Extensions/DotCompute.Linq/ServiceCollectionExtensions.cs:16-38)."""

    def __init__(self, accelerator: CudaAccelerator | None = None):
        self._acc = accelerator

    def CreateComputeQueryable(self, source) -> ComputeQueryable:
        if source is None:
            raise errors.ArgumentNullException("source")
        if not isinstance(source, (np.ndarray, UnifiedBuffer, PinnedArray)):
            source = np.asarray(list(source))
        return ComputeQueryable(source, self._acc)
