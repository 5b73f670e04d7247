"""linq_oracle — TEST INFRASTRUCTURE ONLY: a generic CPU Enumerable with System.Linq semantics.

The reference evaluates AsComputeQueryable() queries with System.Linq (ExecuteFallback<T>,
src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:628-633; scalar results :240-267). This module restates
those operators over numpy arrays so a test can write the same query twice: once as C# text for the GPU, once as a
Python callable here. Callables receive numpy arrays (or numpy scalars) of the element dtype, so `x * np.float32(2)
+ np.float32(1)` rounds after each operation exactly as the C# float expression does (numpy never contracts to FMA).

Sum(float) follows the BCL: sequential accumulation in double, one rounding to float (np.cumsum is sequential).
Integer Sum is checked. Min / Max / Average of an empty sequence raise. Float Min returns NaN if any element is NaN;
Max returns NaN only when every element is NaN.
"""
from __future__ import annotations

import numpy as np


class InvalidOperationError(Exception):
    pass


class Enumerable:
    def __init__(self, data):
        self.data = np.asarray(data).reshape(-1)

    # deferred operators ------------------------------------------------------------------------------
    def Select(self, f):
        out = f(self.data) if self.data.size else f(self.data[:0]) if True else None
        return Enumerable(np.asarray(out))

    def Where(self, pred):
        if self.data.size == 0:
            return Enumerable(self.data)
        mask = np.asarray(pred(self.data), dtype=bool)
        if mask.shape == ():                       # predicate ignored its argument (x => true)
            mask = np.full(self.data.shape, bool(mask))
        return Enumerable(self.data[mask])

    def Zip(self, other, f):
        b = other.data if isinstance(other, Enumerable) else np.asarray(other).reshape(-1)
        n = min(self.data.size, b.size)
        return Enumerable(np.asarray(f(self.data[:n], b[:n])))

    def Take(self, n):
        return Enumerable(self.data[: max(n, 0)])

    def Skip(self, n):
        return Enumerable(self.data[max(n, 0):])

    def _first_failing(self, pred):
        """Position of the first element that fails `pred` (len if none): a plain sequential loop, as System.Linq's
        TakeWhile / SkipWhile iterators do it (the vocabulary of ExpressionTreeVisitor.cs:248-249, 263-265)."""
        for i in range(self.data.size):
            if not bool(pred(self.data[i])):
                return i
        return int(self.data.size)

    def TakeWhile(self, pred):
        return Enumerable(self.data[: self._first_failing(pred)])

    def SkipWhile(self, pred):
        return Enumerable(self.data[self._first_failing(pred):])

    def OrderBy(self, key=None):
        """Stable ascending sort by key (Enumerable.OrderBy is stable; NaN keys order first, as Comparer<float> does)."""
        keys = self.data if key is None else np.asarray(key(self.data))
        if keys.dtype.kind == "f":
            order = np.lexsort((np.arange(keys.size), np.where(np.isnan(keys), -np.inf, keys), ~np.isnan(keys)))
        else:
            order = np.argsort(keys, kind="stable")
        return Enumerable(self.data[order])

    def OrderByDescending(self, key=None):
        keys = self.data if key is None else np.asarray(key(self.data))
        if keys.dtype.kind == "f":
            order = np.lexsort((np.arange(keys.size), np.where(np.isnan(keys), np.inf, -keys), np.isnan(keys)))
        else:
            order = np.lexsort((np.arange(keys.size), -keys.astype(np.int64) if keys.dtype.itemsize < 8 else ~keys))
        return Enumerable(self.data[order])

    def GroupAggregate(self, key, aggregate, value=None):
        """GroupBy(key) followed by an aggregate, as the reference's CPU generator writes it (CpuKernelGenerator.cs:544-659): a
        dictionary filled in one sequential pass and enumerated in insertion order. Returns (keys, aggregates). Sum adds in
        the value type with wrap-around for integers; floating sums are returned in double (the comparison carries a tolerance)."""
        keys = np.asarray(key(self.data)) if key is not None else self.data
        vals = np.asarray(value(self.data)) if value is not None else self.data
        groups = {}
        for i in range(keys.size):
            k = keys[i].item()
            if isinstance(k, float) and k != k:
                k = "nan"                                     # float.Equals(NaN, NaN) is true: one group
            groups.setdefault(k, []).append(i)
        out_keys, out = [], []
        for k, idx in groups.items():
            v = vals[idx]
            out_keys.append(keys[idx[0]])
            if aggregate == "Count":
                out.append(len(idx))
            elif aggregate == "Sum":
                out.append(v.astype(np.float64).sum() if v.dtype.kind == "f" else int(v.astype(np.int64).sum()))
            elif aggregate == "Min":
                out.append(v.min())
            elif aggregate == "Max":
                out.append(v.max())
            else:
                out.append(v.astype(np.float64).sum() / len(idx))
        return np.asarray(out_keys, dtype=keys.dtype), out

    def Join(self, inner, outer_key, inner_key, result):
        """Enumerable.Join: for every outer element in order, every inner element with an equal key in inner order."""
        b = inner.data if isinstance(inner, Enumerable) else np.asarray(inner).reshape(-1)
        ok = np.asarray(outer_key(self.data)) if outer_key is not None else self.data
        ik = np.asarray(inner_key(b)) if inner_key is not None else b
        lookup = {}
        for j in range(ik.size):
            lookup.setdefault(ik[j].item(), []).append(j)
        oi, ii = [], []
        for i in range(ok.size):
            for j in lookup.get(ok[i].item(), ()):
                oi.append(i)
                ii.append(j)
        oi, ii = np.asarray(oi, dtype=np.int64), np.asarray(ii, dtype=np.int64)
        return Enumerable(np.asarray(result(self.data[oi], b[ii])))

    def First(self, pred=None):
        e = self.Where(pred) if pred else self
        if e.data.size == 0:
            raise InvalidOperationError("Sequence contains no elements")
        return e.data[0]

    def Last(self, pred=None):
        e = self.Where(pred) if pred else self
        if e.data.size == 0:
            raise InvalidOperationError("Sequence contains no elements")
        return e.data[-1]

    def LastOrDefault(self, pred=None):
        e = self.Where(pred) if pred else self
        return e.data[-1] if e.data.size else self.data.dtype.type(0)

    # terminals -----------------------------------------------------------------------------------------
    def ToArray(self):
        return self.data.copy()

    def Count(self, pred=None):
        return int((self.Where(pred) if pred else self).data.size)

    def Any(self, pred=None):
        return self.Count(pred) > 0

    def All(self, pred):
        return self.Where(pred).data.size == self.data.size

    def Scan(self, inclusive=True):
        """Running sum. Integers add in their own width and wrap (the arithmetic of the reference's generated scan kernel,
        CudaKernelGenerator.cs:499-576); floats are summed sequentially in fp64 and rounded per element."""
        d = self.data
        if d.dtype in (np.int32, np.int64):
            u = d.view(np.uint32 if d.dtype == np.int32 else np.uint64)
            c = np.cumsum(u, dtype=u.dtype)
            if not inclusive:
                c = np.concatenate([np.zeros(1, u.dtype), c[:-1]]) if c.size else c
            return Enumerable(c.view(d.dtype))
        if d.dtype in (np.float32, np.float64):
            c = np.cumsum(d.astype(np.float64))
            if not inclusive:
                c = np.concatenate([np.zeros(1), c[:-1]]) if c.size else c
            return Enumerable(c.astype(d.dtype))
        raise TypeError(f"Scan is not defined for {d.dtype}")

    def Sum(self):
        d = self.data
        if d.dtype in (np.float32, np.float64):
            s = np.cumsum(d.astype(np.float64))[-1] if d.size else np.float64(0)
            return d.dtype.type(s)
        if d.dtype in (np.int32, np.int64):
            info = np.iinfo(d.dtype)
            if d.dtype == np.int32:
                pref = np.cumsum(d.astype(np.int64))
                if pref.size and (pref.max() > info.max or pref.min() < info.min):
                    raise OverflowError("Arithmetic operation resulted in an overflow.")
                return int(pref[-1]) if pref.size else 0
            total = 0
            for v in d.tolist():               # Python ints: exact, checked against the long range
                total += v
                if total > info.max or total < info.min:
                    raise OverflowError("Arithmetic operation resulted in an overflow.")
            return total
        raise TypeError(f"Sum is not defined for {d.dtype}")

    def Average(self):
        d = self.data
        if d.size == 0:
            raise InvalidOperationError("Sequence contains no elements")
        if d.dtype == np.float32:
            return np.float32(np.cumsum(d.astype(np.float64))[-1] / d.size)
        if d.dtype == np.float64:
            return float(np.cumsum(d)[-1] / d.size)
        return float(int(np.sum(d.astype(object))) / d.size) if d.dtype == np.int64 else float(np.sum(d.astype(np.int64)) / d.size)

    def Min(self):
        d = self.data
        if d.size == 0:
            raise InvalidOperationError("Sequence contains no elements")
        if d.dtype.kind == "f":
            if np.isnan(d).any():
                return d.dtype.type(np.nan)
            return _first_of_equals(d, d.min())
        return d.min()

    def Max(self):
        d = self.data
        if d.size == 0:
            raise InvalidOperationError("Sequence contains no elements")
        if d.dtype.kind == "f":
            if np.isnan(d).all():
                return d.dtype.type(np.nan)
            return _first_of_equals(d, np.nanmax(d))
        return d.max()


def _first_of_equals(d, m):
    """Enumerable.Min / Max replace their candidate only on a strict comparison (`x < value`, `value < x`), so of several
    elements that compare equal to the result the earliest one is returned. Only -0 and +0 can tell: same value, other bits."""
    if m == 0:
        return d[np.flatnonzero(d == 0)[0]]
    return m


def scalar_enumerable_where_select(data, pred, sel):
    """Pure-Python element-by-element loop (small inputs): the literal shape of Enumerable.Where(...).Select(...)."""
    out = []
    for x in np.asarray(data).reshape(-1):
        if pred(x):
            out.append(sel(x))
    return out
