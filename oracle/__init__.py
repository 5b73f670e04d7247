"""oracle — TEST INFRASTRUCTURE ONLY.

CPU restatement of the reference's semantics for the LINQ hot path, used as the checker by tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline legs. Nothing under dotcompute_b200/ imports it.

  c_oracle      ctypes view of dc_oracle.c (sequential System.Linq semantics for the benchmark configurations)
  cpu_simd      ctypes view of cpu_simd.cpp (restated CPU SIMD backend loops; the timed CPU baseline)
  linq_oracle   generic numpy / pure-Python Enumerable for arbitrary lambdas
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")


def build() -> None:
    """Compile the C / C++ sources with gcc (make -C oracle)."""
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)


def _load(name: str) -> C.CDLL:
    path = os.path.join(_HERE, name)
    if not os.path.exists(path):
        build()
    return C.CDLL(path)


class _COracle:
    def __init__(self):
        L = _load("liboracle.so")
        self.L = L
        L.oracle_select_mul_add_f32.argtypes = [_f32p, C.c_int64, C.c_float, C.c_float, _f32p]
        L.oracle_where_gt_select_sq_add_f32.argtypes = [_f32p, C.c_int64, C.c_float, C.c_float, _f32p]
        L.oracle_where_gt_select_sq_add_f32.restype = C.c_int64
        L.oracle_where_gt_select_sq_add_sum_f32.argtypes = [_f32p, C.c_int64, C.c_float, C.c_float, C.POINTER(C.c_double), C.POINTER(C.c_int64)]
        L.oracle_where_gt_select_sq_add_sum_f32.restype = C.c_float
        L.oracle_sum_f32.argtypes = [_f32p, C.c_int64, C.POINTER(C.c_double)]
        L.oracle_sum_f32.restype = C.c_float
        L.oracle_sum_abs_f64.argtypes = [_f32p, C.c_int64]
        L.oracle_sum_abs_f64.restype = C.c_double
        for nm in ("average", "min", "max"):
            getattr(L, f"oracle_{nm}_f32").argtypes = [_f32p, C.c_int64, C.POINTER(C.c_float)]
        for nm in ("sum", "min", "max"):
            getattr(L, f"oracle_{nm}_i32").argtypes = [_i32p, C.c_int64, C.POINTER(C.c_int32)]
        L.oracle_average_i32.argtypes = [_i32p, C.c_int64, C.POINTER(C.c_double)]
        L.oracle_zip_mul_sum_f32.argtypes = [_f32p, _f32p, C.c_int64, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        L.oracle_zip_mul_sum_f32.restype = C.c_float
        L.oracle_where_mask_eq_i64.argtypes = [_i64p, C.c_int64, C.c_int64, C.c_int64, _i64p]
        L.oracle_where_mask_eq_i64.restype = C.c_int64
        L.oracle_fingerprint_u32.argtypes = [_u32p, C.c_int64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]

    # Each wrapper returns numpy values; status codes become the exceptions System.Linq throws.
    @staticmethod
    def _raise(st):
        if st == 501:
            raise InvalidOperationError("Sequence contains no elements")
        if st == 502:
            raise OverflowError("Arithmetic operation resulted in an overflow.")

    def select_mul_add(self, x, a, b):
        out = np.empty_like(x)
        self.L.oracle_select_mul_add_f32(x, x.size, a, b, out)
        return out

    def where_gt_select_sq_add(self, x, thr, c):
        out = np.empty_like(x)
        k = self.L.oracle_where_gt_select_sq_add_f32(x, x.size, thr, c, out)
        return out[:k].copy()

    def where_gt_select_sq_add_sum(self, x, thr, c):
        raw, cnt = C.c_double(), C.c_int64()
        v = self.L.oracle_where_gt_select_sq_add_sum_f32(x, x.size, thr, c, C.byref(raw), C.byref(cnt))
        return np.float32(v), raw.value, cnt.value

    def sum_f32(self, x):
        raw = C.c_double()
        v = self.L.oracle_sum_f32(x, x.size, C.byref(raw))
        return np.float32(v), raw.value

    def sum_abs(self, x):
        return self.L.oracle_sum_abs_f64(x, x.size)

    def _f32(self, nm, x):
        out = C.c_float()
        self._raise(getattr(self.L, f"oracle_{nm}_f32")(x, x.size, C.byref(out)))
        return np.float32(out.value)

    def average_f32(self, x):
        return self._f32("average", x)

    def min_f32(self, x):
        return self._f32("min", x)

    def max_f32(self, x):
        return self._f32("max", x)

    def _i32(self, nm, x):
        out = C.c_int32()
        self._raise(getattr(self.L, f"oracle_{nm}_i32")(x, x.size, C.byref(out)))
        return int(out.value)

    def sum_i32(self, x):
        return self._i32("sum", x)

    def min_i32(self, x):
        return self._i32("min", x)

    def max_i32(self, x):
        return self._i32("max", x)

    def average_i32(self, x):
        out = C.c_double()
        self._raise(self.L.oracle_average_i32(x, x.size, C.byref(out)))
        return out.value

    def zip_mul_sum(self, a, b):
        n = min(a.size, b.size)
        raw, sa = C.c_double(), C.c_double()
        v = self.L.oracle_zip_mul_sum_f32(a, b, n, C.byref(raw), C.byref(sa))
        return np.float32(v), raw.value, sa.value

    def where_mask_eq_i64(self, k, mask, val):
        out = np.empty_like(k)
        n = self.L.oracle_where_mask_eq_i64(k, k.size, mask, val, out)
        return out[:n].copy()

    def fingerprint(self, arr):
        u = np.ascontiguousarray(arr).view(np.uint32).reshape(-1)
        p, w = C.c_uint64(), C.c_uint64()
        self.L.oracle_fingerprint_u32(u, u.size, C.byref(p), C.byref(w))
        return p.value, w.value


class InvalidOperationError(Exception):
    """System.InvalidOperationException as thrown by Enumerable.Min/Max/Average on an empty sequence."""


class _CpuSimd:
    def __init__(self):
        flags = ""
        try:
            with open("/proc/cpuinfo") as f:
                for line in f:
                    if line.startswith("flags"):
                        flags = line
                        break
        except OSError:
            pass
        variant = "avx512" if " avx512f" in flags else ("avx2" if " avx2" in flags else "base")
        L = _load(f"libcpusimd_{variant}.so")
        self.L, self.variant = L, variant
        L.cpu_simd_sum_f32.argtypes = [_f32p, C.c_int64, C.c_int]
        L.cpu_simd_sum_f32.restype = C.c_float
        L.cpu_simd_where_select_sum_f32.argtypes = [_f32p, C.c_int64, C.c_float, C.c_float, C.c_int]
        L.cpu_simd_where_select_sum_f32.restype = C.c_float
        L.cpu_simd_where_select_toarray_f32.argtypes = [_f32p, C.c_int64, C.c_float, C.c_float, _f32p, C.c_int]
        L.cpu_simd_where_select_toarray_f32.restype = C.c_int64
        L.cpu_scalar_where_select_sum_f32.argtypes = [_f32p, C.c_int64, C.c_float, C.c_float]
        L.cpu_scalar_where_select_sum_f32.restype = C.c_float
        self.threads = L.cpu_simd_threads()
        self.width = L.cpu_simd_width()

    def where_select_sum(self, x, thr, c, threads=None):
        return np.float32(self.L.cpu_simd_where_select_sum_f32(x, x.size, thr, c, threads or self.threads))

    def where_select_toarray(self, x, thr, c, threads=None):
        out = np.empty_like(x)
        k = self.L.cpu_simd_where_select_toarray_f32(x, x.size, thr, c, out, threads or self.threads)
        return out[:k]

    def scalar_where_select_sum(self, x, thr, c):
        return np.float32(self.L.cpu_scalar_where_select_sum_f32(x, x.size, thr, c))

    def sum(self, x, threads=None):
        return np.float32(self.L.cpu_simd_sum_f32(x, x.size, threads or self.threads))


_c = None
_s = None


def c_oracle() -> _COracle:
    global _c
    if _c is None:
        _c = _COracle()
    return _c


def cpu_simd() -> _CpuSimd:
    global _s
    if _s is None:
        _s = _CpuSimd()
    return _s
