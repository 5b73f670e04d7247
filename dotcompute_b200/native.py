"""ctypes binding of libdcb200.so — exactly the entry points include/dcb200.h declares.

This is the Python stand-in for the `[LibraryImport("dcb200")]` class the managed side would hold. It adds
nothing: handles are opaque pointers, every call returns a status, and a non-zero status is turned into the
exception the reference's callers expect (see errors.py). There is no fallback: if the shared library is
missing, importing a symbol from here raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

from . import errors

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdcb200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "dcb200.h")

# ---- constants (values mirror dcb200.h) -------------------------------------------------------------------
T_NONE, T_I8, T_U8, T_I16, T_U16, T_I32, T_U32, T_I64, T_U64, T_F32, T_F64, T_BOOL = range(12)
OP_SELECT, OP_WHERE, OP_ZIP = 1, 2, 3
OP_TOARRAY, OP_SUM, OP_MIN, OP_MAX, OP_AVERAGE, OP_COUNT, OP_FIRST_INDEX, OP_LAST_INDEX = 16, 17, 18, 19, 20, 21, 22, 23
PIPE_FORCE_JIT = 1
RUN_TAKE = 1
AGG_COUNT, AGG_SUM, AGG_MIN, AGG_MAX, AGG_AVERAGE = 0, 1, 2, 3, 4
JOIN_INNER, JOIN_SEMI, JOIN_ANTI = 0, 2, 3
RES_SAW_NAN, RES_TRUNCATED, RES_TIMEOUT, RES_OVERFLOW = 1, 2, 4, 8
RES_PREFIX_RANGE = 32
SLOT_PREFIX_MIN_LO, SLOT_PREFIX_MIN_HI, SLOT_PREFIX_MAX_LO, SLOT_PREFIX_MAX_HI = 12, 13, 14, 15
DEVICE_RESULT_BYTES = 128
SLOT_FSUM, SLOT_COUNT_F, SLOT_ISUM_LO, SLOT_ISUM_HI, SLOT_COUNT = 0, 1, 2, 3, 4
SLOT_FMIN, SLOT_FMAX, SLOT_IMIN, SLOT_IMAX, SLOT_FLAGS, SLOT_OFFSET, SLOT_LOCAL_COUNT, SLOT_NSLOTS = 5, 6, 7, 8, 9, 10, 11, 16
OPT_COMPACT_KERNEL, OPT_FORCE_SCALAR, OPT_BLOCKS_PER_SM, OPT_WITHHOLD_FIRST_COUNT, OPT_CACHE_MAX_ENTRIES, OPT_CACHE_ENTRIES, OPT_OVERLAP_LAUNCHES = 1, 2, 3, 4, 5, 6, 7


class Op(C.Structure):
    _fields_ = [("kind", C.c_int32), ("lambda_", C.c_char_p)]


class PipelineDesc(C.Structure):
    _fields_ = [("elem_type0", C.c_int32), ("elem_type1", C.c_int32), ("n_ops", C.c_int32),
                ("ops", C.POINTER(Op)), ("flags", C.c_uint32)]


class PipelineInfo(C.Structure):
    _fields_ = [("terminal", C.c_int32), ("out_type", C.c_int32), ("result_type", C.c_int32),
                ("has_filter", C.c_int32), ("n_inputs", C.c_int32), ("precompiled", C.c_int32),
                ("tile_elems", C.c_int64), ("compile_ms", C.c_double)]


class Result(C.Structure):
    _fields_ = [("count", C.c_int64), ("f64", C.c_double), ("i64", C.c_int64), ("u64", C.c_uint64),
                ("flags", C.c_uint32), ("launches", C.c_uint32), ("kernel_ms", C.c_float), ("total_ms", C.c_float)]


_vp, _i32, _i64, _sz, _u32 = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_uint32
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes). Every prototype of dcb200.h appears here; a test checks the two lists agree.
PROTOTYPES = {
    "dcb_status_class": (_i32, [_i32]),
    "dcb_status_name": (C.c_char_p, [_i32]),
    "dcb_abi_version": (_i32, []),
    "dcb_type_size": (_i32, [_i32]),
    "dcb_init": (_i32, [_i32, _pp]),
    "dcb_shutdown": (_i32, [_vp]),
    "dcb_last_error": (_i32, [_vp, C.c_char_p, _sz]),
    "dcb_device_count": (_i32, [C.POINTER(_i32)]),
    "dcb_device_info": (_i32, [_vp, C.c_char_p, _sz, C.POINTER(_i32), C.POINTER(_i64), C.POINTER(_i32), C.POINTER(_i32)]),
    "dcb_set_stream": (_i32, [_vp, _vp]),
    "dcb_stream_sync": (_i32, [_vp, _vp]),
    "dcb_set_spin_limit": (_i32, [_vp, _u32]),
    "dcb_set_option": (_i32, [_vp, _i32, _i64]),
    "dcb_get_option": (_i32, [_vp, _i32, C.POINTER(_i64)]),
    "dcb_alloc": (_i32, [_vp, _sz, _pp]),
    "dcb_free": (_i32, [_vp, _vp]),
    "dcb_buf_wrap": (_i32, [_vp, _vp, _sz, _pp]),
    "dcb_buf_slice": (_i32, [_vp, _vp, _sz, _sz, _pp]),
    "dcb_devptr": (_vp, [_vp]),
    "dcb_buf_bytes": (_sz, [_vp]),
    "dcb_h2d_async": (_i32, [_vp, _vp, _sz, _vp, _sz, _vp]),
    "dcb_d2h_async": (_i32, [_vp, _vp, _vp, _sz, _sz, _vp]),
    "dcb_d2d_async": (_i32, [_vp, _vp, _sz, _vp, _sz, _sz, _vp]),
    "dcb_fill_async": (_i32, [_vp, _vp, _sz, _vp, _i32, _sz, _vp]),
    "dcb_host_alloc_pinned": (_i32, [_vp, _sz, _pp]),
    "dcb_host_free_pinned": (_i32, [_vp, _vp]),
    "dcb_pin_host": (_i32, [_vp, _vp, _sz]),
    "dcb_unpin_host": (_i32, [_vp, _vp]),
    "dcb_memory_stats": (_i32, [_vp, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "dcb_translate_lambda": (_i32, [C.c_char_p, C.POINTER(_i32), _i32, C.c_char_p, _sz, C.POINTER(_i32), C.c_char_p, _sz]),
    "dcb_translate_kernel_method": (_i32, [C.c_char_p, C.c_char_p, _sz, C.POINTER(_sz), C.c_char_p, _sz, C.c_char_p, _sz]),
    "dcb_pipeline_compile": (_i32, [_vp, C.POINTER(PipelineDesc), _pp]),
    "dcb_pipeline_destroy": (_i32, [_vp]),
    "dcb_pipeline_info_get": (_i32, [_vp, C.POINTER(PipelineInfo)]),
    "dcb_pipeline_source": (_i32, [_vp, C.c_char_p, _sz, C.POINTER(_sz)]),
    "dcb_pipeline_generate_source": (_i32, [C.POINTER(PipelineDesc), C.c_char_p, _sz, C.POINTER(_sz), C.c_char_p, _sz]),
    "dcb_pipeline_run_async": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _vp]),
    "dcb_pipeline_run": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, C.POINTER(Result), _vp]),
    "dcb_pipeline_run_ex": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, _u32, C.POINTER(Result), _vp]),
    "dcb_result_finalize": (_i32, [_vp, _vp, C.POINTER(Result)]),
    "dcb_record_finalize": (_i32, [_i32, _i32, _vp, C.POINTER(Result)]),
    "dcb_pipeline_run_host": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, C.POINTER(Result)]),
    "dcb_pipeline_run_host_ex": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, _u32, C.POINTER(Result)]),
    "dcb_peer_area_create": (_i32, [_vp, _vp, _sz]),
    "dcb_peer_connect": (_i32, [_vp, _i32, _i32, _vp, _sz]),
    "dcb_peer_area_ptr": (_i32, [_vp, _pp, C.POINTER(_sz)]),
    "dcb_peer_connect_local": (_i32, [_vp, _i32, _i32, _pp]),
    "dcb_peer_exchange_async": (_i32, [_vp, _vp, _i32, _vp]),
    "dcb_peer_disconnect": (_i32, [_vp]),
    "dcb_sort_indices": (_i32, [_vp, _i32, _vp, _i64, _i32, _vp, _vp]),
    "dcb_sort_by_key": (_i32, [_vp, _i32, _vp, _i64, _i32, _i32, _vp, _vp, _vp]),
    "dcb_prefix_sum": (_i32, [_vp, _i32, _vp, _i64, _i32, _vp, _vp]),
    "dcb_gather": (_i32, [_vp, _i32, _vp, _vp, _i64, _vp, _vp]),
    "dcb_group_aggregate": (_i32, [_vp, _i32, _vp, _i32, _vp, _i64, _i32, _i64, _vp, _vp, _vp, _vp, C.POINTER(_i64), _vp]),
    "dcb_join_indices": (_i32, [_vp, _i32, _vp, _i64, _vp, _i64, _i32, _i64, _vp, _vp, C.POINTER(_i64), _vp]),
    "dcb_compact_noalloc": (_i32, [_i32, C.POINTER(PipelineDesc), _vp, _vp, _i64, _vp, _i64, _vp, _vp]),
    "dcb_kernel_compile": (_i32, [_vp, C.c_char_p, C.c_char_p, _pp]),
    "dcb_kernel_launch": (_i32, [_vp, C.POINTER(_u32), C.POINTER(_u32), _u32, _pp, _vp]),
    "dcb_kernel_destroy": (_i32, [_vp]),
    "dcb_event_create": (_i32, [_vp, _pp]),
    "dcb_event_record": (_i32, [_vp, _vp, _vp]),
    "dcb_event_elapsed_ms": (_i32, [_vp, _vp, _vp, C.POINTER(C.c_float)]),
    "dcb_event_destroy": (_i32, [_vp, _vp]),
    "dcb_launch_count": (_i32, [_vp, C.POINTER(_i64)]),
}

_lib = None


def declared_symbols(header_path: str = HEADER_PATH):
    """Names of the functions include/dcb200.h declares (parsed from the header text)."""
    with open(header_path) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dcb_[a-z0-9_]+)\s*\(", text)))


def lib() -> C.CDLL:
    """Load libdcb200.so (once). Raises if it has not been built: there is no other implementation to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise errors.DotComputeException(
                f"{LIB_PATH} is missing: build it with `python -m dotcompute_b200.build` (needs nvcc); "
                "this package has no CPU or PyTorch fallback")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error(ctx=None) -> str:
    buf = C.create_string_buffer(1024)
    lib().dcb_last_error(ctx, buf, len(buf))
    return buf.value.decode("utf-8", "replace")


def check(status: int, ctx=None) -> None:
    """Raise the managed-side exception that corresponds to a non-zero status."""
    if status != 0:
        raise errors.from_status(status, last_error(ctx), lib().dcb_status_name(status).decode())
