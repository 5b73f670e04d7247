"""The C ABI without a GPU: the library loads, exports every function include/dcb200.h declares, the Python prototype
table covers the same set, and the host-only entry points (status helpers, translator, generator, finalizer) work."""
import ctypes as C

import numpy as np
import pytest

from dotcompute_b200 import (NotSupportedException, InvalidOperationException, OverflowException, generate_source,
                             native as N, translate_lambda)
from dotcompute_b200.sharded import finalize_record


def test_library_exports_every_declared_symbol(built_library):
    lib = C.CDLL(built_library)
    declared = N.declared_symbols()
    assert len(declared) >= 45
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in dcb200.h but not exported"
    assert sorted(N.PROTOTYPES) == declared, "native.PROTOTYPES and dcb200.h disagree"


def test_status_helpers(built_library):
    L = N.lib()
    assert L.dcb_abi_version() == 1
    assert L.dcb_status_class(0) == 0 and L.dcb_status_class(102) == 1 and L.dcb_status_class(201) == 2
    assert L.dcb_status_class(302) == 3 and L.dcb_status_class(402) == 4 and L.dcb_status_class(501) == 5
    assert L.dcb_status_name(502) == b"DCB_ERR_OVERFLOW"
    assert [L.dcb_type_size(t) for t in range(1, 12)] == [1, 1, 2, 2, 4, 4, 8, 8, 4, 8, 1]


def test_no_gpu_means_an_error_not_a_fallback(built_library):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    ctx = C.c_void_p()
    st = N.lib().dcb_init(0, C.byref(ctx))
    assert st == 401 and not ctx.value            # DCB_ERR_NO_DEVICE: nothing computes on the host instead


@pytest.mark.parametrize("lam,types,code,rtype", [
    ("x => x * 2f + 1f", [np.float32], "((p0 * 2.0f) + 1.0f)", np.float32),
    ("x => x * x + 3f", [np.float32], "((p0 * p0) + 3.0f)", np.float32),
    ("k => (k & 0xF) == 3", [np.int64], "((p0 & ((long long)(15))) == ((long long)(3)))", np.bool_),
    ("(x, y) => x * y", [np.float32, np.float32], "(p0 * p1)", np.float32),
    ("(float a, float b) => a + b", [np.float32, np.float32], "(p0 + p1)", np.float32),
    ("x => x / 2", [np.int32], "(p0 / 2)", np.int32),
    ("x => x & 0xFF", [np.uint32], "(p0 & ((unsigned int)(255)))", np.uint32),
    ("x => x >> 3", [np.int64], "(p0 >> (((int)(3)) & 63))", np.int64),
])
def test_translate_lambda_text(lam, types, code, rtype):
    got, rt = translate_lambda(lam, *types)
    assert got == code and rt == np.dtype(rtype)


@pytest.mark.parametrize("lam,types,rtype", [
    ("x => x + 1", [np.uint8], np.int32),             # byte + int -> int
    ("x => x + 1", [np.int16], np.int32),
    ("x => x + 1u", [np.int32], np.int64),            # int + uint -> long
    ("x => x + 1", [np.uint32], np.uint32),           # uint + constant int that fits -> uint
    ("x => x + 1L", [np.int32], np.int64),
    ("x => x * 0.5", [np.float32], np.float64),       # float * double literal -> double
    ("x => x * 0.5f", [np.int64], np.float32),        # long * float -> float
    ("x => -x", [np.uint32], np.int64),
    ("x => ~x", [np.uint8], np.int32),
    ("x => x << 2", [np.uint8], np.int32),
    ("x => x > 1 ? x : 0", [np.int16], np.int16),     # ?: with a constant that fits keeps short
    ("x => x > 1 ? 1.0f : 2.0", [np.int32], np.float64),
    ("x => Math.Sqrt(x)", [np.float32], np.float64),
    ("x => MathF.Sqrt(x)", [np.float32], np.float32),
    ("x => Math.Abs(x)", [np.uint8], np.int16),       # byte -> Abs(short)
    ("x => Math.Max(x, 0)", [np.int32], np.int32),
    ("x => Math.Sign(x)", [np.float64], np.int32),
    ("x => (byte)(x * 2)", [np.int32], np.uint8),
    ("x => x == 3 || !(x < 10)", [np.int32], np.bool_),
    ("x => float.IsNaN(x)", [np.float32], np.bool_),
    ("x => x * Math.PI", [np.float32], np.float64),
    ("x => x + int.MaxValue", [np.int32], np.int32),
    ("x => 1_000 + 0b101 + 0x10 + x", [np.int32], np.int32),
    ("x => x >>> 1", [np.int32], np.int32),
])
def test_translate_lambda_result_types_follow_csharp(lam, types, rtype):
    _, rt = translate_lambda(lam, *types)
    assert rt == np.dtype(rtype), lam


@pytest.mark.parametrize("lam,types", [
    ("x => x.ToString()", [np.int32]),
    ("x => x * 1.5m", [np.float32]),
    ("x => DateTime.Now.Ticks + x", [np.int64]),
    ("x => Guid.NewGuid()", [np.int32]),
    ("x => captured + x", [np.int32]),
    ("x => x + ", [np.int32]),
    ("x => x & 1.5f", [np.int32]),
    ("x => -x", [np.uint64]),
    ("x => x + 1", [np.bool_]),
    ("x x", [np.int32]),
    ("(x, y) => x", [np.int32]),
    ("x => x ? 1 : 2", [np.int32]),
])
def test_untranslatable_lambdas_are_not_supported(lam, types):
    with pytest.raises(NotSupportedException):
        translate_lambda(lam, *types)


def test_generated_source_shape():
    src = generate_source(np.float32, [(N.OP_WHERE, "x => x > 0.5f"), (N.OP_SELECT, "x => x * x + 3f"), (N.OP_SUM, None)])
    assert "struct dcb_chain" in src and "keep = keep & (p0 > 0.5f);" in src
    assert "dcb::reduce_body<dcb_chain, 1, 256, 4, true>" in src and 'extern "C" __global__' in src
    assert "atomicAdd" not in src                       # no float atomics: reductions are deterministic
    src = generate_source(np.int64, [(N.OP_WHERE, "k => (k & 0xF) == 3"), (N.OP_TOARRAY, None)])
    assert "dcb::compact_body<dcb_chain" in src and "typedef long long in0_t" in src
    src = generate_source(np.float32, [(N.OP_ZIP, "(x, y) => x * y"), (N.OP_SUM, None)], np.float32)
    assert "static constexpr int n_in = 2;" in src
    src = generate_source(np.float32, [(N.OP_SELECT, "x => x * 2f + 1f"), (N.OP_TOARRAY, None)])
    assert "dcb::map_body<dcb_chain" in src
    # two different lambdas of the same shape must give different cache keys (the reference's key ignores the lambda)
    a = generate_source(np.float32, [(N.OP_SELECT, "x => x * 2f"), (N.OP_TOARRAY, None)])
    b = generate_source(np.float32, [(N.OP_SELECT, "x => x * 3f"), (N.OP_TOARRAY, None)])
    assert a.splitlines()[1] != b.splitlines()[1] and a.splitlines()[1].startswith("// key:")


def test_streamed_compaction_kernel_is_generated_where_it_applies():
    """The persistent, bulk-copy fed compaction kernel stages survivors over the input it has read, so it exists only
    for queries whose output element is no wider than the first input's; every compaction query keeps the
    one-tile-per-block kernels (vector and scalar) as the route for everything else."""
    src = generate_source(np.int64, [(N.OP_WHERE, "k => (k & 0xF) == 3"), (N.OP_TOARRAY, None)])
    assert "dcb::compact_stream_body<dcb_chain, 4, 10, 3, 5, 3, " in src and "__launch_bounds__(256, 2) dcb_compact_stream(" in src
    assert "dcb_compact_vec(" in src and "dcb_compact_scalar(" in src
    src = generate_source(np.float32, [(N.OP_ZIP, "(x, y) => x * y"), (N.OP_WHERE, "v => v > 0f"), (N.OP_TOARRAY, None)], np.float32)
    assert "dcb::compact_stream_body<dcb_chain, 4, 5, 3, 5, 3, " in src          # two inputs: half the rows, same bytes per slot
    src = generate_source(np.int32, [(N.OP_WHERE, "x => x > 7"), (N.OP_SELECT, "x => (long)x * 3L"), (N.OP_TOARRAY, None)])
    assert "compact_stream_body" not in src and "dcb_compact_vec(" in src     # widening Select: no in-place staging
    src = generate_source(np.float32, [(N.OP_WHERE, "x => x > 0.5f"), (N.OP_SUM, None)])
    assert "compact_stream_body" not in src and "dcb_reduce_vec(" in src


def test_operator_order_rules():
    with pytest.raises(NotSupportedException):
        generate_source(np.float32, [(N.OP_SELECT, "x => x"), (N.OP_ZIP, "(x, y) => x * y"), (N.OP_SUM, None)], np.float32)
    with pytest.raises(NotSupportedException):
        generate_source(np.uint8, [(N.OP_SUM, None)])                 # Sum(byte) does not exist in System.Linq
    with pytest.raises(NotSupportedException):
        generate_source(np.float32, [(N.OP_WHERE, "x => x + 1f"), (N.OP_TOARRAY, None)])   # predicate must be bool
    generate_source(np.uint8, [(N.OP_SELECT, "x => (int)x"), (N.OP_SUM, None)])


def _record(**slots):
    rec = np.zeros(16, dtype=np.int64)
    f = rec.view(np.float64)
    for k, v in slots.items():
        idx = getattr(N, "SLOT_" + k)
        if k in ("FSUM", "COUNT_F", "FMIN", "FMAX"):
            f[idx] = v
        else:
            rec[idx] = v
    return rec


def test_record_finalize_semantics():
    r = finalize_record(_record(FSUM=1.0 + 2**-30, COUNT=4), N.OP_SUM, N.T_F32)
    assert r.f64 == 1.0                                   # one rounding to float
    r = finalize_record(_record(FSUM=10.0, COUNT=4), N.OP_AVERAGE, N.T_F64)
    assert r.f64 == 2.5
    with pytest.raises(InvalidOperationException):
        finalize_record(_record(COUNT=0), N.OP_AVERAGE, N.T_F32)
    with pytest.raises(InvalidOperationException):
        finalize_record(_record(COUNT=0), N.OP_MIN, N.T_I32)
    assert finalize_record(_record(COUNT=0), N.OP_SUM, N.T_I32).i64 == 0     # Sum of nothing is 0
    with pytest.raises(OverflowException):
        finalize_record(_record(ISUM_LO=2**31, ISUM_HI=0), N.OP_SUM, N.T_I32)
    assert finalize_record(_record(ISUM_LO=2**31, ISUM_HI=0), N.OP_SUM, N.T_I64).i64 == 2**31
    with pytest.raises(OverflowException):
        finalize_record(_record(ISUM_LO=5, ISUM_HI=1), N.OP_SUM, N.T_I64)
    assert finalize_record(_record(ISUM_LO=7, COUNT=2), N.OP_AVERAGE, N.T_I32).f64 == 3.5
    nanrec = _record(FMIN=-2.0, FMAX=7.5, COUNT=4, FLAGS=1 | 16)
    assert np.isnan(finalize_record(nanrec, N.OP_MIN, N.T_F32).f64)
    assert finalize_record(nanrec, N.OP_MAX, N.T_F32).f64 == 7.5
    assert np.isnan(finalize_record(_record(COUNT=2, FLAGS=1), N.OP_MAX, N.T_F32).f64)
