"""Every kind of program the generator emits must compile under NVRTC for sm_100a. NVRTC needs no GPU, so this runs
on any machine that has the CUDA toolkit's Python bindings; it catches a template or translator change that would only
fail at the first JIT compilation on a GPU box otherwise (the ahead-of-time table covers the listed queries only).
"""
import os

import numpy as np
import pytest

from dotcompute_b200 import generate_source, native as N

nvrtc = pytest.importorskip("cuda.bindings.nvrtc")

HEADER = os.path.join(os.path.dirname(os.path.abspath(N.__file__)), "csrc", "dcb_kernels.cuh")

QUERIES = [
    ("map", np.float32, None, [(N.OP_SELECT, "x => MathF.Sqrt(x) * 2f + 1f"), (N.OP_TOARRAY, None)]),
    ("reduce-minmax-f64", np.float64, None, [(N.OP_WHERE, "x => x > 0.25"), (N.OP_MAX, None)]),
    ("reduce-sum-i32", np.int32, None, [(N.OP_SELECT, "x => x % 7"), (N.OP_SUM, None)]),
    ("reduce-sum-i64-checked", np.int64, None, [(N.OP_WHERE, "x => x != 0L"), (N.OP_SUM, None)]),
    ("reduce-sum-zip-i32-checked", np.int32, np.int32, [(N.OP_ZIP, "(a, b) => a * b"), (N.OP_SUM, None)]),
    ("reduce-sum-u8-to-i32-checked", np.uint8, None, [(N.OP_SELECT, "x => (int)x * 3"), (N.OP_SUM, None)]),
    ("zip-sum", np.float32, np.float32, [(N.OP_ZIP, "(a, b) => a * b"), (N.OP_SUM, None)]),
    ("compact-f32", np.float32, None, [(N.OP_WHERE, "x => x > 0.5f"), (N.OP_SELECT, "x => x * x + 3f"), (N.OP_TOARRAY, None)]),
    ("compact-i64", np.int64, None, [(N.OP_WHERE, "k => (k & 0xF) == 3"), (N.OP_TOARRAY, None)]),
    ("compact-zip", np.float32, np.int32, [(N.OP_ZIP, "(a, b) => a * b"), (N.OP_WHERE, "v => v > 0f"), (N.OP_TOARRAY, None)]),
    ("compact-u8", np.uint8, None, [(N.OP_WHERE, "x => x > 7"), (N.OP_TOARRAY, None)]),
    ("compact-widening", np.int32, None, [(N.OP_WHERE, "x => x > 7"), (N.OP_SELECT, "x => (long)x * 3L"), (N.OP_TOARRAY, None)]),
    ("count", np.uint16, None, [(N.OP_WHERE, "x => (x & 1) == 0"), (N.OP_COUNT, None)]),
]


def compile_for_sm100a(src: str, extra=()):
    err, prog = nvrtc.nvrtcCreateProgram(src.encode(), b"pipeline.cu", 0, [], [])
    assert err == nvrtc.nvrtcResult.NVRTC_SUCCESS
    opts = [b"--gpu-architecture=sm_100a", b"-std=c++17", b"-fmad=false", b"-default-device", *extra]
    (res,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    _, n = nvrtc.nvrtcGetProgramLogSize(prog)
    log = b" " * n
    nvrtc.nvrtcGetProgramLog(prog, log)
    nvrtc.nvrtcDestroyProgram(prog)
    return res, log.decode(errors="replace")


@pytest.mark.parametrize("name,dt0,dt1,ops", QUERIES, ids=[q[0] for q in QUERIES])
def test_generated_program_compiles(name, dt0, dt1, ops):
    with open(HEADER) as f:
        header = f.read()
    src = generate_source(dt0, ops, dt1)
    assert '#include "dcb_kernels.cuh"' in src
    res, log = compile_for_sm100a(src.replace('#include "dcb_kernels.cuh"', header))
    assert res == nvrtc.nvrtcResult.NVRTC_SUCCESS, log[:2000]


def test_pack_ranking_variant_still_compiles():
    """The build knob that switches the pipelined compaction kernel back to ranking by 16-byte packs."""
    with open(HEADER) as f:
        header = f.read()
    src = generate_source(np.float32, [(N.OP_WHERE, "x => x > 0.5f"), (N.OP_TOARRAY, None)])
    res, log = compile_for_sm100a(src.replace('#include "dcb_kernels.cuh"', header), extra=(b"-DDCB_PIPE_PACK_RANKS",))
    assert res == nvrtc.nvrtcResult.NVRTC_SUCCESS, log[:2000]


KERNEL_METHODS = {
    "add": """
public static void Add(ReadOnlySpan<float> a, ReadOnlySpan<float> b, Span<float> c)
{
    int i = KernelContext.ThreadId.X;
    if (i < c.Length)
        c[i] = a[i] + b[i];
}""",
    "transpose": """
public static void TransposeNaive(ReadOnlySpan<float> input, Span<float> output, int rows, int cols)
{
    int row = KernelContext.ThreadId.Y + KernelContext.BlockId.Y * KernelContext.BlockDim.Y;
    int col = KernelContext.ThreadId.X + KernelContext.BlockId.X * KernelContext.BlockDim.X;
    if (row < rows && col < cols)
        output[col * rows + row] = input[row * cols + col];
}""",
    "statements": """
public static void Mix(Span<double> y, ReadOnlySpan<int> k, double scale, int n)
{
    var i = Kernel.ThreadId.X;
    if (i >= n) { return; }
    double acc = 0.0;
    for (int j = 0; j < 4; j++) { acc += (double)k[i] * scale; }
    int t = k[i];
    while (t > 100) { t /= 2; }
    if (t < 0) { acc = -acc; } else if (t == 0) { acc = 1.0; } else { acc *= 2.0; }
    t++;
    t <<= 1;
    y[i] = acc + (t > 5 ? Math.Sqrt((double)t) : Math.Abs(acc));
}""",
}


@pytest.mark.parametrize("name", sorted(KERNEL_METHODS))
def test_translated_kernel_method_compiles(name):
    from dotcompute_b200 import translate_kernel_method
    reg = translate_kernel_method(KERNEL_METHODS[name])
    res, log = compile_for_sm100a(reg.CudaSource)
    assert res == nvrtc.nvrtcResult.NVRTC_SUCCESS, reg.CudaSource + "\n" + log[:2000]


def test_integer_sum_uses_the_ordered_kernel():
    """Sum over int / long must track the running sum in source order; Sum over float, and Average, must not."""
    assert "sum_checked_body" in generate_source(np.int32, [(N.OP_SUM, None)])
    assert "sum_checked_body" in generate_source(np.int64, [(N.OP_SELECT, "x => x + 1L"), (N.OP_SUM, None)])
    assert "sum_checked_body" not in generate_source(np.float32, [(N.OP_SUM, None)])
    assert "sum_checked_body" not in generate_source(np.int32, [(N.OP_AVERAGE, None)])


def test_integer_division_is_checked_only_where_the_divisor_can_be_zero():
    """C# throws on x / 0 and on int.MinValue / -1: a division whose divisor is not a non-zero constant goes through the
    helper that records either; constant divisors and floating division stay plain; such a program still compiles."""
    assert "dcb_idiv<int>" in generate_source(np.int32, [(N.OP_SELECT, "x => 100 / x"), (N.OP_TOARRAY, None)])
    assert "dcb_irem<long long>" in generate_source(np.int64, [(N.OP_WHERE, "k => k % (k >> 3) == 0L"), (N.OP_COUNT, None)])
    assert "dcb_idiv<" not in generate_source(np.int32, [(N.OP_SELECT, "x => x / 7 + x % 3"), (N.OP_TOARRAY, None)])
    assert "dcb_idiv<" not in generate_source(np.float32, [(N.OP_SELECT, "x => 1f / x"), (N.OP_TOARRAY, None)])
    with open(HEADER) as f:
        header = f.read()
    for ops, second in (([(N.OP_ZIP, "(a, b) => a / b + a % b"), (N.OP_WHERE, "v => v != 0"), (N.OP_SUM, None)], np.int32),
                        ([(N.OP_SELECT, "x => 100 / x"), (N.OP_TOARRAY, None)], None)):          # with and without a filter
        src = generate_source(np.int32, ops, second)
        res, log = compile_for_sm100a(src.replace('#include "dcb_kernels.cuh"', header))
        assert res == nvrtc.nvrtcResult.NVRTC_SUCCESS, log[:2000]
