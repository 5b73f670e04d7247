"""[Kernel] methods: the C# -> CUDA translator (no GPU) and IComputeOrchestrator.ExecuteAsync on the GPU.
The two kernels are the ones the reference's generator tests use
(tests/Unit/DotCompute.Generators.Tests/Generator/KernelExecutionMetadataTests.cs:20-35, 61-75)."""
import numpy as np
import pytest

from dotcompute_b200 import (ArgumentException, ComputeOrchestrator, KernelRegistry, NotSupportedException,
                             translate_kernel_method)

ADD = """
[Kernel(Backends = KernelBackends.CPU | KernelBackends.CUDA, VectorSize = 8, IsParallel = true)]
public static void Add(ReadOnlySpan<float> a, ReadOnlySpan<float> b, Span<float> c)
{
    int i = KernelContext.ThreadId.X;
    if (i < c.Length)
        c[i] = a[i] + b[i];
}"""

TRANSPOSE = """
[Kernel(Backends = KernelBackends.CPU | KernelBackends.CUDA, VectorSize = 8, IsParallel = true)]
public static void TransposeNaive(ReadOnlySpan<float> input, Span<float> output, int rows, int cols)
{
    int row = KernelContext.ThreadId.Y + KernelContext.BlockId.Y * KernelContext.BlockDim.Y;
    int col = KernelContext.ThreadId.X + KernelContext.BlockId.X * KernelContext.BlockDim.X;
    if (row < rows && col < cols)
        output[col * rows + row] = input[row * cols + col];
}"""

SAXPY = """
public static void Saxpy(Span<float> y, ReadOnlySpan<float> x, float a, int n)
{
    var i = Kernel.ThreadId.X;
    if (i >= n) { return; }
    for (int k = 0; k < 2; k++) { y[i] += a * x[i]; }
    for (int k = 0; k < 1; k++) { y[i] = y[i] + 1f; }
}"""


def test_vector_add_gets_an_implicit_length_parameter():
    reg = translate_kernel_method(ADD)
    assert reg.CudaEntryPoint == "Add" and reg.CudaNeedsLength and reg.Dimensions == 1
    assert "__global__ void Add(const float* a, const float* b, float* c, const unsigned int __length)" in reg.CudaSource
    assert "if ((i < ((int)__length)))" in reg.CudaSource
    assert [(p.Name, p.IsBuffer, p.IsReadOnly, p.ElementType) for p in reg.Parameters] == [
        ("a", True, True, "float"), ("b", True, True, "float"), ("c", True, False, "float")]
    # ThreadId alone is the global work-item index, as in the reference's CPU invoker
    assert "blockIdx.x * blockDim.x + threadIdx.x" in reg.CudaSource


def test_transpose_is_two_dimensional_and_keeps_block_arithmetic():
    reg = translate_kernel_method(TRANSPOSE)
    assert reg.Dimensions == 2 and not reg.CudaNeedsLength
    assert "__global__ void TransposeNaive(const float* input, float* output, int rows, int cols)" in reg.CudaSource
    assert "threadIdx.y" in reg.CudaSource and "blockIdx.y" in reg.CudaSource and "blockDim.y" in reg.CudaSource
    assert [p.IsBuffer for p in reg.Parameters] == [True, True, False, False]


@pytest.mark.parametrize("src", [
    "public static void K(Span<float> y) { y[0] = Math.Foo(1); }",
    "public static void K(Span<float> y) { y[0] = y; }",
    "public static void K(Span<float> y) { string s = \"x\"; }",
    "public static int K(Span<float> y) { return 1; }",
    "public static void K(List<float> y) { }",
    "public static void K(Span<float> y, int n) { n = 1.5f; }",
    "public static void K(ReadOnlySpan<float> y) { foreach (var v in y) { } }",
])
def test_unsupported_constructs_are_rejected(src):
    with pytest.raises(NotSupportedException):
        translate_kernel_method(src)


def test_launch_derivation_follows_the_reference():
    reg = translate_kernel_method(ADD)
    a, c = np.zeros(1000, np.float32), np.zeros(1000, np.float32)
    assert ComputeOrchestrator.DeriveWorkSize(reg, (a, a, c)) == 1000
    assert ComputeOrchestrator.DeriveLaunch(reg, (a, a, c), 1000) == ((4, 1, 1), (256, 1, 1))
    reg2 = translate_kernel_method(TRANSPOSE)
    inp, out = np.zeros(30 * 50, np.float32), np.zeros(30 * 50, np.float32)
    grid, block = ComputeOrchestrator.DeriveLaunch(reg2, (inp, out, 30, 50), 1500)
    assert block == (16, 16, 1) and grid == (4, 2, 1)          # x extent = last int (cols = 50), y = rows = 30


def test_unknown_kernel_and_bad_arguments():
    orch = ComputeOrchestrator(registry=KernelRegistry())
    orch.Registry.Register(ADD)
    with pytest.raises(ArgumentException):
        orch._resolve("Nope")
    assert not orch.ValidateKernelArgsAsync("Add", np.zeros(4, np.float32))
    assert not orch.ValidateKernelArgsAsync("Add", np.zeros(4, np.float64), np.zeros(4, np.float32), np.zeros(4, np.float32))
    assert orch.ValidateKernelArgsAsync("Add", np.zeros(4, np.float32), np.zeros(4, np.float32), np.zeros(4, np.float32))


@pytest.mark.gpu
def test_execute_async_on_gpu(acc):
    orch = ComputeOrchestrator(acc)
    for src in (ADD, TRANSPOSE, SAXPY):
        orch.Registry.Register(src)
    r = np.random.Generator(np.random.PCG64(1))
    a, b = r.random(100_003, dtype=np.float32), r.random(100_003, dtype=np.float32)
    c = np.zeros_like(a)
    out = orch.ExecuteAsync("Add", a, b, c)
    assert out is c and np.array_equal(c, a + b)                 # more than one block: ThreadId is global
    rows, cols = 37, 53
    m = r.random(rows * cols, dtype=np.float32)
    t = np.zeros_like(m)
    orch.ExecuteAsync("TransposeNaive", m, t, rows, cols)
    assert np.array_equal(t.reshape(cols, rows), m.reshape(rows, cols).T)
    y, x = r.random(5000, dtype=np.float32), r.random(5000, dtype=np.float32)
    want = y.copy()
    for _ in range(2):
        want = want + np.float32(1.5) * x
    want = want + np.float32(1)
    orch.ExecuteAsync("Saxpy", y, x, 1.5, 5000)
    assert np.array_equal(y, want)
    # device-resident buffers are used in place, nothing is copied back
    dy = acc.Memory.AllocateAndCopyAsync(np.zeros(1000, np.float32))
    orch.ExecuteAsync("Add", a[:1000].copy(), b[:1000].copy(), dy)
    assert np.array_equal(dy.ToArray(), a[:1000] + b[:1000])
    dy.Dispose()
    with pytest.raises(ArgumentException):
        orch.ExecuteAsync("Add", a, b)
    orch.Dispose()


def test_preferred_backend_is_a_wish():
    orch = ComputeOrchestrator.__new__(ComputeOrchestrator)     # no device needed for the argument check
    orch._disposed = False
    with pytest.raises(ArgumentException):
        orch.ExecuteAsync("Add", preferredBackend=3)
