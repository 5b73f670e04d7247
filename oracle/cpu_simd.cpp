// cpu_simd.cpp — TEST / BENCH INFRASTRUCTURE ONLY: C++ restatement of the reference's CPU SIMD backend loops,
// used as the timed CPU baseline ("port") next to the GPU numbers. The product never calls it.
//
// The reference's CPU backend is C# (System.Runtime.Intrinsics) and cannot run without a .NET runtime, so its
// loops are restated with the same shapes:
//   * partitioning: Parallel.For over Environment.ProcessorCount contiguous partitions, the last one taking the
//     remainder (src/Backends/DotCompute.Backends.CPU/Kernels/Optimized/OptimizedReductionKernel.cs:69-95,
//     src/Backends/DotCompute.Backends.CPU/Kernels/Simd/SimdHorizontalOperations.cs:462-575)
//   * Sum: per-thread fp32 vector lanes (AVX-512 16 lanes / AVX2 8 lanes), horizontal add, scalar tail, per-thread
//     result kept as double, partials added in partition order, cast to float
//     (SimdHorizontalOperations.cs:483-575; src/Backends/DotCompute.Backends.CPU/Kernels/Simd/SimdVectorOperations.cs:298-420)
//   * fused Where -> Select: vector compare to a mask, then the surviving lanes handled one by one, scalar remainder
//     (src/Extensions/DotCompute.Linq/CodeGeneration/CpuKernelGenerator.cs:1266-1334); with a Sum terminal the lanes are
//     added instead of stored (CpuKernelGenerator.cs:362-454)
// plus a one-thread scalar loop, which is what the shipped provider actually runs for these queries (System.Linq on
// one thread, src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:240-267).
#include <immintrin.h>

#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

namespace {

template <class F>
void parallel_for(int parts, F&& f) {
    std::vector<std::thread> th;
    th.reserve(parts > 0 ? parts - 1 : 0);
    for (int p = 1; p < parts; ++p) th.emplace_back([&, p] { f(p); });
    f(0);
    for (auto& t : th) t.join();
}

inline float hsum256(__m256 v) {
    __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
    lo = _mm_add_ps(lo, hi);
    lo = _mm_hadd_ps(lo, lo);
    lo = _mm_hadd_ps(lo, lo);
    return _mm_cvtss_f32(lo);
}

// One partition of Where(x > thr).Select(x*x + c).Sum(): vector mask, masked lanes accumulate in fp32 lanes.
double part_where_select_sum(const float* in, int64_t start, int64_t end, float thr, float c) {
    int64_t i = start;
    double tail = 0.0;
#if defined(__AVX512F__)
    __m512 acc = _mm512_setzero_ps();
    const __m512 vthr = _mm512_set1_ps(thr), vc = _mm512_set1_ps(c);
    for (; i + 16 <= end; i += 16) {
        __m512 x = _mm512_loadu_ps(in + i);
        __mmask16 m = _mm512_cmp_ps_mask(x, vthr, _CMP_GT_OQ);
        __m512 v = _mm512_add_ps(_mm512_mul_ps(x, x), vc);
        acc = _mm512_mask_add_ps(acc, m, acc, v);
    }
    double s = (double)_mm512_reduce_add_ps(acc);
#elif defined(__AVX2__)
    __m256 acc = _mm256_setzero_ps();
    const __m256 vthr = _mm256_set1_ps(thr), vc = _mm256_set1_ps(c);
    for (; i + 8 <= end; i += 8) {
        __m256 x = _mm256_loadu_ps(in + i);
        __m256 m = _mm256_cmp_ps(x, vthr, _CMP_GT_OQ);
        __m256 v = _mm256_add_ps(_mm256_mul_ps(x, x), vc);
        acc = _mm256_add_ps(acc, _mm256_and_ps(v, m));
    }
    double s = (double)hsum256(acc);
#else
    double s = 0.0;
#endif
    for (; i < end; ++i) { float x = in[i]; if (x > thr) tail += (double)(x * x + c); }
    return s + tail;
}

double part_sum(const float* in, int64_t start, int64_t end) {
    int64_t i = start;
#if defined(__AVX512F__)
    __m512 acc = _mm512_setzero_ps();
    for (; i + 16 <= end; i += 16) acc = _mm512_add_ps(acc, _mm512_loadu_ps(in + i));
    double s = (double)_mm512_reduce_add_ps(acc);
#elif defined(__AVX2__)
    __m256 acc = _mm256_setzero_ps();
    for (; i + 8 <= end; i += 8) acc = _mm256_add_ps(acc, _mm256_loadu_ps(in + i));
    double s = (double)hsum256(acc);
#else
    double s = 0.0;
#endif
    for (; i < end; ++i) s += (double)in[i];
    return s;
}

}  // namespace

extern "C" {

int cpu_simd_threads() { return (int)std::max(1u, std::thread::hardware_concurrency()); }

int cpu_simd_width() {
#if defined(__AVX512F__)
    return 16;
#elif defined(__AVX2__)
    return 8;
#else
    return 1;
#endif
}

// ParallelTreeReduction shape (SimdHorizontalOperations.cs:462-575).
float cpu_simd_sum_f32(const float* in, int64_t n, int threads) {
    if (n == 0) return 0.f;
    threads = (int)std::max<int64_t>(1, std::min<int64_t>(threads, n / 32));
    std::vector<double> partial((size_t)threads, 0.0);
    const int64_t per = n / threads;
    parallel_for(threads, [&](int t) {
        const int64_t s = t * per, e = (t == threads - 1) ? n : s + per;
        partial[(size_t)t] = part_sum(in, s, e);
    });
    double total = 0.0;
    for (double p : partial) total += p;
    return (float)total;
}

// Fused Where -> Select -> Sum over partitions (CpuKernelGenerator.cs:1266-1334 + 362-454, partitioned as
// OptimizedReductionKernel.cs:69-95).
float cpu_simd_where_select_sum_f32(const float* in, int64_t n, float thr, float c, int threads) {
    if (n == 0) return 0.f;
    threads = (int)std::max<int64_t>(1, std::min<int64_t>(threads, n / 32));
    std::vector<double> partial((size_t)threads, 0.0);
    const int64_t per = n / threads;
    parallel_for(threads, [&](int t) {
        const int64_t s = t * per, e = (t == threads - 1) ? n : s + per;
        partial[(size_t)t] = part_where_select_sum(in, s, e, thr, c);
    });
    double total = 0.0;
    for (double p : partial) total += p;
    return (float)total;
}

// Fused Where -> Select -> ToArray: each partition compacts into its own slice (mask, then lane by lane), slices are
// concatenated in partition order. Returns the survivor count. `out` needs room for n elements.
int64_t cpu_simd_where_select_toarray_f32(const float* in, int64_t n, float thr, float c, float* out, int threads) {
    if (n == 0) return 0;
    threads = (int)std::max<int64_t>(1, std::min<int64_t>(threads, n / 32));
    std::vector<int64_t> counts((size_t)threads, 0);
    std::vector<std::vector<float>> tmp((size_t)threads);
    const int64_t per = n / threads;
    parallel_for(threads, [&](int t) {
        const int64_t s = t * per, e = (t == threads - 1) ? n : s + per;
        std::vector<float>& v = tmp[(size_t)t];
        v.resize((size_t)(e - s));
        int64_t k = 0;
        for (int64_t i = s; i < e; ++i) { float x = in[i]; if (x > thr) v[(size_t)k++] = x * x + c; }
        counts[(size_t)t] = k;
    });
    int64_t off = 0;
    for (int t = 0; t < threads; ++t) {
        std::copy(tmp[(size_t)t].begin(), tmp[(size_t)t].begin() + counts[(size_t)t], out + off);
        off += counts[(size_t)t];
    }
    return off;
}

// What the shipped provider runs today: one thread, scalar, double accumulator.
float cpu_scalar_where_select_sum_f32(const float* in, int64_t n, float thr, float c) {
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) { float x = in[i]; if (x > thr) s += (double)(x * x + c); }
    return (float)s;
}

}  // extern "C"
