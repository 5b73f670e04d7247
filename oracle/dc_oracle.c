/*
 * dc_oracle.c — TEST INFRASTRUCTURE ONLY. CPU restatement of what DotCompute computes for the LINQ hot path.
 *
 * Nothing in the product (dotcompute_b200/, libdcb200.so) may call, link or import this file; it is the checker
 * the tests and bench.py's cpu_baseline leg compare the CUDA path against.
 *
 * What is restated. For AsComputeQueryable() queries over unmanaged element types the reference ends in
 * System.Linq: collection results go through ExecuteFallback<T>
 * (src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:344-352, 628-633) and scalar results through
 * Expression.Lambda(expr).Compile().DynamicInvoke() (ComputeQueryableExtensions.cs:240-267). So the observable
 * arithmetic is that of System.Linq.Enumerable in the .NET 10 BCL (SDK 10.0.0 per global.json:3), a dependency
 * whose source is NOT in the reference tree. Its published behaviour is restated here:
 *   Select      one IEEE operation per C# operator, in the lambda's own type, no FMA contraction
 *   Where       keeps the surviving elements in source order
 *   Zip         pairs by index up to the shorter length
 *   Sum(float)  accumulates sequentially in double, rounds once to float; Sum(double) sequential in double
 *   Sum(int)    checked: leaving the int range at any prefix throws OverflowException; Sum(long) likewise
 *   Average     Sum (double / checked long) divided by the count; float result rounded once
 *   Min/Max     sequential compare; empty sequence throws; for float Min any NaN gives NaN, Max ignores NaN
 *               unless every element is NaN
 * Pinning: the functions below are checked against the reference's own test fixtures (tests/golden/, taken from
 * tests/Unit/DotCompute.Linq.Tests/ComputeQueryProviderTests.cs:340-366,560-613,
 * tests/Integration/DotCompute.Linq.Integration.Tests/RuntimeOrchestrationTests.cs:112-209 and
 * tests/Integration/DotCompute.Linq.Tests/CpuIntegrationTests.cs:490-581). Zip, Min, Max, Average, float Sum order,
 * NaN handling and int64 predicates have no reference test: for those, parity is unpinned.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC (see Makefile). -ffp-contract=off matters: a
 * contracted x*x+3 would round differently from the C# lambda.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>

#define ORACLE_OK 0
#define ORACLE_EMPTY 501     /* InvalidOperationException: sequence contains no elements */
#define ORACLE_OVERFLOW 502  /* OverflowException */

/* ---- Select: x => x * a + b (config 1: a = 2f, b = 1f; CpuIntegrationTests.cs:544-561) */
void oracle_select_mul_add_f32(const float* in, int64_t n, float a, float b, float* out) {
    for (int64_t i = 0; i < n; ++i) { float t = in[i] * a; out[i] = t + b; }
}

/* ---- Where(x => x > thr).Select(x => x * x + c).ToArray()  (config 3). Returns the survivor count. */
int64_t oracle_where_gt_select_sq_add_f32(const float* in, int64_t n, float thr, float c, float* out) {
    int64_t k = 0;
    for (int64_t i = 0; i < n; ++i) {
        float x = in[i];
        if (x > thr) { float t = x * x; out[k++] = t + c; }
    }
    return k;
}

/* ---- Where(x => x > thr).Select(x => x * x + c).Sum(): Enumerable.Sum(IEnumerable<float>) accumulates in double. */
float oracle_where_gt_select_sq_add_sum_f32(const float* in, int64_t n, float thr, float c, double* raw_sum, int64_t* count) {
    double s = 0.0; int64_t k = 0;
    for (int64_t i = 0; i < n; ++i) {
        float x = in[i];
        if (x > thr) { float t = x * x; float v = t + c; s += (double)v; ++k; }
    }
    if (raw_sum) *raw_sum = s;
    if (count) *count = k;
    return (float)s;
}

/* ---- plain reductions over float (config 2) */
float oracle_sum_f32(const float* in, int64_t n, double* raw_sum) {
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += (double)in[i];
    if (raw_sum) *raw_sum = s;
    return (float)s;
}
double oracle_sum_abs_f64(const float* in, int64_t n) {   /* the tolerance scale: sum of |x| in fp64 */
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += fabs((double)in[i]);
    return s;
}
int oracle_average_f32(const float* in, int64_t n, float* out) {
    if (n == 0) return ORACLE_EMPTY;
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += (double)in[i];
    *out = (float)(s / (double)n);
    return ORACLE_OK;
}
int oracle_min_f32(const float* in, int64_t n, float* out) {
    if (n == 0) return ORACLE_EMPTY;
    float v = in[0];
    if (isnan(v)) { *out = v; return ORACLE_OK; }
    for (int64_t i = 1; i < n; ++i) {
        float x = in[i];
        if (x < v) v = x;
        else if (isnan(x)) { *out = x; return ORACLE_OK; }
    }
    *out = v;
    return ORACLE_OK;
}
int oracle_max_f32(const float* in, int64_t n, float* out) {
    if (n == 0) return ORACLE_EMPTY;
    int64_t i = 0;
    float v = in[0];
    while (isnan(v)) { if (++i >= n) { *out = v; return ORACLE_OK; } v = in[i]; }
    for (; i < n; ++i) if (in[i] > v) v = in[i];
    *out = v;
    return ORACLE_OK;
}

/* ---- int reductions (config 2): Sum is checked */
int oracle_sum_i32(const int32_t* in, int64_t n, int32_t* out) {
    int64_t s = 0;
    for (int64_t i = 0; i < n; ++i) {
        s += in[i];
        if (s > INT32_MAX || s < INT32_MIN) return ORACLE_OVERFLOW;
    }
    *out = (int32_t)s;
    return ORACLE_OK;
}
int oracle_min_i32(const int32_t* in, int64_t n, int32_t* out) {
    if (n == 0) return ORACLE_EMPTY;
    int32_t v = in[0];
    for (int64_t i = 1; i < n; ++i) if (in[i] < v) v = in[i];
    *out = v;
    return ORACLE_OK;
}
int oracle_max_i32(const int32_t* in, int64_t n, int32_t* out) {
    if (n == 0) return ORACLE_EMPTY;
    int32_t v = in[0];
    for (int64_t i = 1; i < n; ++i) if (in[i] > v) v = in[i];
    *out = v;
    return ORACLE_OK;
}
int oracle_average_i32(const int32_t* in, int64_t n, double* out) {   /* Average(int) returns double */
    if (n == 0) return ORACLE_EMPTY;
    int64_t s = 0;
    for (int64_t i = 0; i < n; ++i) s += in[i];
    *out = (double)s / (double)n;
    return ORACLE_OK;
}

/* ---- a.Zip(b, (x, y) => x * y).Sum()  (config 4) */
float oracle_zip_mul_sum_f32(const float* a, const float* b, int64_t n, double* raw_sum, double* sum_abs) {
    double s = 0.0, sa = 0.0;
    for (int64_t i = 0; i < n; ++i) { float p = a[i] * b[i]; s += (double)p; sa += fabs((double)p); }
    if (raw_sum) *raw_sum = s;
    if (sum_abs) *sum_abs = sa;
    return (float)s;
}

/* ---- keys.Where(k => (k & mask) == val).ToArray() over long  (config 4) */
int64_t oracle_where_mask_eq_i64(const int64_t* in, int64_t n, int64_t mask, int64_t val, int64_t* out) {
    int64_t k = 0;
    for (int64_t i = 0; i < n; ++i) if ((in[i] & mask) == val) out[k++] = in[i];
    return k;
}

/* ---- order-independent fingerprints for full-size checks (sum of elements mod 2^64 and a position-weighted sum) */
void oracle_fingerprint_u32(const uint32_t* in, int64_t n, uint64_t* plain, uint64_t* weighted) {
    uint64_t p = 0, w = 0;
    for (int64_t i = 0; i < n; ++i) { p += in[i]; w += (uint64_t)in[i] * (uint64_t)(i + 1); }
    *plain = p; *weighted = w;
}
