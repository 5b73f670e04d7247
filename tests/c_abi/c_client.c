/* A plain C client of libdcb200.so: what a non-Python host does through the C ABI. Builds with
 *   gcc -std=c99 -I include tests/c_abi/c_client.c -L dotcompute_b200 -ldcb200 -lm
 * Runs Where(x => x > 0.5f).Select(x => x * x + 3f) as ToArray and as Sum over a small seeded array, checks both against a
 * loop written here (separate multiply and add, double accumulation), and prints "c_client ok". Exit code 0 on success. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "dcb200.h"

#define CHECK(call)                                                                   \
    do {                                                                              \
        dcb_status st_ = (call);                                                      \
        if (st_ != DCB_OK) {                                                          \
            char msg[512];                                                            \
            dcb_last_error(ctx, msg, sizeof msg);                                     \
            fprintf(stderr, "%s -> %s: %s\n", #call, dcb_status_name(st_), msg);      \
            return 1;                                                                 \
        }                                                                             \
    } while (0)

int main(void) {
    dcb_ctx* ctx = NULL;
    const int64_t n = 1000003;
    float* x = (float*)malloc(sizeof(float) * (size_t)n);
    float* got = (float*)malloc(sizeof(float) * (size_t)n);
    float* want = (float*)malloc(sizeof(float) * (size_t)n);
    unsigned int s = 12345u;
    int64_t i, k = 0;
    double acc = 0.0;
    dcb_op ops_arr[3], ops_sum[3];
    dcb_pipeline_desc d_arr, d_sum;
    dcb_pipeline *p_arr = NULL, *p_sum = NULL;
    dcb_result r;

    for (i = 0; i < n; ++i) { s = s * 1664525u + 1013904223u; x[i] = (float)(s >> 8) * (1.0f / 16777216.0f); }
    for (i = 0; i < n; ++i) {
        if (x[i] > 0.5f) { volatile float t = x[i] * x[i]; float v = t + 3.0f; want[k++] = v; acc += (double)v; }
    }

    CHECK(dcb_init(0, &ctx));
    ops_arr[0].kind = DCB_OP_WHERE;  ops_arr[0].lambda = "x => x > 0.5f";
    ops_arr[1].kind = DCB_OP_SELECT; ops_arr[1].lambda = "x => x * x + 3f";
    ops_arr[2].kind = DCB_OP_TOARRAY; ops_arr[2].lambda = NULL;
    memcpy(ops_sum, ops_arr, sizeof ops_arr);
    ops_sum[2].kind = DCB_OP_SUM;
    d_arr.elem_type0 = DCB_T_F32; d_arr.elem_type1 = DCB_T_NONE; d_arr.n_ops = 3; d_arr.ops = ops_arr; d_arr.flags = 0;
    d_sum = d_arr; d_sum.ops = ops_sum;
    CHECK(dcb_pipeline_compile(ctx, &d_arr, &p_arr));
    CHECK(dcb_pipeline_compile(ctx, &d_sum, &p_sum));

    CHECK(dcb_pipeline_run_host(p_arr, x, NULL, n, got, n, &r));
    if (r.count != k || memcmp(got, want, sizeof(float) * (size_t)k) != 0) { fprintf(stderr, "ToArray differs (%lld vs %lld)\n", (long long)r.count, (long long)k); return 1; }
    CHECK(dcb_pipeline_run_host(p_sum, x, NULL, n, NULL, 0, &r));
    if ((float)r.f64 != (float)acc) { fprintf(stderr, "Sum differs: %.9g vs %.9g\n", r.f64, (double)(float)acc); return 1; }

    CHECK(dcb_shutdown(ctx));
    printf("c_client ok: %lld of %lld kept, sum %.9g\n", (long long)k, (long long)n, r.f64);
    free(x); free(got); free(want);
    return 0;
}
