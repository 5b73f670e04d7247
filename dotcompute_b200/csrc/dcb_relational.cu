// dcb_relational.cu — multi-block OrderBy, GroupBy-with-aggregate and Join for the LINQ surface (see include/dcb200.h).
//
// The reference has generators for these three operators whose kernels are single-block or direct-index
// (src/Extensions/DotCompute.Linq/CodeGeneration/CudaKernelGenerator.cs:613-751 OrderBy, :753-825 GroupBy, :827-900 Join;
// OrderByKernelGenerator.cs:108, GroupByKernelGenerator.cs:152, JoinKernelGenerator.cs:140-239) and whose CPU semantics
// are Array.Sort, a Dictionary in insertion order, and a hash probe (CpuKernelGenerator.cs:475-723). Here all three rest
// on one primitive, a stable least-significant-digit radix sort of (key, index) pairs over any number of blocks:
//
//   OrderBy   keys -> order-preserving unsigned bits -> stable sort -> permutation (the caller gathers the elements)
//   GroupBy   stable sort by key; equal keys are then neighbours in source order: head flags -> group ids (a scan) ->
//             one warp-aggregated atomic per (warp, group); groups are emitted in order of first occurrence, which is
//             what enumerating a Dictionary gives
//   Join      stable sort of the inner keys; every outer element finds its run of equal keys by binary search; counts ->
//             scan -> pairs written in (outer index, inner index) order, the order of Enumerable.Join
//
// Key selectors and result selectors are ordinary fused Select / Zip pipelines run by the caller; the kernels here are
// fixed-function and compiled ahead of time. All streaming kernels are HBM-bound; a radix pass reads the keys twice
// (tile histogram, scatter) and moves key and index once: 4 B + 8 B + 8 B per element and pass for 32-bit keys.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/dcb200.h"
#include "dcb_internal.h"

namespace {

typedef unsigned int u32;
typedef unsigned long long u64;
typedef long long i64;

constexpr int kThreads = 256;
constexpr int kItems = 16;                       // elements per thread and tile in the sort kernels
constexpr int kTile = kThreads * kItems;         // 4096
constexpr int kWarps = kThreads / 32;
constexpr int kScanItems = 16;
constexpr int kScanTile = kThreads * kScanItems;

#define RCU(call)                                                                                   \
    do {                                                                                            \
        cudaError_t e__ = (call);                                                                   \
        if (e__ != cudaSuccess) {                                                                   \
            char msg__[256];                                                                        \
            snprintf(msg__, sizeof msg__, "%s: %s", #call, cudaGetErrorString(e__));                \
            dcb_set_thread_error(msg__);                                                            \
            (void)cudaGetLastError();                                                               \
            return e__ == cudaErrorMemoryAllocation ? DCB_ERR_OUT_OF_MEMORY : DCB_ERR_CUDA;         \
        }                                                                                           \
    } while (0)

dcb_status bad(const char* msg) { dcb_set_thread_error(msg); return DCB_ERR_INVALID_ARGUMENT; }

// ---------------------------------------------------------------------------------------------- sortable keys
// Order-preserving unsigned image of a key. Floating keys follow .NET's comparer: every NaN is equal to every other NaN
// and below all numbers, -0 equals +0 (so both get one image and the stable sort keeps their source order).
template <typename K> struct Sortable;
template <> struct Sortable<u32> {
    static __device__ __forceinline__ u32 of_f32(float f) {
        if (f != f) return 0u;
        if (f == 0.0f) f = 0.0f;
        const u32 b = __float_as_uint(f);
        return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    }
};
template <int TYPE> struct KeyOf;
#define KEY32(T, CT, EXPR) template <> struct KeyOf<T> { typedef CT in_t; typedef u32 bits_t; static __device__ __forceinline__ u32 bits(CT v) { return EXPR; } };
#define KEY64(T, CT, EXPR) template <> struct KeyOf<T> { typedef CT in_t; typedef u64 bits_t; static __device__ __forceinline__ u64 bits(CT v) { return EXPR; } };
KEY32(DCB_T_I8, signed char, (u32)((int)v + 128))
KEY32(DCB_T_U8, unsigned char, (u32)v)
KEY32(DCB_T_BOOL, unsigned char, (u32)(v != 0))
KEY32(DCB_T_I16, short, (u32)((int)v + 32768))
KEY32(DCB_T_U16, unsigned short, (u32)v)
KEY32(DCB_T_I32, int, (u32)v ^ 0x80000000u)
KEY32(DCB_T_U32, u32, v)
KEY32(DCB_T_F32, float, Sortable<u32>::of_f32(v))
KEY64(DCB_T_I64, i64, (u64)v ^ 0x8000000000000000ull)
KEY64(DCB_T_U64, u64, v)
template <> struct KeyOf<DCB_T_F64> {
    typedef double in_t; typedef u64 bits_t;
    static __device__ __forceinline__ u64 bits(double f) {
        if (f != f) return 0ull;
        if (f == 0.0) f = 0.0;
        const u64 b = (u64)__double_as_longlong(f);
        return (b & 0x8000000000000000ull) ? ~b : (b | 0x8000000000000000ull);
    }
};

template <int TYPE>
__global__ void __launch_bounds__(kThreads) prepare_keys(const typename KeyOf<TYPE>::in_t* __restrict__ keys, i64 n, int descending,
                                                         typename KeyOf<TYPE>::bits_t* __restrict__ bits, u32* __restrict__ idx,
                                                         const u32* __restrict__ payload) {
    const i64 stride = (i64)gridDim.x * blockDim.x;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        typename KeyOf<TYPE>::bits_t b = KeyOf<TYPE>::bits(keys[i]);
        bits[i] = descending ? ~b : b;          // descending = ascending in the complement; ties keep source order either way
        if (idx) idx[i] = payload ? payload[i] : (u32)i;   // what travels with the key: its position, or a 4-byte value
    }
}

// ---------------------------------------------------------------------------------------------- radix sort, one pass
// Tile histogram: counts of the pass's digit in one tile, written digit-major (all tiles of digit 0, then digit 1, ...),
// so that ONE exclusive scan over that array gives every (digit, tile) its first output position.
// A block counts kHistTiles consecutive tiles and thread d writes digit d's counts of all of them side by side: whole
// 32-byte sectors instead of one 4-byte word per (tile, digit) at a stride of the number of tiles.
constexpr int kHistTiles = 8;
template <typename K>
__global__ void __launch_bounds__(kThreads) radix_tile_hist(const K* __restrict__ keys, i64 n, int shift, u32 num_tiles, u32* __restrict__ hist) {
    __shared__ u32 s_hist[kHistTiles][256];
#pragma unroll
    for (int t = 0; t < kHistTiles; ++t) s_hist[t][threadIdx.x] = 0;
    __syncthreads();
    const u32 tile0 = blockIdx.x * kHistTiles;
#pragma unroll 1
    for (int t = 0; t < kHistTiles; ++t) {
        const i64 base = (i64)(tile0 + t) * kTile;
        if (base >= n) break;
#pragma unroll 8
        for (int i = 0; i < kItems; ++i) {
            const i64 e = base + (i64)i * kThreads + threadIdx.x;
            if (e < n) atomicAdd(&s_hist[t][(u32)(keys[e] >> shift) & 255u], 1u);
        }
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kHistTiles; ++t)
        if (tile0 + t < num_tiles) hist[(size_t)threadIdx.x * num_tiles + tile0 + t] = s_hist[t][threadIdx.x];
}

// Scatter: warp w of a tile owns a contiguous run of kItems * 32 elements; ranks inside the tile follow element order
// (item, then lane, within a warp; warps in order), so the sort is stable. The tile is first sorted by digit inside
// shared memory; it then leaves in that order, so that consecutive threads write consecutive addresses of one digit's
// run (whole sectors, a few per warp) where a direct scatter sends every lane to a sector of its own.
template <typename K>
__global__ void __launch_bounds__(kThreads, 3) radix_scatter(const K* __restrict__ keys_in, const u32* __restrict__ idx_in, i64 n, int shift,
                                                          u32 num_tiles, const u32* __restrict__ scanned,
                                                          K* __restrict__ keys_out, u32* __restrict__ idx_out) {
    extern __shared__ __align__(16) unsigned char s_dyn[];   // kTile keys, then kTile payloads, in tile-sorted order
    K* s_keys = reinterpret_cast<K*>(s_dyn);
    u32* s_idx = reinterpret_cast<u32*>(s_dyn + (size_t)kTile * sizeof(K));
    __shared__ u32 s_cnt[kWarps][257];           // per warp and digit: elements seen so far; bin 256 = past the end of the array
    __shared__ u32 s_start[257];                 // where digit d starts inside the sorted tile
    __shared__ u32 s_gbase[256];                 // global position of a sorted-tile position p of digit d = s_gbase[d] + p
    __shared__ u32 s_warp_tot[kWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int d = lane; d < 257; d += 32) s_cnt[warp][d] = 0;
    __syncwarp();
    const i64 run = (i64)blockIdx.x * kTile + (i64)warp * (kItems * 32);
    K key[kItems];
    u32 pay[kItems];
    u32 rank[kItems];
    const u32 lt = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const i64 e = run + i * 32 + lane;
        key[i] = e < n ? keys_in[e] : (K)0;
        pay[i] = e < n ? idx_in[e] : 0u;
    }
    // The lanes that hold the same digit: one ballot per bit (nine of them: bin 256 is the ninth bit). match.any walks
    // through the distinct values of the warp one by one, about thirty of them for random digits.
    auto peers_of = [&](u32 d) -> u32 {
        u32 peers = 0xffffffffu;
#pragma unroll
        for (int bit = 0; bit < 9; ++bit) {
            const bool on = ((d >> bit) & 1u) != 0u;
            const u32 m = __ballot_sync(0xffffffffu, on);
            peers &= on ? m : ~m;
        }
        return peers;
    };
    // (Shared-memory atomics whose results are used only after all sixteen are in flight, instead of a read and a write of
    // the counter per item, measured slower twice: 767 against 636 us a pass with match.any, 3.7 against 3.0 ms a sort with
    // the ballots.)
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const i64 e = run + i * 32 + lane;
        const u32 d = e < n ? ((u32)(key[i] >> shift) & 255u) : 256u;
        const u32 peers = peers_of(d);
        const u32 before = s_cnt[warp][d];
        __syncwarp();
        if ((peers & lt) == 0u) s_cnt[warp][d] = before + (u32)__popc(peers);   // the first lane of each group of equal digits
        __syncwarp();
        rank[i] = before + (u32)__popc(peers & lt);
    }
    __syncthreads();
    {   // thread d: the tile's count of digit d; the warps' counts become offsets inside the digit's run
        const int d = threadIdx.x;
        u32 acc = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) { const u32 c = s_cnt[w][d]; s_cnt[w][d] = acc; acc += c; }
        // exclusive scan of the 256 counts over the block: where each digit starts in the sorted tile
        u32 incl = acc;
#pragma unroll
        for (int dd = 1; dd < 32; dd <<= 1) { const u32 t = __shfl_up_sync(0xffffffffu, incl, dd); if (lane >= dd) incl += t; }
        if (lane == 31) s_warp_tot[warp] = incl;
        __syncthreads();
        u32 off = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) if (w < warp) off += s_warp_tot[w];
        const u32 start = off + incl - acc;
        s_start[d] = start;
        s_gbase[d] = scanned[(size_t)d * num_tiles + blockIdx.x] - start;
        if (d == 255) s_start[256] = start + acc;             // elements of the tile that lie inside the array
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const i64 e = run + i * 32 + lane;
        if (e < n) {
            const u32 d = (u32)(key[i] >> shift) & 255u;
            const u32 p = s_start[d] + s_cnt[warp][d] + rank[i];
            s_keys[p] = key[i];
            s_idx[p] = pay[i];
        }
    }
    __syncthreads();
    const u32 valid = s_start[256];
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const u32 p = (u32)i * kThreads + threadIdx.x;
        if (p < valid) {
            const K k = s_keys[p];
            const u32 g = s_gbase[(u32)(k >> shift) & 255u] + p;
            keys_out[g] = k;
            idx_out[g] = s_idx[p];
        }
    }
}
template <typename K> constexpr size_t scatter_smem_bytes() { return (size_t)kTile * (sizeof(K) + sizeof(u32)); }

// ---------------------------------------------------------------------------------------------- exclusive scan of u32
__global__ void __launch_bounds__(kThreads) scan_tiles(const u32* __restrict__ in, u32* __restrict__ out, i64 n, u32* __restrict__ totals) {
    __shared__ u32 s_warp[kWarps];
    const i64 base = (i64)blockIdx.x * kScanTile + (i64)threadIdx.x * kScanItems;
    u32 v[kScanItems];
    u32 sum = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) { v[i] = base + i < n ? in[base + i] : 0u; sum += v[i]; }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    u32 incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const u32 t = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += t; }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    u32 warp_off = 0, block_total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) { if (w < warp) warp_off += s_warp[w]; block_total += s_warp[w]; }
    u32 run = warp_off + incl - sum;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) { if (base + i < n) out[base + i] = run; run += v[i]; }
    if (threadIdx.x == 0) totals[blockIdx.x] = block_total;
}
__global__ void __launch_bounds__(1024) scan_totals(u32* __restrict__ totals, u32 count, u32* __restrict__ grand_total) {
    // one block: exclusive scan of up to a few hundred thousand block totals, 1024 at a time with a running carry
    __shared__ u32 s_warp[32];
    __shared__ u32 s_carry;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (u32 base = 0; base < count; base += 1024) {
        const u32 i = base + threadIdx.x;
        const u32 v = i < count ? totals[i] : 0u;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        u32 incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { const u32 t = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += t; }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            u32 w = s_warp[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const u32 t = __shfl_up_sync(0xffffffffu, w, d); if (lane >= d) w += t; }
            s_warp[lane] = w;                    // inclusive over warps
        }
        __syncthreads();
        const u32 carry = s_carry;
        const u32 warp_off = warp ? s_warp[warp - 1] : 0u;
        if (i < count) totals[i] = carry + warp_off + incl - v;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = carry + warp_off + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0 && grand_total) *grand_total = s_carry;
}
__global__ void __launch_bounds__(kThreads) scan_add(u32* __restrict__ out, i64 n, const u32* __restrict__ totals) {
    const u32 add = totals[blockIdx.x];
    const i64 base = (i64)blockIdx.x * kScanTile + (i64)threadIdx.x * kScanItems;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) if (base + i < n) out[base + i] += add;
}

// out[i] = sum of in[0..i), in place allowed; *d_total (device, optional) = sum of everything. `d_totals` holds one u32 per scan tile.
dcb_status exclusive_scan(const u32* d_in, u32* d_out, i64 n, u32* d_totals, u32* d_total, cudaStream_t s) {
    if (n == 0) { if (d_total) RCU(cudaMemsetAsync(d_total, 0, sizeof(u32), s)); return DCB_OK; }
    const u32 blocks = (u32)((n + kScanTile - 1) / kScanTile);
    scan_tiles<<<blocks, kThreads, 0, s>>>(d_in, d_out, n, d_totals);
    scan_totals<<<1, 1024, 0, s>>>(d_totals, blocks, d_total);
    scan_add<<<blocks, kThreads, 0, s>>>(d_out, n, d_totals);
    RCU(cudaGetLastError());
    return DCB_OK;
}
size_t scan_totals_count(i64 n) { return (size_t)((n + kScanTile - 1) / kScanTile) + 1; }

// ---------------------------------------------------------------------------------------------- prefix sum of a column
// out[i] = in[0] + ... + in[i] (inclusive) or ... + in[i-1] (exclusive), over any number of blocks: tile totals, one scan of
// the totals, then every tile scans itself starting from the sum before it - 12 bytes per 4-byte element. Integers add in
// their own width and wrap (what the reference's generated kernel does, CudaKernelGenerator.cs:499-576, which stops at one
// block of 256); floats add in fp64 and every output is rounded once, so the result does not depend on the grid.
template <typename T> struct ScanAcc;
template <> struct ScanAcc<int> { typedef u32 acc_t; static __device__ __forceinline__ u32 in(int v) { return (u32)v; } static __device__ __forceinline__ int out(u32 a) { return (int)a; } };
template <> struct ScanAcc<i64> { typedef u64 acc_t; static __device__ __forceinline__ u64 in(i64 v) { return (u64)v; } static __device__ __forceinline__ i64 out(u64 a) { return (i64)a; } };
template <> struct ScanAcc<float> { typedef double acc_t; static __device__ __forceinline__ double in(float v) { return (double)v; } static __device__ __forceinline__ float out(double a) { return (float)a; } };
template <> struct ScanAcc<double> { typedef double acc_t; static __device__ __forceinline__ double in(double v) { return v; } static __device__ __forceinline__ double out(double a) { return a; } };

template <typename A> __device__ __forceinline__ A shfl_up_acc(A v, int d);
template <> __device__ __forceinline__ u32 shfl_up_acc<u32>(u32 v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
template <> __device__ __forceinline__ u64 shfl_up_acc<u64>(u64 v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
template <> __device__ __forceinline__ double shfl_up_acc<double>(double v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }

// Sum of the block's values in thread order; every thread gets (sum of the threads before it, block total).
template <typename A>
__device__ __forceinline__ void block_exclusive(A mine, A* s_warp /* kWarps */, A& before, A& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    A incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const A t = shfl_up_acc<A>(incl, d); if (lane >= d) incl = incl + t; }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    A off = A(0); total = A(0);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) { if (w < warp) off = off + s_warp[w]; total = total + s_warp[w]; }
    before = off + incl - mine;
    __syncthreads();
}
// A thread's kItems consecutive elements, with 16-byte accesses when the tile lies inside the array and the column starts
// at a 16-byte boundary (a thread's run then does too), element by element otherwise.
template <typename T>
__device__ __forceinline__ void load_run(const T* __restrict__ in, i64 base, i64 n, bool vec, T (&v)[kItems]) {
    constexpr int VE = 16 / (int)sizeof(T);
    if (vec) {
        const uint4* p = reinterpret_cast<const uint4*>(in + base);
#pragma unroll
        for (int q = 0; q < kItems / VE; ++q) {
            const uint4 w = __ldcs(p + q);
            *reinterpret_cast<uint4*>(&v[q * VE]) = w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < kItems; ++i) v[i] = base + i < n ? in[base + i] : T(0);
    }
}
template <typename T>
__device__ __forceinline__ void store_run(T* __restrict__ out, i64 base, i64 n, bool vec, const T (&v)[kItems]) {
    constexpr int VE = 16 / (int)sizeof(T);
    if (vec) {
        uint4* p = reinterpret_cast<uint4*>(out + base);
#pragma unroll
        for (int q = 0; q < kItems / VE; ++q) __stcs(p + q, *reinterpret_cast<const uint4*>(&v[q * VE]));
    } else {
#pragma unroll
        for (int i = 0; i < kItems; ++i) if (base + i < n) out[base + i] = v[i];
    }
}
template <typename T>
__global__ void __launch_bounds__(kThreads) prefix_tile_totals(const T* __restrict__ in, i64 n, typename ScanAcc<T>::acc_t* __restrict__ totals) {
    typedef typename ScanAcc<T>::acc_t A;
    __shared__ A s_warp[kWarps];
    const i64 base = (i64)blockIdx.x * kTile + (i64)threadIdx.x * kItems;
    const bool vec = (i64)(blockIdx.x + 1) * kTile <= n && (reinterpret_cast<unsigned long long>(in) & 15ull) == 0;
    __align__(16) T x[kItems];
    load_run<T>(in, base, n, vec, x);
    A sum = A(0);
#pragma unroll
    for (int i = 0; i < kItems; ++i) sum = sum + ScanAcc<T>::in(x[i]);   // same order as prefix_tiles: same bits
    A before, total;
    block_exclusive<A>(sum, s_warp, before, total);
    if (threadIdx.x == 0) totals[blockIdx.x] = total;
}
template <typename A>
__global__ void __launch_bounds__(1024) prefix_scan_totals(A* __restrict__ totals, u32 count) {
    // one block: exclusive scan of the tile totals in tile order, 1024 at a time with a running carry
    __shared__ A s_warp[32];
    __shared__ A s_carry;
    if (threadIdx.x == 0) s_carry = A(0);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (u32 base = 0; base < count; base += 1024) {
        const u32 i = base + threadIdx.x;
        const A v = i < count ? totals[i] : A(0);
        A incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { const A t = shfl_up_acc<A>(incl, d); if (lane >= d) incl = incl + t; }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        A off = A(0), all = A(0);
        for (int w = 0; w < 32; ++w) { if (w < warp) off = off + s_warp[w]; all = all + s_warp[w]; }
        const A carry = s_carry;
        if (i < count) totals[i] = carry + off + incl - v;
        __syncthreads();
        if (threadIdx.x == 0) s_carry = carry + all;
        __syncthreads();
    }
}
template <typename T>
__global__ void __launch_bounds__(kThreads) prefix_tiles(const T* __restrict__ in, i64 n, const typename ScanAcc<T>::acc_t* __restrict__ totals_excl,
                                                        int inclusive, T* __restrict__ out) {
    typedef typename ScanAcc<T>::acc_t A;
    __shared__ A s_warp[kWarps];
    const i64 base = (i64)blockIdx.x * kTile + (i64)threadIdx.x * kItems;
    const bool vec = (i64)(blockIdx.x + 1) * kTile <= n && ((reinterpret_cast<unsigned long long>(in) | reinterpret_cast<unsigned long long>(out)) & 15ull) == 0;
    __align__(16) T x[kItems];
    load_run<T>(in, base, n, vec, x);
    A sum = A(0);
#pragma unroll
    for (int i = 0; i < kItems; ++i) sum = sum + ScanAcc<T>::in(x[i]);
    A before, total;
    block_exclusive<A>(sum, s_warp, before, total);
    A run = totals_excl[blockIdx.x] + before;
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const A next = run + ScanAcc<T>::in(x[i]);
        x[i] = ScanAcc<T>::out(inclusive ? next : run);
        run = next;
    }
    store_run<T>(out, base, n, vec, x);
}
template <typename T>
dcb_status prefix_sum_typed(const void* d_in, i64 n, int inclusive, void* d_out, cudaStream_t s) {
    typedef typename ScanAcc<T>::acc_t A;
    const u32 tiles = (u32)((n + kTile - 1) / kTile);
    A* totals = nullptr;
    RCU(cudaMallocAsync((void**)&totals, (size_t)tiles * sizeof(A), s));
    prefix_tile_totals<T><<<tiles, kThreads, 0, s>>>((const T*)d_in, n, totals);
    prefix_scan_totals<A><<<1, 1024, 0, s>>>(totals, tiles);
    prefix_tiles<T><<<tiles, kThreads, 0, s>>>((const T*)d_in, n, totals, inclusive, (T*)d_out);
    const cudaError_t e = cudaGetLastError();
    cudaFreeAsync(totals, s);
    if (e != cudaSuccess) { dcb_set_thread_error(cudaGetErrorString(e)); return DCB_ERR_CUDA; }
    return DCB_OK;
}

// ---------------------------------------------------------------------------------------------- the sort itself
// Which bits differ among the keys: OR of key ^ first key. A pass whose digit is the same in every key would move nothing
// and is skipped (keys below 1000 need two passes of four, `v % 7` one).
template <typename K>
__global__ void __launch_bounds__(kThreads) key_bits_differ(const K* __restrict__ keys, i64 n, u64* __restrict__ out) {
    const K k0 = keys[0];
    K acc = 0;
    const i64 stride = (i64)gridDim.x * blockDim.x;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc |= keys[i] ^ k0;
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) acc |= (K)__shfl_xor_sync(0xffffffffu, acc, m);
    if ((threadIdx.x & 31) == 0 && acc != 0) atomicOr(out, (u64)acc);
}

struct SortScratch {
    void* keys[2] = {nullptr, nullptr};
    u32* idx[2] = {nullptr, nullptr};
    u32* hist = nullptr;
    u32* totals = nullptr;
    u64* differ = nullptr;
    cudaStream_t s = nullptr;
    dcb_status alloc(i64 n, int key_bytes, cudaStream_t stream) {
        s = stream;
        const u32 tiles = (u32)((n + kTile - 1) / kTile);
        const size_t m = (size_t)256 * std::max<u32>(tiles, 1);
        for (int i = 0; i < 2; ++i) {
            RCU(cudaMallocAsync(&keys[i], std::max<size_t>((size_t)n * key_bytes, 16), s));
            RCU(cudaMallocAsync((void**)&idx[i], std::max<size_t>((size_t)n * 4, 16), s));
        }
        RCU(cudaMallocAsync((void**)&hist, m * 4, s));
        RCU(cudaMallocAsync((void**)&totals, scan_totals_count((i64)m) * 4, s));
        RCU(cudaMallocAsync((void**)&differ, 16, s));
        return DCB_OK;
    }
    void release() {
        for (int i = 0; i < 2; ++i) { if (keys[i]) cudaFreeAsync(keys[i], s); if (idx[i]) cudaFreeAsync(idx[i], s); keys[i] = nullptr; idx[i] = nullptr; }
        if (hist) cudaFreeAsync(hist, s);
        if (totals) cudaFreeAsync(totals, s);
        if (differ) cudaFreeAsync(differ, s);
        hist = totals = nullptr; differ = nullptr;
    }
};

// Sorts sc.keys[0] / sc.idx[0] (n pairs of sortable bits and payload); returns which of the two buffers holds the result.
// `final_idx` (optional): where the last pass writes the payloads instead of the scratch buffer. Passes whose digit is
// the same in every key are skipped; finding that out costs one read of the keys and one synchronisation of the stream
// (not done while the stream is being captured into a graph).
template <typename K>
dcb_status radix_sort(SortScratch& sc, i64 n, int* result_buf, u32* final_idx = nullptr, const u64* known_differ = nullptr) {
    const u32 tiles = (u32)((n + kTile - 1) / kTile);
    int cur = 0;
    if (scatter_smem_bytes<K>() + 11 * 1024 > 48 * 1024) {   // static + dynamic shared memory beyond the default 48 KB: opt in (cheap, per device)
        RCU(cudaFuncSetAttribute(radix_scatter<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)scatter_smem_bytes<K>()));
    }
    if (n > 0) {
        u64 differ = ~0ull;
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(sc.s, &cap) != cudaSuccess) { (void)cudaGetLastError(); cap = cudaStreamCaptureStatusNone; }
        if (known_differ) differ = *known_differ;
        else if (cap == cudaStreamCaptureStatusNone && n > 1) {
            RCU(cudaMemsetAsync(sc.differ, 0, 8, sc.s));
            key_bits_differ<K><<<(int)std::min<i64>((n + kThreads - 1) / kThreads, 148 * 8), kThreads, 0, sc.s>>>((const K*)sc.keys[0], n, sc.differ);
            RCU(cudaMemcpyAsync(&differ, sc.differ, 8, cudaMemcpyDeviceToHost, sc.s));
            RCU(cudaStreamSynchronize(sc.s));
        }
        int shifts[8], passes = 0;
        for (int shift = 0; shift < (int)sizeof(K) * 8; shift += 8)
            if ((differ >> shift) & 0xffull) shifts[passes++] = shift;
        for (int p = 0; p < passes; ++p) {
            const int shift = shifts[p];
            const bool last = p + 1 == passes;
            radix_tile_hist<K><<<(tiles + kHistTiles - 1) / kHistTiles, kThreads, 0, sc.s>>>((const K*)sc.keys[cur], n, shift, tiles, sc.hist);
            dcb_status st = exclusive_scan(sc.hist, sc.hist, (i64)256 * tiles, sc.totals, nullptr, sc.s);
            if (st) return st;
            radix_scatter<K><<<tiles, kThreads, scatter_smem_bytes<K>(), sc.s>>>((const K*)sc.keys[cur], sc.idx[cur], n, shift, tiles, sc.hist,
                                                                                 (K*)sc.keys[cur ^ 1], (last && final_idx) ? final_idx : sc.idx[cur ^ 1]);
            cur ^= 1;
        }
        if (passes == 0 && final_idx) RCU(cudaMemcpyAsync(final_idx, sc.idx[0], (size_t)n * 4, cudaMemcpyDeviceToDevice, sc.s));   // all keys equal: source order
        RCU(cudaGetLastError());
    }
    *result_buf = cur;
    return DCB_OK;
}

template <int TYPE>
dcb_status prepare(const void* d_keys, i64 n, int descending, void* bits, u32* idx, const u32* payload, cudaStream_t s) {
    if (n == 0) return DCB_OK;
    const int grid = (int)std::min<i64>((n + kThreads - 1) / kThreads, 148 * 8);
    prepare_keys<TYPE><<<grid, kThreads, 0, s>>>((const typename KeyOf<TYPE>::in_t*)d_keys, n, descending,
                                                (typename KeyOf<TYPE>::bits_t*)bits, idx, payload);
    RCU(cudaGetLastError());
    return DCB_OK;
}
int key_bytes_of(int type) {
    switch (type) {
        case DCB_T_I64: case DCB_T_U64: case DCB_T_F64: return 8;
        case DCB_T_I8: case DCB_T_U8: case DCB_T_BOOL: case DCB_T_I16: case DCB_T_U16: case DCB_T_I32: case DCB_T_U32: case DCB_T_F32: return 4;
        default: return 0;
    }
}
dcb_status prepare_any(int type, const void* d_keys, i64 n, int descending, void* bits, u32* idx, const u32* payload, cudaStream_t s) {
    switch (type) {
        case DCB_T_I8: return prepare<DCB_T_I8>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_U8: return prepare<DCB_T_U8>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_BOOL: return prepare<DCB_T_BOOL>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_I16: return prepare<DCB_T_I16>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_U16: return prepare<DCB_T_U16>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_I32: return prepare<DCB_T_I32>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_U32: return prepare<DCB_T_U32>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_F32: return prepare<DCB_T_F32>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_I64: return prepare<DCB_T_I64>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_U64: return prepare<DCB_T_U64>(d_keys, n, descending, bits, idx, payload, s);
        case DCB_T_F64: return prepare<DCB_T_F64>(d_keys, n, descending, bits, idx, payload, s);
        default: return bad("unsupported key type");
    }
}
// keys (typed, device) -> sorted sortable bits in sc.keys[*buf] and the stable permutation in sc.idx[*buf]
// (`payload`: 4-byte values to carry instead of positions; `final_idx`: where the sorted payloads go, else sc.idx[*buf])
dcb_status sort_keys(SortScratch& sc, int key_type, const void* d_keys, i64 n, int descending, int* buf,
                     const u32* payload = nullptr, u32* final_idx = nullptr) {
    dcb_status st = prepare_any(key_type, d_keys, n, descending, sc.keys[0], sc.idx[0], payload, sc.s);
    if (st) return st;
    return key_bytes_of(key_type) == 8 ? radix_sort<u64>(sc, n, buf, final_idx) : radix_sort<u32>(sc, n, buf, final_idx);
}
// The bits that differ among the prepared keys in sc.keys[0] (synchronises the stream).
dcb_status keys_differ(SortScratch& sc, int key_bytes, i64 n, u64* differ) {
    *differ = 0;
    if (n <= 1) return DCB_OK;
    RCU(cudaMemsetAsync(sc.differ, 0, 8, sc.s));
    const int grid = (int)std::min<i64>((n + kThreads - 1) / kThreads, 148 * 8);
    if (key_bytes == 8) key_bits_differ<u64><<<grid, kThreads, 0, sc.s>>>((const u64*)sc.keys[0], n, sc.differ);
    else key_bits_differ<u32><<<grid, kThreads, 0, sc.s>>>((const u32*)sc.keys[0], n, sc.differ);
    RCU(cudaMemcpyAsync(differ, sc.differ, 8, cudaMemcpyDeviceToHost, sc.s));
    RCU(cudaStreamSynchronize(sc.s));
    return DCB_OK;
}

// ---------------------------------------------------------------------------------------------- gather
template <typename T>
__global__ void __launch_bounds__(kThreads) gather_kernel(const T* __restrict__ src, const u32* __restrict__ idx, i64 n, T* __restrict__ dst) {
    // Eight independent random reads per thread are in flight before the first is used: the kernel is bound by the latency
    // of sector-sized reads all over `src`, not by bytes.
    constexpr int G = 8;
    const i64 stride = (i64)gridDim.x * blockDim.x;
    i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (G - 1) * stride < n; i += G * stride) {
        u32 j[G]; T v[G];
#pragma unroll
        for (int g = 0; g < G; ++g) j[g] = __ldcs(idx + i + g * stride);
#pragma unroll
        for (int g = 0; g < G; ++g) v[g] = src[j[g]];
#pragma unroll
        for (int g = 0; g < G; ++g) dst[i + g * stride] = v[g];
    }
    for (; i < n; i += stride) dst[i] = src[idx[i]];
}

// ---------------------------------------------------------------------------------------------- group by
enum { AGG_COUNT = 0, AGG_SUM = 1, AGG_MIN = 2, AGG_MAX = 3, AGG_AVERAGE = 4 };

template <typename K>
__global__ void __launch_bounds__(kThreads) group_heads(const K* __restrict__ sorted, i64 n, u32* __restrict__ heads) {
    const i64 stride = (i64)gridDim.x * blockDim.x;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) heads[i] = (i == 0 || sorted[i] != sorted[i - 1]) ? 1u : 0u;
}
// Value of element e as a double (floating values) or a 64-bit integer (integer values).
template <typename V> struct ValueOf {
    static __device__ __forceinline__ double f(const V* p, u32 e) { return (double)p[e]; }
    static __device__ __forceinline__ i64 i(const V* p, u32 e) { return (i64)p[e]; }
};
__device__ __forceinline__ void atomic_min_f64(double* addr, double v) {
    u64 old = *(volatile u64*)addr;
    while (__longlong_as_double((i64)old) > v || __longlong_as_double((i64)old) != __longlong_as_double((i64)old)) {
        const u64 seen = atomicCAS((u64*)addr, old, (u64)__double_as_longlong(v));
        if (seen == old) break;
        old = seen;
    }
}
__device__ __forceinline__ void atomic_max_f64(double* addr, double v) {
    u64 old = *(volatile u64*)addr;
    while (__longlong_as_double((i64)old) < v || __longlong_as_double((i64)old) != __longlong_as_double((i64)old)) {
        const u64 seen = atomicCAS((u64*)addr, old, (u64)__double_as_longlong(v));
        if (seen == old) break;
        old = seen;
    }
}
// Sorted position i belongs to group gid[i] (inclusive scan of the head flags, minus one). Lanes of one group are
// neighbours, so a warp folds each of its groups with a segmented shuffle reduction and issues one atomic per group.
template <typename V, bool FP>
__global__ void __launch_bounds__(kThreads) group_reduce(const V* __restrict__ values, const u32* __restrict__ idx, const u32* __restrict__ heads_excl,
                                                         const u32* __restrict__ heads, i64 n, int agg, u32* __restrict__ first_idx,
                                                         u32* __restrict__ counts, double* __restrict__ facc, i64* __restrict__ iacc) {
    const i64 stride = (i64)gridDim.x * blockDim.x;
    const int lane = threadIdx.x & 31;
    for (i64 i0 = ((i64)blockIdx.x * blockDim.x + threadIdx.x) - lane; i0 < n; i0 += stride) {
        const i64 i = i0 + lane;
        const bool live = i < n;
        const u32 e = live ? idx[i] : 0u;
        const u32 g = live ? heads_excl[i] + heads[i] - 1u : 0xffffffffu;
        if (live && heads[i]) first_idx[g] = e;              // stable sort: the head of a group is its first element in the source
        double fv = 0; i64 iv = 0; u32 c = live ? 1u : 0u;
        if (live && agg != AGG_COUNT) { if (FP) fv = ValueOf<V>::f(values, e); else iv = ValueOf<V>::i(values, e); }
        const u32 peers = __match_any_sync(0xffffffffu, g);
        const int last = 31 - __clz((int)peers);             // lanes of a group are contiguous
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const u32 oc = __shfl_down_sync(0xffffffffu, c, d);
            const double of = __shfl_down_sync(0xffffffffu, fv, d);
            const i64 oi = __shfl_down_sync(0xffffffffu, iv, d);
            if (lane + d <= last) {
                c += oc;
                if (agg == AGG_MIN) { if (FP) fv = of < fv ? of : fv; else iv = oi < iv ? oi : iv; }
                else if (agg == AGG_MAX) { if (FP) fv = of > fv ? of : fv; else iv = oi > iv ? oi : iv; }
                else { fv += of; iv += oi; }
            }
        }
        if (live && (peers & ((1u << lane) - 1u)) == 0u) {   // first lane of the group within this warp
            atomicAdd(&counts[g], c);
            if (agg == AGG_SUM || agg == AGG_AVERAGE) { if (FP) atomicAdd(&facc[g], fv); else atomicAdd((u64*)&iacc[g], (u64)iv); }
            else if (agg == AGG_MIN) { if (FP) atomic_min_f64(&facc[g], fv); else atomicMin(&iacc[g], iv); }
            else if (agg == AGG_MAX) { if (FP) atomic_max_f64(&facc[g], fv); else atomicMax(&iacc[g], iv); }
        }
    }
}
__global__ void __launch_bounds__(kThreads) group_init(u32 groups, int agg, bool fp, double* facc, i64* iacc, u32* counts) {
    for (u32 g = blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += gridDim.x * blockDim.x) {
        counts[g] = 0;
        if (agg == AGG_MIN) { facc[g] = __longlong_as_double(0x7ff8000000000000LL); iacc[g] = 0x7fffffffffffffffLL; }
        else if (agg == AGG_MAX) { facc[g] = __longlong_as_double(0x7ff8000000000000LL); iacc[g] = -0x7fffffffffffffffLL - 1; }
        else { facc[g] = 0.0; iacc[g] = 0; }
        (void)fp;
    }
}
// Final order = order of first occurrence: `order` is the argsort of first_idx.
__global__ void __launch_bounds__(kThreads) group_emit(const u32* __restrict__ order, const u32* __restrict__ first_idx, const u32* __restrict__ counts,
                                                       const double* __restrict__ facc, const i64* __restrict__ iacc, u32 groups, int agg, bool fp,
                                                       u32* __restrict__ out_first, i64* __restrict__ out_counts, double* __restrict__ out_f, i64* __restrict__ out_i) {
    for (u32 j = blockIdx.x * blockDim.x + threadIdx.x; j < groups; j += gridDim.x * blockDim.x) {
        const u32 g = order[j];
        out_first[j] = first_idx[g];
        out_counts[j] = (i64)counts[g];
        if (fp) out_f[j] = agg == AGG_AVERAGE ? facc[g] / (double)counts[g] : facc[g];
        else { out_i[j] = iacc[g]; out_f[j] = agg == AGG_AVERAGE ? (double)iacc[g] / (double)counts[g] : (double)iacc[g]; }
    }
}

// Keys that differ in their low bits only (at most 16 of them) need no sort: the low bits index a table directly. Each
// block adds into a table of its own in shared memory when that fits (Count / Sum / Average over at most 2048 slots) and
// flushes it once; otherwise straight into the table in global memory. A group's first index is a minimum that, after
// the group's first few elements, only has to be looked at.
constexpr int kDenseSmemSlots = 2048;
template <typename K, typename V, bool FP>
__global__ void __launch_bounds__(kThreads) group_dense(const K* __restrict__ bits, const V* __restrict__ values, i64 n, int agg, u32 mask, int in_smem,
                                                        u32* __restrict__ first, u32* __restrict__ counts, double* __restrict__ facc, i64* __restrict__ iacc) {
    __shared__ u32 s_cnt[kDenseSmemSlots];
    __shared__ u32 s_first[kDenseSmemSlots];
    __shared__ u64 s_acc[kDenseSmemSlots];                    // double or 64-bit integer sums
    const u32 slots = mask + 1u;
    if (in_smem) {
        for (u32 i = threadIdx.x; i < slots; i += kThreads) { s_cnt[i] = 0; s_first[i] = 0xffffffffu; s_acc[i] = 0; }
        __syncthreads();
    }
    const i64 stride = (i64)gridDim.x * blockDim.x;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const u32 g = (u32)bits[i] & mask;
        double fv = 0; i64 iv = 0;
        if (agg != AGG_COUNT) { if (FP) fv = ValueOf<V>::f(values, (u32)i); else iv = ValueOf<V>::i(values, (u32)i); }
        if (in_smem) {
            atomicAdd(&s_cnt[g], 1u);
            if ((u32)i < s_first[g]) atomicMin(&s_first[g], (u32)i);
            if (agg != AGG_COUNT) { if (FP) atomicAdd(reinterpret_cast<double*>(&s_acc[g]), fv); else atomicAdd(&s_acc[g], (u64)iv); }
        } else {
            atomicAdd(&counts[g], 1u);
            if ((u32)i < *(volatile u32*)&first[g]) atomicMin(&first[g], (u32)i);
            if (agg == AGG_SUM || agg == AGG_AVERAGE) { if (FP) atomicAdd(&facc[g], fv); else atomicAdd((u64*)&iacc[g], (u64)iv); }
            else if (agg == AGG_MIN) { if (FP) atomic_min_f64(&facc[g], fv); else atomicMin(&iacc[g], iv); }
            else if (agg == AGG_MAX) { if (FP) atomic_max_f64(&facc[g], fv); else atomicMax(&iacc[g], iv); }
        }
    }
    if (in_smem) {
        __syncthreads();
        for (u32 g = threadIdx.x; g < slots; g += kThreads) {
            const u32 c = s_cnt[g];
            if (c == 0) continue;
            atomicAdd(&counts[g], c);
            atomicMin(&first[g], s_first[g]);
            if (agg != AGG_COUNT) { if (FP) atomicAdd(&facc[g], __longlong_as_double((i64)s_acc[g])); else atomicAdd((u64*)&iacc[g], s_acc[g]); }
        }
    }
}
__global__ void __launch_bounds__(kThreads) dense_init(u32 slots, int agg, u32* first, u32* counts, double* facc, i64* iacc) {
    for (u32 g = blockIdx.x * blockDim.x + threadIdx.x; g < slots; g += gridDim.x * blockDim.x) {
        first[g] = 0xffffffffu; counts[g] = 0;
        if (agg == AGG_MIN) { facc[g] = __longlong_as_double(0x7ff8000000000000LL); iacc[g] = 0x7fffffffffffffffLL; }
        else if (agg == AGG_MAX) { facc[g] = __longlong_as_double(0x7ff8000000000000LL); iacc[g] = -0x7fffffffffffffffLL - 1; }
        else { facc[g] = 0.0; iacc[g] = 0; }
    }
}
// One block: the table's used slots, packed to the front of the same arrays (slot order; the caller sorts by first index).
__global__ void __launch_bounds__(1024) dense_pack(u32 slots, u32* first, u32* counts, double* facc, i64* iacc, u32* __restrict__ groups_out) {
    __shared__ u32 s_warp[32];
    __shared__ u32 s_carry;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (u32 base = 0; base < slots; base += 1024) {
        const u32 g = base + threadIdx.x;
        const u32 c = g < slots ? counts[g] : 0u;
        const u32 fi = g < slots ? first[g] : 0u;
        const double fa = g < slots ? facc[g] : 0.0;
        const i64 ia = g < slots ? iacc[g] : 0;
        const u32 used = c ? 1u : 0u;
        u32 incl = used;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { const u32 t = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += t; }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();                                     // every slot of this chunk has been read
        u32 off = 0, all = 0;
        for (int w = 0; w < 32; ++w) { if (w < warp) off += s_warp[w]; all += s_warp[w]; }
        const u32 pos = s_carry + off + incl - used;         // pos <= g: packing to the front never overtakes the reads
        if (used) { first[pos] = fi; counts[pos] = c; facc[pos] = fa; iacc[pos] = ia; }
        __syncthreads();
        if (threadIdx.x == 0) s_carry += all;
        __syncthreads();
    }
    if (threadIdx.x == 0) *groups_out = s_carry;
}
template <typename K, typename V, bool FP>
static void launch_group_dense(const void* bits, const void* values, i64 n, int agg, u32 mask, u32* first, u32* counts, double* facc, i64* iacc, cudaStream_t s) {
    const int in_smem = (mask + 1u <= (u32)kDenseSmemSlots && (agg == AGG_COUNT || agg == AGG_SUM || agg == AGG_AVERAGE)) ? 1 : 0;
    const int grid = (int)std::min<i64>((n + kThreads - 1) / kThreads, 148 * 4);
    group_dense<K, V, FP><<<grid, kThreads, 0, s>>>((const K*)bits, (const V*)values, n, agg, mask, in_smem, first, counts, facc, iacc);
}
template <typename K>
static bool launch_group_dense_typed(int value_type, const void* d_keys_for_count, const void* bits, const void* values, i64 n, int agg, u32 mask,
                                     u32* first, u32* counts, double* facc, i64* iacc, cudaStream_t s) {
    switch (value_type) {
        case DCB_T_F32: launch_group_dense<K, float, true>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_F64: launch_group_dense<K, double, true>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_I8: launch_group_dense<K, signed char, false>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_U8: case DCB_T_BOOL: launch_group_dense<K, unsigned char, false>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_I16: launch_group_dense<K, short, false>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_U16: launch_group_dense<K, unsigned short, false>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_I32: launch_group_dense<K, int, false>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_U32: launch_group_dense<K, u32, false>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        case DCB_T_I64: case DCB_T_U64: launch_group_dense<K, i64, false>(bits, values, n, agg, mask, first, counts, facc, iacc, s); return true;
        default:
            if (agg == AGG_COUNT) { launch_group_dense<K, u32, false>(bits, d_keys_for_count, n, agg, mask, first, counts, facc, iacc, s); return true; }
            return false;
    }
}

// ---------------------------------------------------------------------------------------------- join
enum { JOIN_INNER = 0, JOIN_SEMI = 2, JOIN_ANTI = 3 };
// Every outer element looks its key up in the sorted inner keys. The first ten steps of each search run over 1024 pivots
// kept in shared memory (every 1/1024th of the array), the rest in the slice between two pivots; the end of the run of
// equal keys is found by doubling steps from its start, not by a second search over the whole array.
constexpr int kJoinPivots = 1024;
template <typename K>
__global__ void __launch_bounds__(kThreads) join_count(const K* __restrict__ outer_bits, i64 n_outer, const K* __restrict__ inner_sorted, u32 n_inner,
                                                       int kind, u32* __restrict__ lo_out, u32* __restrict__ cnt_out) {
    __shared__ K s_piv[kJoinPivots];
    const bool use_piv = n_inner >= 4u * kJoinPivots;
    if (use_piv) {
        for (int j = threadIdx.x; j < kJoinPivots; j += kThreads) s_piv[j] = inner_sorted[(u32)(((u64)j * n_inner) >> 10)];
        __syncthreads();
    }
    const i64 stride = (i64)gridDim.x * blockDim.x;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n_outer; i += stride) {
        const K key = outer_bits[i];
        u32 a = 0, b = n_inner;                               // the first element >= key lies in [a, b]
        if (use_piv) {
            u32 c = 0, h = kJoinPivots;                       // c = number of pivots below the key
            while (c < h) { const u32 mid = (c + h) >> 1; if (s_piv[mid] < key) c = mid + 1; else h = mid; }
            a = c == 0 ? 0u : (u32)(((u64)(c - 1) * n_inner) >> 10) + 1u;
            b = c == (u32)kJoinPivots ? n_inner : (u32)(((u64)c * n_inner) >> 10);
        }
        while (a < b) { const u32 mid = a + ((b - a) >> 1); if (inner_sorted[mid] < key) a = mid + 1; else b = mid; }
        const u32 lo = a;
        // end of the run of keys equal to `key`: doubling steps, then a search inside the last step
        u32 hi = lo;
        if (lo < n_inner && inner_sorted[lo] == key) {
            u32 step = 1, last = lo;                          // inner_sorted[last] == key
            for (;;) {
                const u32 probe = last + step;
                if (probe >= n_inner || inner_sorted[probe] != key) { hi = probe < n_inner ? probe : n_inner; break; }
                last = probe; step <<= 1;
            }
            u32 x = last + 1, y = hi;                         // first index in (last, hi] whose key differs
            while (x < y) { const u32 mid = x + ((y - x) >> 1); if (inner_sorted[mid] == key) x = mid + 1; else y = mid; }
            hi = x;
        }
        lo_out[i] = lo;
        const u32 m = hi - lo;
        cnt_out[i] = kind == JOIN_INNER ? m : (kind == JOIN_SEMI ? (m ? 1u : 0u) : (m ? 0u : 1u));
    }
}
__global__ void __launch_bounds__(kThreads) join_write(const u32* __restrict__ lo, const u32* __restrict__ cnt, const u32* __restrict__ off, i64 n_outer,
                                                       const u32* __restrict__ inner_idx_sorted, int kind, i64 out_cap,
                                                       u32* __restrict__ outer_out, u32* __restrict__ inner_out) {
    const i64 stride = (i64)gridDim.x * blockDim.x;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n_outer; i += stride) {
        const u32 c = cnt[i], o = off[i], l = lo[i];
        for (u32 j = 0; j < c; ++j) {
            if ((i64)o + j >= out_cap) break;
            outer_out[o + j] = (u32)i;
            if (inner_out) inner_out[o + j] = kind == JOIN_INNER ? inner_idx_sorted[l + j] : 0u;
        }
    }
}

int launch_grid(i64 n) { return (int)std::max<i64>(1, std::min<i64>((n + kThreads - 1) / kThreads, 148 * 8)); }

}  // namespace

// ================================================================================================ C ABI
extern "C" dcb_status dcb_sort_indices(dcb_ctx* ctx, int32_t key_type, const void* d_keys, int64_t n, int32_t descending,
                                       uint32_t* d_indices, void* stream) {
    if (!ctx) return bad("ctx is null");
    dcb_status st = (dcb_status)dcb_ctx_make_current(ctx);
    if (st) return st;
    if (n < 0 || n >= (1ll << 32)) return bad("n must lie in [0, 2^32)");
    if (n > 0 && (!d_keys || !d_indices)) return bad("null pointer");
    if (key_bytes_of(key_type) == 0) return bad("unsupported key type");
    cudaStream_t s = (cudaStream_t)dcb_ctx_pick_stream(ctx, stream);
    dcb_ctx_count_launches(ctx, 1 + 5 * key_bytes_of(key_type));
    SortScratch sc;
    if ((st = sc.alloc(n, key_bytes_of(key_type), s))) { sc.release(); return st; }
    int buf = 0;
    st = sort_keys(sc, key_type, d_keys, n, descending, &buf, nullptr, d_indices);   // the last pass writes the permutation in place
    sc.release();
    return st;
}

extern "C" dcb_status dcb_sort_by_key(dcb_ctx* ctx, int32_t key_type, const void* d_keys, int64_t n, int32_t descending,
                                      int32_t value_bytes, const void* d_values, void* d_sorted_values, void* stream) {
    if (!ctx) return bad("ctx is null");
    dcb_status st = (dcb_status)dcb_ctx_make_current(ctx);
    if (st) return st;
    if (n < 0 || n >= (1ll << 32)) return bad("n must lie in [0, 2^32)");
    if (value_bytes != 4) { dcb_set_thread_error("values of 4 bytes travel with the keys; others: dcb_sort_indices + dcb_gather"); return DCB_ERR_NOT_SUPPORTED; }
    if (n > 0 && (!d_keys || !d_values || !d_sorted_values)) return bad("null pointer");
    if (d_values == d_sorted_values && n > 0) return bad("the sorted values need a buffer of their own");
    if (key_bytes_of(key_type) == 0) return bad("unsupported key type");
    cudaStream_t s = (cudaStream_t)dcb_ctx_pick_stream(ctx, stream);
    dcb_ctx_count_launches(ctx, 1 + 5 * key_bytes_of(key_type));
    SortScratch sc;
    if ((st = sc.alloc(n, key_bytes_of(key_type), s))) { sc.release(); return st; }
    int buf = 0;
    st = sort_keys(sc, key_type, d_keys, n, descending, &buf, (const u32*)d_values, (u32*)d_sorted_values);
    sc.release();
    return st;
}

extern "C" dcb_status dcb_prefix_sum(dcb_ctx* ctx, int32_t elem_type, const void* d_in, int64_t n, int32_t inclusive, void* d_out, void* stream) {
    if (!ctx) return bad("ctx is null");
    if (n < 0) return bad("n is negative");
    if (!(elem_type == DCB_T_I32 || elem_type == DCB_T_I64 || elem_type == DCB_T_F32 || elem_type == DCB_T_F64)) {
        dcb_set_thread_error("prefix sums are defined for int, long, float and double (project with Select first)");
        return DCB_ERR_NOT_SUPPORTED;
    }
    if (n == 0) return DCB_OK;
    if (!d_in || !d_out) return bad("null pointer");
    if (n > (int64_t)kTile * 0x7fffffffll) return bad("n is too large");
    if (dcb_ctx_make_current(ctx)) return DCB_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)dcb_ctx_pick_stream(ctx, stream);
    dcb_ctx_count_launches(ctx, 3);
    switch (elem_type) {
        case DCB_T_I32: return prefix_sum_typed<int>(d_in, n, inclusive, d_out, s);
        case DCB_T_I64: return prefix_sum_typed<i64>(d_in, n, inclusive, d_out, s);
        case DCB_T_F32: return prefix_sum_typed<float>(d_in, n, inclusive, d_out, s);
        default: return prefix_sum_typed<double>(d_in, n, inclusive, d_out, s);
    }
}

extern "C" dcb_status dcb_gather(dcb_ctx* ctx, int32_t elem_bytes, const void* d_src, const uint32_t* d_indices, int64_t n, void* d_dst, void* stream) {
    if (!ctx) return bad("ctx is null");
    if (n < 0) return bad("n is negative");
    if (n == 0) return DCB_OK;
    if (!d_src || !d_indices || !d_dst) return bad("null pointer");
    if (dcb_ctx_make_current(ctx)) return DCB_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)dcb_ctx_pick_stream(ctx, stream);
    dcb_ctx_count_launches(ctx, 1);
    const int grid = launch_grid(n);
    switch (elem_bytes) {
        case 1: gather_kernel<unsigned char><<<grid, kThreads, 0, s>>>((const unsigned char*)d_src, d_indices, n, (unsigned char*)d_dst); break;
        case 2: gather_kernel<unsigned short><<<grid, kThreads, 0, s>>>((const unsigned short*)d_src, d_indices, n, (unsigned short*)d_dst); break;
        case 4: gather_kernel<u32><<<grid, kThreads, 0, s>>>((const u32*)d_src, d_indices, n, (u32*)d_dst); break;
        case 8: gather_kernel<u64><<<grid, kThreads, 0, s>>>((const u64*)d_src, d_indices, n, (u64*)d_dst); break;
        default: return bad("element size must be 1, 2, 4 or 8 bytes");
    }
    RCU(cudaGetLastError());
    return DCB_OK;
}

template <typename V, bool FP>
static void launch_group_reduce(const void* values, const u32* idx, const u32* excl, const u32* heads, i64 n, int agg, u32* first_idx, u32* counts,
                                double* facc, i64* iacc, cudaStream_t s) {
    group_reduce<V, FP><<<launch_grid(n), kThreads, 0, s>>>((const V*)values, idx, excl, heads, n, agg, first_idx, counts, facc, iacc);
}

extern "C" dcb_status dcb_group_aggregate(dcb_ctx* ctx, int32_t key_type, const void* d_keys, int32_t value_type, const void* d_values, int64_t n,
                                          int32_t aggregate, int64_t out_cap, uint32_t* d_out_first, int64_t* d_out_counts, double* d_out_f64,
                                          int64_t* d_out_i64, int64_t* out_groups, void* stream) {
    if (!ctx) return bad("ctx is null");
    if (dcb_ctx_make_current(ctx)) return DCB_ERR_CUDA;
    if (!out_groups) return bad("out_groups is null");
    *out_groups = 0;
    if (n < 0 || n >= (1ll << 32)) return bad("n must lie in [0, 2^32)");
    if (aggregate < AGG_COUNT || aggregate > AGG_AVERAGE) return bad("unknown aggregate");
    if (n == 0) return DCB_OK;
    if (!d_keys || !d_out_first || !d_out_counts || !d_out_f64 || !d_out_i64) return bad("null pointer");
    if (aggregate != AGG_COUNT && !d_values) return bad("values are null");
    const int kb = key_bytes_of(key_type);
    if (kb == 0) return bad("unsupported key type");
    const bool fp = value_type == DCB_T_F32 || value_type == DCB_T_F64;
    cudaStream_t s = (cudaStream_t)dcb_ctx_pick_stream(ctx, stream);
    dcb_ctx_count_launches(ctx, 12 + 5 * kb);
    SortScratch sc;
    dcb_status st = sc.alloc(n, kb, s);
    u32 *heads = nullptr, *excl = nullptr, *totals = nullptr, *d_total = nullptr;
    u32 *first_idx = nullptr, *counts = nullptr, *order = nullptr;
    double* facc = nullptr; i64* iacc = nullptr;
    SortScratch sg;
    auto cleanup = [&]() {
        sc.release(); sg.release();
        for (void* p : {(void*)heads, (void*)excl, (void*)totals, (void*)d_total, (void*)first_idx, (void*)counts, (void*)order, (void*)facc, (void*)iacc})
            if (p) cudaFreeAsync(p, s);
    };
    if (st) { cleanup(); return st; }
    int buf = 0;
    if ((st = prepare_any(key_type, d_keys, n, 0, sc.keys[0], sc.idx[0], nullptr, s))) { cleanup(); return st; }
    u64 differ = 0;
    if ((st = keys_differ(sc, kb, n, &differ))) { cleanup(); return st; }
    cudaError_t e = cudaSuccess;
    if (differ < 65536ull) {
        // Dense keys: no sort. The table is indexed by the keys' low bits, packed, and emitted in order of first occurrence.
        u32 slots = 1; while ((u64)slots <= differ) slots <<= 1;
        const u32 mask = slots - 1u;
        e = cudaMallocAsync((void**)&first_idx, (size_t)slots * 4, s);
        if (e == cudaSuccess) e = cudaMallocAsync((void**)&counts, (size_t)slots * 4, s);
        if (e == cudaSuccess) e = cudaMallocAsync((void**)&facc, (size_t)slots * 8, s);
        if (e == cudaSuccess) e = cudaMallocAsync((void**)&iacc, (size_t)slots * 8, s);
        if (e == cudaSuccess) e = cudaMallocAsync((void**)&d_total, 16, s);
        if (e != cudaSuccess) { cleanup(); (void)cudaGetLastError(); return DCB_ERR_OUT_OF_MEMORY; }
        dense_init<<<launch_grid(slots), kThreads, 0, s>>>(slots, aggregate, first_idx, counts, facc, iacc);
        const bool ok = kb == 8 ? launch_group_dense_typed<u64>(value_type, d_keys, sc.keys[0], d_values, n, aggregate, mask, first_idx, counts, facc, iacc, s)
                                : launch_group_dense_typed<u32>(value_type, d_keys, sc.keys[0], d_values, n, aggregate, mask, first_idx, counts, facc, iacc, s);
        if (!ok) { cleanup(); return bad("unsupported value type"); }
        dense_pack<<<1, 1024, 0, s>>>(slots, first_idx, counts, facc, iacc, d_total);
        u32 groups = 0;
        e = cudaMemcpyAsync(&groups, d_total, 4, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) { cleanup(); (void)cudaGetLastError(); return DCB_ERR_CUDA; }
        *out_groups = groups;
        if ((int64_t)groups > out_cap) { cleanup(); dcb_set_thread_error("more groups than the outputs hold"); return DCB_ERR_OUTPUT_TOO_SMALL; }
        if ((st = sg.alloc(groups, 4, s))) { cleanup(); return st; }
        int gb = 0;
        if ((st = sort_keys(sg, DCB_T_U32, first_idx, groups, 0, &gb))) { cleanup(); return st; }
        group_emit<<<launch_grid(groups), kThreads, 0, s>>>(sg.idx[gb], first_idx, counts, facc, iacc, groups, aggregate, fp, d_out_first, (i64*)d_out_counts, d_out_f64, (i64*)d_out_i64);
        e = cudaGetLastError();
        cleanup();
        return e == cudaSuccess ? DCB_OK : DCB_ERR_CUDA;
    }
    st = kb == 8 ? radix_sort<u64>(sc, n, &buf, nullptr, &differ) : radix_sort<u32>(sc, n, &buf, nullptr, &differ);
    if (st) { cleanup(); return st; }
    e = cudaMallocAsync((void**)&heads, (size_t)n * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&excl, (size_t)n * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&totals, scan_totals_count(n) * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&d_total, 16, s);
    if (e != cudaSuccess) { cleanup(); (void)cudaGetLastError(); return DCB_ERR_OUT_OF_MEMORY; }
    if (kb == 8) group_heads<u64><<<launch_grid(n), kThreads, 0, s>>>((const u64*)sc.keys[buf], n, heads);
    else group_heads<u32><<<launch_grid(n), kThreads, 0, s>>>((const u32*)sc.keys[buf], n, heads);
    if ((st = exclusive_scan(heads, excl, n, totals, d_total, s))) { cleanup(); return st; }
    u32 groups = 0;
    e = cudaMemcpyAsync(&groups, d_total, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { cleanup(); (void)cudaGetLastError(); return DCB_ERR_CUDA; }
    *out_groups = groups;
    if ((int64_t)groups > out_cap) { cleanup(); dcb_set_thread_error("more groups than the outputs hold"); return DCB_ERR_OUTPUT_TOO_SMALL; }
    e = cudaMallocAsync((void**)&first_idx, (size_t)groups * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&counts, (size_t)groups * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&order, (size_t)groups * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&facc, (size_t)groups * 8, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&iacc, (size_t)groups * 8, s);
    if (e != cudaSuccess) { cleanup(); (void)cudaGetLastError(); return DCB_ERR_OUT_OF_MEMORY; }
    group_init<<<launch_grid(groups), kThreads, 0, s>>>(groups, aggregate, fp, facc, iacc, counts);
    const u32* idx = sc.idx[buf];
    switch (value_type) {
        case DCB_T_F32: launch_group_reduce<float, true>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_F64: launch_group_reduce<double, true>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_I8: launch_group_reduce<signed char, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_U8: case DCB_T_BOOL: launch_group_reduce<unsigned char, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_I16: launch_group_reduce<short, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_U16: launch_group_reduce<unsigned short, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_I32: launch_group_reduce<int, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_U32: launch_group_reduce<u32, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_I64: launch_group_reduce<i64, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        case DCB_T_U64: launch_group_reduce<i64, false>(d_values, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break;
        default:
            if (aggregate == AGG_COUNT) { launch_group_reduce<u32, false>(d_keys, idx, excl, heads, n, aggregate, first_idx, counts, facc, iacc, s); break; }
            cleanup(); return bad("unsupported value type");
    }
    // groups in order of first occurrence: argsort of the groups' first indices
    if ((st = sg.alloc(groups, 4, s))) { cleanup(); return st; }
    int gb = 0;
    if ((st = sort_keys(sg, DCB_T_U32, first_idx, groups, 0, &gb))) { cleanup(); return st; }
    group_emit<<<launch_grid(groups), kThreads, 0, s>>>(sg.idx[gb], first_idx, counts, facc, iacc, groups, aggregate, fp, d_out_first, (i64*)d_out_counts, d_out_f64, (i64*)d_out_i64);
    e = cudaGetLastError();
    cleanup();
    if (e != cudaSuccess) return DCB_ERR_CUDA;
    return DCB_OK;
}

extern "C" dcb_status dcb_join_indices(dcb_ctx* ctx, int32_t key_type, const void* d_outer_keys, int64_t n_outer, const void* d_inner_keys,
                                       int64_t n_inner, int32_t join_kind, int64_t out_cap, uint32_t* d_outer_out, uint32_t* d_inner_out,
                                       int64_t* out_pairs, void* stream) {
    if (!ctx) return bad("ctx is null");
    if (dcb_ctx_make_current(ctx)) return DCB_ERR_CUDA;
    if (!out_pairs) return bad("out_pairs is null");
    *out_pairs = 0;
    if (n_outer < 0 || n_inner < 0 || n_outer >= (1ll << 32) || n_inner >= (1ll << 32)) return bad("sizes must lie in [0, 2^32)");
    if (join_kind != JOIN_INNER && join_kind != JOIN_SEMI && join_kind != JOIN_ANTI) return bad("join kind must be inner (0), semi (2) or anti (3)");
    const int kb = key_bytes_of(key_type);
    if (kb == 0) return bad("unsupported key type");
    if (n_outer == 0) return DCB_OK;
    if (!d_outer_keys || (n_inner > 0 && !d_inner_keys)) return bad("null pointer");
    cudaStream_t s = (cudaStream_t)dcb_ctx_pick_stream(ctx, stream);
    dcb_ctx_count_launches(ctx, 6 + 5 * kb);
    SortScratch sc;
    void* outer_bits = nullptr;
    u32 *lo = nullptr, *cnt = nullptr, *off = nullptr, *totals = nullptr, *d_total = nullptr;
    auto cleanup = [&]() {
        sc.release();
        for (void* p : {outer_bits, (void*)lo, (void*)cnt, (void*)off, (void*)totals, (void*)d_total}) if (p) cudaFreeAsync(p, s);
    };
    dcb_status st = sc.alloc(n_inner, kb, s);
    if (st) { cleanup(); return st; }
    int buf = 0;
    if ((st = sort_keys(sc, key_type, d_inner_keys, n_inner, 0, &buf))) { cleanup(); return st; }
    cudaError_t e = cudaMallocAsync(&outer_bits, (size_t)n_outer * kb, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&lo, (size_t)n_outer * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&cnt, (size_t)n_outer * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&off, (size_t)n_outer * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&totals, scan_totals_count(n_outer) * 4, s);
    if (e == cudaSuccess) e = cudaMallocAsync((void**)&d_total, 16, s);
    if (e != cudaSuccess) { cleanup(); (void)cudaGetLastError(); return DCB_ERR_OUT_OF_MEMORY; }
    if ((st = prepare_any(key_type, d_outer_keys, n_outer, 0, outer_bits, nullptr, nullptr, s))) { cleanup(); return st; }
    if (kb == 8) join_count<u64><<<launch_grid(n_outer), kThreads, 0, s>>>((const u64*)outer_bits, n_outer, (const u64*)sc.keys[buf], (u32)n_inner, join_kind, lo, cnt);
    else join_count<u32><<<launch_grid(n_outer), kThreads, 0, s>>>((const u32*)outer_bits, n_outer, (const u32*)sc.keys[buf], (u32)n_inner, join_kind, lo, cnt);
    if ((st = exclusive_scan(cnt, off, n_outer, totals, d_total, s))) { cleanup(); return st; }
    u32 pairs = 0;
    e = cudaMemcpyAsync(&pairs, d_total, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { cleanup(); (void)cudaGetLastError(); return DCB_ERR_CUDA; }
    *out_pairs = pairs;      // a total beyond 2^32 - 1 is not representable here: the counts are 32-bit
    if (d_outer_out && pairs > 0) {
        join_write<<<launch_grid(n_outer), kThreads, 0, s>>>(lo, cnt, off, n_outer, sc.idx[buf], join_kind, out_cap, d_outer_out, d_inner_out);
        e = cudaGetLastError();
    }
    cleanup();
    if (e != cudaSuccess) return DCB_ERR_CUDA;
    if ((int64_t)pairs > out_cap && d_outer_out) { dcb_set_thread_error("more pairs than the outputs hold"); return DCB_ERR_OUTPUT_TOO_SMALL; }
    return DCB_OK;
}
