// dcb_kernels.cuh — hand-written sm_100a templates for the fused LINQ pipelines.
//
// One "chain" type describes what happens to an element between the source array and the
// terminal operator: a sequence of Select (map) and Where (filter) steps, optionally starting
// with a two-input Zip. The host-side translator emits the chain from the C# lambdas; the three
// kernel bodies below are instantiated on it:
//
//   map_body      Select/Zip only, ToArray       : out[i] = f(in[i])
//   reduce_body   any chain, Sum/Min/Max/Avg/Count: one read of the input, nothing written but a record
//   compact_body  chain with a Where, ToArray     : stable stream compaction, single pass
//
// All three are HBM-bound streaming kernels: 128-bit loads with a streaming cache hint, several
// independent loads in flight per thread, no tensor cores. This file is compiled both by nvcc
// (ahead-of-time instantiations) and by NVRTC (chains built at run time), so it includes nothing.
//
// The semantics reproduced are those of System.Linq over the same lambdas, which is what the
// reference executes for these queries (src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:240-267,
// 344-352, 628-633). The kernels replace the generated `Execute` kernels of
// src/Extensions/DotCompute.Linq/CodeGeneration/CudaKernelGenerator.cs:188-214 (map), 351-376 (filter by
// atomicAdd, unordered), 399-463 (block tree + atomicAdd reduce) and 1058-1134 (fused, un-compacted).
#ifndef DCB_KERNELS_CUH
#define DCB_KERNELS_CUH

namespace dcb {

typedef long long i64;
typedef unsigned long long u64;
typedef unsigned int u32;

// ------------------------------------------------------------------ small type traits
template <typename A, typename B> struct same_t { static constexpr bool value = false; };
template <typename A> struct same_t<A, A> { static constexpr bool value = true; };
template <typename T> struct is_fp { static constexpr bool value = same_t<T, float>::value || same_t<T, double>::value; };
template <typename T> struct is_unsigned_t {
    static constexpr bool value = same_t<T, unsigned char>::value || same_t<T, unsigned short>::value ||
                                  same_t<T, unsigned int>::value || same_t<T, u64>::value || same_t<T, bool>::value;
};

// Reduction selector bits.
enum : int { RED_SUM = 1, RED_MIN = 2, RED_MAX = 4, RED_COUNT = 8 };

// Flag bits in the record (low bits match DCB_RES_* of the C ABI).
enum : u32 { FLAG_SAW_NAN = 1u, FLAG_TRUNCATED = 2u, FLAG_TIMEOUT = 4u, FLAG_OVERFLOW = 8u, FLAG_SAW_NUMBER = 16u };

// The record a run leaves in device memory: 16 eight-byte slots (see DCB_SLOT_* in dcb200.h).
struct __align__(16) DeviceResult {
    double fsum;     // 0
    double count_f;  // 1
    i64 isum_lo;     // 2
    i64 isum_hi;     // 3
    i64 count;       // 4
    double fmin;     // 5
    double fmax;     // 6
    i64 imin;        // 7
    i64 imax;        // 8
    u64 flags;       // 9
    i64 pad[6];
};

// Per-block partial of a reduction, also the shared-memory exchange format.
struct __align__(16) Partial {
    double fsum;
    u64 isum_lo;
    i64 isum_hi;
    i64 count;
    i64 mn_bits;   // minimum: raw bits of a double for floating elements, else the sign- or zero-extended integer
    i64 mx_bits;
    u32 flags;
    u32 pad0;
    i64 pad1;
};

// Partials are written by one block and read by another: go through L2 explicitly.
__device__ __forceinline__ void partial_store(Partial* dst, const Partial& p) {
    const uint4* s = reinterpret_cast<const uint4*>(&p);
    uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(Partial) / 16); ++i) __stcg(d + i, s[i]);
}
__device__ __forceinline__ void partial_load(Partial& p, const Partial* src) {
    uint4* d = reinterpret_cast<uint4*>(&p);
    const uint4* s = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(Partial) / 16); ++i) d[i] = __ldcg(s + i);
}

// ------------------------------------------------------------------ packs: E elements moved as one unit
template <typename T, int E>
struct Pack {
    static constexpr int BYTES = (int)sizeof(T) * E;
    static constexpr int NQ = (BYTES + 15) / 16;
    union {
        T e[E];
        uint4 q[NQ];
        uint2 d;
        unsigned int w;
        unsigned short h;
        unsigned char b;
    };
    __device__ __forceinline__ Pack() {}
    // Streaming load: the data is read exactly once, so it is marked evict-first (ld.global.cs).
    __device__ __forceinline__ void load(const T* __restrict__ p) {
        if constexpr (BYTES % 16 == 0) {
#pragma unroll
            for (int i = 0; i < NQ; ++i) q[i] = __ldcs(reinterpret_cast<const uint4*>(p) + i);
        } else if constexpr (BYTES == 8) {
            d = __ldcs(reinterpret_cast<const uint2*>(p));
        } else if constexpr (BYTES == 4) {
            w = __ldcs(reinterpret_cast<const unsigned int*>(p));
        } else if constexpr (BYTES == 2) {
            h = __ldcs(reinterpret_cast<const unsigned short*>(p));
        } else if constexpr (BYTES == 1) {
            b = __ldcs(reinterpret_cast<const unsigned char*>(p));
        } else {
#pragma unroll
            for (int i = 0; i < E; ++i) e[i] = p[i];
        }
    }
    __device__ __forceinline__ void store(T* __restrict__ p) const {
        if constexpr (BYTES % 16 == 0) {
#pragma unroll
            for (int i = 0; i < NQ; ++i) __stcs(reinterpret_cast<uint4*>(p) + i, q[i]);
        } else if constexpr (BYTES == 8) {
            __stcs(reinterpret_cast<uint2*>(p), d);
        } else if constexpr (BYTES == 4) {
            __stcs(reinterpret_cast<unsigned int*>(p), w);
        } else if constexpr (BYTES == 2) {
            __stcs(reinterpret_cast<unsigned short*>(p), h);
        } else if constexpr (BYTES == 1) {
            __stcs(reinterpret_cast<unsigned char*>(p), b);
        } else {
#pragma unroll
            for (int i = 0; i < E; ++i) p[i] = e[i];
        }
    }
};

// Elements per 16-byte vector of the first input; the unit every vector kernel works in.
template <class C, bool VEC> struct pack_elems { static constexpr int value = VEC ? 16 / (int)sizeof(typename C::in0_t) : 1; };

// ------------------------------------------------------------------ accumulator of a reduction
template <typename T, int RED>
struct Acc {
    double fsum;
    u64 isum_lo;
    i64 isum_hi;
    i64 count;
    u32 cnt32;     // per-thread running count; folded into `count` by finish()
    T mn, mx;
    u32 flags;

    __device__ __forceinline__ void finish() { count += (i64)cnt32; cnt32 = 0; }
    __device__ __forceinline__ void init() {
        fsum = 0.0; isum_lo = 0; isum_hi = 0; count = 0; cnt32 = 0; flags = 0;
        if constexpr (same_t<T, float>::value) { mn = __int_as_float(0x7f800000); mx = __int_as_float(0xff800000); }
        else if constexpr (same_t<T, double>::value) { mn = __longlong_as_double(0x7ff0000000000000LL); mx = __longlong_as_double(0xfff0000000000000LL); }
        else if constexpr (same_t<T, bool>::value) { mn = true; mx = false; }
        else if constexpr (is_unsigned_t<T>::value) { mn = (T)~(T)0; mx = (T)0; }
        else if constexpr (sizeof(T) == 1) { mn = (T)127; mx = (T)(-128); }
        else if constexpr (sizeof(T) == 2) { mn = (T)32767; mx = (T)(-32768); }
        else if constexpr (sizeof(T) == 4) { mn = (T)0x7fffffff; mx = (T)(-0x7fffffff - 1); }
        else { mn = (T)0x7fffffffffffffffLL; mx = (T)(-0x7fffffffffffffffLL - 1LL); }
    }
    __device__ __forceinline__ void add(T v) {
        if constexpr ((RED & RED_SUM) != 0) {
            if constexpr (is_fp<T>::value) {
                fsum += (double)v;            // fp64 accumulation, as Enumerable.Sum(float) does
            } else if constexpr (sizeof(T) == 8) {
                const u64 x = (u64)v;         // 128-bit two's complement sum: exact, overflow decided at the end
                const u64 s = isum_lo + x;
                isum_hi += (s < x ? 1 : 0) + ((!is_unsigned_t<T>::value && (i64)x < 0) ? -1 : 0);
                isum_lo = s;
            } else {
                isum_lo += (u64)(i64)v;       // at most 2^63 / 2^32 addends before wrap: exact in 64 bits
            }
        }
        if constexpr ((RED & (RED_MIN | RED_MAX)) != 0) {
            if constexpr (is_fp<T>::value) {
                if (v != v) flags |= FLAG_SAW_NAN;
                else {
                    flags |= FLAG_SAW_NUMBER;
                    if constexpr ((RED & RED_MIN) != 0) mn = v < mn ? v : mn;
                    if constexpr ((RED & RED_MAX) != 0) mx = v > mx ? v : mx;
                }
            } else {
                if constexpr ((RED & RED_MIN) != 0) mn = v < mn ? v : mn;
                if constexpr ((RED & RED_MAX) != 0) mx = v > mx ? v : mx;
            }
        }
        if constexpr ((RED & (RED_COUNT | RED_MIN | RED_MAX)) != 0) cnt32 += 1u;   // Sum alone needs no count
    }
    // Fixed-shape combine: `this` is the left (lower-index) operand.
    __device__ __forceinline__ void merge(const Acc& o) {
        if constexpr ((RED & RED_SUM) != 0) {
            if constexpr (is_fp<T>::value) fsum += o.fsum;
            else {
                const u64 s = isum_lo + o.isum_lo;
                isum_hi += o.isum_hi + (s < o.isum_lo ? 1 : 0);
                isum_lo = s;
            }
        }
        if constexpr ((RED & RED_MIN) != 0) mn = o.mn < mn ? o.mn : mn;
        if constexpr ((RED & RED_MAX) != 0) mx = o.mx > mx ? o.mx : mx;
        flags |= o.flags;
        count += o.count + (i64)o.cnt32;
    }
    __device__ __forceinline__ Acc shuffled(int lane_mask) const {
        Acc r;
        r.fsum = 0.0; r.isum_lo = 0; r.isum_hi = 0; r.mn = mn; r.mx = mx; r.cnt32 = 0;
        if constexpr ((RED & RED_SUM) != 0) {
            if constexpr (is_fp<T>::value) r.fsum = __shfl_xor_sync(0xffffffffu, fsum, lane_mask);
            else {
                r.isum_lo = __shfl_xor_sync(0xffffffffu, isum_lo, lane_mask);
                if constexpr (sizeof(T) == 8) r.isum_hi = __shfl_xor_sync(0xffffffffu, isum_hi, lane_mask);
            }
        }
        if constexpr ((RED & RED_MIN) != 0) r.mn = shfl_val(mn, lane_mask);
        if constexpr ((RED & RED_MAX) != 0) r.mx = shfl_val(mx, lane_mask);
        r.flags = __shfl_xor_sync(0xffffffffu, flags, lane_mask);
        r.count = __shfl_xor_sync(0xffffffffu, count + (i64)cnt32, lane_mask);
        return r;
    }
    static __device__ __forceinline__ T shfl_val(T v, int lane_mask) {
        if constexpr (sizeof(T) == 8) {
            union { T t; u64 u; } a; a.t = v;
            a.u = __shfl_xor_sync(0xffffffffu, a.u, lane_mask);
            return a.t;
        } else if constexpr (same_t<T, float>::value) {
            return __shfl_xor_sync(0xffffffffu, v, lane_mask);
        } else {
            return (T)__shfl_xor_sync(0xffffffffu, (int)v, lane_mask);
        }
    }
    __device__ __forceinline__ void to_partial(Partial& p) const {
        p.fsum = fsum; p.isum_lo = isum_lo; p.isum_hi = isum_hi; p.count = count + (i64)cnt32; p.flags = flags;
        p.pad0 = 0; p.pad1 = 0;
        if constexpr (is_fp<T>::value) { p.mn_bits = __double_as_longlong((double)mn); p.mx_bits = __double_as_longlong((double)mx); }
        else { p.mn_bits = (i64)mn; p.mx_bits = (i64)mx; }
    }
    __device__ __forceinline__ void from_partial(const Partial& p) {
        fsum = p.fsum; isum_lo = p.isum_lo; isum_hi = p.isum_hi; count = p.count; cnt32 = 0; flags = p.flags;
        if constexpr (is_fp<T>::value) { mn = (T)__longlong_as_double(p.mn_bits); mx = (T)__longlong_as_double(p.mx_bits); }
        else { mn = (T)p.mn_bits; mx = (T)p.mx_bits; }
    }
};

// Warp butterfly in a fixed order, then one shared-memory stage: the value every block computes
// depends only on the data and the launch shape, never on timing.
template <typename T, int RED, int BLOCK>
__device__ __forceinline__ Acc<T, RED> block_reduce(Acc<T, RED> a, Partial* smem /* BLOCK/32 entries */) {
    a.finish();
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
        Acc<T, RED> o = a.shuffled(m);
        // Keep left/right order stable so that floating sums are reproducible.
        if ((threadIdx.x & m) == 0) a.merge(o); else { o.merge(a); a = o; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) a.to_partial(smem[warp]);
    __syncthreads();
    if (warp == 0) {
        Acc<T, RED> b; b.init();
        if (lane < BLOCK / 32) b.from_partial(smem[lane]);
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
            Acc<T, RED> o = b.shuffled(m);
            if ((lane & m) == 0) b.merge(o); else { o.merge(b); b = o; }
        }
        a = b;
    }
    __syncthreads();
    return a;   // valid in warp 0 (all lanes hold the block total)
}

// ------------------------------------------------------------------ chain application helpers
template <class C>
__device__ __forceinline__ bool apply_chain(const typename C::in0_t& a, const typename C::in1_t& b, typename C::out_t& o) {
    return C::apply(a, b, o);
}

// ------------------------------------------------------------------ map: out[i] = f(in0[i] [, in1[i]])
// Grid-stride over tiles of BLOCK*UNROLL packs; all UNROLL loads of a thread are issued before the first use.
template <class C, int BLOCK, int UNROLL, bool VEC>
__device__ __forceinline__ void map_body(const typename C::in0_t* __restrict__ in0, const typename C::in1_t* __restrict__ in1,
                                         i64 n, typename C::out_t* __restrict__ out) {
    typedef typename C::in0_t A; typedef typename C::in1_t B; typedef typename C::out_t O;
    constexpr int E = pack_elems<C, VEC>::value;
    const i64 nitems = n / E;
    const i64 tile_items = (i64)BLOCK * UNROLL;
    const i64 ntiles = nitems / tile_items;
    for (i64 t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const i64 base = t * tile_items + threadIdx.x;
        Pack<A, E> a[UNROLL]; Pack<B, E> b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            a[u].load(in0 + (base + (i64)u * BLOCK) * E);
            if constexpr (C::n_in == 2) b[u].load(in1 + (base + (i64)u * BLOCK) * E);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            Pack<O, E> o;
#pragma unroll
            for (int k = 0; k < E; ++k) {
                if constexpr (C::n_in == 2) C::apply(a[u].e[k], b[u].e[k], o.e[k]);
                else C::apply(a[u].e[k], B(), o.e[k]);
            }
            o.store(out + (base + (i64)u * BLOCK) * E);
        }
    }
    const i64 gtid = (i64)blockIdx.x * BLOCK + threadIdx.x, gsize = (i64)gridDim.x * BLOCK;
    for (i64 it = ntiles * tile_items + gtid; it < nitems; it += gsize) {
        Pack<A, E> a; Pack<B, E> b; Pack<O, E> o;
        a.load(in0 + it * E);
        if constexpr (C::n_in == 2) b.load(in1 + it * E);
#pragma unroll
        for (int k = 0; k < E; ++k) {
            if constexpr (C::n_in == 2) C::apply(a.e[k], b.e[k], o.e[k]);
            else C::apply(a.e[k], B(), o.e[k]);
        }
        o.store(out + it * E);
    }
    for (i64 i = nitems * E + gtid; i < n; i += gsize) {
        O o;
        if constexpr (C::n_in == 2) C::apply(in0[i], in1[i], o); else C::apply(in0[i], B(), o);
        out[i] = o;
    }
}

// ------------------------------------------------------------------ reduce: chain + Sum/Min/Max/Count in one read
// Persistent grid. Each block leaves its partial in slot blockIdx.x; the block that takes the last
// ticket combines the slots in index order. Nothing depends on which block finishes first.
template <class C, int RED, int BLOCK, int UNROLL, bool VEC>
__device__ __forceinline__ void reduce_body(const typename C::in0_t* __restrict__ in0, const typename C::in1_t* __restrict__ in1,
                                            i64 n, Partial* __restrict__ partials, unsigned int* __restrict__ ticket,
                                            DeviceResult* __restrict__ res) {
    typedef typename C::in0_t A; typedef typename C::in1_t B; typedef typename C::out_t O;
    constexpr int E = pack_elems<C, VEC>::value;
    __shared__ Partial s_part[BLOCK / 32];
    __shared__ bool s_last;

    Acc<O, RED> acc; acc.init();
    const i64 nitems = n / E;
    const i64 tile_items = (i64)BLOCK * UNROLL;
    const i64 ntiles = nitems / tile_items;
    for (i64 t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const i64 base = t * tile_items + threadIdx.x;
        Pack<A, E> a[UNROLL]; Pack<B, E> b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            a[u].load(in0 + (base + (i64)u * BLOCK) * E);
            if constexpr (C::n_in == 2) b[u].load(in1 + (base + (i64)u * BLOCK) * E);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int k = 0; k < E; ++k) {
                O o; bool keep;
                if constexpr (C::n_in == 2) keep = C::apply(a[u].e[k], b[u].e[k], o);
                else keep = C::apply(a[u].e[k], B(), o);
                if (keep) acc.add(o);
            }
        }
    }
    const i64 gtid = (i64)blockIdx.x * BLOCK + threadIdx.x, gsize = (i64)gridDim.x * BLOCK;
    for (i64 it = ntiles * tile_items + gtid; it < nitems; it += gsize) {
        Pack<A, E> a; Pack<B, E> b;
        a.load(in0 + it * E);
        if constexpr (C::n_in == 2) b.load(in1 + it * E);
#pragma unroll
        for (int k = 0; k < E; ++k) {
            O o; bool keep;
            if constexpr (C::n_in == 2) keep = C::apply(a.e[k], b.e[k], o); else keep = C::apply(a.e[k], B(), o);
            if (keep) acc.add(o);
        }
    }
    for (i64 i = nitems * E + gtid; i < n; i += gsize) {
        O o; bool keep;
        if constexpr (C::n_in == 2) keep = C::apply(in0[i], in1[i], o); else keep = C::apply(in0[i], B(), o);
        if (keep) acc.add(o);
    }

    acc = block_reduce<O, RED, BLOCK>(acc, s_part);
    if (threadIdx.x == 0) {
        Partial p; acc.to_partial(p);
        partial_store(partials + blockIdx.x, p);
        __threadfence();
        const unsigned int t = atomicAdd(ticket, 1u);
        s_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Last block: thread k folds slots k, k+BLOCK, ... in increasing order, then the same block tree.
    Acc<O, RED> tot; tot.init();
    for (unsigned int s = threadIdx.x; s < gridDim.x; s += BLOCK) {
        Partial p; partial_load(p, partials + s);
        Acc<O, RED> o; o.from_partial(p);
        tot.merge(o);
    }
    tot = block_reduce<O, RED, BLOCK>(tot, s_part);
    if (threadIdx.x == 0) {
        Partial p; tot.to_partial(p);
        res->fsum = p.fsum; res->count_f = (double)p.count;
        res->isum_lo = (i64)p.isum_lo; res->isum_hi = (sizeof(O) == 8) ? p.isum_hi : ((i64)p.isum_lo < 0 ? -1 : 0);
        res->count = p.count;
        if constexpr (is_fp<O>::value) { res->fmin = __longlong_as_double(p.mn_bits); res->fmax = __longlong_as_double(p.mx_bits); res->imin = 0; res->imax = 0; }
        else { res->fmin = 0; res->fmax = 0; res->imin = p.mn_bits; res->imax = p.mx_bits; }
        res->flags = p.flags;
        *ticket = 0;   // ready for the next launch on this stream
    }
}

// ------------------------------------------------------------------ compact: stable Where [-> Select] -> ToArray
// Tile descriptors for the decoupled look-back: one 64-bit word = epoch(14) | status(2) | value(48),
// written and read with single relaxed accesses, so status and value can never be seen torn.
enum : u64 { DESC_VALUE_MASK = (1ull << 48) - 1ull };
enum : u32 { ST_INVALID = 0, ST_AGGREGATE = 1, ST_INCLUSIVE = 2 };

__device__ __forceinline__ u64 desc_make(u32 epoch, u32 status, u64 value) {
    return ((u64)(epoch & 0x3fffu) << 50) | ((u64)status << 48) | (value & DESC_VALUE_MASK);
}
__device__ __forceinline__ void desc_store(u64* p, u64 v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 desc_load(const u64* p) {
    u64 v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ u32 desc_status(u64 d, u32 epoch) {
    return ((u32)(d >> 50) & 0x3fffu) == (epoch & 0x3fffu) ? (u32)((d >> 48) & 3u) : (u32)ST_INVALID;
}

// Rows per warp: as many as keep the staging tile within 32 KB of shared memory, at most 4 (64 bytes in flight per thread).
template <class C, int BLOCK, bool VEC> struct compact_rows {
    static constexpr int per_row = BLOCK * pack_elems<C, VEC>::value * (int)sizeof(typename C::out_t);
    static constexpr int fit = 32768 / per_row;
    static constexpr int value = fit < 1 ? 1 : (fit > 4 ? 4 : fit);
};

// Tile = BLOCK threads, each warp owns ROWS rows of 32 packs (a contiguous run of ROWS*32*E elements).
// Element order inside a warp's run is row, then lane, then position in the pack; ranks follow it.
template <class C, int BLOCK, int ROWS, bool VEC>
__device__ __forceinline__ void compact_body(const typename C::in0_t* __restrict__ in0, const typename C::in1_t* __restrict__ in1,
                                             i64 n, typename C::out_t* __restrict__ out, i64 out_cap,
                                             u64* __restrict__ desc, unsigned int* __restrict__ tile_counter,
                                             u32 epoch, u32 spin_limit, i64 num_tiles,
                                             const DeviceResult* __restrict__ prev, DeviceResult* __restrict__ res,
                                             unsigned int* __restrict__ abort_flag) {
    typedef typename C::in0_t A; typedef typename C::in1_t B; typedef typename C::out_t O;
    constexpr int E = pack_elems<C, VEC>::value;
    constexpr int WARPS = BLOCK / 32;
    constexpr int WARP_ELEMS = ROWS * 32 * E;
    constexpr int TILE = WARPS * WARP_ELEMS;

    __shared__ O s_stage[TILE];
    __shared__ int s_warp_tot[WARPS];
    __shared__ i64 s_tile_prefix;
    __shared__ i64 s_tile;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(tile_counter, 1u);   // ids in arrival order: a tile's predecessors already run
        if ((i64)t == num_tiles - 1) *tile_counter = 0;       // every other tile has drawn its id by now
        s_tile = (i64)t;
    }
    __syncthreads();
    const i64 tile = s_tile;
    const i64 tile_base = tile * TILE;
    const i64 warp_base = tile_base + (i64)warp * WARP_ELEMS;

    // 1. loads
    Pack<A, E> a[ROWS]; Pack<B, E> b[ROWS];
    const bool full = tile_base + TILE <= n;
    if (full) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const i64 idx = warp_base + ((i64)r * 32 + lane) * E;
            a[r].load(in0 + idx);
            if constexpr (C::n_in == 2) b[r].load(in1 + idx);
        }
    } else {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const i64 idx = warp_base + ((i64)r * 32 + lane) * E;
#pragma unroll
            for (int k = 0; k < E; ++k) {
                if (idx + k < n) {
                    a[r].e[k] = in0[idx + k];
                    if constexpr (C::n_in == 2) b[r].e[k] = in1[idx + k];
                } else {
                    a[r].e[k] = A();
                    if constexpr (C::n_in == 2) b[r].e[k] = B();
                }
            }
        }
    }

    // 2. chain + ranks inside the warp (ballot / popc)
    O val[ROWS][E];
    u64 keepbits = 0;                      // bit r*E+k
    int rank[ROWS];                        // rank of this lane's first survivor in row r, within the warp run
    int warp_run = 0;
    const unsigned int lt_mask = (1u << lane) - 1u;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        int before = 0, row_total = 0;
#pragma unroll
        for (int k = 0; k < E; ++k) {
            bool keep;
            if constexpr (C::n_in == 2) keep = C::apply(a[r].e[k], b[r].e[k], val[r][k]);
            else keep = C::apply(a[r].e[k], B(), val[r][k]);
            if (!full) keep = keep && (warp_base + ((i64)r * 32 + lane) * E + k < n);
            const unsigned int bal = __ballot_sync(0xffffffffu, keep);
            before += __popc(bal & lt_mask);
            row_total += __popc(bal);
            keepbits |= (u64)(keep ? 1u : 0u) << (r * E + k);
        }
        rank[r] = warp_run + before;
        warp_run += row_total;
    }
    if (lane == 0) s_warp_tot[warp] = warp_run;
    __syncthreads();
    int warp_off = 0, tile_total = 0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        const int t = s_warp_tot[w];
        if (w < warp) warp_off += t;
        tile_total += t;
    }

    // 3. publish the aggregate, stage survivors, and let warp 0 look back meanwhile
    if (threadIdx.x == 0) {
        if (tile == 0) {
            const i64 base0 = prev ? prev->count : 0;
            desc_store(desc + tile, desc_make(epoch, ST_INCLUSIVE, (u64)tile_total));
            s_tile_prefix = base0;
        } else {
            desc_store(desc + tile, desc_make(epoch, ST_AGGREGATE, (u64)tile_total));
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        int pos = warp_off + rank[r];
#pragma unroll
        for (int k = 0; k < E; ++k) {
            if ((keepbits >> (r * E + k)) & 1ull) { s_stage[pos] = val[r][k]; ++pos; }
        }
    }
    if (warp == 0 && tile > 0) {
        // Each lane inspects one predecessor; the window slides back 32 tiles at a time until a
        // tile with an inclusive prefix is met.
        i64 exclusive = 0;
        i64 look = tile - 1;
        bool failed = false;
        while (true) {
            const i64 idx = look - lane;
            u64 d = 0; u32 st = ST_INCLUSIVE;
            if (idx >= 0) {
                u32 polls = 0;
                d = desc_load(desc + idx);
                st = desc_status(d, epoch);
                while (st == ST_INVALID) {
                    if (++polls > spin_limit || *(volatile unsigned int*)abort_flag == epoch) { failed = true; break; }
                    if (polls > 16) __nanosleep(polls > 1024 ? 256 : 32);
                    d = desc_load(desc + idx);
                    st = desc_status(d, epoch);
                }
            }
            if (__any_sync(0xffffffffu, failed)) { failed = true; break; }
            const unsigned int incl = __ballot_sync(0xffffffffu, st == ST_INCLUSIVE);
            const int first = incl ? (__ffs(incl) - 1) : 32;
            i64 contrib = (lane <= first && idx >= 0) ? (i64)(d & DESC_VALUE_MASK) : 0;
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, m);
            exclusive += contrib;
            if (incl) break;
            look -= 32;
        }
        if (lane == 0) {
            if (failed) {
                // A wait ran out (or another tile's did). Tell the tiles still waiting, and leave a record that says
                // so; every tile after the stuck one ends here too, so the last tile cannot overwrite it with success.
                atomicExch(abort_flag, epoch);
                res->count = 0; res->count_f = 0; res->flags = (u64)FLAG_TIMEOUT;
                s_tile_prefix = -1;
            } else {
                const i64 base0 = prev ? prev->count : 0;
                desc_store(desc + tile, desc_make(epoch, ST_INCLUSIVE, (u64)(exclusive + tile_total)));
                s_tile_prefix = base0 + exclusive;
            }
        }
    }
    __syncthreads();
    const i64 prefix = s_tile_prefix;
    if (prefix < 0) return;                 // a bounded wait ran out: leave without writing

    // 4. coalesced write of the staged survivors
    for (int i = threadIdx.x; i < tile_total; i += BLOCK) {
        const i64 pos = prefix + i;
        if (pos < out_cap) out[pos] = s_stage[i];
    }
    if (tile == num_tiles - 1 && threadIdx.x == 0) {
        const i64 total = prefix + tile_total;
        res->count = total; res->count_f = (double)total;
        res->fsum = 0; res->isum_lo = 0; res->isum_hi = 0; res->fmin = 0; res->fmax = 0; res->imin = 0; res->imax = 0;
        res->flags = total > out_cap ? (u64)FLAG_TRUNCATED : 0ull;
    }
}

}  // namespace dcb
#endif  // DCB_KERNELS_CUH
