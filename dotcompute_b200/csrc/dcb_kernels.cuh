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
//   compact_stream_body  the same, warp-specialised persistent blocks whose input arrives by asynchronous bulk copies
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

// The bits of a value in an unsigned integer of the same size (what memcpy would give).
template <typename U, typename T>
__device__ __forceinline__ void memcpy_bits(U& dst, const T& src) {
    static_assert(sizeof(U) == sizeof(T), "same size");
    union { T t; U u; } c;
    c.t = src;
    dst = c.u;
}

// Reduction selector bits.
enum : int { RED_SUM = 1, RED_MIN = 2, RED_MAX = 4, RED_COUNT = 8, RED_FIRST = 16, RED_LAST = 32 };   // FIRST / LAST: smallest / largest index of a surviving element

// Flag bits in the record (low bits match DCB_RES_* of the C ABI).
enum : u32 { FLAG_SAW_NAN = 1u, FLAG_TRUNCATED = 2u, FLAG_TIMEOUT = 4u, FLAG_OVERFLOW = 8u, FLAG_SAW_NUMBER = 16u,
             FLAG_PREFIX = 32u,     // PREFIX: slots 12..15 hold the smallest and the largest running sum (checked integer Sum)
             FLAG_DIV0 = 64u, FLAG_DIV_OVERFLOW = 128u };   // an integer / or % of a lambda: zero divisor, MinValue / -1

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
    i64 offset;      // 10: after an exchange between GPUs: survivors (elements counted) on lower ranks; else 0
    i64 local_count; // 11: after an exchange: this GPU's own count (slot 4 then holds the total); else equal to slot 4
    i64 pad[4];      // 12..15: checked integer Sum: smallest running sum (low, high word), largest running sum (low, high word)
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
    // Plain load, for a pack that lies in shared memory (the cache hints above exist for global memory only).
    __device__ __forceinline__ void load_shared(const T* p) {
        if constexpr (BYTES % 16 == 0) {
#pragma unroll
            for (int i = 0; i < NQ; ++i) q[i] = reinterpret_cast<const uint4*>(p)[i];
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
    i64 ifirst, ilast;   // RED_FIRST / RED_LAST: index of the first / last element that passed the chain
    i64 zfirst;          // floating Min / Max: 2 * index + sign bit of the earliest zero seen (see zero_sign below)
    u32 flags;

    __device__ __forceinline__ void finish() { count += (i64)cnt32; cnt32 = 0; }
    __device__ __forceinline__ void init() {
        fsum = 0.0; isum_lo = 0; isum_hi = 0; count = 0; cnt32 = 0; flags = 0;
        ifirst = 0x7fffffffffffffffLL; ilast = -1; zfirst = 0x7fffffffffffffffLL;
        if constexpr (same_t<T, float>::value) { mn = __int_as_float(0x7f800000); mx = __int_as_float(0xff800000); }
        else if constexpr (same_t<T, double>::value) { mn = __longlong_as_double(0x7ff0000000000000LL); mx = __longlong_as_double(0xfff0000000000000LL); }
        else if constexpr (same_t<T, bool>::value) { mn = true; mx = false; }
        else if constexpr (is_unsigned_t<T>::value) { mn = (T)~(T)0; mx = (T)0; }
        else if constexpr (sizeof(T) == 1) { mn = (T)127; mx = (T)(-128); }
        else if constexpr (sizeof(T) == 2) { mn = (T)32767; mx = (T)(-32768); }
        else if constexpr (sizeof(T) == 4) { mn = (T)0x7fffffff; mx = (T)(-0x7fffffff - 1); }
        else { mn = (T)0x7fffffffffffffffLL; mx = (T)(-0x7fffffffffffffffLL - 1LL); }
    }
    __device__ __forceinline__ void add(T v, i64 idx) {
        if constexpr ((RED & RED_FIRST) != 0) ifirst = idx < ifirst ? idx : ifirst;
        if constexpr ((RED & RED_LAST) != 0) ilast = idx > ilast ? idx : ilast;
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
        if constexpr ((RED & (RED_COUNT | RED_MIN | RED_MAX | RED_FIRST | RED_LAST)) != 0) cnt32 += 1u;   // Sum alone needs no count
    }
    // Enumerable.Min / Max replace their candidate only on a strict comparison, so among -0 and +0 (equal to each other)
    // the one that comes first in the sequence is returned. note_zero remembers which that is; callers test a whole pack
    // for zeros with one branch and call it only then (a branch per element costs a quarter of the kernel's time).
    static constexpr bool TRACK_ZERO = is_fp<T>::value && (RED & (RED_MIN | RED_MAX)) != 0;
    __device__ __forceinline__ void note_zero(T v, i64 idx) {
        if (v == T(0)) {
            const i64 z = idx * 2 + (signbit_of(v) ? 1 : 0);
            zfirst = z < zfirst ? z : zfirst;
        }
    }
    static __device__ __forceinline__ bool signbit_of(T v) {
        if constexpr (same_t<T, float>::value) return (__float_as_uint(v) >> 31) != 0u;
        else if constexpr (same_t<T, double>::value) return ((u64)__double_as_longlong(v) >> 63) != 0ull;
        else return false;
    }
    // The sign a zero result of Min / Max carries: that of the earliest zero in the sequence.
    __device__ __forceinline__ void zero_sign() {
        if constexpr (is_fp<T>::value && (RED & (RED_MIN | RED_MAX)) != 0) {
            if (zfirst != 0x7fffffffffffffffLL) {
                const T z = (zfirst & 1) ? -T(0) : T(0);
                if constexpr ((RED & RED_MIN) != 0) { if (mn == T(0)) mn = z; }
                if constexpr ((RED & RED_MAX) != 0) { if (mx == T(0)) mx = z; }
            }
        }
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
        if constexpr ((RED & RED_FIRST) != 0) ifirst = o.ifirst < ifirst ? o.ifirst : ifirst;
        if constexpr ((RED & RED_LAST) != 0) ilast = o.ilast > ilast ? o.ilast : ilast;
        if constexpr (is_fp<T>::value && (RED & (RED_MIN | RED_MAX)) != 0) zfirst = o.zfirst < zfirst ? o.zfirst : zfirst;
        flags |= o.flags;
        count += o.count + (i64)o.cnt32;
    }
    __device__ __forceinline__ Acc shuffled(int lane_mask) const {
        Acc r;
        r.fsum = 0.0; r.isum_lo = 0; r.isum_hi = 0; r.mn = mn; r.mx = mx; r.cnt32 = 0; r.ifirst = ifirst; r.ilast = ilast; r.zfirst = zfirst;
        if constexpr (is_fp<T>::value && (RED & (RED_MIN | RED_MAX)) != 0) r.zfirst = __shfl_xor_sync(0xffffffffu, zfirst, lane_mask);
        if constexpr ((RED & RED_FIRST) != 0) r.ifirst = __shfl_xor_sync(0xffffffffu, ifirst, lane_mask);
        if constexpr ((RED & RED_LAST) != 0) r.ilast = __shfl_xor_sync(0xffffffffu, ilast, lane_mask);
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
        if constexpr (is_fp<T>::value && (RED & (RED_MIN | RED_MAX)) != 0) p.pad1 = zfirst;
        if constexpr ((RED & (RED_FIRST | RED_LAST)) != 0) { p.mn_bits = ifirst; p.mx_bits = ilast; }   // index reductions use the Min / Max slots
        else if constexpr (is_fp<T>::value) { p.mn_bits = __double_as_longlong((double)mn); p.mx_bits = __double_as_longlong((double)mx); }
        else { p.mn_bits = (i64)mn; p.mx_bits = (i64)mx; }
    }
    // Read from a block's slot only what this reduction accumulates (the slot was written by another block: via L2).
    __device__ __forceinline__ void load_live(const Partial* p) {
        if constexpr ((RED & RED_SUM) != 0) {
            if constexpr (is_fp<T>::value) fsum = __ldcg(&p->fsum);
            else { isum_lo = __ldcg(&p->isum_lo); if constexpr (sizeof(T) == 8) isum_hi = __ldcg(&p->isum_hi); }
        }
        if constexpr ((RED & (RED_COUNT | RED_MIN | RED_MAX | RED_FIRST | RED_LAST)) != 0) count = __ldcg(&p->count);
        if constexpr ((RED & RED_FIRST) != 0) ifirst = __ldcg(&p->mn_bits);
        if constexpr ((RED & RED_LAST) != 0) ilast = __ldcg(&p->mx_bits);
        if constexpr ((RED & RED_MIN) != 0) {
            const i64 b = __ldcg(&p->mn_bits);
            if constexpr (is_fp<T>::value) mn = (T)__longlong_as_double(b); else mn = (T)b;
        }
        if constexpr ((RED & RED_MAX) != 0) {
            const i64 b = __ldcg(&p->mx_bits);
            if constexpr (is_fp<T>::value) mx = (T)__longlong_as_double(b); else mx = (T)b;
        }
        if constexpr ((RED & (RED_MIN | RED_MAX)) != 0 && is_fp<T>::value) { flags = __ldcg(&p->flags); zfirst = __ldcg(&p->pad1); }
    }
    __device__ __forceinline__ void from_partial(const Partial& p) {
        fsum = p.fsum; isum_lo = p.isum_lo; isum_hi = p.isum_hi; count = p.count; cnt32 = 0; flags = p.flags;
        ifirst = 0x7fffffffffffffffLL; ilast = -1; zfirst = 0x7fffffffffffffffLL;
        if constexpr (is_fp<T>::value && (RED & (RED_MIN | RED_MAX)) != 0) zfirst = p.pad1;
        if constexpr ((RED & (RED_FIRST | RED_LAST)) != 0) { ifirst = p.mn_bits; ilast = p.mx_bits; mn = T(); mx = T(); }
        else if constexpr (is_fp<T>::value) { mn = (T)__longlong_as_double(p.mn_bits); mx = (T)__longlong_as_double(p.mx_bits); }
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

// Which block is the last of the grid to get here? All blocks of a launch finish within a microsecond of each other, and
// several hundred atomics on one word are served one after the other: the last ticket would be drawn microseconds after
// the last block was ready. So the blocks take tickets in 64 groups (word 1 + blockIdx % 64) and only the last of each
// group goes on to the main word (word 0): a microsecond less per launch at 888 blocks than one word for all, measured
// three times in turn on one GPU (74.7 against 75.8 us a step over 2^27 floats; sixteen groups: no gain). Call from one thread, after the block's partial is stored; the caller
// puts a __threadfence() before it and another one before reading other blocks' partials. Resets the words when last.
#ifndef DCB_TICKET_GROUPS
#define DCB_TICKET_GROUPS 64
#endif
__device__ __forceinline__ bool last_block_ticket(unsigned int* ticket) {
    constexpr unsigned int G = DCB_TICKET_GROUPS;
    const unsigned int g = blockIdx.x % G;
    const unsigned int in_group = (gridDim.x + G - 1u - g) / G;          // blocks with this residue
    if (atomicAdd(ticket + 1 + g, 1u) != in_group - 1u) return false;
    __threadfence();
    const unsigned int groups = gridDim.x < G ? gridDim.x : G;           // residues that have a block at all
    if (atomicAdd(ticket, 1u) != groups - 1u) return false;
    for (unsigned int i = 0; i <= G; ++i) ticket[i] = 0;                   // ready for the next launch on this stream
    return true;
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

    // Programmatic dependent launch (only when the host asked for it at launch; otherwise both instructions do nothing):
    // the next kernel on the stream may start while this one runs, and this one may have started while its predecessor
    // was still running. What such a pair shares - the partials, the ticket, the record - is touched only after the wait
    // below, which returns once the predecessor has completed and its writes are visible; the input is read before it, so
    // the host sets the launch attribute only when the caller has said the inputs are not written by the work just before.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    Acc<O, RED> acc; acc.init();
    // Whole tiles of BLOCK*UNROLL packs are dealt round-robin, the same number to every block, so that at any moment all
    // blocks read from one compact window that moves through the array (measured faster than giving each block its own
    // distant range). What is left over, less than one tile per block, is split evenly so all blocks finish together.
    const i64 nitems = n / E;
    const i64 tile_items = (i64)BLOCK * UNROLL;
    const i64 rounds = (nitems / tile_items) / gridDim.x;
    for (i64 r = 0; r < rounds; ++r) {
        const i64 base = (r * gridDim.x + blockIdx.x) * tile_items + threadIdx.x;
        Pack<A, E> a[UNROLL]; Pack<B, E> b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            a[u].load(in0 + (base + (i64)u * BLOCK) * E);
            if constexpr (C::n_in == 2) b[u].load(in1 + (base + (i64)u * BLOCK) * E);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            O ov[E]; bool kv[E]; bool zero = false;
#pragma unroll
            for (int k = 0; k < E; ++k) {
                if constexpr (C::n_in == 2) kv[k] = C::apply(a[u].e[k], b[u].e[k], ov[k]);
                else kv[k] = C::apply(a[u].e[k], B(), ov[k]);
                if (kv[k]) acc.add(ov[k], (base + (i64)u * BLOCK) * E + k);
                if constexpr (Acc<O, RED>::TRACK_ZERO) zero = zero || (kv[k] && ov[k] == O(0));
            }
            if constexpr (Acc<O, RED>::TRACK_ZERO) {
                if (zero) {
#pragma unroll
                    for (int k = 0; k < E; ++k) if (kv[k]) acc.note_zero(ov[k], (base + (i64)u * BLOCK) * E + k);
                }
            }
        }
    }
    const i64 rest_lo = rounds * gridDim.x * tile_items;
    const i64 per_block = (nitems - rest_lo + gridDim.x - 1) / gridDim.x;          // < tile_items + 1
    const i64 off = rest_lo + (i64)blockIdx.x * per_block < nitems ? rest_lo + (i64)blockIdx.x * per_block : nitems;
    const i64 range_hi = off + per_block < nitems ? off + per_block : nitems;
    {   // the block's share of the leftover: at most UNROLL packs per thread, still issued together
        Pack<A, E> a[UNROLL]; Pack<B, E> b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const i64 it = off + threadIdx.x + (i64)u * BLOCK;
            if (it < range_hi) {
                a[u].load(in0 + it * E);
                if constexpr (C::n_in == 2) b[u].load(in1 + it * E);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const i64 it = off + threadIdx.x + (i64)u * BLOCK;
            if (it < range_hi) {
#pragma unroll
                for (int k = 0; k < E; ++k) {
                    O o; bool keep;
                    if constexpr (C::n_in == 2) keep = C::apply(a[u].e[k], b[u].e[k], o);
                    else keep = C::apply(a[u].e[k], B(), o);
                    if (keep) { acc.add(o, it * E + k); if constexpr (Acc<O, RED>::TRACK_ZERO) acc.note_zero(o, it * E + k); }
                }
            }
        }
    }
    const i64 gtid = (i64)blockIdx.x * BLOCK + threadIdx.x, gsize = (i64)gridDim.x * BLOCK;
    for (i64 i = nitems * E + gtid; i < n; i += gsize) {   // the last n % E elements
        O o; bool keep;
        if constexpr (C::n_in == 2) keep = C::apply(in0[i], in1[i], o); else keep = C::apply(in0[i], B(), o);
        if (keep) { acc.add(o, i); if constexpr (Acc<O, RED>::TRACK_ZERO) acc.note_zero(o, i); }
    }

    acc = block_reduce<O, RED, BLOCK>(acc, s_part);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        Partial p; acc.to_partial(p);
        partial_store(partials + blockIdx.x, p);
        __threadfence();
        s_last = last_block_ticket(ticket);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Last block: thread k folds slots k, k+BLOCK, ... in increasing order, then the same block tree. Only the fields
    // this reduction uses are read, FOLD slots at a time so that their loads are in flight together.
    Acc<O, RED> tot; tot.init();
    constexpr int FOLD = 6;
    for (unsigned int s0 = threadIdx.x; s0 < gridDim.x; s0 += BLOCK * FOLD) {
        Acc<O, RED> o[FOLD];
#pragma unroll
        for (int f = 0; f < FOLD; ++f) {
            o[f].init();
            const unsigned int sl = s0 + (unsigned int)f * BLOCK;
            if (sl < gridDim.x) o[f].load_live(partials + sl);
        }
#pragma unroll
        for (int f = 0; f < FOLD; ++f) tot.merge(o[f]);
    }
    tot = block_reduce<O, RED, BLOCK>(tot, s_part);
    if (threadIdx.x == 0) {
        tot.zero_sign();
        Partial p; tot.to_partial(p);
        res->fsum = p.fsum; res->count_f = (double)p.count;
        res->isum_lo = (i64)p.isum_lo; res->isum_hi = (sizeof(O) == 8) ? p.isum_hi : ((i64)p.isum_lo < 0 ? -1 : 0);
        res->count = p.count;
        if constexpr ((RED & (RED_FIRST | RED_LAST)) != 0) { res->fmin = 0; res->fmax = 0; res->imin = p.mn_bits; res->imax = p.mx_bits; }
        else if constexpr (is_fp<O>::value) { res->fmin = __longlong_as_double(p.mn_bits); res->fmax = __longlong_as_double(p.mx_bits); res->imin = 0; res->imax = 0; }
        else { res->fmin = 0; res->fmax = 0; res->imin = p.mn_bits; res->imax = p.mx_bits; }
        res->flags = p.flags;
        res->offset = 0; res->local_count = p.count;
    }
}

// ------------------------------------------------------------------ checked integer Sum: the range of the running sum
// Enumerable.Sum(int) and Sum(long) add in a checked context, element by element in source order: the call throws as soon
// as a *running* sum leaves the element type's range, even if later elements would bring the total back. So the kernel
// needs, beside the total, the smallest and the largest running sum. Per segment that is a triple (s, lo, hi) with lo and
// hi relative to the segment's start and counting the empty prefix (lo <= 0 <= hi); two adjacent segments combine as
// (s1 + s2, min(lo1, s1 + lo2), max(hi1, s1 + hi2)) - associative, not commutative, so everything below keeps source order.
// Wide arithmetic: 64 bits for elements of up to 32 bits, 128 bits for 64-bit elements; neither can wrap for n < 2^63.
struct Wide128 {
    u64 lo; i64 hi;
    __device__ __forceinline__ Wide128() {}
    __device__ __forceinline__ explicit Wide128(i64 v) : lo((u64)v), hi(v < 0 ? -1 : 0) {}
    __device__ __forceinline__ Wide128 operator+(const Wide128& o) const {
        Wide128 r; r.lo = lo + o.lo; r.hi = hi + o.hi + (r.lo < lo ? 1 : 0); return r;
    }
    __device__ __forceinline__ bool operator<(const Wide128& o) const { return hi < o.hi || (hi == o.hi && lo < o.lo); }
};
template <typename O> struct prefix_wide { typedef i64 type; };
template <> struct prefix_wide<long long> { typedef Wide128 type; };
__device__ __forceinline__ i64 wide_shfl_xor(i64 v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
__device__ __forceinline__ Wide128 wide_shfl_xor(const Wide128& v, int m) {
    Wide128 r; r.lo = __shfl_xor_sync(0xffffffffu, v.lo, m); r.hi = __shfl_xor_sync(0xffffffffu, v.hi, m); return r;
}
__device__ __forceinline__ u64 wide_low(i64 v) { return (u64)v; }
__device__ __forceinline__ i64 wide_high(i64 v) { return v < 0 ? -1 : 0; }
__device__ __forceinline__ u64 wide_low(const Wide128& v) { return v.lo; }
__device__ __forceinline__ i64 wide_high(const Wide128& v) { return v.hi; }
__device__ __forceinline__ void wide_set(i64& w, u64 lo, i64) { w = (i64)lo; }
__device__ __forceinline__ void wide_set(Wide128& w, u64 lo, i64 hi) { w.lo = lo; w.hi = hi; }

template <typename W>
struct PrefixTriple {
    W s, lo, hi;
    __device__ __forceinline__ void zero() { s = W(0); lo = W(0); hi = W(0); }
    __device__ __forceinline__ void push(i64 v) {            // one more element at the end
        s = s + W(v);
        if (s < lo) lo = s;
        if (hi < s) hi = s;
    }
    __device__ __forceinline__ void append(const PrefixTriple& b) {   // `b` is the segment right after this one
        const W l = s + b.lo, h = s + b.hi;
        if (l < lo) lo = l;
        if (hi < h) hi = h;
        s = s + b.s;
    }
};
// One lane's CNT consecutive values. When all of them are small enough for every running sum to fit the element type
// itself, the arithmetic is done in that type (a third of the instructions); else in the wide type.
template <typename O, int CNT>
__device__ __forceinline__ void lane_prefix(const O (&v)[CNT], PrefixTriple<typename prefix_wide<O>::type>& t) {
    typedef typename prefix_wide<O>::type W;
    constexpr int LOG2 = CNT <= 1 ? 0 : CNT <= 2 ? 1 : CNT <= 4 ? 2 : CNT <= 8 ? 3 : CNT <= 16 ? 4 : CNT <= 32 ? 5 : CNT <= 64 ? 6 : 7;
    static_assert(CNT <= 128, "too many elements per lane");
    if constexpr (sizeof(O) == 4) {
        u32 m = 0;
#pragma unroll
        for (int i = 0; i < CNT; ++i) m |= (u32)((int)v[i] ^ ((int)v[i] >> 31));      // magnitude bits of every value
        if (m < (1u << (31 - LOG2))) {
            int s = 0, lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < CNT; ++i) { s += (int)v[i]; lo = s < lo ? s : lo; hi = s > hi ? s : hi; }
            t.s = W((i64)s); t.lo = W((i64)lo); t.hi = W((i64)hi);
            return;
        }
    } else {
        u64 m = 0;
#pragma unroll
        for (int i = 0; i < CNT; ++i) m |= (u64)((i64)v[i] ^ ((i64)v[i] >> 63));
        if (m < (1ull << (63 - LOG2))) {
            i64 s = 0, lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < CNT; ++i) { s += (i64)v[i]; lo = s < lo ? s : lo; hi = s > hi ? s : hi; }
            t.s = W(s); t.lo = W(lo); t.hi = W(hi);
            return;
        }
    }
    t.zero();
#pragma unroll
    for (int i = 0; i < CNT; ++i) t.push((i64)v[i]);
}

// The slot a block leaves for the fold: same 64 bytes as a Partial.
struct __align__(16) PrefixPartial { u64 s_lo; i64 s_hi; u64 mn_lo; i64 mn_hi; u64 mx_lo; i64 mx_hi; u64 pad[2]; };
static_assert(sizeof(PrefixPartial) == sizeof(Partial), "the checked Sum reuses the reduction's partial slots");

// Warp-wide minimum / maximum of wide integers: the high words first (one redux), then the low words of the lanes that tie.
__device__ __forceinline__ i64 warp_min_wide(i64 v) {
    const int h = (int)(v >> 32), mh = __reduce_min_sync(0xffffffffu, h);
    const u32 ml = __reduce_min_sync(0xffffffffu, h == mh ? (u32)v : 0xffffffffu);
    return (i64)(((u64)(u32)mh << 32) | ml);
}
__device__ __forceinline__ i64 warp_max_wide(i64 v) {
    const int h = (int)(v >> 32), mh = __reduce_max_sync(0xffffffffu, h);
    const u32 ml = __reduce_max_sync(0xffffffffu, h == mh ? (u32)v : 0u);
    return (i64)(((u64)(u32)mh << 32) | ml);
}
__device__ __forceinline__ u64 warp_min_u64(u64 v) {
    const u32 h = (u32)(v >> 32), mh = __reduce_min_sync(0xffffffffu, h);
    const u32 ml = __reduce_min_sync(0xffffffffu, h == mh ? (u32)v : 0xffffffffu);
    return ((u64)mh << 32) | ml;
}
__device__ __forceinline__ u64 warp_max_u64(u64 v) {
    const u32 h = (u32)(v >> 32), mh = __reduce_max_sync(0xffffffffu, h);
    const u32 ml = __reduce_max_sync(0xffffffffu, h == mh ? (u32)v : 0u);
    return ((u64)mh << 32) | ml;
}
__device__ __forceinline__ Wide128 warp_min_wide(const Wide128& v) {
    Wide128 r; r.hi = warp_min_wide(v.hi); r.lo = warp_min_u64(v.hi == r.hi ? v.lo : ~0ull); return r;
}
__device__ __forceinline__ Wide128 warp_max_wide(const Wide128& v) {
    Wide128 r; r.hi = warp_max_wide(v.hi); r.lo = warp_max_u64(v.hi == r.hi ? v.lo : 0ull); return r;
}
__device__ __forceinline__ i64 wide_shfl_up(i64 v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ __forceinline__ Wide128 wide_shfl_up(const Wide128& v, int d) {
    Wide128 r; r.lo = __shfl_up_sync(0xffffffffu, v.lo, d); r.hi = __shfl_up_sync(0xffffffffu, v.hi, d); return r;
}
__device__ __forceinline__ i64 wide_shfl(i64 v, int src) { return __shfl_sync(0xffffffffu, v, src); }
__device__ __forceinline__ Wide128 wide_shfl(const Wide128& v, int src) {
    Wide128 r; r.lo = __shfl_sync(0xffffffffu, v.lo, src); r.hi = __shfl_sync(0xffffffffu, v.hi, src); return r;
}

// The lanes' segments appended in lane order; every lane gets the warp's triple. Instead of appending triples pairwise
// (three wide values through every shuffle step), the totals alone are scanned; a lane's extremes, moved by the sum of
// the lanes before it, are then absolute within the warp and an ordinary minimum / maximum finishes the job.
template <typename W>
__device__ __forceinline__ PrefixTriple<W> warp_prefix_append(const PrefixTriple<W>& t) {
    const int lane = threadIdx.x & 31;
    W incl = t.s;
#pragma unroll
    for (int d = 1; d <= 16; d <<= 1) {
        const W up = wide_shfl_up(incl, d);
        if (lane >= d) incl = incl + up;
    }
    W before = wide_shfl_up(incl, 1);
    if (lane == 0) before = W(0);
    PrefixTriple<W> r;
    r.lo = warp_min_wide(before + t.lo);
    r.hi = warp_max_wide(before + t.hi);
    r.s = wide_shfl(incl, 31);
    return r;
}
template <typename W>
__device__ __forceinline__ void prefix_to_slot(PrefixPartial* dst, const PrefixTriple<W>& t) {
    uint4 q0, q1, q2;
    const u64 a = wide_low(t.s), c = wide_low(t.lo), e = wide_low(t.hi);
    const i64 b = wide_high(t.s), d = wide_high(t.lo), f = wide_high(t.hi);
    q0.x = (u32)a; q0.y = (u32)(a >> 32); q0.z = (u32)(u64)b; q0.w = (u32)((u64)b >> 32);
    q1.x = (u32)c; q1.y = (u32)(c >> 32); q1.z = (u32)(u64)d; q1.w = (u32)((u64)d >> 32);
    q2.x = (u32)e; q2.y = (u32)(e >> 32); q2.z = (u32)(u64)f; q2.w = (u32)((u64)f >> 32);
    uint4* p = reinterpret_cast<uint4*>(dst);
    __stcg(p, q0); __stcg(p + 1, q1); __stcg(p + 2, q2);
}
template <typename W>
__device__ __forceinline__ void prefix_from_slot(PrefixTriple<W>& t, const PrefixPartial* src) {
    const uint4* p = reinterpret_cast<const uint4*>(src);
    const uint4 q0 = __ldcg(p), q1 = __ldcg(p + 1), q2 = __ldcg(p + 2);
    wide_set(t.s, (u64)q0.x | ((u64)q0.y << 32), (i64)((u64)q0.z | ((u64)q0.w << 32)));
    wide_set(t.lo, (u64)q1.x | ((u64)q1.y << 32), (i64)((u64)q1.z | ((u64)q1.w << 32)));
    wide_set(t.hi, (u64)q2.x | ((u64)q2.y << 32), (i64)((u64)q2.z | ((u64)q2.w << 32)));
}
// Warp triples -> block triple, in warp order. Valid in warp 0.
template <typename W, int BLOCK>
__device__ __forceinline__ PrefixTriple<W> block_prefix_append(PrefixTriple<W> a, PrefixTriple<W>* smem /* BLOCK/32 */) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    a = warp_prefix_append(a);
    if (lane == 0) smem[warp] = a;
    __syncthreads();
    PrefixTriple<W> b; b.zero();
    if (warp == 0) {
        if (lane < BLOCK / 32) b = smem[lane];
        b = warp_prefix_append(b);
    }
    __syncthreads();
    return b;
}

// Persistent grid, same launch and same scratch as reduce_body. Every *warp* owns one contiguous range of the input and
// every lane UNROLL consecutive packs of each warp tile, so that a lane's elements, a warp's lanes, a block's warps and the
// grid's blocks are each in source order; the last block appends the block triples in index order. The record carries the
// exact total (slots 2, 3), the smallest and largest running sum (slots 12..15) and FLAG_OVERFLOW if either left O's range.
template <class C, int BLOCK, int UNROLL, bool VEC>
__device__ __forceinline__ void sum_checked_body(const typename C::in0_t* __restrict__ in0, const typename C::in1_t* __restrict__ in1,
                                                 i64 n, Partial* __restrict__ partials, unsigned int* __restrict__ ticket,
                                                 DeviceResult* __restrict__ res) {
    typedef typename C::in0_t A; typedef typename C::in1_t B; typedef typename C::out_t O;
    typedef typename prefix_wide<O>::type W;
    static_assert(sizeof(O) == 4 || sizeof(O) == 8, "checked Sum is defined for int and long");
    constexpr int E = pack_elems<C, VEC>::value;
    constexpr int WARPS = BLOCK / 32;
    __shared__ PrefixTriple<W> s_tri[WARPS];
    __shared__ bool s_last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // same launch protocol as reduce_body

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const i64 nitems = n / E;
    const i64 total_warps = (i64)gridDim.x * WARPS, gw = (i64)blockIdx.x * WARPS + warp;
    constexpr i64 WTILE = 32 * UNROLL;                                 // packs per warp tile
    i64 per = (nitems + total_warps - 1) / total_warps;
    per = (per + WTILE - 1) / WTILE * WTILE;
    const i64 lo_pack = gw * per < nitems ? gw * per : nitems;
    const i64 hi_pack = lo_pack + per < nitems ? lo_pack + per : nitems;

    PrefixTriple<W> run; run.zero();
    for (i64 base = lo_pack; base < hi_pack; base += WTILE) {
        const i64 p0 = base + (i64)lane * UNROLL;
        Pack<A, E> a[UNROLL]; Pack<B, E> b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (p0 + u < hi_pack) {
                a[u].load(in0 + (p0 + u) * E);
                if constexpr (C::n_in == 2) b[u].load(in1 + (p0 + u) * E);
            }
        }
        // An element the chain drops, or beyond the range, counts as 0: adding 0 changes neither the sum nor its range.
        O vals[UNROLL * E];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int k = 0; k < E; ++k) {
                O o = O(0); bool keep = false;
                if (p0 + u < hi_pack) {
                    if constexpr (C::n_in == 2) keep = C::apply(a[u].e[k], b[u].e[k], o);
                    else keep = C::apply(a[u].e[k], B(), o);
                }
                vals[u * E + k] = keep ? o : O(0);
            }
        }
        PrefixTriple<W> t;
        if constexpr (sizeof(O) == 8) {
            // 64-bit elements: when every lane's values are small enough for the whole warp's running sums to fit 64 bits
            // (magnitudes below 2^54 for eight elements a lane: always, in practice), the warp-wide append is done in 64
            // bits as well - a third of the instructions of the 128-bit one, which otherwise dominates this kernel.
            constexpr int CNT = UNROLL * E;
            constexpr int LOG2 = CNT <= 1 ? 0 : CNT <= 2 ? 1 : CNT <= 4 ? 2 : CNT <= 8 ? 3 : CNT <= 16 ? 4 : CNT <= 32 ? 5 : 6;
            u64 m = 0;
#pragma unroll
            for (int i = 0; i < CNT; ++i) m |= (u64)((i64)vals[i] ^ ((i64)vals[i] >> 63));
            if (__all_sync(0xffffffffu, m < (1ull << (57 - LOG2)))) {
                PrefixTriple<i64> n; n.zero();
#pragma unroll
                for (int i = 0; i < CNT; ++i) n.push((i64)vals[i]);
                n = warp_prefix_append(n);
                t.s = W(n.s); t.lo = W(n.lo); t.hi = W(n.hi);
            } else {
                lane_prefix<O, CNT>(vals, t);
                t = warp_prefix_append(t);
            }
        } else {
            lane_prefix<O, UNROLL * E>(vals, t);
            t = warp_prefix_append(t);
        }
        run.append(t);
    }
    if (gw == total_warps - 1) {   // the last n % E elements come after every pack: the last warp appends them
        PrefixTriple<W> t; t.zero();
        if (lane == 0) {
            for (i64 i = nitems * E; i < n; ++i) {
                O o; bool keep;
                if constexpr (C::n_in == 2) keep = C::apply(in0[i], in1[i], o); else keep = C::apply(in0[i], B(), o);
                if (keep) t.push((i64)o);
            }
        }
        t = warp_prefix_append(t);
        run.append(t);
    }
    // every lane of a warp holds the warp's triple; make lane 0's the one that counts and the others empty
    if (lane != 0) run.zero();
    PrefixTriple<W> blk = block_prefix_append<W, BLOCK>(run, s_tri);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    PrefixPartial* slots = reinterpret_cast<PrefixPartial*>(partials);
    if (threadIdx.x == 0) {
        prefix_to_slot(slots + blockIdx.x, blk);
        __threadfence();
        s_last = last_block_ticket(ticket);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Last block: thread k appends the slots of its own contiguous run, then the block appends the threads' triples in order.
    const unsigned int per_thread = (gridDim.x + BLOCK - 1) / BLOCK;
    PrefixTriple<W> tot; tot.zero();
    for (unsigned int j = 0; j < per_thread; ++j) {
        const unsigned int sl = threadIdx.x * per_thread + j;
        if (sl < gridDim.x) { PrefixTriple<W> o; prefix_from_slot(o, slots + sl); tot.append(o); }
    }
    tot = block_prefix_append<W, BLOCK>(tot, s_tri);
    if (threadIdx.x == 0) {
        W mn, mx;
        if constexpr (sizeof(O) == 4) { mn = W(-2147483647LL - 1LL); mx = W(2147483647LL); }
        else { mn = W(-0x7fffffffffffffffLL - 1LL); mx = W(0x7fffffffffffffffLL); }
        const bool overflow = (tot.lo < mn) || (mx < tot.hi);
        res->fsum = 0.0; res->count_f = 0.0;
        res->isum_lo = (i64)wide_low(tot.s); res->isum_hi = wide_high(tot.s);
        res->count = 0; res->fmin = 0; res->fmax = 0; res->imin = 0; res->imax = 0;
        res->flags = (u64)(FLAG_PREFIX | (overflow ? FLAG_OVERFLOW : 0u));
        res->offset = 0; res->local_count = 0;
        res->pad[0] = (i64)wide_low(tot.lo); res->pad[1] = wide_high(tot.lo);
        res->pad[2] = (i64)wide_low(tot.hi); res->pad[3] = wide_high(tot.hi);
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

// Compaction tile shape: 256 threads, 8 rows per warp (128 bytes in flight per thread), fewer rows if the staging tile
// would exceed 32 KB of shared memory; four such blocks share an SM. Of the shapes measured on B200 (128 / 256 threads,
// 2 / 4 / 8 rows, 4 to 16 resident blocks) this one was fastest. One definition for device templates and host launch code.
__host__ __device__ constexpr int compact_rows_for(int block, int elems_per_pack, int out_bytes) {
    return 32768 / (block * elems_per_pack * out_bytes) < 1 ? 1
         : (32768 / (block * elems_per_pack * out_bytes) > 8 ? 8 : 32768 / (block * elems_per_pack * out_bytes));
}
template <class C, int BLOCK, bool VEC> struct compact_rows {
    static constexpr int value = compact_rows_for(BLOCK, pack_elems<C, VEC>::value, (int)sizeof(typename C::out_t));
};

// Chain, ranks and staging of one warp's run of a tile, whose packs the lanes hold in registers (row r of lane l is
// pack r*32+l of the run); returns the number of survivors the warp staged, compacted and in source order, at `stage`.
// FULL = the whole tile lies inside the array, so no element needs a bound check.
template <class C, int ROWS, int E, bool FULL>
__device__ __forceinline__ int compact_rank_and_stage(const Pack<typename C::in0_t, E> (&a)[ROWS], const Pack<typename C::in1_t, E> (&b)[ROWS],
                                                      i64 n, i64 warp_base, int lane, typename C::out_t* stage, i64 lo = 0) {
    typedef typename C::in0_t A; typedef typename C::in1_t B; typedef typename C::out_t O;
    // Per-row survivor counts of a lane are packed FIELD bits apiece into 32-bit words, so one shuffle scan ranks
    // several rows at once. A row total is at most 32*E, which fits 8 bits up to E = 4 (128 = 0x80), else 16.
    constexpr int FIELD = (32 * E <= 128) ? 8 : 16;
    constexpr int PER_WORD = 32 / FIELD;
    constexpr int WORDS = (ROWS + PER_WORD - 1) / PER_WORD;
    constexpr u32 FMASK = (FIELD == 8) ? 0xffu : 0xffffu;
    // 2. chain, per-lane survivor bits and counts
    O val[ROWS][E];
    u32 keepbits[ROWS];
    u32 packed[WORDS];
#pragma unroll
    for (int w = 0; w < WORDS; ++w) packed[w] = 0;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        u32 bits = 0;
#pragma unroll
        for (int k = 0; k < E; ++k) {
            bool keep;
            if constexpr (C::n_in == 2) keep = C::apply(a[r].e[k], b[r].e[k], val[r][k]);
            else keep = C::apply(a[r].e[k], B(), val[r][k]);
            if constexpr (!FULL) {
                const i64 idx = warp_base + ((i64)r * 32 + lane) * E + k;
                keep = keep && idx < n && idx >= lo;
            }
            bits |= (keep ? 1u : 0u) << k;
        }
        keepbits[r] = bits;
        packed[r / PER_WORD] |= (u32)__popc(bits) << ((r % PER_WORD) * FIELD);
    }
    // 3. ranks: inclusive scan of the packed counts across the warp (fields cannot carry into each other)
    u32 incl[WORDS];
#pragma unroll
    for (int w = 0; w < WORDS; ++w) {
        u32 v = packed[w];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d) v += t;
        }
        incl[w] = v;
    }
    int row_start = 0;
    int rank[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int w = r / PER_WORD, sh = (r % PER_WORD) * FIELD;
        const u32 tot_word = __shfl_sync(0xffffffffu, incl[w], 31);
        const int before = (int)(((incl[w] - packed[w]) >> sh) & FMASK);
        rank[r] = row_start + before;
        row_start += (int)((tot_word >> sh) & FMASK);
    }
    const int warp_run = row_start;
    // 4. stage the survivors, compacted, in the warp's run
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        int pos = rank[r];
#pragma unroll
        for (int k = 0; k < E; ++k) {
            if ((keepbits[r] >> k) & 1u) { stage[pos] = val[r][k]; ++pos; }
        }
    }
    return warp_run;
}

// Loads of one warp's run from global memory, then compact_rank_and_stage.
template <class C, int BLOCK, int ROWS, bool VEC, bool FULL>
__device__ __forceinline__ int compact_count_and_stage(const typename C::in0_t* __restrict__ in0, const typename C::in1_t* __restrict__ in1,
                                                       i64 n, i64 warp_base, int lane, typename C::out_t* __restrict__ stage) {
    typedef typename C::in0_t A; typedef typename C::in1_t B;
    constexpr int E = pack_elems<C, VEC>::value;
    // all rows of the thread are in flight before the first is used
    Pack<A, E> a[ROWS]; Pack<B, E> b[ROWS];
    if constexpr (FULL) {
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

    return compact_rank_and_stage<C, ROWS, E, FULL>(a, b, n, warp_base, lane, stage);
}


// Decoupled look-back of tile `tile` (> 0), run by one whole warp after the tile's own descriptor was published:
// returns, in every lane, the number of survivors of all earlier tiles, or sets `failed` when a bounded wait ran out.
__device__ __forceinline__ i64 compact_lookback(const u64* __restrict__ desc, i64 tile, int lane, u32 epoch, u32 spin_limit,
                                                const unsigned int* abort_flag, bool& failed_out) {
    // One step inspects LOOK_WIN*32 predecessors, nearest first: sub-window j holds tiles look-32j-lane. All loads
    // of a step are issued before the first is examined. The walk stops at the nearest tile whose inclusive
    // prefix is known. Every poll loop is bounded.
    constexpr int LOOK_WIN = 2;
    i64 exclusive = 0;
    i64 look = tile - 1;
    bool failed = false, done = false;
    while (!done && !failed) {

        u64 d[LOOK_WIN];
#pragma unroll
        for (int j = 0; j < LOOK_WIN; ++j) {
            const i64 idx = look - (i64)j * 32 - lane;
            d[j] = idx >= 0 ? desc_load(desc + idx) : desc_make(epoch, ST_INCLUSIVE, 0);   // before tile 0: empty, inclusive
        }
#pragma unroll
        for (int j = 0; j < LOOK_WIN; ++j) {
            if (done || failed) break;
            const i64 idx = look - (i64)j * 32 - lane;
            u32 st = desc_status(d[j], epoch);
            u32 polls = 0;
            while (st == ST_INVALID) {
                // the abort word is looked at every 16th poll only: every poller shares its L2 path
                if (++polls > spin_limit || ((polls & 15u) == 0u && *(volatile unsigned int*)abort_flag == epoch)) { failed = true; break; }
                // Back off before asking again: a poll is an L2 round trip, and hundreds of warps share these lines.
#ifndef DCB_POLL_SLEEP_NS
#define DCB_POLL_SLEEP_NS 200
#endif
                __nanosleep(polls > 4096 ? 4 * DCB_POLL_SLEEP_NS : DCB_POLL_SLEEP_NS);

                d[j] = desc_load(desc + idx);
                st = desc_status(d[j], epoch);
            }
            if (__any_sync(0xffffffffu, failed)) { failed = true; break; }
            const unsigned int inc = __ballot_sync(0xffffffffu, st == ST_INCLUSIVE);
            const int first = inc ? (__ffs(inc) - 1) : 32;
            if (lane <= first) exclusive += (i64)(d[j] & DESC_VALUE_MASK);
            if (inc) done = true;
        }
        look -= 32 * LOOK_WIN;
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) exclusive += __shfl_xor_sync(0xffffffffu, exclusive, m);
    failed_out = failed;
    return exclusive;
}

// A warp copies its staged run of `warp_run` survivors to out[base ...]; consecutive lanes write consecutive elements.
template <typename O, bool VEC>
__device__ __forceinline__ void compact_copy_out(O* __restrict__ out, i64 out_cap, i64 base, int warp_run, int lane, const O* stage) {
    if (base + warp_run <= out_cap) {                      // the usual case: no per-element bound check
        O* __restrict__ dst = out + base;
        constexpr int VO = (sizeof(O) == 4 || sizeof(O) == 8) ? 16 / (int)sizeof(O) : 1;
        if constexpr (VEC && VO > 1) {
            // A few single elements up to the next 16-byte boundary of the destination, then 16-byte stores (one
            // instruction moves VO elements), then the last few. Works for any element-aligned `out`.
            const int mis = (int)(((unsigned long long)dst & 15ull) / sizeof(O));
            int head = (VO - mis) & (VO - 1);
            if (head > warp_run) head = warp_run;
            if (lane < head) dst[lane] = stage[lane];
            const int nvec = (warp_run - head) / VO;
#pragma unroll 2
            for (int v = lane; v < nvec; v += 32) {
                Pack<O, VO> q;
#pragma unroll
                for (int k = 0; k < VO; ++k) q.e[k] = stage[head + v * VO + k];
                q.store(dst + head + v * VO);
            }
            const int done = head + nvec * VO;
            if (lane < warp_run - done) dst[done + lane] = stage[done + lane];
        } else {
            // Batches of eight per lane: all loads of a batch are issued before its first store, so a batch pays the
            // shared-memory latency once (a rolled loop pays it on every element).
            constexpr int BATCH = 8;
            for (int i0 = 0; i0 < warp_run; i0 += 32 * BATCH) {
                O v[BATCH];
#pragma unroll
                for (int j = 0; j < BATCH; ++j) {
                    const int i = i0 + j * 32 + lane;
                    if (i < warp_run) v[j] = stage[i];
                }
#pragma unroll
                for (int j = 0; j < BATCH; ++j) {
                    const int i = i0 + j * 32 + lane;
                    if (i < warp_run) dst[i] = v[j];
                }
            }
        }
    } else {
        for (int i = lane; i < warp_run; i += 32) {
            const i64 pos = base + i;
            if (pos < out_cap) out[pos] = stage[i];
        }
    }
}

// Tile = BLOCK threads; each warp owns ROWS rows of 32 packs, a contiguous run of ROWS*32*E elements. Element order
// inside a warp's run is row, then lane, then position in the pack; ranks follow it, so the output keeps source order.
//
// One tile per block, tile id = blockIdx.x. The look-back waits on tiles with smaller ids, i.e. on blocks the hardware
// dispatched earlier (a 1-D grid is dispatched in index order; NVIDIA's own single-pass scan relies on the same). Should
// that ever not hold, the bounded polls below end the launch with FLAG_TIMEOUT instead of hanging the GPU.
template <class C, int BLOCK, int ROWS, bool VEC>
__device__ __forceinline__ void compact_body(const typename C::in0_t* __restrict__ in0, const typename C::in1_t* __restrict__ in1,
                                             i64 n, typename C::out_t* __restrict__ out, i64 out_cap,
                                             u64* __restrict__ desc, u32 epoch, u32 spin_limit, i64 num_tiles,
                                             const DeviceResult* __restrict__ prev, DeviceResult* __restrict__ res,
                                             unsigned int* __restrict__ abort_flag) {
    typedef typename C::in0_t A; typedef typename C::in1_t B; typedef typename C::out_t O;
    constexpr int E = pack_elems<C, VEC>::value;
    constexpr int WARPS = BLOCK / 32;
    constexpr int WARP_ELEMS = ROWS * 32 * E;
    constexpr int TILE = WARPS * WARP_ELEMS;

    __shared__ O s_stage[TILE];           // warp w stages its survivors, compacted, at [w*WARP_ELEMS, ...)
    __shared__ int s_warp_tot[WARPS];
    __shared__ i64 s_prefix;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const i64 tile = blockIdx.x;
    const i64 tile_base = tile * TILE;
    const i64 warp_base = tile_base + (i64)warp * WARP_ELEMS;
    const bool full = tile_base + TILE <= n;

    // 0. Pull a tile far ahead of this one into L2. A tile's look-back cannot finish before every earlier tile has
    //    counted its survivors, so one slow HBM access holds up all tiles behind it; with the input already in L2 the
    //    loads of all tiles take about the same, short time (measured: 8 % faster at 8 MB ahead, no gain beyond).
#ifndef DCB_COMPACT_AHEAD_BYTES
#define DCB_COMPACT_AHEAD_BYTES (8 << 20)
#endif
    if (DCB_COMPACT_AHEAD_BYTES > 0) {
        const i64 ahead = tile + (i64)(DCB_COMPACT_AHEAD_BYTES) / (i64)(TILE * sizeof(A)) + 1;
        if ((ahead + 1) * TILE <= n) {
            const char* p0 = reinterpret_cast<const char*>(in0 + ahead * TILE);
            for (int l = threadIdx.x; l < (int)(TILE * sizeof(A) / 128); l += BLOCK)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p0 + (i64)l * 128));
            if constexpr (C::n_in == 2) {
                const char* p1 = reinterpret_cast<const char*>(in1 + ahead * TILE);
                for (int l = threadIdx.x; l < (int)(TILE * sizeof(B) / 128); l += BLOCK)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(p1 + (i64)l * 128));
            }
        }
    }
    // 1-4. loads, chain, ranks, staging (specialised on whether the tile needs bound checks)
    O* stage = s_stage + warp * WARP_ELEMS;
    const int warp_run = full ? compact_count_and_stage<C, BLOCK, ROWS, VEC, true>(in0, in1, n, warp_base, lane, stage)
                              : compact_count_and_stage<C, BLOCK, ROWS, VEC, false>(in0, in1, n, warp_base, lane, stage);
    if (lane == 0) s_warp_tot[warp] = warp_run;
    __syncthreads();                                       // warp totals and staged runs are visible
    int warp_off = 0, tile_total = 0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        const int t = s_warp_tot[w];
        if (w < warp) warp_off += t;
        tile_total += t;
    }

    // 5. publish the aggregate, look back
    if (warp == 0) {
        if (tile == 0) {
            if (lane == 0) {
                // abort_flag[1] == epoch withholds this count: a host-driven test of the time-out path (every later tile
                // then waits, bounded, for a count that never comes)
                if (*(volatile unsigned int*)(abort_flag + 1) != epoch)
                    desc_store(desc + tile, desc_make(epoch, ST_INCLUSIVE, (u64)tile_total));
                s_prefix = prev ? prev->count : 0;
            }
        } else {
            if (lane == 0) desc_store(desc + tile, desc_make(epoch, ST_AGGREGATE, (u64)tile_total));
            bool failed = false;
            const i64 exclusive = compact_lookback(desc, tile, lane, epoch, spin_limit, abort_flag, failed);
            if (lane == 0) {
                if (failed) {
                    // A wait ran out (or another tile's did). Tell the tiles still waiting, and leave a record that says
                    // so; every tile after the stuck one ends here too, so the last tile cannot overwrite it with success.
                    atomicExch(abort_flag, epoch);
                    res->count = 0; res->count_f = 0; res->flags = (u64)FLAG_TIMEOUT;
                    s_prefix = -1;
                } else {
                    desc_store(desc + tile, desc_make(epoch, ST_INCLUSIVE, (u64)(exclusive + tile_total)));
                    s_prefix = (prev ? prev->count : 0) + exclusive;
                }
            }
        }
    }
    __syncthreads();                                       // the tile's output offset is known
    const i64 prefix = s_prefix;
    if (prefix < 0) return;                                // a bounded wait ran out: leave without writing

    // 6. each warp copies its compacted run
    compact_copy_out<O, VEC>(out, out_cap, prefix + warp_off, warp_run, lane, stage);
    if (tile == num_tiles - 1 && threadIdx.x == 0) {
        const i64 total = prefix + tile_total;
        res->count = total; res->count_f = (double)total;
        res->fsum = 0; res->isum_lo = 0; res->isum_hi = 0; res->fmin = 0; res->fmax = 0; res->imin = 0; res->imax = 0;
        res->offset = 0; res->local_count = total;
        res->flags = total > out_cap ? (u64)FLAG_TRUNCATED : 0ull;
        // A tile that gave up left FLAG_TIMEOUT and raised the abort word; do not cover that with a success record.
        if (*(volatile unsigned int*)abort_flag == epoch) { res->count = 0; res->count_f = 0; res->local_count = 0; res->flags = (u64)FLAG_TIMEOUT; }
    }
}


// ------------------------------------------------------------------ bulk copies, shared-memory barriers, descriptor range sums
// Asynchronous bulk copies (the TMA unit, untiled form) and the shared-memory barriers they complete on.
__device__ __forceinline__ u32 smem_addr(const void* p) { return (u32)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(u64* bar, u32 arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(u64* bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(u64* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(u64* bar, u32 parity) {
    u32 ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Global -> shared copy of `bytes` (a multiple of 16, both addresses 16-byte aligned), completing on `bar`.
// The same with a suspend-time hint: the hardware may keep the thread asleep, off the issue slots, for up to `hint_ns`
// or until the phase completes, whichever comes first.
__device__ __forceinline__ bool mbar_try_wait_hint(u64* bar, u32 parity, u32 hint_ns) {
    u32 ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_global, u32 bytes, u64* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst_smem)), "l"(src_global), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// Orders this thread's earlier shared-memory accesses before later accesses made by bulk copies.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Sum of the survivor counts of tiles [lo, hi), run by one whole warp: the look-back of a persistent block. Such a block
// knows the prefix after its own previous tile, so what it needs is the counts of the tiles drawn since, a known range,
// read with all loads in flight at once rather than window by window. Returns the sum in every lane, or sets `failed`
// when a bounded wait for a count that was not yet published ran out.
__device__ __forceinline__ i64 compact_range_sum(const u64* __restrict__ desc, i64 lo, i64 hi, int lane, u32 epoch, u32 spin_limit,
                                                 const unsigned int* abort_flag, bool& failed_out) {
#ifndef DCB_RANGE_DEPTH
#define DCB_RANGE_DEPTH 8
#endif
    constexpr int DEPTH = DCB_RANGE_DEPTH;                    // descriptors per lane per step: 256 tiles per round trip
    i64 sum = 0;
    bool failed = false;
    for (i64 base = lo; base < hi && !failed; base += 32 * DEPTH) {
        u64 d[DEPTH];
#pragma unroll
        for (int u = 0; u < DEPTH; ++u) {
            const i64 idx = base + (i64)u * 32 + lane;
            d[u] = idx < hi ? desc_load(desc + idx) : desc_make(epoch, ST_AGGREGATE, 0);
        }
#pragma unroll
        for (int u = 0; u < DEPTH; ++u) {
            const i64 idx = base + (i64)u * 32 + lane;
            u32 polls = 0;
            while (!failed && desc_status(d[u], epoch) == ST_INVALID) {
                if (++polls > spin_limit || ((polls & 15u) == 0u && *(volatile unsigned int*)abort_flag == epoch)) { failed = true; break; }
                __nanosleep(polls > 4096 ? 4 * DCB_POLL_SLEEP_NS : DCB_POLL_SLEEP_NS);
                d[u] = desc_load(desc + idx);
            }
            if (!failed) sum += (i64)(d[u] & DESC_VALUE_MASK);
        }
        failed = __any_sync(0xffffffffu, failed);
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
    failed_out = failed;
    return sum;
}

// ------------------------------------------------------------------ compact, streamed: warp-specialised persistent blocks
// Same result as compact_body, built so that nothing on the data path waits for anything but data.
//
// A block is WARPS worker warps, one offsets warp and one loader thread. It works through tiles of WARPS * ROWS * 512
// bytes whose ids the loader draws from a counter; tile r of the block lives in slot r % NBUF of a ring of shared-memory
// buffers. Four shared-memory barriers per slot hand a tile from one role to the next; there is no block-wide barrier
// between the first and the last tile:
//
//   loader    waits for `empty` (the slot's previous tile has been written out), draws an id, starts the bulk copy of the
//             tile's input into the slot (completing on `full`), and asks L2 for a tile some block will draw a few rounds
//             from now, so that the copies themselves are served from L2;
//   worker w  waits for `full`, ranks its 1/WARPS of the tile and stages the survivors in place, over the input it has just
//             read (hence sizeof(out) <= sizeof(in0)), leaves its count in shared memory and arrives on `ranked`; then it
//             turns to the tile it ranked LAG rounds ago, waits for `offs` (normally long complete), copies its run to the
//             output with 16-byte stores and arrives on `empty`. Workers never wait for each other;
//   offsets   waits for `ranked`, publishes the tile's count (one relaxed 64-bit store), then works on the two tiles before
//             it. A tile's output offset is the offset after the block's previous tile plus the counts of the tiles
//             drawn in between, a known range of descriptors read with all loads in flight at once. Those loads are
//             issued one round after the tile was ranked (by then its neighbours in id order have published their
//             counts) and summed one round later still (a round trip to L2 takes about a round), so the warp never
//             waits for memory; it leaves one offset per worker in shared memory and arrives on `offs`.
//
// A tile's offset is thus ready two rounds after the tile was ranked, which is when a worker asks for it (LAG = 2). Progress:
// a tile's offset needs only counts of tiles with smaller ids; an id is drawn by a running block at the moment its copy
// is started, and ranking never waits for another block, so the smallest id not yet counted is always about to be.
// Nothing is assumed about how many blocks are resident. Every wait is bounded: polls of a descriptor by `spin_limit`,
// waits on the block's own barriers and copies by a fixed number of clock cycles; a wait that runs out marks the block dead, raises the
// epoch-tagged abort word for the other blocks, and the launch ends with FLAG_TIMEOUT in the record.
//
// Alignment: bulk copies need 16-byte aligned sources, so the kernel works in a shifted index space that starts `head`
// elements before in0 (at the 16-byte boundary below it; in1 must be displaced by the same number of elements). Tiles
// that are not wholly inside [head, head + n) - the first one if head > 0, the last one if ragged - are read with plain
// bounds-checked loads. `out` needs element alignment only.
//
// `counters[0]` hands out tile ids, `counters[1]` counts finished blocks; both are zero at launch and the last block
// to finish zeroes them again. `abort_flag[1] == epoch` withholds the count of tile 0 (a host-driven test of the time-out
// path: every offset then waits for a count that never comes). With STREAM_TAKE in `run_flags` (Take(k) after a Where,
// k = out_cap) the scan ends early: the offsets warp that finds a tile starting at or beyond k raises abort_flag[2] to
// the epoch and leaves a record with a count >= k; loaders look at that word before they draw an id and stop drawing.
// Ids already drawn are finished as usual (their writes are clipped at k), so nothing waits for a count that never comes.
// Launch with (WARPS + 2) * 32 threads and NBUF * tile bytes of dynamic shared memory for each input.
// Limit of one wait on a block's own barrier or bulk copy, in SM clock cycles (about two seconds). It is measured with
// the SM's cycle counter, which costs a few cycles to read; the nanosecond timer shared by the whole GPU takes microseconds
// per read, which a wait on the data path cannot afford.
#ifndef DCB_STREAM_VEC_OUT
#define DCB_STREAM_VEC_OUT 0
#endif
#ifndef DCB_STREAM_WAIT_CYCLES
#define DCB_STREAM_WAIT_CYCLES 4000000000ll
#endif
// Store of one survivor into a warp's staging run in shared memory, as straight-line code: the store and the advance
// of the write position are predicated on bit `mask` of `keepbits` (a branch per element, which is what the plain C++
// form compiles to, costs several times as many instructions). `addr` is a shared-space byte address.
template <typename O>
__device__ __forceinline__ void stage_if(u32& addr, const O& v, u32 keepbits, u32 mask) {
    if constexpr (sizeof(O) == 4) {
        u32 w; memcpy_bits(w, v);
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\tand.b32 t, %2, %3;\n\tsetp.ne.b32 p, t, 0;\n\t@p st.shared.b32 [%0], %1;\n\t@p add.u32 %0, %0, 4;\n\t}"
                     : "+r"(addr) : "r"(w), "r"(keepbits), "r"(mask) : "memory");
    } else if constexpr (sizeof(O) == 8) {
        u64 w; memcpy_bits(w, v);
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\tand.b32 t, %2, %3;\n\tsetp.ne.b32 p, t, 0;\n\t@p st.shared.b64 [%0], %1;\n\t@p add.u32 %0, %0, 8;\n\t}"
                     : "+r"(addr) : "l"(w), "r"(keepbits), "r"(mask) : "memory");
    } else if constexpr (sizeof(O) == 2) {
        unsigned short w; memcpy_bits(w, v);
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\tand.b32 t, %2, %3;\n\tsetp.ne.b32 p, t, 0;\n\t@p st.shared.b16 [%0], %1;\n\t@p add.u32 %0, %0, 2;\n\t}"
                     : "+r"(addr) : "h"(w), "r"(keepbits), "r"(mask) : "memory");
    } else {
        unsigned char b; memcpy_bits(b, v);
        const u32 w = b;
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\tand.b32 t, %2, %3;\n\tsetp.ne.b32 p, t, 0;\n\t@p st.shared.u8 [%0], %1;\n\t@p add.u32 %0, %0, 1;\n\t}"
                     : "+r"(addr) : "r"(w), "r"(keepbits), "r"(mask) : "memory");
    }
}

// Chain, ranks and staging of one warp's run of a tile for the streamed kernel: as compact_rank_and_stage, with the
// whole run inside the array (no bound checks) and the survivors stored by stage_if.
template <class C, int ROWS, int E>
__device__ __forceinline__ int stream_rank_and_stage(const Pack<typename C::in0_t, E> (&a)[ROWS], const Pack<typename C::in1_t, E> (&b)[ROWS],
                                                     int lane, u32 stage_addr) {
    typedef typename C::in1_t B; typedef typename C::out_t O;
    constexpr int FIELD = (32 * E <= 128) ? 8 : 16;
    constexpr int PER_WORD = 32 / FIELD;
    constexpr int WORDS = (ROWS + PER_WORD - 1) / PER_WORD;
    constexpr u32 FMASK = (FIELD == 8) ? 0xffu : 0xffffu;
    O val[ROWS][E];
    u32 keepbits[ROWS];
    u32 packed[WORDS];
#pragma unroll
    for (int w = 0; w < WORDS; ++w) packed[w] = 0;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        u32 bits = 0;
#pragma unroll
        for (int k = 0; k < E; ++k) {
            bool keep;
            if constexpr (C::n_in == 2) keep = C::apply(a[r].e[k], b[r].e[k], val[r][k]);
            else keep = C::apply(a[r].e[k], B(), val[r][k]);
            bits |= keep ? (1u << k) : 0u;
        }
        keepbits[r] = bits;
        packed[r / PER_WORD] += (u32)__popc(bits) << ((r % PER_WORD) * FIELD);
    }
    u32 incl[WORDS];
#pragma unroll
    for (int w = 0; w < WORDS; ++w) {
        u32 v = packed[w];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d) v += t;
        }
        incl[w] = v;
    }
    u32 tot[WORDS];
#pragma unroll
    for (int w = 0; w < WORDS; ++w) tot[w] = __shfl_sync(0xffffffffu, incl[w], 31);
    int row_start = 0;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int w = r / PER_WORD, sh = (r % PER_WORD) * FIELD;
        const u32 tot_word = tot[w];
        const int before = (int)(((incl[w] - packed[w]) >> sh) & FMASK);
        u32 addr = stage_addr + (u32)(row_start + before) * (u32)sizeof(O);
#pragma unroll
        for (int k = 0; k < E; ++k) stage_if<O>(addr, val[r][k], keepbits[r], 1u << k);
        row_start += (int)((tot_word >> sh) & FMASK);
    }
    return row_start;
}

// Count descriptors of the streamed kernel: one 32-bit word per tile = epoch(12) | written(1) | count(19), four to a
// 16-byte load, so that the counts of 128 tiles come back with one instruction per warp.
__device__ __forceinline__ u32 cdesc_make(u32 epoch, u32 count) { return ((epoch & 0xfffu) << 20) | 0x80000u | (count & 0x7ffffu); }
__device__ __forceinline__ bool cdesc_written(u32 d, u32 epoch) { return (d >> 19) == (((epoch & 0xfffu) << 1) | 1u); }
__device__ __forceinline__ void cdesc_store(u32* p, u32 v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void cdesc_load4(const u32* p, u32 (&v)[4]) {
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(p) : "memory");
}
// Loads of the window of D4 * 128 descriptors that starts at the 16-byte boundary at or below tile `lo`, cut at `hi`.
template <int D4>
__device__ __forceinline__ void cdesc_issue(const u32* __restrict__ cdesc, i64 lo, i64 hi, int lane, u32 (&d)[D4][4]) {
    const i64 base = lo & ~(i64)3;
    const int span = (int)(hi - base < (i64)D4 * 128 ? hi - base : (i64)D4 * 128);   // descriptors of the window that matter
#pragma unroll
    for (int u = 0; u < D4; ++u) {
        const int rel = (u * 32 + lane) * 4;
        if (rel < span) cdesc_load4(cdesc + base + rel, d[u]);
        else { d[u][0] = 0; d[u][1] = 0; d[u][2] = 0; d[u][3] = 0; }
    }
}
// Sum of the counts of tiles [lo, hi) by one whole warp; `d` holds the loads cdesc_issue made for (lo, hi). Counts that
// were not there yet are asked for again, all together, with a bounded number of polls; a range longer than one window
// is finished window by window. Returns the sum in every lane, or sets `failed`.
// The offsets warp is one warp working through dependent instructions, and what it does per tile sets the length of every
// round of its block (measured: 1900 cycles a round whatever the tile size, 1100 of them in here with the loads long
// back). So the common case is kept short: a 16-byte group that lies inside the range is tested with four XORs against
// the expected top bits and summed raw, the warp-wide results come from one redux each.
template <int D4>
__device__ __forceinline__ i64 cdesc_finish(const u32* __restrict__ cdesc, i64 lo, i64 hi, int lane, u32 epoch, u32 spin_limit,
                                            const unsigned int* abort_flag, volatile int* dead, u32 (&d)[D4][4], bool& failed) {
    i64 total = 0;
    const u32 tag = (((epoch & 0xfffu) << 1) | 1u) << 19;      // the top 13 bits of a descriptor written by this launch
    for (;;) {
        const i64 base = lo & ~(i64)3;
        const int first = (int)(lo - base);
        const int span = (int)(hi - base < (i64)D4 * 128 ? hi - base : (i64)D4 * 128);
        u32 warp_sum = 0;
        for (u32 polls = 0;;) {
            u32 bad = 0, sum = 0;
#pragma unroll
            for (int u = 0; u < D4; ++u) {
                const int rel = (u * 32 + lane) * 4;
                if (rel >= first && rel + 4 <= span) {        // the whole group matters: the usual case
                    bad |= ((d[u][0] ^ tag) | (d[u][1] ^ tag) | (d[u][2] ^ tag) | (d[u][3] ^ tag)) >> 19;
                    sum += d[u][0] + d[u][1] + d[u][2] + d[u][3] - 4u * tag;   // the counts, if all four carry the tag
                } else if (rel < span && rel + 4 > first) {   // a group on the range's edge
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (rel + e >= first && rel + e < span) { bad |= (d[u][e] ^ tag) >> 19; sum += d[u][e] & 0x7ffffu; }
                    }
                }
            }
            const u32 warp_bad = __reduce_or_sync(0xffffffffu, bad);   // the two reductions are independent: issued back to back
            warp_sum = __reduce_add_sync(0xffffffffu, sum);           // at most D4 * 128 counts below 2^19 each
            if (warp_bad == 0u) break;
            if (++polls > spin_limit || *dead || ((polls & 15u) == 0u && *(volatile unsigned int*)abort_flag == epoch)) { failed = true; break; }
            __nanosleep(polls > 4096 ? 4 * DCB_POLL_SLEEP_NS : DCB_POLL_SLEEP_NS);
#pragma unroll
            for (int u = 0; u < D4; ++u) {
                const int rel = (u * 32 + lane) * 4;
                bool again = false;
#pragma unroll
                for (int e = 0; e < 4; ++e) again = again || (rel + e >= first && rel + e < span && !cdesc_written(d[u][e], epoch));
                if (again) cdesc_load4(cdesc + base + rel, d[u]);
            }
        }
        if (failed) break;
        total += (i64)warp_sum;
        lo = base + (i64)D4 * 128;
        if (lo >= hi) break;
        cdesc_issue<D4>(cdesc, lo, hi, lane, d);              // the rare long range: the next window, waited for in place
    }
    return total;
}

enum : u32 { STREAM_TAKE = 1u };
__device__ __forceinline__ void l2_prefetch_bulk(const void* src_global, u32 bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_global), "r"(bytes) : "memory");
}

template <class C, int WARPS, int ROWS, int LAG, int NBUF, int DEPTH, int AHEAD_BYTES, int DRAW_AHEAD, int COPY_WARPS>
__device__ __forceinline__ void compact_stream_body(const typename C::in0_t* __restrict__ in0, const typename C::in1_t* __restrict__ in1,
                                                    i64 n, typename C::out_t* __restrict__ out, i64 out_cap,
                                                    u64* __restrict__ desc, u32 epoch, u32 spin_limit, i64 num_tiles,
                                                    const DeviceResult* __restrict__ prev, DeviceResult* __restrict__ res,
                                                    unsigned int* __restrict__ abort_flag, unsigned int* __restrict__ counters, u32 head,
                                                    u32 run_flags) {
    typedef typename C::in0_t A; typedef typename C::in1_t B; typedef typename C::out_t O;
    static_assert(sizeof(O) <= sizeof(A), "in-place staging needs an output element no larger than the input element");
    static_assert(COPY_WARPS > 0 || (LAG >= 2 && NBUF >= LAG + 2), "workers that also write: an offset is ready two rounds after its tile was ranked; NBUF = LAG + 1 + tiles on their way in");
    static_assert(NBUF >= 3 && NBUF <= 16, "one slot on its way in, one being ranked, one waiting to be written");
    static_assert(WARPS >= 1 && WARPS <= 30 && DEPTH >= 1 && DEPTH <= 8, "one offsets lane per worker warp; DEPTH * 128 tiles per window");
    static_assert(COPY_WARPS >= 0 && COPY_WARPS <= WARPS, "copy warps share the worker warps' runs among them");
    static_assert(WARPS * ROWS * 32 * (16 / (int)sizeof(typename C::in0_t)) < (1 << 19), "a tile's count must fit the descriptor");
    constexpr int E = 16 / (int)sizeof(A);
    constexpr int WARP_ELEMS = ROWS * 32 * E;
    constexpr int TILE = WARPS * WARP_ELEMS;
    constexpr u32 BYTES_A = (u32)(TILE * sizeof(A));
    constexpr u32 BYTES_B = C::n_in == 2 ? (u32)(TILE * sizeof(B)) : 0u;
    static_assert(BYTES_A % 16 == 0 && BYTES_B % 16 == 0, "bulk copies move multiples of 16 bytes");
    constexpr i64 AHEAD_TILES = AHEAD_BYTES > 0 ? ((i64)AHEAD_BYTES / (i64)BYTES_A > 0 ? (i64)AHEAD_BYTES / (i64)BYTES_A : 1) : 0;

    extern __shared__ __align__(128) unsigned char s_dyn[];   // NBUF buffers of in0, then NBUF buffers of in1
    // Round r of the block uses slot r % NBUF and phase (r / NBUF) & 1 of each barrier.
    __shared__ __align__(8) u64 s_full[NBUF], s_ranked[NBUF], s_offs[NBUF], s_empty[NBUF];
    __shared__ i64 s_tile[NBUF];                              // tile id held by the slot (num_tiles = none left)
    __shared__ int s_cnt[NBUF][WARPS];                        // survivors per worker of that tile
    __shared__ i64 s_off[NBUF][WARPS];                        // output offset of each worker's run; -1 = gave up
    __shared__ int s_dead;                                    // a wait ran out somewhere in this block

    const int warp_id = (int)(threadIdx.x >> 5), lane = (int)(threadIdx.x & 31);
    volatile int* dead = &s_dead;
    const i64 lo = (i64)head, hi = n + (i64)head;             // the array in the shifted index space
    const A* in0a = in0 - head;
    const B* in1a = in1 - (C::n_in == 2 ? head : 0u);

    // Bounded wait for phase `parity` of one of the block's barriers: false when another warp of the block gave up or
    // the fixed time limit passed (one try may itself suspend the thread for a while).
    // A waiting warp is put to sleep by the barrier itself (a try with a suspend-time hint: it wakes when the phase
    // completes or the hint runs out): a warp that spins takes issue slots from the very warps it is waiting for.
#ifndef DCB_STREAM_WAIT_HINT_NS
#define DCB_STREAM_WAIT_HINT_NS 2000
#endif
    auto wait = [&](u64* bar, u32 parity, bool heed_dead) -> bool {
        if (mbar_try_wait(bar, parity)) return true;
        const i64 t0 = clock64();
        for (u32 i = 0; i < (1u << 30); ++i) {
            if (mbar_try_wait_hint(bar, parity, DCB_STREAM_WAIT_HINT_NS)) return true;
            if (heed_dead && *dead) return false;
            if ((i & 15u) == 15u && clock64() - t0 > DCB_STREAM_WAIT_CYCLES) return false;
        }
        return false;
    };

    if (threadIdx.x == 0) {
#pragma unroll
        for (int st = 0; st < NBUF; ++st) {
            mbar_init(&s_full[st], 1u); mbar_init(&s_ranked[st], (u32)WARPS); mbar_init(&s_offs[st], 1u); mbar_init(&s_empty[st], (u32)(COPY_WARPS > 0 ? COPY_WARPS : WARPS));
        }
        s_dead = 0;
        fence_async_smem();                                   // the barriers exist before a copy can complete on them
    }
    __syncthreads();

    // DCB_STREAM_STATS = 1 / 2 / 3 (profiling builds only) adds up, over all blocks, clock cycles the offsets warp / worker 0
    // / the loader spent in each of its waits and work phases, in the four spare slots of the record.
#ifdef DCB_STREAM_STATS
    i64 stat[4] = {0, 0, 0, 0};
#define DCB_STAT_BEGIN const i64 stat_t0 = clock64()
#define DCB_STAT_END(role, i) do { if (DCB_STREAM_STATS == (role)) stat[i] += clock64() - stat_t0; } while (0)
#define DCB_STAT_ADD(role, i, v) do { if (DCB_STREAM_STATS == (role)) stat[i] += (v); } while (0)
#else
#define DCB_STAT_BEGIN
#define DCB_STAT_END(role, i)
#define DCB_STAT_ADD(role, i, v)
#endif
    i64 issued = 0;                                           // loader thread: rounds it has started
    if (warp_id == 1) {
        // ---------------------------------------------------------------- loader (one thread)
        if (lane == 0) {
            int st = 0; u32 ph = 0;
            for (i64 r = 0;; ++r) {
                // DRAW_AHEAD > 0 paces the draws: the id of round r is not asked for before round r - DRAW_AHEAD has been
                // ranked, so a block never holds ids far ahead of the tiles it is ranking (other blocks' offsets wait
                // for the counts of all smaller ids). 0 = draw as soon as a slot is free.
                if (DRAW_AHEAD > 0 && r >= DRAW_AHEAD) {
                    const i64 rr = r - DRAW_AHEAD;
                    if (!wait(&s_ranked[(int)(rr % NBUF)], (u32)((rr / NBUF) & 1), true)) { *dead = 1; break; }
                }
                // The id is asked for before the wait for the slot: the counter's round trip overlaps that wait. (Asking one
                // round earlier still changed nothing: the counter is not what a round waits for.)
                i64 t = num_tiles;
                if (!((run_flags & STREAM_TAKE) && *(volatile unsigned int*)(abort_flag + 2) == epoch)) {   // Take(k) already satisfied?
                    t = (i64)atomicAdd(counters, 1u);
                    if (t > num_tiles) t = num_tiles;
                }
                { DCB_STAT_BEGIN;
                  if (r >= NBUF && !wait(&s_empty[st], ph ^ 1u, true)) { *dead = 1; break; }
                  DCB_STAT_END(3, 0); DCB_STAT_ADD(3, 1, 1); }
                s_tile[st] = t;
                const bool whole = t < num_tiles && t * TILE >= lo && (t + 1) * TILE <= hi;
                if (whole) {
                    mbar_expect_tx(&s_full[st], BYTES_A + BYTES_B);
                    bulk_load(s_dyn + (size_t)st * BYTES_A, in0a + t * TILE, BYTES_A, &s_full[st]);
                    if constexpr (C::n_in == 2)
                        bulk_load(s_dyn + (size_t)NBUF * BYTES_A + (size_t)st * BYTES_B, in1a + t * TILE, BYTES_B, &s_full[st]);
                } else {
                    mbar_arrive(&s_full[st]);                 // ragged tile (plain loads) or no tile left: the id alone
                }
                issued = r + 1;
                if (t >= num_tiles) break;
                if constexpr (AHEAD_TILES > 0) {
                    const i64 ta = t + AHEAD_TILES;
                    if ((ta + 1) * TILE <= hi) {
                        l2_prefetch_bulk(in0a + ta * TILE, BYTES_A);
                        if constexpr (C::n_in == 2) l2_prefetch_bulk(in1a + ta * TILE, BYTES_B);
                    }
                }
                if (++st == NBUF) { st = 0; ph ^= 1u; }
            }
        }
    } else if (warp_id == 0) {
        // ---------------------------------------------------------------- offsets warp
        const i64 base_prev = prev ? prev->count : 0;
        i64 last_tile = -1, run_incl = 0;                     // the block's previous finished tile, survivors up to and including it
        // Two tiles are in the works besides the one just ranked: `c_` has its descriptor loads in flight (issued a round
        // ago, summed now), `i_` was ranked a round ago and gets its loads issued now. A round trip to L2 takes about as
        // long as a round, so it is never waited for; and a tile's loads go out a round after its neighbours in id order
        // published their counts, so they rarely come back empty.
        bool c_have = false, i_have = false;
        i64 c_tile = 0, c_lo = 0, i_tile = 0;
        int c_st = 0, c_excl = 0, c_total = 0, i_st = 0, i_excl = 0, i_total = 0;
        u32 d[DEPTH][4];
        u32* cdesc = reinterpret_cast<u32*>(desc);            // this kernel's descriptors are 32-bit counts
        int st = 0; u32 ph = 0;
        bool failed = false;
        for (bool more = true; more && !failed;) {
            { DCB_STAT_BEGIN;
              if (!wait(&s_ranked[st], ph, true)) { *dead = 1; break; }
              DCB_STAT_END(1, 0); DCB_STAT_ADD(1, 3, 1); }
            const i64 tile = s_tile[st];
            const bool valid = tile < num_tiles;
            int cnt = 0, incl = 0, total = 0;
            if (valid) {
                cnt = lane < WARPS ? s_cnt[st][lane] : 0;
                incl = cnt;
#pragma unroll
                for (int dd = 1; dd < WARPS; dd <<= 1) {      // only the first WARPS lanes hold anything
                    const int t = __shfl_up_sync(0xffffffffu, incl, dd);
                    if (lane >= dd) incl += t;
                }
                total = __shfl_sync(0xffffffffu, incl, WARPS - 1);
                if (lane == 0 && !(tile == 0 && *(volatile unsigned int*)(abort_flag + 1) == epoch))
                    cdesc_store(cdesc + tile, cdesc_make(epoch, (u32)total));
            }
            more = valid;
            // After the block's last tile the two tiles still in the works are finished one after the other.
            for (int pass = 0; pass < (valid ? 1 : 3) && !failed; ++pass) {
                if (c_have) {
                    DCB_STAT_BEGIN;
                    // Sum the counts of (last_tile, c_tile): the loads went out a round ago.
                    const i64 sum = cdesc_finish<DEPTH>(cdesc, c_lo, c_tile, lane, epoch, spin_limit, abort_flag, dead, d, failed);
                    DCB_STAT_END(1, 1);
                    const i64 exclusive = run_incl + sum;
                    if (lane < WARPS) s_off[c_st][lane] = failed ? -1 : base_prev + exclusive + c_excl;
                    __syncwarp();
                    if (lane == 0) {
                        if (!failed && c_tile == num_tiles - 1) {
                            const i64 total_all = base_prev + exclusive + c_total;
                            res->count = total_all; res->count_f = (double)total_all;
                            res->fsum = 0; res->isum_lo = 0; res->isum_hi = 0; res->fmin = 0; res->fmax = 0; res->imin = 0; res->imax = 0;
                            res->offset = 0; res->local_count = total_all;
                            res->flags = total_all > out_cap ? (u64)FLAG_TRUNCATED : 0ull;
                        }
                        if (!failed && (run_flags & STREAM_TAKE) && base_prev + exclusive >= out_cap &&
                            *(volatile unsigned int*)(abort_flag + 2) != epoch) {
                            // Take(k): everything asked for lies in tiles before this one. Tell the loaders, and leave a
                            // record in case the array's last tile is never reached.
                            *(volatile unsigned int*)(abort_flag + 2) = epoch;
                            const i64 seen = base_prev + exclusive + c_total;
                            res->count = seen; res->count_f = (double)seen; res->local_count = seen; res->offset = 0;
                            res->fsum = 0; res->isum_lo = 0; res->isum_hi = 0; res->fmin = 0; res->fmax = 0; res->imin = 0; res->imax = 0;
                            res->flags = seen > out_cap ? (u64)FLAG_TRUNCATED : 0ull;
                        }
                        if (failed) { *dead = 1; atomicExch(abort_flag, epoch); }
                        mbar_arrive(&s_offs[c_st]);           // the workers read s_off after this
                    }
                    run_incl = exclusive + c_total;
                    last_tile = c_tile;
                    c_have = false;
                    DCB_STAT_END(1, 2);
                }
                if (i_have && !failed) {
                    c_lo = last_tile + 1;
                    cdesc_issue<DEPTH>(cdesc, c_lo, i_tile, lane, d);
                    c_have = true; c_tile = i_tile; c_st = i_st; c_excl = i_excl; c_total = i_total;
                    i_have = false;
                }
            }
            if (valid) {
                i_have = true; i_tile = tile; i_st = st; i_excl = incl - cnt; i_total = total;
                if (++st == NBUF) { st = 0; ph ^= 1u; }
            }
        }
    } else if (COPY_WARPS > 0 && warp_id >= 2 + WARPS) {
        // ---------------------------------------------------------------- copy warps (COPY_WARPS > 0)
        // Writing a tile out is mostly waiting - for shared memory, then for room in the store queue - and ranking is
        // mostly arithmetic; in one warp the two only take turns. Here they are different warps' work: these warps move
        // the runs the workers staged, the workers go straight on to the next tile.
        const int c = warp_id - 2 - WARPS;
        int sj = 0; u32 pj = 0;
        for (;;) {
            // The round's tile id: its `full` phase completed LAG rounds ago and cannot complete again before these warps
            // give the slot back.
            if (!wait(&s_full[sj], pj, true)) { *dead = 1; break; }
            if (s_tile[sj] >= num_tiles) break;
            { DCB_STAT_BEGIN;
              if (!wait(&s_offs[sj], pj, true)) { *dead = 1; break; }
              if (c == 0) DCB_STAT_END(4, 2); }
            DCB_STAT_BEGIN;
            bool gave_up = false;
#pragma unroll 1
            for (int w = c; w < WARPS; w += COPY_WARPS) {
                const i64 off = s_off[sj][w];
                if (off < 0) { gave_up = true; break; }
                const O* stage0 = reinterpret_cast<const O*>(reinterpret_cast<const A*>(s_dyn + (size_t)sj * BYTES_A) + w * WARP_ELEMS);
                compact_copy_out<O, DCB_STREAM_VEC_OUT != 0>(out, out_cap, off, s_cnt[sj][w], lane, stage0);
            }
            if (gave_up) { *dead = 1; break; }
            fence_async_smem();                               // this warp's reads of the slot come before the next copy into it
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[sj]);
            if (c == 0) DCB_STAT_END(4, 3);
            if (++sj == NBUF) { sj = 0; pj ^= 1u; }
        }
    } else {
        // ---------------------------------------------------------------- workers
        const int w = warp_id - 2;
        i64 nvalid = (i64)1 << 62;                            // rounds in which this block has a tile
        int st = 0, sj = 0; u32 ph = 0, pj = 0;               // slot and phase of round k, and of round k - LAG
        for (i64 k = 0; k < nvalid + (COPY_WARPS > 0 ? 0 : LAG); ++k) {
            if (k < nvalid) {
                { DCB_STAT_BEGIN;
                  if (!wait(&s_full[st], ph, true)) { *dead = 1; break; }
                  if (w == 0) DCB_STAT_END(2, 0); }
                const i64 tile = s_tile[st];
                if (tile >= num_tiles) {
                    nvalid = k;
                } else {
                    DCB_STAT_BEGIN;
                    const i64 warp_base = tile * TILE + (i64)w * WARP_ELEMS;
                    A* bufA = reinterpret_cast<A*>(s_dyn + (size_t)st * BYTES_A) + w * WARP_ELEMS;
                    const B* bufB = reinterpret_cast<const B*>(s_dyn + (size_t)NBUF * BYTES_A + (size_t)st * BYTES_B) + w * WARP_ELEMS;
                    O* stage = reinterpret_cast<O*>(bufA);
                    Pack<A, E> a[ROWS]; Pack<B, E> b[ROWS];
                    int run;
                    if (tile * TILE >= lo && (tile + 1) * TILE <= hi) {
#pragma unroll
                        for (int r = 0; r < ROWS; ++r) {
                            a[r].load_shared(bufA + (r * 32 + lane) * E);
                            if constexpr (C::n_in == 2) b[r].load_shared(bufB + (r * 32 + lane) * E);
                        }
                        __syncwarp();                         // every lane holds its packs before any lane overwrites the run
                        run = stream_rank_and_stage<C, ROWS, E>(a, b, lane, smem_addr(stage));
                    } else {
#pragma unroll
                        for (int r = 0; r < ROWS; ++r) {
#pragma unroll
                            for (int e = 0; e < E; ++e) {
                                const i64 idx = warp_base + ((i64)r * 32 + lane) * E + e;
                                const bool in_range = idx >= lo && idx < hi;
                                a[r].e[e] = in_range ? in0a[idx] : A();
                                if constexpr (C::n_in == 2) b[r].e[e] = in_range ? in1a[idx] : B();
                            }
                        }
                        run = compact_rank_and_stage<C, ROWS, E, false>(a, b, hi, warp_base, lane, stage, lo);
                    }
                    if (lane == 0) s_cnt[st][w] = run;
                    if (w == 0) DCB_STAT_END(2, 1);
                }
                if (COPY_WARPS > 0) fence_async_smem();       // the staged run was written here and is read, and the slot given back, elsewhere
                __syncwarp();                                 // the staged run and its count are written
                if (lane == 0) mbar_arrive(&s_ranked[st]);    // also for the round without a tile: it ends the offsets warp
                if (++st == NBUF) { st = 0; ph ^= 1u; }
            }
            if (COPY_WARPS == 0 && k >= LAG) {
                if (k - LAG < nvalid) {                       // write the tile ranked LAG rounds ago, give its slot back
                    { DCB_STAT_BEGIN;
                      if (!wait(&s_offs[sj], pj, true)) { *dead = 1; break; }
                      if (w == 0) DCB_STAT_END(2, 2); }
                    DCB_STAT_BEGIN;
                    const i64 off = s_off[sj][w];
                    if (off < 0) { *dead = 1; break; }
                    const O* stage0 = reinterpret_cast<const O*>(reinterpret_cast<const A*>(s_dyn + (size_t)sj * BYTES_A) + w * WARP_ELEMS);
                    // Consecutive lanes move consecutive survivors: no bank conflicts on the way out of shared memory, whole
                    // 128-byte lines on the way into L2 (16-byte stores would read shared memory four lanes to a bank).
                    compact_copy_out<O, DCB_STREAM_VEC_OUT != 0>(out, out_cap, off, s_cnt[sj][w], lane, stage0);
#ifndef DCB_STREAM_NO_PROXY_FENCE
                    fence_async_smem();                       // this warp's accesses to the slot come before the next copy into it
#endif
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&s_empty[sj]);
                    if (w == 0) DCB_STAT_END(2, 3);
                }
                if (++sj == NBUF) { sj = 0; pj ^= 1u; }
            }
        }
    }

#ifdef DCB_STREAM_STATS
    if (lane == 0 && (warp_id == 0 ? DCB_STREAM_STATS == 1 : (warp_id == 1 ? DCB_STREAM_STATS == 3 : (warp_id == 2 ? DCB_STREAM_STATS == 2 : (warp_id == 2 + WARPS && DCB_STREAM_STATS == 4)))))
        for (int i = 0; i < 4; ++i) atomicAdd((u64*)&res->pad[i], (u64)stat[i]);
#endif
    __syncthreads();
    if (s_dead) {
        // Tell the blocks still waiting. Copies this block started must land before its shared memory is given to another
        // block: wait for the rounds that may still be on their way, each with the fixed limit.
        if (threadIdx.x == 0) atomicExch(abort_flag, epoch);
        if (threadIdx.x == 32)
            for (i64 r = issued > NBUF ? issued - NBUF : 0; r < issued; ++r)
                (void)wait(&s_full[(int)(r % NBUF)], (u32)((r / NBUF) & 1), false);
    }
    // Sign off. The last block to do so resets the counters for the next launch and has the final say on the record.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int finished = atomicAdd(counters + 1, 1u);
        if (finished == gridDim.x - 1) {
            __threadfence();
            if (*(volatile unsigned int*)abort_flag == epoch) { res->count = 0; res->count_f = 0; res->local_count = 0; res->flags = (u64)FLAG_TIMEOUT; }
            counters[0] = 0; counters[1] = 0;
        }
    }
}

}  // namespace dcb
#endif  // DCB_KERNELS_CUH
