// dcb_peer.cuh - exchange of reduction partials between the GPUs of one node (compiled by nvcc only).
//
// A sharded reduction ends with every GPU holding the total. The reduce kernel itself is the single-GPU kernel; the
// exchange is a one-warp kernel that the host enqueues on a side stream behind it. That kernel stores this GPU's
// partial into an exchange area in every peer's memory (plain NVLink peer stores), waits - with a bounded poll - for
// the peers' partials to land in its own area, folds them in rank order (so every GPU computes the bit-identical
// total) and rewrites the record. Because it needs one warp, it runs beside the next query's reduce kernel: neither
// NVLink latency nor the skew between GPUs is on the critical path of a stream of queries.
// Slots form a ring indexed by a launch counter kept in device memory (the same on every rank); a slot is valid when
// its stamp equals the counter. A rank cannot post launch s+1 before every peer has posted s, so ranks are never
// more than one launch apart and a ring of PEER_RING slots cannot be overrun.
#ifndef DCB_PEER_CUH
#define DCB_PEER_CUH
#include "dcb_kernels.cuh"

namespace dcb {

enum : int { PEER_MAX = 8, PEER_RING = 4 };
struct __align__(16) PeerSlot {   // 64 bytes: one rank's partial for one launch; valid when stamp == launch number
    double fsum; u64 isum_lo; i64 isum_hi; i64 count; i64 mn_bits; i64 mx_bits; u64 flags; u64 stamp;
};
enum : u64 { SLOT_IS_FP = 1ull << 32, SLOT_IS_U64 = 1ull << 33,     // how to compare mn_bits / mx_bits
             SLOT_IS_I32 = 1ull << 34 };                             // a checked Sum's range is int's, not long's
struct PeerState { u64 seq; u64 pad; };                              // device memory, one per context
struct PeerTable {                // passed by value as a kernel parameter
    int world, rank;
    u32 spin_limit, pad;
    PeerState* state;
    PeerSlot* area[PEER_MAX];     // area[r]: base of rank r's exchange area = PeerSlot[PEER_RING][PEER_MAX], peer-mapped
};
__device__ __forceinline__ void st_release_sys(u64* p, u64 v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 ld_acquire_sys(const u64* p) {
    u64 v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// One warp. `rec` holds this GPU's partial on entry and the global result on exit. `tag` = SLOT_IS_FP / SLOT_IS_U64.
__device__ __forceinline__ void peer_exchange_body(const PeerTable& pt, DeviceResult* rec, u64 tag) {
    __shared__ PeerSlot slots[PEER_MAX];
    __shared__ int failed;
    const int lane = threadIdx.x;
    const u64 seq = pt.state->seq + 1;                 // every lane reads the same value; lane 0 stores it at the end
    if (lane == 0) failed = 0;
    __syncwarp();
    if (lane < pt.world) {
        // post: payload with plain stores, then the stamp with release semantics (orders this lane's earlier stores)
        PeerSlot* dst = pt.area[lane] + (seq % PEER_RING) * PEER_MAX + pt.rank;
        volatile PeerSlot* vd = dst;
        const bool fp = (tag & SLOT_IS_FP) != 0;
        vd->fsum = rec->fsum; vd->isum_lo = (u64)rec->isum_lo; vd->isum_hi = rec->isum_hi; vd->count = rec->count;
        vd->mn_bits = fp ? __double_as_longlong(rec->fmin) : rec->imin;
        vd->mx_bits = fp ? __double_as_longlong(rec->fmax) : rec->imax;
        if (rec->flags & (u64)FLAG_PREFIX) {
            // a checked integer Sum: the fields a Sum leaves unused carry the range of the running sum (two words each)
            vd->mn_bits = rec->pad[0]; vd->fsum = __longlong_as_double(rec->pad[1]);
            vd->mx_bits = rec->pad[2]; vd->count = rec->pad[3];
        }
        vd->flags = (rec->flags & 0xffffffffull) | tag;
        st_release_sys(&dst->stamp, seq);
        // collect: rank `lane`'s partial in my own area
        const PeerSlot* src = pt.area[pt.rank] + (seq % PEER_RING) * PEER_MAX + lane;
        u32 polls = 0; bool ok = true;
        while (ld_acquire_sys(&src->stamp) != seq) {
            if (++polls > pt.spin_limit) { ok = false; break; }
            if (polls > 64) __nanosleep(polls > 65536 ? 1000 : 100);
        }
        if (ok) {
            const volatile PeerSlot* vs = src;
            slots[lane].fsum = vs->fsum; slots[lane].isum_lo = vs->isum_lo; slots[lane].isum_hi = vs->isum_hi; slots[lane].count = vs->count;
            slots[lane].mn_bits = vs->mn_bits; slots[lane].mx_bits = vs->mx_bits; slots[lane].flags = vs->flags;
        } else {
            atomicExch(&failed, 1);
        }
    }
    __syncwarp();
    if (lane == 0) {
        if (failed) {                                  // a peer never showed up: say so, keep the local partial
            rec->flags = rec->flags | (u64)FLAG_TIMEOUT;
        } else if (slots[0].flags & (u64)FLAG_PREFIX) {
            // checked integer Sum: the ranks' (total, smallest, largest running sum) appended in rank order, exactly
            Wide128 s(0), lo(0), hi(0);
            u64 fl = 0;
            for (int r = 0; r < pt.world; ++r) {
                const PeerSlot& o = slots[r];
                Wide128 os, olo, ohi;
                os.lo = o.isum_lo; os.hi = o.isum_hi;
                olo.lo = (u64)o.mn_bits; olo.hi = __double_as_longlong(o.fsum);
                ohi.lo = (u64)o.mx_bits; ohi.hi = o.count;
                const Wide128 l = s + olo, h = s + ohi;
                if (l < lo) lo = l;
                if (hi < h) hi = h;
                s = s + os;
                fl |= o.flags;
            }
            const bool is32 = (fl & SLOT_IS_I32) != 0;
            const Wide128 mn(is32 ? -2147483647LL - 1LL : -0x7fffffffffffffffLL - 1LL), mx(is32 ? 2147483647LL : 0x7fffffffffffffffLL);
            fl = (fl & 0xffffffffull & ~(u64)FLAG_OVERFLOW) | ((lo < mn || mx < hi) ? (u64)FLAG_OVERFLOW : 0ull);
            rec->fsum = 0; rec->count_f = 0; rec->isum_lo = (i64)s.lo; rec->isum_hi = s.hi; rec->count = 0;
            rec->fmin = 0; rec->fmax = 0; rec->imin = 0; rec->imax = 0;
            rec->flags = fl;
            rec->offset = 0; rec->local_count = 0;
            rec->pad[0] = (i64)lo.lo; rec->pad[1] = lo.hi; rec->pad[2] = (i64)hi.lo; rec->pad[3] = hi.hi;
        } else {
            PeerSlot g = slots[0];
            const bool fp = (g.flags & SLOT_IS_FP) != 0, u64cmp = (g.flags & SLOT_IS_U64) != 0;
            i64 below = pt.rank > 0 ? slots[0].count : 0;   // elements counted on lower ranks: this rank's output offset
            for (int r = 1; r < pt.world; ++r) {       // rank order: the same arithmetic on every GPU
                const PeerSlot& o = slots[r];
                if (r < pt.rank) below += o.count;
                g.fsum += o.fsum;
                const u64 lo = g.isum_lo + o.isum_lo;
                g.isum_hi += o.isum_hi + (lo < o.isum_lo ? 1 : 0);
                g.isum_lo = lo;
                g.count += o.count;
                if (fp) {
                    if (__longlong_as_double(o.mn_bits) < __longlong_as_double(g.mn_bits)) g.mn_bits = o.mn_bits;
                    if (__longlong_as_double(o.mx_bits) > __longlong_as_double(g.mx_bits)) g.mx_bits = o.mx_bits;
                } else if (u64cmp) {
                    if ((u64)o.mn_bits < (u64)g.mn_bits) g.mn_bits = o.mn_bits;
                    if ((u64)o.mx_bits > (u64)g.mx_bits) g.mx_bits = o.mx_bits;
                } else {
                    if (o.mn_bits < g.mn_bits) g.mn_bits = o.mn_bits;
                    if (o.mx_bits > g.mx_bits) g.mx_bits = o.mx_bits;
                }
                g.flags |= o.flags;
            }
            rec->fsum = g.fsum; rec->count_f = (double)g.count; rec->isum_lo = (i64)g.isum_lo; rec->isum_hi = g.isum_hi;
            rec->count = g.count;
            if (fp) { rec->fmin = __longlong_as_double(g.mn_bits); rec->fmax = __longlong_as_double(g.mx_bits); rec->imin = 0; rec->imax = 0; }
            else { rec->fmin = 0; rec->fmax = 0; rec->imin = g.mn_bits; rec->imax = g.mx_bits; }
            rec->flags = g.flags & 0xffffffffull;
            rec->offset = below; rec->local_count = slots[pt.rank].count;
        }
        pt.state->seq = seq;
    }
}

}  // namespace dcb
#endif
