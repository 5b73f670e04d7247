// dcb_noalloc.cu — dcb_compact_noalloc(): stable Where [-> Select] -> ToArray without a single device allocation.
//
// Who needs this. Some hosts of this library may not let it allocate device memory: a service that reserved the whole
// of HBM for its own buffer pool at start-up (so any later cudaMalloc fails or breaks its accounting), or a caller on a
// latency-critical path where an allocation's implicit device synchronisation is not acceptable. The ordinary entry
// points allocate look-back descriptors on demand; this one keeps them in a fixed array that is part of the library
// image, and accepts only the queries compiled ahead of time (loading an NVRTC module allocates too).
//
// The scratch is shared by every call on a device and keeps the previous call's contents. Descriptors carry a launch
// epoch, so stale ones read as "not written yet"; the three control words are cleared on the stream before each launch.
// Two calls that overlap on the same GPU (different streams, or different host threads) race on the scratch: callers
// must serialise them. Every GPU that loads the library holds the array (512 KiB + 256 bytes) until the process exits.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/dcb200.h"
#include "dcb_builtin.h"
#include "dcb_internal.h"
#include "dcb_kernels.cuh"
#include "dcb_translate.h"

namespace {

constexpr int kMaxDevices = 64;

// Look-back descriptors for DCB_NOALLOC_MAX_TILES tiles, followed by 256 bytes of control words
// (word 32 is the abort flag; the rest is spare). File scope, device memory, lives as long as the module.
static __device__ __align__(256) unsigned long long g_noalloc_scratch[DCB_NOALLOC_MAX_TILES + 32];

struct DeviceState {
    bool ready = false;
    unsigned long long* scratch = nullptr;   // device address of g_noalloc_scratch on this device
    unsigned int epoch = 0;
};
DeviceState g_state[kMaxDevices];
std::mutex g_mu;
dcb_status fail(dcb_status st, const char* msg) {
    dcb_set_thread_error(msg);   // read back with dcb_last_error(NULL, ...)
    return st;
}

}  // namespace

extern "C" dcb_status dcb_compact_noalloc(int32_t device, const dcb_pipeline_desc* desc, const void* in0, const void* in1,
                                          int64_t n, void* out, int64_t out_cap, void* d_record, void* stream) {
    if (device < 0 || device >= kMaxDevices) return fail(DCB_ERR_INVALID_ARGUMENT, "device index out of range");
    if (!desc || !desc->ops || desc->n_ops <= 0) return fail(DCB_ERR_INVALID_ARGUMENT, "pipeline description is null or empty");
    if (n < 0 || out_cap < 0) return fail(DCB_ERR_INVALID_ARGUMENT, "negative size");
    if (!d_record) return fail(DCB_ERR_INVALID_ARGUMENT, "d_record (device pointer to 128 bytes) is required");
    if (n > 0 && (!in0 || (!out && out_cap > 0))) return fail(DCB_ERR_INVALID_ARGUMENT, "null input or output pointer");

    // Which precompiled kernel? (host-side string work only)
    std::vector<dcbt::OpSpec> ops;
    for (int i = 0; i < desc->n_ops; ++i) {
        dcbt::OpSpec o;
        o.kind = desc->ops[i].kind;
        if (desc->ops[i].lambda) o.lambda = desc->ops[i].lambda;
        ops.push_back(o);
    }
    dcbt::ChainInfo info;
    std::string err;
    int st2 = 0;
    if (!dcbt::build_chain(desc->elem_type0, desc->elem_type1, ops, &info, &err, &st2)) return fail(st2, err.c_str());
    if (!(info.terminal == DCB_OP_TOARRAY && info.has_filter))
        return fail(DCB_ERR_NOT_SUPPORTED, "dcb_compact_noalloc runs Where[->Select]->ToArray queries only");
    if (info.n_in == 2 && n > 0 && !in1) return fail(DCB_ERR_INVALID_ARGUMENT, "in1 is null for a Zip pipeline");
    const dcb_builtin_entry* b = dcb_builtin_find(info.key.c_str());
    if (!b) return fail(DCB_ERR_NOT_SUPPORTED, "this query is not in the precompiled table; building it would allocate");

    // The caller's current device is put back on every way out: with no context object, changing it behind the caller's
    // back would redirect the caller's next CUDA call.
    struct DeviceGuard {
        int prev = -1;
        DeviceGuard() { if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; (void)cudaGetLastError(); } }
        ~DeviceGuard() { if (prev >= 0) (void)cudaSetDevice(prev); }
    } restore_device;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return fail(DCB_ERR_NO_DEVICE, cudaGetErrorString(e)); }
    cudaStream_t s = (cudaStream_t)stream;   // NULL is the default stream here: there is no context object to own one

    // Shape of the launch: same rules as the allocating path (vector kernel when every pointer is 16-byte aligned).
    const int esz = dcbt::type_size(info.in0), osz = dcbt::type_size(info.out_type);
    const int e_vec = 16 / esz;
    auto aligned = [](const void* p, size_t a) { return a <= 1 || ((uintptr_t)p % a) == 0; };
    bool vec = aligned(in0, 16) && aligned(out, (size_t)(e_vec * osz < 16 ? e_vec * osz : 16));
    if (info.n_in == 2) { const int b1 = e_vec * dcbt::type_size(info.in1); vec = vec && aligned(in1, (size_t)(b1 < 16 ? b1 : 16)); }
    const int E = vec ? e_vec : 1;
    const int block = b->compact_block;
    const int rows = dcb::compact_rows_for(block, E, osz);
    const int64_t tile = (int64_t)(block / 32) * rows * 32 * E;
    long long num_tiles = (n + tile - 1) / tile;
    if (num_tiles > DCB_NOALLOC_MAX_TILES) {
        char msg[512];
        snprintf(msg, sizeof msg, "n = %lld needs %lld tiles of %lld elements; the fixed scratch holds %d tiles (at most %lld elements for this query)",
                 (long long)n, num_tiles, (long long)tile, DCB_NOALLOC_MAX_TILES, (long long)tile * DCB_NOALLOC_MAX_TILES);
        return fail(DCB_ERR_INVALID_ARGUMENT, msg);
    }

    unsigned long long* scratch = nullptr;
    unsigned int epoch = 0;
    {
        std::lock_guard<std::mutex> g(g_mu);
        DeviceState& d = g_state[device];
        if (!d.ready) {
            // Once per device, with that device current: the array's name is only a host-side stand-in in host code;
            // the address a kernel can use comes from cudaGetSymbolAddress.
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess) { (void)cudaGetLastError(); return fail(DCB_ERR_CUDA, cudaGetErrorString(e)); }
            d.scratch = (unsigned long long*)p;
            d.epoch = 0;
            d.ready = true;
        }
        d.epoch += 1;
        if (d.epoch >= 0x3fffu) {
            // the epoch field of a descriptor is 14 bits: wipe the descriptors before a value is used again
            e = cudaMemsetAsync(d.scratch, 0, sizeof(unsigned long long) * DCB_NOALLOC_MAX_TILES, s);
            if (e != cudaSuccess) { (void)cudaGetLastError(); return fail(DCB_ERR_CUDA, cudaGetErrorString(e)); }
            d.epoch = 1;
        }
        scratch = d.scratch;
        epoch = d.epoch;
    }
    if (num_tiles == 0) {
        e = cudaMemsetAsync(d_record, 0, DCB_DEVICE_RESULT_BYTES, s);
        if (e != cudaSuccess) { (void)cudaGetLastError(); return fail(DCB_ERR_CUDA, cudaGetErrorString(e)); }
        return DCB_OK;
    }
    unsigned int* words = (unsigned int*)(scratch + DCB_NOALLOC_MAX_TILES);
    e = cudaMemsetAsync(words, 0, 256, s);   // the abort flag must start at zero
    if (e != cudaSuccess) { (void)cudaGetLastError(); return fail(DCB_ERR_CUDA, cudaGetErrorString(e)); }
    unsigned int* abort_flag = words + 32;
    unsigned int spin = 1u << 22;
    long long nn = n, cap = out_cap;
    const void* prev = nullptr;
    void* args[] = {(void*)&in0, (void*)&in1, (void*)&nn, (void*)&out, (void*)&cap, (void*)&scratch,
                    (void*)&epoch, (void*)&spin, (void*)&num_tiles, (void*)&prev, (void*)&d_record, (void*)&abort_flag};
    e = cudaLaunchKernel(vec ? b->k_vec : b->k_scalar, dim3((unsigned)num_tiles), dim3(block), args, 0, s);   // one tile per block
    if (e != cudaSuccess) { (void)cudaGetLastError(); return fail(DCB_ERR_CUDA, cudaGetErrorString(e)); }
    return DCB_OK;
}
