// dcb_api.cu — the C ABI of libdcb200.so (see include/dcb200.h).
//
// Host side of the engine: context and stream per GPU, stream-ordered device memory and pinned staging,
// translation of a query's lambdas into one fused kernel (NVRTC, or the ahead-of-time table), launch
// shaping, and the semantics of the terminal operators. Everything here runs on the GPU or fails with a
// status; there is no host computation path.
#include <cuda_runtime.h>
#include <nvrtc.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../include/dcb200.h"
#include "dcb_builtin.h"
#include "dcb_internal.h"
#include "dcb_kernels.cuh"
#include "dcb_peer.cuh"
#include "dcb_translate.h"

// Text of dcb_kernels.cuh, generated at build time, handed to NVRTC in front of every chain.
static const char* const kKernelsHeaderText =
#include "build/dcb_kernels_embed.inc"
    ;

namespace {

constexpr int kBlock = 256;
constexpr int kMaxPartials = 8192;
constexpr size_t kHostChunkBytes = 32u << 20;

thread_local char tl_error[1024] = "";

// Device scratch of one pipeline on one stream. Launches on one stream run one after the other and may share it; launches
// of the same pipeline on different streams may overlap on the GPU, so every stream gets a set of its own.
struct Scratch {
    dcb::Partial* partials = nullptr;
    unsigned int* words = nullptr;      // 512 bytes: [0] reduce ticket, [32] [33] tile-id and finished-block counters of the
                                        // persistent compaction kernels, [64] compaction abort flag, [65] "withhold the first
                                        // count" word of the time-out test (separate 128-byte lines)
    unsigned long long* desc = nullptr; // look-back descriptors of the one-tile-per-block kernel (64-bit), followed by
    unsigned int* cdesc = nullptr;      // the 32-bit count descriptors of the streamed kernel (same allocation)
    size_t desc_cap = 0;
    unsigned int epoch = 0;
};

// Pipelines that exist, so that a handle used after dcb_shutdown or after its eviction is refused instead of followed.
std::mutex g_live_mu;
std::set<const void*> g_live_pipelines;

}  // namespace

struct dcb_ctx {
    int device = 0;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    cudaStream_t own_stream = nullptr, stream = nullptr, copy_stream = nullptr, out_stream = nullptr;
    cudaMemPool_t pool = nullptr;
    uint32_t spin_limit = 1u << 22;
    uint32_t peer_spin_limit = 1u << 20;   // polls of one wait for a peer's partial (about a second with the back-off)
    char err[1024] = "";
    std::mutex mu;
    std::map<std::string, dcb_pipeline*> cache;
    int64_t bytes_in_use = 0, peak_bytes = 0, n_allocs = 0;
    std::atomic<int64_t> launches{0};
    // Options (dcb_set_option); the initial values come from the environment once, at dcb_init.
    int opt_compact_kernel = 0;            // DCB_OPT_COMPACT_KERNEL
    int opt_force_scalar = 0;              // DCB_OPT_FORCE_SCALAR
    int opt_blocks_per_sm = 0;             // DCB_OPT_BLOCKS_PER_SM (0 = what fits)
    int opt_withhold_first_count = 0;      // DCB_OPT_WITHHOLD_FIRST_COUNT
    int opt_cache_max = 100;               // DCB_OPT_CACHE_MAX_ENTRIES (the reference: new KernelCache(maxEntries: 100))
    int opt_overlap_launches = 0;          // DCB_OPT_OVERLAP_LAUNCHES
    uint64_t cache_clock = 0;              // use counter behind the cache's least-recently-used order
    std::mutex host_mu;                    // serialises dcb_pipeline_run_host: the staging buffers belong to the context
    // Staging ring of the host path: kRingIn chunk buffers per input, kRingOut chunk buffers for the output, with the
    // events that hand a slot from the copy engine to the kernel and back. Allocated on first use, kept until shutdown.
    void* ring_in[2][3] = {{nullptr, nullptr, nullptr}, {nullptr, nullptr, nullptr}};
    void* ring_out[2] = {nullptr, nullptr};
    size_t ring_in_bytes = 0, ring_out_bytes = 0;
    cudaEvent_t ev_copied[3] = {nullptr, nullptr, nullptr};    // H2D of the chunk in input slot i has landed
    cudaEvent_t ev_computed[3] = {nullptr, nullptr, nullptr};  // the kernel that read input slot i is done
    cudaEvent_t ev_filled[2] = {nullptr, nullptr};             // the kernel that wrote output slot i is done
    cudaEvent_t ev_drained[2] = {nullptr, nullptr};            // D2H of output slot i is done
    cudaEvent_t ev_record[2] = {nullptr, nullptr};             // the record of the chunk in output slot i is on the host
    void* host_recs = nullptr;             // pinned: per-chunk records of the host path (grow-only)
    void* dev_recs = nullptr;
    size_t recs_cap = 0;                   // in records
    bool alive = true;
    // exchange of partials between GPUs (see PeerTable in dcb_kernels.cuh)
    dcb::PeerTable peers = {};
    void* peer_area = nullptr;             // this GPU's exchange area (cudaMalloc, exported over CUDA IPC)
    void* peer_state = nullptr;            // launch counter and pending record (device memory)
    std::vector<void*> peer_opened;        // areas of other ranks opened here
};

struct dcb_buf {
    dcb_ctx* ctx = nullptr;
    void* ptr = nullptr;
    size_t bytes = 0;
    bool owned = false;
};

struct dcb_pipeline {
    dcb_ctx* ctx = nullptr;
    dcbt::ChainInfo info;
    std::string source;
    cudaLibrary_t lib = nullptr;
    const void* k_vec = nullptr;
    const void* k_scalar = nullptr;
    bool precompiled = false;
    int unroll = 4;
    int occ_vec = 1, occ_scalar = 1;     // resident blocks per SM
    int rows_vec = 1, rows_scalar = 1;   // compaction rows per warp
    int jit_rows = 0;                    // rows forced by a tuning experiment (0 = automatic)
    int compact_block = 256;             // threads per block of the compaction kernels
    const void* k_stream = nullptr;      // streamed compaction kernel (null: the query has none)
    unsigned int* fault_word = nullptr;  // device word the lambdas' checked integer divisions set (null: the query has none)
    int stream_rows = 0, stream_warps = 0, stream_nbuf = 0, stream_copy_warps = 0, occ_stream = 1;
    std::mutex mu;                       // guards `scratch` and every enqueue that uses it
    std::map<cudaStream_t, Scratch> scratch;
    std::mutex run_mu;                   // serialises the blocking calls, which share d_result / h_record / ev0 / ev1
    uint64_t last_use = 0;
    dcb::DeviceResult* d_result = nullptr;
    void* h_record = nullptr;            // pinned, DCB_DEVICE_RESULT_BYTES * kMaxChunks
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    double compile_ms = 0;
    int refs = 1;
    bool alive = true;
};

struct dcb_kernel {
    dcb_ctx* ctx = nullptr;
    cudaLibrary_t lib = nullptr;
    const void* fn = nullptr;
};

namespace {

dcb_status set_err(dcb_ctx* ctx, dcb_status st, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    snprintf(tl_error, sizeof tl_error, "%s", buf);
    if (ctx) snprintf(ctx->err, sizeof ctx->err, "%s", buf);
    return st;
}

dcb_status cuda_fail(dcb_ctx* ctx, cudaError_t e, const char* what) {
    dcb_status st = DCB_ERR_CUDA;
    if (e == cudaErrorMemoryAllocation) st = DCB_ERR_OUT_OF_MEMORY;
    else if (e == cudaErrorNotReady) st = DCB_ERR_NOT_READY;
    else if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) st = DCB_ERR_NO_DEVICE;
    else if (e == cudaErrorInvalidValue) st = DCB_ERR_INVALID_ARGUMENT;
    (void)cudaGetLastError();
    return set_err(ctx, st, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

#define CU(ctx, call)                                                \
    do {                                                             \
        cudaError_t e__ = (call);                                    \
        if (e__ != cudaSuccess) return cuda_fail((ctx), e__, #call); \
    } while (0)

#define NEED(ctx, cond, what)                                                         \
    do {                                                                              \
        if (!(cond)) return set_err((ctx), DCB_ERR_INVALID_ARGUMENT, "%s", (what));   \
    } while (0)

dcb_status use(dcb_ctx* ctx) {
    if (!ctx) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "ctx is null");
    if (!ctx->alive) return set_err(nullptr, DCB_ERR_DISPOSED, "context was shut down");
    CU(ctx, cudaSetDevice(ctx->device));
    return DCB_OK;
}

cudaStream_t pick(dcb_ctx* ctx, void* stream) { return stream ? (cudaStream_t)stream : ctx->stream; }

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

__global__ void fill_kernel(unsigned char* dst, size_t count, unsigned long long pattern, int pattern_bytes) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        switch (pattern_bytes) {
            case 1: dst[i] = (unsigned char)pattern; break;
            case 2: reinterpret_cast<unsigned short*>(dst)[i] = (unsigned short)pattern; break;
            case 4: reinterpret_cast<unsigned int*>(dst)[i] = (unsigned int)pattern; break;
            default: reinterpret_cast<unsigned long long*>(dst)[i] = pattern; break;
        }
    }
}

// Bytes a pointer must be aligned to for the vector variant: one pack of E elements, at most 16.
size_t pack_align(int elems, int type) { return (size_t)std::min(16, elems * dcbt::type_size(type)); }

int compact_rows(int block, int elems, int out_type) { return dcb::compact_rows_for(block, elems, dcbt::type_size(out_type)); }

// The scratch set of pipeline `p` for stream `s` (p->mu held), with room for `num_tiles` descriptors. What must start at
// zero is cleared ON `s`, so the clearing is ordered before the launch that follows on the same stream.
dcb_status ensure_scratch(dcb_pipeline* p, int64_t num_tiles, cudaStream_t s, Scratch** out) {
    dcb_ctx* ctx = p->ctx;
    Scratch& sc = p->scratch[s];
    *out = &sc;
    if (!sc.partials) {
        CU(ctx, cudaMalloc(&sc.partials, sizeof(dcb::Partial) * kMaxPartials));
        CU(ctx, cudaMalloc(&sc.words, 1024));   // words 0..127: compaction (counters at 32, abort word at 64); 128..192: the reductions' tickets
        CU(ctx, cudaMemsetAsync(sc.words, 0, 1024, s));
    }
    if ((size_t)num_tiles > sc.desc_cap) {
        size_t cap = std::max<size_t>((size_t)num_tiles, 1024);
        cap = std::max(cap, sc.desc_cap * 2);
        if (sc.desc) { CU(ctx, cudaStreamSynchronize(s)); CU(ctx, cudaFree(sc.desc)); sc.desc = nullptr; sc.desc_cap = 0; }
        cap = (cap + 3) & ~(size_t)3;
        const size_t bytes = cap * sizeof(unsigned long long) + (cap + 8) * sizeof(unsigned int);   // the streamed kernel reads 16 bytes at a time
        CU(ctx, cudaMalloc(&sc.desc, bytes));
        CU(ctx, cudaMemsetAsync(sc.desc, 0, bytes, s));
        sc.cdesc = reinterpret_cast<unsigned int*>(sc.desc + cap);
        sc.desc_cap = cap;
        sc.epoch = 0;
    }
    return DCB_OK;
}

dcb_status load_jit(dcb_ctx* ctx, dcb_pipeline* p) {
    dcbt::Tuning tuning;   // the defaults, unless a tuning experiment overrides them through the environment
    tuning.unroll = env_int("DCB200_UNROLL", tuning.unroll);
    tuning.reduce_min_blocks = env_int("DCB200_REDUCE_MINBLOCKS", 0);
    tuning.compact_block = env_int("DCB200_COMPACT_BLOCK", tuning.compact_block);
    tuning.compact_rows = env_int("DCB200_COMPACT_ROWS", 0);
    tuning.compact_min_blocks = env_int("DCB200_COMPACT_MINBLOCKS", tuning.compact_min_blocks);
    p->compact_block = tuning.compact_block;
    tuning.stream = env_int("DCB200_STREAM", tuning.stream);
    tuning.stream_warps = env_int("DCB200_STREAM_WARPS", tuning.stream_warps);
    tuning.stream_rows = env_int("DCB200_STREAM_ROWS", 0);
    tuning.stream_lag = env_int("DCB200_STREAM_LAG", tuning.stream_lag);
    tuning.stream_nbuf = env_int("DCB200_STREAM_NBUF", tuning.stream_nbuf);
    tuning.stream_copy_warps = env_int("DCB200_STREAM_COPY_WARPS", tuning.stream_copy_warps);
    tuning.stream_depth = env_int("DCB200_STREAM_DEPTH", tuning.stream_depth);
    tuning.stream_ahead_mb = env_int("DCB200_STREAM_AHEAD_MB", tuning.stream_ahead_mb);
    tuning.stream_min_blocks = env_int("DCB200_STREAM_MINBLOCKS", tuning.stream_min_blocks);
    tuning.stream_draw_ahead = env_int("DCB200_STREAM_DRAW_AHEAD", tuning.stream_draw_ahead);
    p->stream_warps = tuning.stream_warps;
    p->stream_nbuf = tuning.stream_nbuf;
    p->stream_copy_warps = tuning.stream_copy_warps;
    p->stream_rows = (tuning.stream && dcbt::stream_rows_for(p->info, tuning.stream_warps) > 0)
                         ? (tuning.stream_rows > 0 ? tuning.stream_rows : dcbt::stream_rows_for(p->info, tuning.stream_warps)) : 0;
    p->unroll = tuning.unroll;
    p->jit_rows = tuning.compact_rows;
    p->source = dcbt::build_program(p->info, "", kKernelsHeaderText, tuning, true);
    nvrtcProgram prog = nullptr;
    if (nvrtcCreateProgram(&prog, p->source.c_str(), "dcb_pipeline.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
        return set_err(ctx, DCB_ERR_COMPILE, "nvrtcCreateProgram failed");
    // No --use_fast_math and no FMA contraction: a Select must round exactly like the C# lambda does.
    // Extra options for tuning experiments, space separated (the counterpart of CompilationOptions.AdditionalFlags,
    // consumed by the reference at src/Backends/DotCompute.Backends.CUDA/Compilation/PTXCompiler.cs:251-270).
    std::vector<std::string> extra;
    if (const char* ev = getenv("DCB200_NVRTC_FLAGS")) {
        std::string cur;
        for (const char* c = ev;; ++c) {
            if (*c == ' ' || *c == '\0') { if (!cur.empty()) extra.push_back(cur); cur.clear(); if (!*c) break; }
            else cur += *c;
        }
    }
    std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-fmad=false", "-lineinfo"};
    for (const auto& e : extra) opts.push_back(e.c_str());
    nvrtcResult r = nvrtcCompileProgram(prog, (int)opts.size(), opts.data());
    if (r != NVRTC_SUCCESS) {
        size_t n = 0;
        nvrtcGetProgramLogSize(prog, &n);
        std::string log(n + 1, '\0');
        nvrtcGetProgramLog(prog, &log[0]);
        nvrtcDestroyProgram(&prog);
        return set_err(ctx, DCB_ERR_COMPILE, "NVRTC: %s: %.800s", nvrtcGetErrorString(r), log.c_str());
    }
    size_t sz = 0;
    nvrtcGetCUBINSize(prog, &sz);
    std::vector<char> cubin(sz);
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    CU(ctx, cudaLibraryLoadData(&p->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    const char* stem = (p->info.terminal == DCB_OP_TOARRAY) ? (p->info.has_filter ? "dcb_compact_" : "dcb_map_") : "dcb_reduce_";
    cudaKernel_t kv = nullptr, ks = nullptr;
    CU(ctx, cudaLibraryGetKernel(&kv, p->lib, (std::string(stem) + "vec").c_str()));
    CU(ctx, cudaLibraryGetKernel(&ks, p->lib, (std::string(stem) + "scalar").c_str()));
    p->k_vec = (const void*)kv;
    p->k_scalar = (const void*)ks;
    if (p->info.checked_div) {
        void* w = nullptr; size_t bytes = 0;
        CU(ctx, cudaLibraryGetGlobal(&w, &bytes, p->lib, "dcb_fault_word"));
        p->fault_word = (unsigned int*)w;
    }
    if (p->stream_rows > 0) {
        cudaKernel_t kst = nullptr;
        CU(ctx, cudaLibraryGetKernel(&kst, p->lib, "dcb_compact_stream"));
        p->k_stream = (const void*)kst;
    }
    return DCB_OK;
}

dcb_status finish_pipeline(dcb_ctx* ctx, dcb_pipeline* p) {
    const int e_vec = 16 / dcbt::type_size(p->info.in0);
    p->rows_vec = p->jit_rows > 0 ? p->jit_rows : compact_rows(p->compact_block, e_vec, p->info.out_type);
    p->rows_scalar = p->jit_rows > 0 ? p->jit_rows : compact_rows(p->compact_block, 1, p->info.out_type);
    const int blk = (p->info.terminal == DCB_OP_TOARRAY && p->info.has_filter) ? p->compact_block : kBlock;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, p->k_vec, blk, 0) == cudaSuccess && occ > 0) p->occ_vec = occ;
    else { (void)cudaGetLastError(); p->occ_vec = 4; }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, p->k_scalar, blk, 0) == cudaSuccess && occ > 0) p->occ_scalar = occ;
    else { (void)cudaGetLastError(); p->occ_scalar = 4; }
    // More than 48 KB of dynamic shared memory has to be asked for once per kernel.
    if (p->k_stream) {
        const int dyn = (int)dcbt::stream_smem_bytes(p->info, p->stream_rows, p->stream_warps, p->stream_nbuf);
        if (cudaFuncSetAttribute(p->k_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) == cudaSuccess &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, p->k_stream, dcbt::stream_block_threads(p->stream_warps, p->stream_copy_warps), (size_t)dyn) == cudaSuccess && occ > 0) p->occ_stream = occ;
        else { (void)cudaGetLastError(); p->k_stream = nullptr; }
    }
    CU(ctx, cudaMalloc(&p->d_result, DCB_DEVICE_RESULT_BYTES));
    CU(ctx, cudaMemsetAsync(p->d_result, 0, DCB_DEVICE_RESULT_BYTES, ctx->stream));
    CU(ctx, cudaHostAlloc(&p->h_record, DCB_DEVICE_RESULT_BYTES, cudaHostAllocDefault));
    CU(ctx, cudaEventCreate(&p->ev0));
    CU(ctx, cudaEventCreate(&p->ev1));
    {
        std::lock_guard<std::mutex> g(g_live_mu);
        g_live_pipelines.insert(p);
    }
    return DCB_OK;
}

void free_pipeline(dcb_pipeline* p) {
    if (!p) return;
    {
        std::lock_guard<std::mutex> g(g_live_mu);
        g_live_pipelines.erase(p);
    }
    for (auto& kv : p->scratch) {
        if (kv.second.partials) cudaFree(kv.second.partials);
        if (kv.second.words) cudaFree(kv.second.words);
        if (kv.second.desc) cudaFree(kv.second.desc);
    }
    if (p->d_result) cudaFree(p->d_result);
    if (p->h_record) cudaFreeHost(p->h_record);
    if (p->ev0) cudaEventDestroy(p->ev0);
    if (p->ev1) cudaEventDestroy(p->ev1);
    if (p->lib) cudaLibraryUnload(p->lib);
    p->alive = false;
    delete p;
}

dcb_status desc_to_ops(const dcb_pipeline_desc* desc, std::vector<dcbt::OpSpec>* ops, char* err, size_t err_cap) {
    if (!desc || desc->n_ops <= 0 || !desc->ops) { snprintf(err, err_cap, "pipeline description is null or empty"); return DCB_ERR_INVALID_ARGUMENT; }
    for (int i = 0; i < desc->n_ops; ++i) {
        dcbt::OpSpec o;
        o.kind = desc->ops[i].kind;
        const bool needs_lambda = o.kind == DCB_OP_SELECT || o.kind == DCB_OP_WHERE || o.kind == DCB_OP_ZIP;
        if (needs_lambda && !desc->ops[i].lambda) { snprintf(err, err_cap, "operator %d has a null lambda", i); return DCB_ERR_INVALID_ARGUMENT; }
        if (desc->ops[i].lambda) o.lambda = desc->ops[i].lambda;
        ops->push_back(o);
    }
    return DCB_OK;
}

}  // namespace

void dcb_set_thread_error(const char* msg) { snprintf(tl_error, sizeof tl_error, "%s", msg ? msg : ""); }
int dcb_ctx_make_current(dcb_ctx* ctx) { return (int)use(ctx); }
void* dcb_ctx_pick_stream(dcb_ctx* ctx, void* stream) { return (void*)pick(ctx, stream); }
void dcb_ctx_count_launches(dcb_ctx* ctx, int n) { ctx->launches += n; }

// ============================================================================================ status
extern "C" int32_t dcb_abi_version(void) { return DCB_ABI_VERSION; }

extern "C" int32_t dcb_status_class(dcb_status s) {
    if (s == DCB_OK) return DCB_CLASS_NONE;
    switch (s / 100) {
        case 1: return DCB_CLASS_TRANSIENT;
        case 2: return DCB_CLASS_RESOURCE;
        case 3: return DCB_CLASS_PROGRAMMER;
        case 4: return DCB_CLASS_FATAL;
        case 5: return DCB_CLASS_QUERY;
        default: return DCB_CLASS_FATAL;
    }
}

extern "C" const char* dcb_status_name(dcb_status s) {
    switch (s) {
        case DCB_OK: return "DCB_OK";
        case DCB_ERR_NOT_READY: return "DCB_ERR_NOT_READY";
        case DCB_ERR_TIMEOUT: return "DCB_ERR_TIMEOUT";
        case DCB_ERR_OUT_OF_MEMORY: return "DCB_ERR_OUT_OF_MEMORY";
        case DCB_ERR_OUTPUT_TOO_SMALL: return "DCB_ERR_OUTPUT_TOO_SMALL";
        case DCB_ERR_INVALID_ARGUMENT: return "DCB_ERR_INVALID_ARGUMENT";
        case DCB_ERR_NOT_SUPPORTED: return "DCB_ERR_NOT_SUPPORTED";
        case DCB_ERR_COMPILE: return "DCB_ERR_COMPILE";
        case DCB_ERR_DISPOSED: return "DCB_ERR_DISPOSED";
        case DCB_ERR_NO_DEVICE: return "DCB_ERR_NO_DEVICE";
        case DCB_ERR_CUDA: return "DCB_ERR_CUDA";
        case DCB_ERR_EMPTY_SEQUENCE: return "DCB_ERR_EMPTY_SEQUENCE";
        case DCB_ERR_OVERFLOW: return "DCB_ERR_OVERFLOW";
        case DCB_ERR_DIVIDE_BY_ZERO: return "DCB_ERR_DIVIDE_BY_ZERO";
        default: return "DCB_ERR_UNKNOWN";
    }
}

extern "C" int32_t dcb_type_size(int32_t type) { return dcbt::type_size(type); }

// ========================================================================================= lifecycle
extern "C" dcb_status dcb_device_count(int32_t* out_count) {
    if (!out_count) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "out_count is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    *out_count = (e == cudaSuccess) ? n : 0;
    if (e != cudaSuccess || n == 0) { (void)cudaGetLastError(); return set_err(nullptr, DCB_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e)); }
    return DCB_OK;
}

extern "C" dcb_status dcb_init(int32_t device, dcb_ctx** out_ctx) {
    if (!out_ctx) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "out_ctx is null");
    *out_ctx = nullptr;
    int n = 0;
    dcb_status st = dcb_device_count(&n);
    if (st != DCB_OK) return st;
    if (device < 0 || device >= n) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "device %d out of range (0..%d)", device, n - 1);
    dcb_ctx* ctx = new dcb_ctx();
    ctx->device = device;
    cudaError_t e = cudaSetDevice(device);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->out_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaDeviceGetDefaultMemPool(&ctx->pool, device);
    if (e == cudaSuccess) {
        // Keep freed blocks in the pool: a query allocates and frees the same sizes over and over.
        unsigned long long keep = ~0ull;
        e = cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    if (e != cudaSuccess) { dcb_status s = cuda_fail(nullptr, e, "dcb_init"); delete ctx; return s; }
    ctx->stream = ctx->own_stream;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->spin_limit = (uint32_t)env_int("DCB200_SPIN_LIMIT", 1 << 22);
    // The environment is read here, once; afterwards these are changed with dcb_set_option.
    ctx->opt_compact_kernel = env_int("DCB200_COMPACT_KERNEL", 0);
    ctx->opt_force_scalar = env_int("DCB200_FORCE_SCALAR", 0);
    ctx->opt_blocks_per_sm = env_int("DCB200_BLOCKS_PER_SM", 0);
    ctx->opt_cache_max = std::max(1, env_int("DCB200_CACHE_MAX_ENTRIES", 100));
    if (prop.major != 10) {
        delete ctx;
        return set_err(nullptr, DCB_ERR_NO_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
    }
    *out_ctx = ctx;
    return DCB_OK;
}

extern "C" dcb_status dcb_shutdown(dcb_ctx* ctx) {
    if (!ctx) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "ctx is null");
    if (!ctx->alive) return DCB_ERR_DISPOSED;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    for (auto& kv : ctx->cache) free_pipeline(kv.second);
    ctx->cache.clear();
    for (void* p : ctx->peer_opened) cudaIpcCloseMemHandle(p);
    if (ctx->peer_area) cudaFree(ctx->peer_area);
    if (ctx->peer_state) cudaFree(ctx->peer_state);
    for (int i = 0; i < 2; ++i) for (int j = 0; j < 3; ++j) if (ctx->ring_in[i][j]) cudaFree(ctx->ring_in[i][j]);
    for (int i = 0; i < 2; ++i) if (ctx->ring_out[i]) cudaFree(ctx->ring_out[i]);
    for (int i = 0; i < 3; ++i) { if (ctx->ev_copied[i]) cudaEventDestroy(ctx->ev_copied[i]); if (ctx->ev_computed[i]) cudaEventDestroy(ctx->ev_computed[i]); }
    for (int i = 0; i < 2; ++i) {
        if (ctx->ev_filled[i]) cudaEventDestroy(ctx->ev_filled[i]);
        if (ctx->ev_drained[i]) cudaEventDestroy(ctx->ev_drained[i]);
        if (ctx->ev_record[i]) cudaEventDestroy(ctx->ev_record[i]);
    }
    if (ctx->dev_recs) cudaFree(ctx->dev_recs);
    if (ctx->host_recs) cudaFreeHost(ctx->host_recs);
    cudaStreamDestroy(ctx->own_stream);
    cudaStreamDestroy(ctx->copy_stream);
    cudaStreamDestroy(ctx->out_stream);
    ctx->alive = false;
    delete ctx;
    return DCB_OK;
}

extern "C" dcb_status dcb_last_error(dcb_ctx* ctx, char* buf, size_t cap) {
    if (!buf || cap == 0) return DCB_ERR_INVALID_ARGUMENT;
    snprintf(buf, cap, "%s", (ctx && ctx->alive) ? ctx->err : tl_error);
    return DCB_OK;
}

extern "C" dcb_status dcb_device_info(dcb_ctx* ctx, char* name, size_t name_cap, int32_t* sm_count, int64_t* total_mem,
                                      int32_t* cc_major, int32_t* cc_minor) {
    dcb_status st = use(ctx);
    if (st) return st;
    cudaDeviceProp prop;
    CU(ctx, cudaGetDeviceProperties(&prop, ctx->device));
    if (name && name_cap) snprintf(name, name_cap, "%s", prop.name);
    if (sm_count) *sm_count = prop.multiProcessorCount;
    if (total_mem) *total_mem = (int64_t)prop.totalGlobalMem;
    if (cc_major) *cc_major = prop.major;
    if (cc_minor) *cc_minor = prop.minor;
    return DCB_OK;
}

extern "C" dcb_status dcb_set_stream(dcb_ctx* ctx, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    ctx->stream = stream ? (cudaStream_t)stream : ctx->own_stream;
    return DCB_OK;
}

extern "C" dcb_status dcb_stream_sync(dcb_ctx* ctx, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    CU(ctx, cudaStreamSynchronize(pick(ctx, stream)));
    return DCB_OK;
}

extern "C" dcb_status dcb_set_spin_limit(dcb_ctx* ctx, uint32_t max_polls) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, max_polls > 0, "max_polls must be positive");
    ctx->spin_limit = max_polls;
    ctx->peer_spin_limit = max_polls;
    ctx->peers.spin_limit = max_polls;
    return DCB_OK;
}

extern "C" dcb_status dcb_set_option(dcb_ctx* ctx, int32_t option, int64_t value) {
    dcb_status st = use(ctx);
    if (st) return st;
    std::lock_guard<std::mutex> g(ctx->mu);
    switch (option) {
        case DCB_OPT_COMPACT_KERNEL:
            NEED(ctx, value >= 0 && value <= 1, "DCB_OPT_COMPACT_KERNEL takes 0 (automatic) or 1 (one tile per block)");
            ctx->opt_compact_kernel = (int)value; return DCB_OK;
        case DCB_OPT_FORCE_SCALAR: ctx->opt_force_scalar = value != 0; return DCB_OK;
        case DCB_OPT_BLOCKS_PER_SM:
            NEED(ctx, value >= 0 && value <= 32, "DCB_OPT_BLOCKS_PER_SM takes 0 (what fits) to 32");
            ctx->opt_blocks_per_sm = (int)value; return DCB_OK;
        case DCB_OPT_WITHHOLD_FIRST_COUNT: ctx->opt_withhold_first_count = value != 0; return DCB_OK;
        case DCB_OPT_CACHE_MAX_ENTRIES:
            NEED(ctx, value >= 1 && value <= (1 << 20), "DCB_OPT_CACHE_MAX_ENTRIES takes 1 to 2^20");
            ctx->opt_cache_max = (int)value; return DCB_OK;
        case DCB_OPT_OVERLAP_LAUNCHES: ctx->opt_overlap_launches = value != 0; return DCB_OK;
        default: return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "unknown option %d", (int)option);
    }
}

extern "C" dcb_status dcb_get_option(dcb_ctx* ctx, int32_t option, int64_t* out_value) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_value != nullptr, "out_value is null");
    std::lock_guard<std::mutex> g(ctx->mu);
    switch (option) {
        case DCB_OPT_COMPACT_KERNEL: *out_value = ctx->opt_compact_kernel; return DCB_OK;
        case DCB_OPT_FORCE_SCALAR: *out_value = ctx->opt_force_scalar; return DCB_OK;
        case DCB_OPT_BLOCKS_PER_SM: *out_value = ctx->opt_blocks_per_sm; return DCB_OK;
        case DCB_OPT_WITHHOLD_FIRST_COUNT: *out_value = ctx->opt_withhold_first_count; return DCB_OK;
        case DCB_OPT_CACHE_MAX_ENTRIES: *out_value = ctx->opt_cache_max; return DCB_OK;
        case DCB_OPT_CACHE_ENTRIES: *out_value = (int64_t)ctx->cache.size(); return DCB_OK;
        case DCB_OPT_OVERLAP_LAUNCHES: *out_value = ctx->opt_overlap_launches; return DCB_OK;
        default: return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "unknown option %d", (int)option);
    }
}

// ============================================================================================ memory
extern "C" dcb_status dcb_alloc(dcb_ctx* ctx, size_t bytes, dcb_buf** out_buf) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_buf != nullptr, "out_buf is null");
    *out_buf = nullptr;
    void* p = nullptr;
    if (bytes > 0) {
        CU(ctx, cudaMallocAsync(&p, bytes, ctx->stream));
    }
    dcb_buf* b = new dcb_buf();
    b->ctx = ctx; b->ptr = p; b->bytes = bytes; b->owned = true;
    {
        std::lock_guard<std::mutex> g(ctx->mu);
        ctx->bytes_in_use += (int64_t)bytes;
        ctx->peak_bytes = std::max(ctx->peak_bytes, ctx->bytes_in_use);
        ctx->n_allocs += 1;
    }
    *out_buf = b;
    return DCB_OK;
}

extern "C" dcb_status dcb_free(dcb_ctx* ctx, dcb_buf* buf) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, buf != nullptr, "buf is null");
    if (buf->ctx != ctx) return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "buffer belongs to another context");
    if (buf->owned && buf->ptr) {
        CU(ctx, cudaFreeAsync(buf->ptr, ctx->stream));
        std::lock_guard<std::mutex> g(ctx->mu);
        ctx->bytes_in_use -= (int64_t)buf->bytes;
    }
    delete buf;
    return DCB_OK;
}

extern "C" dcb_status dcb_buf_wrap(dcb_ctx* ctx, void* device_ptr, size_t bytes, dcb_buf** out_buf) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_buf != nullptr, "out_buf is null");
    NEED(ctx, device_ptr != nullptr || bytes == 0, "device_ptr is null");
    dcb_buf* b = new dcb_buf();
    b->ctx = ctx; b->ptr = device_ptr; b->bytes = bytes; b->owned = false;
    *out_buf = b;
    return DCB_OK;
}

extern "C" dcb_status dcb_buf_slice(dcb_ctx* ctx, dcb_buf* parent, size_t byte_offset, size_t bytes, dcb_buf** out_buf) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, parent != nullptr && out_buf != nullptr, "parent or out_buf is null");
    if (byte_offset > parent->bytes || bytes > parent->bytes - byte_offset)
        return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "slice [%zu, +%zu) outside a buffer of %zu bytes", byte_offset, bytes, parent->bytes);
    dcb_buf* b = new dcb_buf();
    b->ctx = ctx; b->ptr = (char*)parent->ptr + byte_offset; b->bytes = bytes; b->owned = false;
    *out_buf = b;
    return DCB_OK;
}

extern "C" void* dcb_devptr(const dcb_buf* buf) { return buf ? buf->ptr : nullptr; }
extern "C" size_t dcb_buf_bytes(const dcb_buf* buf) { return buf ? buf->bytes : 0; }

static dcb_status check_range(dcb_ctx* ctx, const dcb_buf* b, size_t off, size_t bytes, const char* what) {
    if (!b) return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "%s buffer is null", what);
    if (off > b->bytes || bytes > b->bytes - off)
        return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "%s range [%zu, +%zu) outside a buffer of %zu bytes", what, off, bytes, b->bytes);
    return DCB_OK;
}

extern "C" dcb_status dcb_h2d_async(dcb_ctx* ctx, dcb_buf* dst, size_t dst_off, const void* host, size_t bytes, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    if ((st = check_range(ctx, dst, dst_off, bytes, "destination"))) return st;
    NEED(ctx, host != nullptr || bytes == 0, "host pointer is null");
    if (bytes) CU(ctx, cudaMemcpyAsync((char*)dst->ptr + dst_off, host, bytes, cudaMemcpyHostToDevice, pick(ctx, stream)));
    return DCB_OK;
}

extern "C" dcb_status dcb_d2h_async(dcb_ctx* ctx, void* host, const dcb_buf* src, size_t src_off, size_t bytes, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    if ((st = check_range(ctx, src, src_off, bytes, "source"))) return st;
    NEED(ctx, host != nullptr || bytes == 0, "host pointer is null");
    if (bytes) CU(ctx, cudaMemcpyAsync(host, (const char*)src->ptr + src_off, bytes, cudaMemcpyDeviceToHost, pick(ctx, stream)));
    return DCB_OK;
}

extern "C" dcb_status dcb_d2d_async(dcb_ctx* ctx, dcb_buf* dst, size_t dst_off, const dcb_buf* src, size_t src_off, size_t bytes, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    if ((st = check_range(ctx, dst, dst_off, bytes, "destination"))) return st;
    if ((st = check_range(ctx, src, src_off, bytes, "source"))) return st;
    if (bytes) CU(ctx, cudaMemcpyAsync((char*)dst->ptr + dst_off, (const char*)src->ptr + src_off, bytes, cudaMemcpyDeviceToDevice, pick(ctx, stream)));
    return DCB_OK;
}

extern "C" dcb_status dcb_fill_async(dcb_ctx* ctx, dcb_buf* dst, size_t dst_off, const void* pattern, int32_t pattern_bytes, size_t count, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, pattern != nullptr, "pattern is null");
    NEED(ctx, pattern_bytes == 1 || pattern_bytes == 2 || pattern_bytes == 4 || pattern_bytes == 8, "pattern must be 1, 2, 4 or 8 bytes");
    if ((st = check_range(ctx, dst, dst_off, count * (size_t)pattern_bytes, "destination"))) return st;
    NEED(ctx, dst_off % (size_t)pattern_bytes == 0, "offset must be a multiple of the pattern size");
    if (count == 0) return DCB_OK;
    unsigned long long pat = 0;
    memcpy(&pat, pattern, (size_t)pattern_bytes);
    const int grid = (int)std::min<size_t>((count + 255) / 256, (size_t)ctx->sm_count * 8);
    fill_kernel<<<grid, 256, 0, pick(ctx, stream)>>>((unsigned char*)dst->ptr + dst_off, count, pat, pattern_bytes);
    CU(ctx, cudaGetLastError());
    ctx->launches += 1;
    return DCB_OK;
}

extern "C" dcb_status dcb_host_alloc_pinned(dcb_ctx* ctx, size_t bytes, void** out_host) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_host != nullptr, "out_host is null");
    *out_host = nullptr;
    if (bytes == 0) return DCB_OK;
    CU(ctx, cudaHostAlloc(out_host, bytes, cudaHostAllocPortable));
    return DCB_OK;
}

extern "C" dcb_status dcb_host_free_pinned(dcb_ctx* ctx, void* host) {
    dcb_status st = use(ctx);
    if (st) return st;
    if (host) CU(ctx, cudaFreeHost(host));
    return DCB_OK;
}

extern "C" dcb_status dcb_pin_host(dcb_ctx* ctx, void* host, size_t bytes) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, host != nullptr && bytes > 0, "host range is empty");
    CU(ctx, cudaHostRegister(host, bytes, cudaHostRegisterPortable));
    return DCB_OK;
}

extern "C" dcb_status dcb_unpin_host(dcb_ctx* ctx, void* host) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, host != nullptr, "host pointer is null");
    CU(ctx, cudaHostUnregister(host));
    return DCB_OK;
}

extern "C" dcb_status dcb_memory_stats(dcb_ctx* ctx, int64_t* bytes_in_use, int64_t* peak_bytes, int64_t* n_allocs) {
    dcb_status st = use(ctx);
    if (st) return st;
    std::lock_guard<std::mutex> g(ctx->mu);
    if (bytes_in_use) *bytes_in_use = ctx->bytes_in_use;
    if (peak_bytes) *peak_bytes = ctx->peak_bytes;
    if (n_allocs) *n_allocs = ctx->n_allocs;
    return DCB_OK;
}

// =========================================================================================== compile
extern "C" dcb_status dcb_translate_lambda(const char* lambda, const int32_t* param_types, int32_t n_params, char* out_code,
                                           size_t out_cap, int32_t* result_type, char* err, size_t err_cap) {
    if (err && err_cap) err[0] = '\0';
    if (!lambda || !param_types || n_params < 1 || n_params > 2 || !out_code || out_cap == 0)
        return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "bad argument to dcb_translate_lambda");
    std::vector<std::string> args;
    std::vector<int> types;
    for (int i = 0; i < n_params; ++i) { args.push_back("p" + std::to_string(i)); types.push_back(param_types[i]); }
    std::string code, e;
    int rt = 0;
    if (!dcbt::translate_lambda(lambda, args, types, &code, &rt, &e)) {
        if (err && err_cap) snprintf(err, err_cap, "%s", e.c_str());
        return set_err(nullptr, DCB_ERR_NOT_SUPPORTED, "%s", e.c_str());
    }
    if (code.size() + 1 > out_cap) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "output buffer too small (%zu needed)", code.size() + 1);
    memcpy(out_code, code.c_str(), code.size() + 1);
    if (result_type) *result_type = rt;
    return DCB_OK;
}

extern "C" dcb_status dcb_translate_kernel_method(const char* csharp_method, char* cuda_out, size_t cuda_cap, size_t* cuda_needed,
                                                  char* meta_json, size_t meta_cap, char* err, size_t err_cap) {
    if (err && err_cap) err[0] = '\0';
    if (!csharp_method) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "csharp_method is null");
    dcbt::KernelMethod km;
    std::string e;
    if (!dcbt::translate_kernel_method(csharp_method, &km, &e)) {
        if (err && err_cap) snprintf(err, err_cap, "%s", e.c_str());
        return set_err(nullptr, DCB_ERR_NOT_SUPPORTED, "%s", e.c_str());
    }
    if (cuda_needed) *cuda_needed = km.cuda_source.size() + 1;
    if (cuda_out && cuda_cap) snprintf(cuda_out, cuda_cap, "%s", km.cuda_source.c_str());
    if (meta_json && meta_cap) {
        std::string j = "{\"name\": \"" + km.name + "\", \"needs_length\": " + (km.needs_length ? "true" : "false") +
                        ", \"dimensions\": " + std::to_string(km.dimensions) + ", \"params\": [";
        for (size_t i = 0; i < km.params.size(); ++i) {
            const auto& p = km.params[i];
            j += std::string(i ? ", " : "") + "{\"name\": \"" + p.name + "\", \"is_buffer\": " + (p.is_buffer ? "true" : "false") +
                 ", \"is_readonly\": " + (p.is_readonly ? "true" : "false") + ", \"element_type\": \"" + dcbt::csharp_name(p.elem_type) + "\"}";
        }
        j += "]}";
        snprintf(meta_json, meta_cap, "%s", j.c_str());
    }
    return DCB_OK;
}

extern "C" dcb_status dcb_pipeline_generate_source(const dcb_pipeline_desc* desc, char* buf, size_t cap, size_t* needed,
                                                   char* err, size_t err_cap) {
    char e[512] = "";
    std::vector<dcbt::OpSpec> ops;
    dcb_status st = desc_to_ops(desc, &ops, e, sizeof e);
    dcbt::ChainInfo info;
    std::string es;
    if (st == DCB_OK) {
        int s2 = 0;
        if (!dcbt::build_chain(desc->elem_type0, desc->elem_type1, ops, &info, &es, &s2)) { st = s2; snprintf(e, sizeof e, "%s", es.c_str()); }
    }
    if (st != DCB_OK) {
        if (err && err_cap) snprintf(err, err_cap, "%s", e);
        return set_err(nullptr, st, "%s", e);
    }
    std::string src = dcbt::build_program(info, "", "", dcbt::Tuning(), true);
    if (needed) *needed = src.size() + 1;
    if (buf && cap) { snprintf(buf, cap, "%s", src.c_str()); }
    return DCB_OK;
}

extern "C" dcb_status dcb_pipeline_compile(dcb_ctx* ctx, const dcb_pipeline_desc* desc, dcb_pipeline** out_pipeline) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_pipeline != nullptr, "out_pipeline is null");
    *out_pipeline = nullptr;
    const auto t0 = std::chrono::steady_clock::now();
    char e[512] = "";
    std::vector<dcbt::OpSpec> ops;
    if ((st = desc_to_ops(desc, &ops, e, sizeof e))) return set_err(ctx, st, "%s", e);
    dcbt::ChainInfo info;
    std::string es;
    int s2 = 0;
    if (!dcbt::build_chain(desc->elem_type0, desc->elem_type1, ops, &info, &es, &s2)) return set_err(ctx, s2, "%s", es.c_str());
    const bool force_jit = (desc->flags & DCB_PIPE_FORCE_JIT) != 0 || env_int("DCB200_FORCE_JIT", 0) != 0;
    const std::string cache_key = info.key + (force_jit ? "#jit" : "");

    std::lock_guard<std::mutex> g(ctx->mu);
    auto it = ctx->cache.find(cache_key);
    if (it != ctx->cache.end()) {
        it->second->refs += 1;
        it->second->last_use = ++ctx->cache_clock;
        *out_pipeline = it->second;
        return DCB_OK;
    }
    // Bounded cache, as the reference's KernelCache(maxEntries: 100): before a new entry goes in, the least recently
    // used entries that nobody holds (every dcb_pipeline_compile matched by a dcb_pipeline_destroy) are dropped with
    // their module and scratch. Entries still held stay, so the bound can be exceeded while handles are outstanding.
    while ((int)ctx->cache.size() >= ctx->opt_cache_max) {
        auto victim = ctx->cache.end();
        for (auto c = ctx->cache.begin(); c != ctx->cache.end(); ++c)
            if (c->second->refs == 0 && (victim == ctx->cache.end() || c->second->last_use < victim->second->last_use)) victim = c;
        if (victim == ctx->cache.end()) break;
        CU(ctx, cudaDeviceSynchronize());     // nothing of the victim's may still be running when its memory goes
        free_pipeline(victim->second);
        ctx->cache.erase(victim);
    }
    dcb_pipeline* p = new dcb_pipeline();
    p->ctx = ctx;
    p->info = info;
    const dcb_builtin_entry* b = force_jit ? nullptr : dcb_builtin_find(info.key.c_str());
    if (b) {
        p->precompiled = true;
        p->k_vec = b->k_vec;
        p->k_scalar = b->k_scalar;
        p->unroll = b->unroll;
        p->compact_block = b->compact_block;
        p->k_stream = b->k_stream;
        p->stream_rows = b->stream_rows;
        p->stream_warps = b->stream_warps;
        p->stream_nbuf = b->stream_nbuf;
        p->stream_copy_warps = b->stream_copy_warps;
        p->source.clear();
    } else if ((st = load_jit(ctx, p)) != DCB_OK) {
        free_pipeline(p);
        return st;
    }
    if ((st = finish_pipeline(ctx, p)) != DCB_OK) { free_pipeline(p); return st; }
    p->compile_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    p->last_use = ++ctx->cache_clock;
    ctx->cache[cache_key] = p;
    *out_pipeline = p;
    return DCB_OK;
}

extern "C" dcb_status dcb_pipeline_destroy(dcb_pipeline* p) {
    if (!p) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "pipeline is null");
    // A pipeline stays in its context's cache; destroy only drops the caller's reference, after which the cache may
    // evict it. A handle whose pipeline is already gone (its context was shut down) is refused, not followed.
    {
        std::lock_guard<std::mutex> live(g_live_mu);
        if (!g_live_pipelines.count(p)) return set_err(nullptr, DCB_ERR_DISPOSED, "pipeline was already released with its context");
    }
    std::lock_guard<std::mutex> g(p->ctx->mu);   // the caller's reference keeps the cache from evicting it meanwhile
    if (p->refs > 0) p->refs -= 1;
    return DCB_OK;
}

extern "C" dcb_status dcb_pipeline_info_get(const dcb_pipeline* p, dcb_pipeline_info* out) {
    if (!p || !out) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "null argument");
    out->terminal = p->info.terminal;
    out->out_type = p->info.out_type;
    out->result_type = p->info.result_type;
    out->has_filter = p->info.has_filter ? 1 : 0;
    out->n_inputs = p->info.n_in;
    out->precompiled = p->precompiled ? 1 : 0;
    out->tile_elems = (p->info.terminal == DCB_OP_TOARRAY && p->info.has_filter)
                          ? (int64_t)(p->compact_block / 32) * p->rows_vec * 32 * (16 / dcbt::type_size(p->info.in0)) : 0;
    out->compile_ms = p->compile_ms;
    return DCB_OK;
}

extern "C" dcb_status dcb_pipeline_source(const dcb_pipeline* p, char* buf, size_t cap, size_t* needed) {
    if (!p) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "pipeline is null");
    // Only the generated part is returned (chain + kernel entry points), not the template header in front of it.
    dcbt::Tuning tuning;
    tuning.unroll = p->unroll;
    tuning.compact_rows = p->jit_rows;
    tuning.compact_block = p->compact_block;
    const std::string src = dcbt::build_program(p->info, "", "", tuning, true);
    if (needed) *needed = src.size() + 1;
    if (buf && cap) snprintf(buf, cap, "%s", src.c_str());
    return DCB_OK;
}

// =============================================================================================== run
namespace {

bool aligned_to(const void* p, size_t a) { return a <= 1 || ((uintptr_t)p % a) == 0; }

dcb_status launch(dcb_ctx* ctx, const void* fn, unsigned grid, void** args, cudaStream_t s, int block = kBlock) {
    CU(ctx, cudaLaunchKernel(fn, dim3(grid), dim3(block), args, 0, s));
    ctx->launches += 1;
    return DCB_OK;
}

__global__ void fold_fault_kernel(unsigned int* word, dcb::DeviceResult* rec) {
    // behind the query's kernel on the same stream: what the lambdas' integer divisions noted goes into the record's flags
    const unsigned int f = *word;
    if (f) {
        rec->flags = rec->flags | ((f & 1u) ? (unsigned long long)dcb::FLAG_DIV0 : 0ull) | ((f & 2u) ? (unsigned long long)dcb::FLAG_DIV_OVERFLOW : 0ull);
        *word = 0;
    }
}

dcb_status run_async_launch(dcb_pipeline* p, const void* in0, const void* in1, int64_t n, void* out, int64_t out_cap,
                            void* d_result, const void* d_prev, cudaStream_t s, uint32_t* launches, uint32_t run_flags);

dcb_status run_async_impl(dcb_pipeline* p, const void* in0, const void* in1, int64_t n, void* out, int64_t out_cap,
                          void* d_result, const void* d_prev, cudaStream_t s, uint32_t* launches, uint32_t run_flags = 0) {
    dcb_status st = run_async_launch(p, in0, in1, n, out, out_cap, d_result, d_prev, s, launches, run_flags);
    if (st != DCB_OK || !p->fault_word || n == 0) return st;
    // A map writes no record of its own: its faults are read from the word itself by the blocking calls, and reach a
    // caller's record only if one was given.
    const bool plain_map = p->info.terminal == DCB_OP_TOARRAY && !p->info.has_filter;
    if (plain_map && !d_result) return st;
    dcb::DeviceResult* res = d_result ? (dcb::DeviceResult*)d_result : p->d_result;
    fold_fault_kernel<<<1, 1, 0, s>>>(p->fault_word, res);
    CU(p->ctx, cudaGetLastError());
    if (launches) *launches += 1;
    p->ctx->launches += 1;
    return DCB_OK;
}

dcb_status run_async_launch(dcb_pipeline* p, const void* in0, const void* in1, int64_t n, void* out, int64_t out_cap,
                            void* d_result, const void* d_prev, cudaStream_t s, uint32_t* launches, uint32_t run_flags) {
    dcb_ctx* ctx = p->ctx;
    const dcbt::ChainInfo& I = p->info;
    NEED(ctx, n >= 0, "element count is negative");
    NEED(ctx, n == 0 || in0 != nullptr, "in0 is null");
    NEED(ctx, I.n_in == 1 || n == 0 || in1 != nullptr, "in1 is null for a Zip pipeline");
    const bool to_array = I.terminal == DCB_OP_TOARRAY;
    if (to_array) {
        NEED(ctx, out_cap >= 0, "output capacity is negative");
        NEED(ctx, out != nullptr || out_cap == 0 || n == 0, "out is null");
    }
    dcb::DeviceResult* res = d_result ? (dcb::DeviceResult*)d_result : p->d_result;
    const int e_vec = 16 / dcbt::type_size(I.in0);
    bool vec = aligned_to(in0, 16);
    if (I.n_in == 2) vec = vec && aligned_to(in1, pack_align(e_vec, I.in1));
    if (to_array) vec = vec && aligned_to(out, pack_align(e_vec, I.out_type)) ;
    if (ctx->opt_force_scalar) vec = false;
    const void* fn = vec ? p->k_vec : p->k_scalar;
    const int E = vec ? e_vec : 1;
    long long nn = n;
    const int occ_cap = ctx->opt_blocks_per_sm > 0 ? ctx->opt_blocks_per_sm : (1 << 20);
    std::lock_guard<std::mutex> guard(p->mu);   // the scratch of (pipeline, stream) and the order of enqueues that use it

    if (to_array && !I.has_filter) {
        NEED(ctx, out_cap >= n, "output capacity below the element count");
        if (n == 0) return DCB_OK;
        const int unroll = vec ? p->unroll : p->unroll * 2;
        const int64_t tiles = (n / E + (int64_t)kBlock * unroll - 1) / ((int64_t)kBlock * unroll);
        const int64_t max_grid = (int64_t)ctx->sm_count * std::min(occ_cap, vec ? p->occ_vec : p->occ_scalar);
        const unsigned grid = (unsigned)std::max<int64_t>(1, std::min(tiles, max_grid));
        void* args[] = {(void*)&in0, (void*)&in1, (void*)&nn, (void*)&out};
        if (launches) *launches += 1;
        return launch(ctx, fn, grid, args, s);
    }
    if (to_array) {
        // Which kernel. The streamed kernel takes any element-aligned pointers as long as both inputs sit at the same
        // element offset from a 16-byte boundary (its bulk copies start at that boundary); the one-tile-per-block kernel
        // takes anything (scalar variant if unaligned).
        const size_t sz0 = (size_t)dcbt::type_size(I.in0), sz1 = I.n_in == 2 ? (size_t)dcbt::type_size(I.in1) : 1;
        unsigned int head = (unsigned int)(((uintptr_t)in0 % 16) / sz0);
        const bool stream_ok = p->k_stream && ctx->opt_compact_kernel == 0 && !ctx->opt_force_scalar && (uintptr_t)in0 % sz0 == 0 &&
                               (I.n_in == 1 || ((uintptr_t)in1 - (uintptr_t)head * sz1) % 16 == 0);
        const int rows = vec ? p->rows_vec : p->rows_scalar;
        if (!stream_ok) head = 0;
        const int64_t tile = stream_ok ? (int64_t)dcbt::stream_tile_elems(I, p->stream_rows, p->stream_warps)
                                       : (int64_t)(p->compact_block / 32) * rows * 32 * E;
        long long num_tiles = (n + (int64_t)head + tile - 1) / tile;
        if (n == 0) num_tiles = 0;
        if (num_tiles == 0) {
            // Nothing to scan: the record is the previous one (or zero).
            if (d_prev) CU(ctx, cudaMemcpyAsync(res, d_prev, DCB_DEVICE_RESULT_BYTES, cudaMemcpyDeviceToDevice, s));
            else CU(ctx, cudaMemsetAsync(res, 0, DCB_DEVICE_RESULT_BYTES, s));
            return DCB_OK;
        }
        NEED(ctx, num_tiles < (1ll << 31), "too many tiles for one launch");
        Scratch* scp = nullptr;
        dcb_status st = ensure_scratch(p, num_tiles, s, &scp);
        if (st) return st;
        Scratch& sc = *scp;
        sc.epoch += 1;
        if (sc.epoch >= 0xfffu) {    // the narrower epoch field is 12 bits: wipe the descriptors before reusing a value
            CU(ctx, cudaMemsetAsync(sc.desc, 0, sc.desc_cap * sizeof(unsigned long long) + (sc.desc_cap + 8) * sizeof(unsigned int), s));
            CU(ctx, cudaMemsetAsync(sc.words, 0, 512, s));
            sc.epoch = 1;
        }
        unsigned int epoch = sc.epoch, spin = ctx->spin_limit;
        unsigned int* abort_flag = sc.words + 64;
        if (ctx->opt_withhold_first_count) {
            // Time-out test switch: the kernel that handles tile 0 finds this launch's epoch in the word next to the abort
            // flag and keeps that tile's count to itself, so every bounded wait for it runs out.
            fill_kernel<<<1, 32, 0, s>>>((unsigned char*)(sc.words + 65), 1, (unsigned long long)epoch, 4);
            CU(ctx, cudaGetLastError());
        }
        long long cap = out_cap;
        void* args[] = {(void*)&in0, (void*)&in1, (void*)&nn, (void*)&out, (void*)&cap, (void*)&sc.desc,
                        (void*)&epoch, (void*)&spin, (void*)&num_tiles, (void*)&d_prev, (void*)&res, (void*)&abort_flag};
        if (launches) *launches += 1;
        if (stream_ok) {
            // Persistent blocks, as many as fit the GPU at once (fewer for a small input); tile ids come from counters[0].
            unsigned int* counters = sc.words + 32;
            unsigned int kernel_flags = (run_flags & DCB_RUN_TAKE) ? (unsigned int)dcb::STREAM_TAKE : 0u;
            void* pargs[] = {(void*)&in0, (void*)&in1, (void*)&nn, (void*)&out, (void*)&cap, (void*)&sc.cdesc, (void*)&epoch, (void*)&spin,
                             (void*)&num_tiles, (void*)&d_prev, (void*)&res, (void*)&abort_flag, (void*)&counters, (void*)&head, (void*)&kernel_flags};
            const unsigned grid = (unsigned)std::min<int64_t>(num_tiles, (int64_t)ctx->sm_count * std::min(occ_cap, p->occ_stream));
            CU(ctx, cudaLaunchKernel(p->k_stream, dim3(grid), dim3(dcbt::stream_block_threads(p->stream_warps, p->stream_copy_warps)), pargs,
                                     (size_t)dcbt::stream_smem_bytes(I, p->stream_rows, p->stream_warps, p->stream_nbuf), s));
            ctx->launches += 1;
            return DCB_OK;
        }
        return launch(ctx, fn, (unsigned)num_tiles, args, s, p->compact_block);   // one tile per block, ids in dispatch order
    }
    // reductions
    {
        Scratch* scp = nullptr;
        dcb_status st = ensure_scratch(p, 0, s, &scp);
        if (st) return st;
        const int unroll = vec ? p->unroll : p->unroll * 2;
        const int64_t tiles = (n / E + (int64_t)kBlock * unroll - 1) / ((int64_t)kBlock * unroll);
        int64_t max_grid = (int64_t)ctx->sm_count * std::min(occ_cap, vec ? p->occ_vec : p->occ_scalar);
        max_grid = std::min<int64_t>(max_grid, kMaxPartials);
        const unsigned grid = (unsigned)std::max<int64_t>(1, std::min(tiles, max_grid));
        unsigned int* ticket = scp->words + 128;   // main word and one word per group of blocks (last_block_ticket)
        void* args[] = {(void*)&in0, (void*)&in1, (void*)&nn, (void*)&scp->partials, (void*)&ticket, (void*)&res};
        if (launches) *launches += 1;
        if (ctx->opt_overlap_launches) {
            // Programmatic dependent launch: this kernel may begin while the kernel before it on the stream is still running
            // (it reads its input at once and touches scratch and record only after its grid-dependency wait).
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kBlock); cfg.dynamicSmemBytes = 0; cfg.stream = s;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
            CU(ctx, cudaLaunchKernelExC(&cfg, fn, args));
            ctx->launches += 1;
            return DCB_OK;
        }
        return launch(ctx, fn, grid, args, s);
    }
}

float round_f32(double v) { return (float)v; }

}  // namespace

extern "C" dcb_status dcb_record_finalize(int32_t terminal, int32_t out_type, const void* host_record, dcb_result* r) {
    if (!host_record || !r) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "null argument");
    dcb_ctx* ctx = nullptr;
    const dcb::DeviceResult* d = (const dcb::DeviceResult*)host_record;
    const uint32_t keep_launches = r->launches;
    const float km = r->kernel_ms, tm = r->total_ms;
    memset(r, 0, sizeof *r);
    r->launches = keep_launches; r->kernel_ms = km; r->total_ms = tm;
    r->count = d->count;
    const uint64_t fl = d->flags;
    if (fl & dcb::FLAG_SAW_NAN) r->flags |= DCB_RES_SAW_NAN;
    const bool fp = out_type == DCB_T_F32 || out_type == DCB_T_F64;
    if (fl & dcb::FLAG_TIMEOUT) {
        r->flags |= DCB_RES_TIMEOUT;
        return set_err(ctx, DCB_ERR_TIMEOUT, terminal == DCB_OP_TOARRAY ? "a look-back wait in the compaction kernel ran out"
                                                                        : "a peer's partial did not arrive in time");
    }
    if (fl & dcb::FLAG_DIV0) { r->flags |= DCB_RES_DIVIDE_BY_ZERO; return set_err(ctx, DCB_ERR_DIVIDE_BY_ZERO, "attempted to divide by zero in a lambda"); }
    if (fl & dcb::FLAG_DIV_OVERFLOW) { r->flags |= DCB_RES_DIVIDE_OVERFLOW; return set_err(ctx, DCB_ERR_OVERFLOW, "MinValue / -1 in a lambda"); }
    switch (terminal) {
        case DCB_OP_TOARRAY:
            if (fl & dcb::FLAG_TRUNCATED) { r->flags |= DCB_RES_TRUNCATED; return set_err(ctx, DCB_ERR_OUTPUT_TOO_SMALL, "%lld elements survive, the output holds fewer", (long long)d->count); }
            return DCB_OK;
        case DCB_OP_COUNT:
            r->i64 = d->count; r->u64 = (uint64_t)d->count;
            return DCB_OK;
        case DCB_OP_FIRST_INDEX:
        case DCB_OP_LAST_INDEX:
            r->i64 = d->count == 0 ? -1 : (terminal == DCB_OP_FIRST_INDEX ? d->imin : d->imax);
            r->u64 = (uint64_t)r->i64;
            return DCB_OK;
        case DCB_OP_SUM:
        case DCB_OP_AVERAGE: {
            const bool avg = terminal == DCB_OP_AVERAGE;
            if (!(out_type == DCB_T_I32 || out_type == DCB_T_I64 || fp)) return set_err(ctx, DCB_ERR_NOT_SUPPORTED, "Sum/Average are defined for int, long, float, double");
            if (avg && d->count == 0) return set_err(ctx, DCB_ERR_EMPTY_SEQUENCE, "Average of an empty sequence");
            if (fp) {
                const double v = avg ? d->fsum / (double)d->count : d->fsum;
                r->f64 = (out_type == DCB_T_F32) ? (double)round_f32(v) : v;   // one rounding, as (float)sum in the BCL
                return DCB_OK;
            }
            // integer Sum is checked in System.Linq: a running sum that leaves the element type's range is an error
            // (the Sum kernel flags it; Average adds in long, where only the total can leave the range)
            bool overflow = d->isum_hi != ((d->isum_lo < 0) ? -1 : 0) || (!avg && (fl & dcb::FLAG_OVERFLOW) != 0);
            if (out_type == DCB_T_I32 && !avg) overflow = overflow || d->isum_lo > 2147483647LL || d->isum_lo < -2147483648LL;
            if (overflow) { r->flags |= DCB_RES_OVERFLOW; return set_err(ctx, DCB_ERR_OVERFLOW, "integer Sum overflowed %s", dcbt::csharp_name(out_type)); }
            if (avg) r->f64 = (double)d->isum_lo / (double)d->count;
            else { r->i64 = d->isum_lo; r->u64 = (uint64_t)d->isum_lo; }
            return DCB_OK;
        }
        case DCB_OP_MIN:
        case DCB_OP_MAX: {
            const bool mn = terminal == DCB_OP_MIN;
            if (d->count == 0) return set_err(ctx, DCB_ERR_EMPTY_SEQUENCE, "%s of an empty sequence", mn ? "Min" : "Max");
            if (fp) {
                // Enumerable.Min returns NaN if any element is NaN; Enumerable.Max only if all are.
                const double nan = std::numeric_limits<double>::quiet_NaN();
                if (mn) r->f64 = (fl & dcb::FLAG_SAW_NAN) ? nan : d->fmin;
                else r->f64 = (fl & dcb::FLAG_SAW_NUMBER) ? d->fmax : nan;
            } else {
                r->i64 = mn ? d->imin : d->imax;
                r->u64 = (uint64_t)r->i64;
            }
            return DCB_OK;
        }
        default: return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "unknown terminal operator %d", terminal);
    }
}

extern "C" dcb_status dcb_result_finalize(const dcb_pipeline* p, const void* host_record, dcb_result* r) {
    if (!p) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "pipeline is null");
    dcb_status st = dcb_record_finalize(p->info.terminal, p->info.out_type, host_record, r);
    if (st != DCB_OK) snprintf(p->ctx->err, sizeof p->ctx->err, "%s", tl_error);
    return st;
}

extern "C" dcb_status dcb_pipeline_run_async(dcb_pipeline* p, const void* in0, const void* in1, int64_t n, void* out,
                                             int64_t out_cap, void* d_result, const void* d_prev, void* stream) {
    if (!p) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "pipeline is null");
    dcb_status st = use(p->ctx);
    if (st) return st;
    return run_async_impl(p, in0, in1, n, out, out_cap, d_result, d_prev, pick(p->ctx, stream), nullptr);
}

extern "C" dcb_status dcb_pipeline_run(dcb_pipeline* p, const void* in0, const void* in1, int64_t n, void* out,
                                       int64_t out_cap, dcb_result* result, void* stream) {
    return dcb_pipeline_run_ex(p, in0, in1, n, out, out_cap, 0u, result, stream);
}

// Take(k): more survivors than k is what was asked for, not an error; the count reported is what was written.
static dcb_status finish_take(dcb_status st, int64_t cap, dcb_result* result) {
    if (st == DCB_ERR_OUTPUT_TOO_SMALL) st = DCB_OK;
    if (st == DCB_OK && result->count > cap) result->count = cap;
    result->flags &= ~(uint32_t)DCB_RES_TRUNCATED;
    return st;
}

namespace {
// A map's integer-division faults, read from the module's word after the stream has been synchronised.
dcb_status map_faults(dcb_pipeline* p, cudaStream_t s) {
    dcb_ctx* ctx = p->ctx;
    unsigned int f = 0;
    CU(ctx, cudaMemcpyAsync(&f, p->fault_word, 4, cudaMemcpyDeviceToHost, s));
    CU(ctx, cudaStreamSynchronize(s));
    if (!f) return DCB_OK;
    CU(ctx, cudaMemsetAsync(p->fault_word, 0, 4, s));
    if (f & 1u) return set_err(ctx, DCB_ERR_DIVIDE_BY_ZERO, "attempted to divide by zero in a lambda");
    return set_err(ctx, DCB_ERR_OVERFLOW, "MinValue / -1 in a lambda");
}
}  // namespace

extern "C" dcb_status dcb_pipeline_run_ex(dcb_pipeline* p, const void* in0, const void* in1, int64_t n, void* out,
                                          int64_t out_cap, uint32_t flags, dcb_result* result, void* stream) {
    if (!p) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "pipeline is null");
    dcb_ctx* ctx = p->ctx;
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, result != nullptr, "result is null");
    memset(result, 0, sizeof *result);
    cudaStream_t s = pick(ctx, stream);
    const bool plain_map = p->info.terminal == DCB_OP_TOARRAY && !p->info.has_filter;
    std::lock_guard<std::mutex> run_guard(p->run_mu);   // this pipeline's record, host mirror and events are in use until we return
    CU(ctx, cudaEventRecord(p->ev0, s));
    uint32_t launches = 0;
    const bool take = (flags & DCB_RUN_TAKE) != 0 && p->info.terminal == DCB_OP_TOARRAY && p->info.has_filter;
    if ((st = run_async_impl(p, in0, in1, n, out, out_cap, nullptr, nullptr, s, &launches, take ? DCB_RUN_TAKE : 0u))) return st;
    const bool index_terminal = p->info.terminal == DCB_OP_FIRST_INDEX || p->info.terminal == DCB_OP_LAST_INDEX;   // indices are local to a shard
    if (ctx->peers.world > 1 && p->info.terminal != DCB_OP_TOARRAY && !index_terminal) {   // blocking call: exchange on the same stream
        if ((st = dcb_peer_exchange_async(ctx, p->d_result, p->info.out_type, (void*)s))) return st;
        launches += 1;
    }
    CU(ctx, cudaEventRecord(p->ev1, s));
    if (!plain_map) CU(ctx, cudaMemcpyAsync(p->h_record, p->d_result, DCB_DEVICE_RESULT_BYTES, cudaMemcpyDeviceToHost, s));
    CU(ctx, cudaStreamSynchronize(s));
    float ms = 0;
    CU(ctx, cudaEventElapsedTime(&ms, p->ev0, p->ev1));
    result->launches = launches; result->kernel_ms = ms; result->total_ms = ms;
    if (plain_map) {
        result->count = n;
        return p->fault_word ? map_faults(p, s) : DCB_OK;
    }
    st = dcb_result_finalize(p, p->h_record, result);
    return take ? finish_take(st, out_cap, result) : st;
}

namespace {

// Fold the per-chunk records of a chunked reduction in chunk order (deterministic).
void fold_records(const dcbt::ChainInfo& I, const dcb::DeviceResult* recs, int n, int64_t chunk, dcb::DeviceResult* out) {
    *out = recs[0];
    if (I.terminal == DCB_OP_FIRST_INDEX || I.terminal == DCB_OP_LAST_INDEX) {
        // a chunk reports indices relative to its own start
        out->imin = 0x7fffffffffffffffLL; out->imax = -1; out->count = 0;
        for (int i = 0; i < n; ++i) {
            if (recs[i].count == 0) continue;
            out->count += recs[i].count;
            out->imin = std::min<int64_t>(out->imin, recs[i].imin + (int64_t)i * chunk);
            out->imax = std::max<int64_t>(out->imax, recs[i].imax + (int64_t)i * chunk);
        }
        out->count_f = (double)out->count;
        return;
    }
    if (I.checked_sum) {
        // running-sum range over the chunks, in chunk order: (s, lo, hi) of a chunk is relative to the chunk's start
        typedef __int128 wide;
        auto w = [](int64_t lo, int64_t hi) { return (wide)(((unsigned __int128)(uint64_t)hi << 64) | (uint64_t)lo); };
        wide s = 0, lo = 0, hi = 0;
        uint64_t flags = 0;
        for (int i = 0; i < n; ++i) {
            const dcb::DeviceResult& r = recs[i];
            const wide rs = w(r.isum_lo, r.isum_hi);
            wide rlo = w(r.pad[0], r.pad[1]), rhi = w(r.pad[2], r.pad[3]);
            if (!(r.flags & dcb::FLAG_PREFIX)) { rlo = rs < 0 ? rs : 0; rhi = rs > 0 ? rs : 0; }   // an empty chunk's record
            lo = std::min(lo, s + rlo); hi = std::max(hi, s + rhi); s += rs;
            flags |= r.flags;
        }
        const wide mn = I.out_type == DCB_T_I32 ? (wide)INT32_MIN : (wide)INT64_MIN, mx = I.out_type == DCB_T_I32 ? (wide)INT32_MAX : (wide)INT64_MAX;
        out->isum_lo = (int64_t)(uint64_t)(unsigned __int128)s; out->isum_hi = (int64_t)(uint64_t)((unsigned __int128)s >> 64);
        out->pad[0] = (int64_t)(uint64_t)(unsigned __int128)lo; out->pad[1] = (int64_t)(uint64_t)((unsigned __int128)lo >> 64);
        out->pad[2] = (int64_t)(uint64_t)(unsigned __int128)hi; out->pad[3] = (int64_t)(uint64_t)((unsigned __int128)hi >> 64);
        out->flags = (flags & ~(uint64_t)dcb::FLAG_OVERFLOW) | dcb::FLAG_PREFIX | ((lo < mn || hi > mx) ? (uint64_t)dcb::FLAG_OVERFLOW : 0);
        out->count = 0; out->count_f = 0;
        return;
    }
    for (int i = 1; i < n; ++i) {
        const dcb::DeviceResult& r = recs[i];
        out->fsum += r.fsum;
        const unsigned long long lo = (unsigned long long)out->isum_lo + (unsigned long long)r.isum_lo;
        out->isum_hi += r.isum_hi + (lo < (unsigned long long)r.isum_lo ? 1 : 0);
        out->isum_lo = (long long)lo;
        out->count += r.count;
        if (r.fmin < out->fmin) out->fmin = r.fmin;
        if (r.fmax > out->fmax) out->fmax = r.fmax;
        if (I.out_type == DCB_T_U64) {
            if ((unsigned long long)r.imin < (unsigned long long)out->imin) out->imin = r.imin;
            if ((unsigned long long)r.imax > (unsigned long long)out->imax) out->imax = r.imax;
        } else {
            if (r.imin < out->imin) out->imin = r.imin;
            if (r.imax > out->imax) out->imax = r.imax;
        }
        out->flags |= r.flags;
    }
    out->count_f = (double)out->count;
}

}  // namespace

extern "C" dcb_status dcb_pipeline_run_host(dcb_pipeline* p, const void* host_in0, const void* host_in1, int64_t n,
                                            void* host_out, int64_t host_out_cap, dcb_result* result) {
    return dcb_pipeline_run_host_ex(p, host_in0, host_in1, n, host_out, host_out_cap, 0u, result);
}

extern "C" dcb_status dcb_pipeline_run_host_ex(dcb_pipeline* p, const void* host_in0, const void* host_in1, int64_t n,
                                               void* host_out, int64_t host_out_cap, uint32_t flags, dcb_result* result) {
    if (!p) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "pipeline is null");
    dcb_ctx* ctx = p->ctx;
    dcb_status st = use(ctx);
    if (st) return st;
    const dcbt::ChainInfo& I = p->info;
    NEED(ctx, result != nullptr, "result is null");
    NEED(ctx, n >= 0, "element count is negative");
    NEED(ctx, n == 0 || host_in0 != nullptr, "host_in0 is null");
    NEED(ctx, I.n_in == 1 || n == 0 || host_in1 != nullptr, "host_in1 is null for a Zip pipeline");
    memset(result, 0, sizeof *result);
    std::lock_guard<std::mutex> host_guard(ctx->host_mu);   // the staging buffers and chunk records belong to the context
    std::lock_guard<std::mutex> run_guard(p->run_mu);
    const bool to_array = I.terminal == DCB_OP_TOARRAY;
    const bool compaction = to_array && I.has_filter;
    const bool take = (flags & DCB_RUN_TAKE) != 0 && compaction;
    const size_t sz0 = (size_t)dcbt::type_size(I.in0), sz1 = I.n_in == 2 ? (size_t)dcbt::type_size(I.in1) : 0;
    const size_t szo = (size_t)dcbt::type_size(I.out_type);
    if (to_array) {
        NEED(ctx, host_out_cap >= 0 && (host_out != nullptr || host_out_cap == 0), "host_out is null");
        if (!I.has_filter) NEED(ctx, host_out_cap >= n, "output capacity below the element count");
    }
    // Chunks are whole tiles of the widest kernel shape so that every chunk but the last starts 16-byte aligned.
    int64_t chunk = (int64_t)(kHostChunkBytes / std::max(std::max(sz0, sz1), szo));
    chunk = std::max<int64_t>(chunk - chunk % 16384, 16384);
    const int n_chunks = (int)std::max<int64_t>(1, (n + chunk - 1) / chunk);
    constexpr int kRingIn = 3, kRingOut = 2;
    // The ring: whatever the size of the query, the device holds three chunks of every input and two of the output.
    {
        const size_t in_bytes = (size_t)chunk * std::max(sz0, sz1), out_bytes = (size_t)chunk * szo;
        if (ctx->ring_in_bytes < in_bytes || (I.n_in == 2 && !ctx->ring_in[1][0])) {
            CU(ctx, cudaDeviceSynchronize());
            for (int i = 0; i < 2; ++i) for (int j = 0; j < kRingIn; ++j) if (ctx->ring_in[i][j]) { cudaFree(ctx->ring_in[i][j]); ctx->ring_in[i][j] = nullptr; }
            for (int i = 0; i < I.n_in; ++i) for (int j = 0; j < kRingIn; ++j) CU(ctx, cudaMalloc(&ctx->ring_in[i][j], std::max(in_bytes, ctx->ring_in_bytes)));
            ctx->ring_in_bytes = std::max(in_bytes, ctx->ring_in_bytes);
        }
        if (to_array && ctx->ring_out_bytes < out_bytes) {
            CU(ctx, cudaDeviceSynchronize());
            for (int j = 0; j < kRingOut; ++j) { if (ctx->ring_out[j]) cudaFree(ctx->ring_out[j]); ctx->ring_out[j] = nullptr; CU(ctx, cudaMalloc(&ctx->ring_out[j], out_bytes)); }
            ctx->ring_out_bytes = out_bytes;
        }
        if (!ctx->ev_copied[0]) {
            for (int j = 0; j < kRingIn; ++j) {
                CU(ctx, cudaEventCreateWithFlags(&ctx->ev_copied[j], cudaEventDisableTiming));
                CU(ctx, cudaEventCreateWithFlags(&ctx->ev_computed[j], cudaEventDisableTiming));
            }
            for (int j = 0; j < kRingOut; ++j) {
                CU(ctx, cudaEventCreateWithFlags(&ctx->ev_filled[j], cudaEventDisableTiming));
                CU(ctx, cudaEventCreateWithFlags(&ctx->ev_drained[j], cudaEventDisableTiming));
                CU(ctx, cudaEventCreateWithFlags(&ctx->ev_record[j], cudaEventDisableTiming));
            }
        }
    }
    // Per-chunk records: device array + pinned host mirror, kept on the context and grown when a larger input comes.
    if ((size_t)n_chunks > ctx->recs_cap) {
        CU(ctx, cudaDeviceSynchronize());
        if (ctx->dev_recs) cudaFree(ctx->dev_recs);
        if (ctx->host_recs) cudaFreeHost(ctx->host_recs);
        ctx->dev_recs = ctx->host_recs = nullptr; ctx->recs_cap = 0;
        const size_t cap = std::max<size_t>((size_t)n_chunks, 256);
        CU(ctx, cudaMalloc(&ctx->dev_recs, sizeof(dcb::DeviceResult) * cap));
        CU(ctx, cudaHostAlloc(&ctx->host_recs, sizeof(dcb::DeviceResult) * cap, cudaHostAllocDefault));
        ctx->recs_cap = cap;
    }
    dcb::DeviceResult* d_recs = (dcb::DeviceResult*)ctx->dev_recs;
    dcb::DeviceResult* h_recs = (dcb::DeviceResult*)ctx->host_recs;

    cudaStream_t cs = ctx->copy_stream, ks = ctx->stream, os = ctx->out_stream;
    cudaEvent_t t0 = p->ev0, t1 = p->ev1;
    uint32_t launches = 0;
    st = DCB_OK;
    int64_t out_written = 0, survivors = 0;    // compaction: elements copied to host_out so far / counted so far
    int last_chunk = n_chunks - 1;             // last chunk whose kernel ran (Take may stop earlier)
    uint64_t flags_seen = 0;
    // Output of a compaction chunk leaves one chunk behind the kernels: its record (the survivor count) has to reach the
    // host before the size and the destination of its copy are known.
    auto drain_compacted = [&](int c) -> cudaError_t {
        const int so = c % kRingOut;
        cudaError_t e = cudaEventSynchronize(ctx->ev_record[so]);
        if (e != cudaSuccess) return e;
        const dcb::DeviceResult& r = h_recs[c];
        flags_seen |= r.flags;
        const int64_t cnt = (r.flags & dcb::FLAG_TIMEOUT) ? 0 : r.count;
        survivors += cnt;
        const int64_t room = std::max<int64_t>(0, host_out_cap - out_written);
        const int64_t ncopy = std::min(cnt, room);
        if (ncopy > 0) {
            e = cudaMemcpyAsync((char*)host_out + (size_t)out_written * szo, ctx->ring_out[so], (size_t)ncopy * szo, cudaMemcpyDeviceToHost, os);
            if (e != cudaSuccess) return e;
            out_written += ncopy;
        }
        return cudaEventRecord(ctx->ev_drained[so], os);
    };
    cudaError_t ce = cudaEventRecord(t0, ks);
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(cs, t0, 0);   // copies start after earlier work on the compute stream
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(os, t0, 0);
    for (int c = 0; c < n_chunks && ce == cudaSuccess && st == DCB_OK; ++c) {
        const int64_t off = (int64_t)c * chunk, len = std::max<int64_t>(0, std::min<int64_t>(chunk, n - off));
        const int si = c % kRingIn, so = c % kRingOut;
        if (c >= kRingIn) ce = cudaStreamWaitEvent(cs, ctx->ev_computed[si], 0);   // the slot's previous chunk has been read
        if (len > 0 && ce == cudaSuccess) {
            ce = cudaMemcpyAsync(ctx->ring_in[0][si], (const char*)host_in0 + off * sz0, (size_t)len * sz0, cudaMemcpyHostToDevice, cs);
            if (ce == cudaSuccess && I.n_in == 2)
                ce = cudaMemcpyAsync(ctx->ring_in[1][si], (const char*)host_in1 + off * sz1, (size_t)len * sz1, cudaMemcpyHostToDevice, cs);
        }
        if (ce == cudaSuccess) ce = cudaEventRecord(ctx->ev_copied[si], cs);
        if (ce == cudaSuccess) ce = cudaStreamWaitEvent(ks, ctx->ev_copied[si], 0);
        if (ce != cudaSuccess) break;
        const void* a = ctx->ring_in[0][si];
        const void* b = I.n_in == 2 ? ctx->ring_in[1][si] : nullptr;
        if (to_array) {
            if (compaction && c >= 1 && (ce = drain_compacted(c - 1)) != cudaSuccess) break;
            if (take && survivors >= host_out_cap) { last_chunk = c - 1; break; }   // Take(k) is satisfied: this chunk's kernel is not needed
            if (c >= kRingOut && (ce = cudaStreamWaitEvent(ks, ctx->ev_drained[so], 0)) != cudaSuccess) break;   // the slot's previous output has left
            if (compaction) {
                st = run_async_impl(p, a, b, len, ctx->ring_out[so], chunk, d_recs + c, nullptr, ks, &launches);
                if (st == DCB_OK) ce = cudaMemcpyAsync(h_recs + c, d_recs + c, sizeof(dcb::DeviceResult), cudaMemcpyDeviceToHost, ks);
                if (st == DCB_OK && ce == cudaSuccess) ce = cudaEventRecord(ctx->ev_record[so], ks);
            } else {
                st = run_async_impl(p, a, b, len, ctx->ring_out[so], len, nullptr, nullptr, ks, &launches);
                if (st == DCB_OK && len > 0) {
                    // results of a plain map leave chunk by chunk on a third stream, overlapping the uploads
                    ce = cudaEventRecord(ctx->ev_filled[so], ks);
                    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(os, ctx->ev_filled[so], 0);
                    if (ce == cudaSuccess)
                        ce = cudaMemcpyAsync((char*)host_out + off * szo, ctx->ring_out[so], (size_t)len * szo, cudaMemcpyDeviceToHost, os);
                    if (ce == cudaSuccess) ce = cudaEventRecord(ctx->ev_drained[so], os);
                }
            }
        } else {
            st = run_async_impl(p, a, b, len, nullptr, 0, d_recs + c, nullptr, ks, &launches);
        }
        if (st == DCB_OK && ce == cudaSuccess) ce = cudaEventRecord(ctx->ev_computed[si], ks);
    }
    if (ce != cudaSuccess) { cudaDeviceSynchronize(); return cuda_fail(ctx, ce, "dcb_pipeline_run_host"); }
    if (st != DCB_OK) { cudaDeviceSynchronize(); return st; }
    const bool plain_map = to_array && !compaction;
    dcb::DeviceResult total;
    memset(&total, 0, sizeof total);
    if (compaction) {
        if (last_chunk == n_chunks - 1) ce = drain_compacted(n_chunks - 1);
        total.count = survivors; total.count_f = (double)survivors; total.local_count = survivors;
        total.flags = flags_seen & (uint64_t)(dcb::FLAG_TIMEOUT | dcb::FLAG_DIV0 | dcb::FLAG_DIV_OVERFLOW);
        if (survivors > host_out_cap) total.flags |= dcb::FLAG_TRUNCATED;
    } else if (!plain_map) {
        ce = cudaMemcpyAsync(h_recs, d_recs, sizeof(dcb::DeviceResult) * (size_t)n_chunks, cudaMemcpyDeviceToHost, ks);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(ks);
        if (ce != cudaSuccess) return cuda_fail(ctx, ce, "reading the records back");
        fold_records(I, h_recs, n_chunks, chunk, &total);
    }
    if (ce == cudaSuccess && to_array) ce = cudaStreamWaitEvent(ks, ctx->ev_drained[last_chunk % kRingOut], 0);
    if (ce == cudaSuccess && to_array && last_chunk >= 1) ce = cudaStreamWaitEvent(ks, ctx->ev_drained[(last_chunk - 1) % kRingOut], 0);
    if (ce == cudaSuccess) ce = cudaEventRecord(t1, ks);
    if (ce == cudaSuccess && to_array) ce = cudaStreamSynchronize(os);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(ks);
    if (ce != cudaSuccess) return cuda_fail(ctx, ce, "dcb_pipeline_run_host");
    float ms = 0;
    cudaEventElapsedTime(&ms, t0, t1);
    result->launches = launches; result->total_ms = ms; result->kernel_ms = 0;
    if (plain_map) { result->count = n; return p->fault_word ? map_faults(p, ks) : DCB_OK; }
    st = dcb_result_finalize(p, &total, result);
    return take ? finish_take(st, host_out_cap, result) : st;
}

// ===================================================================================== peer exchange
static dcb_status ensure_peer_area(dcb_ctx* ctx);
extern "C" dcb_status dcb_peer_area_create(dcb_ctx* ctx, void* handle_out, size_t handle_cap) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, handle_out != nullptr && handle_cap >= sizeof(cudaIpcMemHandle_t), "handle buffer must hold 64 bytes");
    if ((st = ensure_peer_area(ctx))) return st;
    cudaIpcMemHandle_t h;
    CU(ctx, cudaIpcGetMemHandle(&h, ctx->peer_area));
    memcpy(handle_out, &h, sizeof h);
    return DCB_OK;
}

static dcb_status ensure_peer_area(dcb_ctx* ctx) {
    if (!ctx->peer_area) {
        const size_t bytes = sizeof(dcb::PeerSlot) * dcb::PEER_RING * dcb::PEER_MAX;
        CU(ctx, cudaMalloc(&ctx->peer_area, bytes));
        CU(ctx, cudaMemset(ctx->peer_area, 0, bytes));
        CU(ctx, cudaMalloc(&ctx->peer_state, sizeof(dcb::PeerState)));
        CU(ctx, cudaMemset(ctx->peer_state, 0, sizeof(dcb::PeerState)));
        CU(ctx, cudaDeviceSynchronize());
    }
    return DCB_OK;
}

extern "C" dcb_status dcb_peer_area_ptr(dcb_ctx* ctx, void** out_area, size_t* out_bytes) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_area != nullptr, "out_area is null");
    if ((st = ensure_peer_area(ctx))) return st;
    *out_area = ctx->peer_area;
    if (out_bytes) *out_bytes = sizeof(dcb::PeerSlot) * dcb::PEER_RING * dcb::PEER_MAX;
    return DCB_OK;
}

extern "C" dcb_status dcb_peer_connect_local(dcb_ctx* ctx, int32_t world, int32_t rank, void* const* areas) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, world >= 1 && world <= dcb::PEER_MAX, "world must be between 1 and 8");
    NEED(ctx, rank >= 0 && rank < world, "rank outside the world");
    NEED(ctx, areas != nullptr, "areas is null");
    if ((st = ensure_peer_area(ctx))) return st;
    dcb::PeerTable t = {};
    t.world = world; t.rank = rank; t.spin_limit = ctx->peer_spin_limit; t.state = (dcb::PeerState*)ctx->peer_state;
    CU(ctx, cudaMemsetAsync(ctx->peer_state, 0, sizeof(dcb::PeerState), ctx->stream));
    CU(ctx, cudaStreamSynchronize(ctx->stream));
    for (int r = 0; r < world; ++r) {
        NEED(ctx, areas[r] != nullptr, "an area pointer is null");
        t.area[r] = (dcb::PeerSlot*)(r == rank ? ctx->peer_area : areas[r]);
    }
    ctx->peers = t;
    return DCB_OK;
}

extern "C" dcb_status dcb_peer_connect(dcb_ctx* ctx, int32_t world, int32_t rank, const void* handles, size_t handle_stride) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, world >= 1 && world <= dcb::PEER_MAX, "world must be between 1 and 8");
    NEED(ctx, rank >= 0 && rank < world, "rank outside the world");
    NEED(ctx, ctx->peer_area != nullptr, "call dcb_peer_area_create first");
    NEED(ctx, handles != nullptr && handle_stride >= sizeof(cudaIpcMemHandle_t), "bad handle table");
    dcb::PeerTable t = {};
    t.world = world; t.rank = rank; t.spin_limit = ctx->peer_spin_limit; t.state = (dcb::PeerState*)ctx->peer_state;
    CU(ctx, cudaMemsetAsync(ctx->peer_state, 0, sizeof(dcb::PeerState), ctx->stream));
    CU(ctx, cudaStreamSynchronize(ctx->stream));
    for (int r = 0; r < world; ++r) {
        if (r == rank) { t.area[r] = (dcb::PeerSlot*)ctx->peer_area; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)r * handle_stride, sizeof h);
        void* p = nullptr;
        CU(ctx, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        ctx->peer_opened.push_back(p);
        t.area[r] = (dcb::PeerSlot*)p;
    }
    ctx->peers = t;
    return DCB_OK;
}

__global__ void __launch_bounds__(32) peer_exchange_kernel(const __grid_constant__ dcb::PeerTable pt, dcb::DeviceResult* rec, unsigned long long tag) {
    dcb::peer_exchange_body(pt, rec, tag);
}

extern "C" dcb_status dcb_peer_exchange_async(dcb_ctx* ctx, void* d_record, int32_t out_type, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, d_record != nullptr, "d_record is null");
    if (ctx->peers.world <= 1) return DCB_OK;
    unsigned long long tag = 0;
    if (out_type == DCB_T_F32 || out_type == DCB_T_F64) tag |= dcb::SLOT_IS_FP;
    if (out_type == DCB_T_U64) tag |= dcb::SLOT_IS_U64;
    if (out_type == DCB_T_I32) tag |= dcb::SLOT_IS_I32;
    peer_exchange_kernel<<<1, 32, 0, pick(ctx, stream)>>>(ctx->peers, (dcb::DeviceResult*)d_record, tag);
    CU(ctx, cudaGetLastError());
    ctx->launches += 1;
    return DCB_OK;
}

extern "C" dcb_status dcb_peer_disconnect(dcb_ctx* ctx) {
    dcb_status st = use(ctx);
    if (st) return st;
    CU(ctx, cudaDeviceSynchronize());
    for (void* p : ctx->peer_opened) cudaIpcCloseMemHandle(p);
    ctx->peer_opened.clear();
    ctx->peers = {};
    return DCB_OK;
}

// ============================================================================== [Kernel] source kernels
extern "C" dcb_status dcb_kernel_compile(dcb_ctx* ctx, const char* cuda_source, const char* entry_point, dcb_kernel** out_kernel) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, cuda_source != nullptr && entry_point != nullptr && out_kernel != nullptr, "null argument");
    *out_kernel = nullptr;
    nvrtcProgram prog = nullptr;
    if (nvrtcCreateProgram(&prog, cuda_source, "kernel.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
        return set_err(ctx, DCB_ERR_COMPILE, "nvrtcCreateProgram failed");
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-fmad=false", "-lineinfo"};
    nvrtcResult r = nvrtcCompileProgram(prog, 4, opts);
    if (r != NVRTC_SUCCESS) {
        size_t n = 0;
        nvrtcGetProgramLogSize(prog, &n);
        std::string log(n + 1, '\0');
        nvrtcGetProgramLog(prog, &log[0]);
        nvrtcDestroyProgram(&prog);
        return set_err(ctx, DCB_ERR_COMPILE, "NVRTC: %s: %.800s", nvrtcGetErrorString(r), log.c_str());
    }
    size_t sz = 0;
    nvrtcGetCUBINSize(prog, &sz);
    std::vector<char> cubin(sz);
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    dcb_kernel* k = new dcb_kernel();
    k->ctx = ctx;
    cudaError_t e = cudaLibraryLoadData(&k->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    cudaKernel_t fn = nullptr;
    if (e == cudaSuccess) e = cudaLibraryGetKernel(&fn, k->lib, entry_point);
    if (e != cudaSuccess) {
        if (k->lib) cudaLibraryUnload(k->lib);
        delete k;
        if (e == cudaErrorSymbolNotFound) { (void)cudaGetLastError(); return set_err(ctx, DCB_ERR_INVALID_ARGUMENT, "entry point '%s' not found (it must be extern \"C\")", entry_point); }
        return cuda_fail(ctx, e, "loading the compiled kernel");
    }
    k->fn = (const void*)fn;
    *out_kernel = k;
    return DCB_OK;
}

extern "C" dcb_status dcb_kernel_launch(dcb_kernel* k, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_bytes,
                                        void** args, void* stream) {
    if (!k) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "kernel is null");
    dcb_ctx* ctx = k->ctx;
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, grid != nullptr && block != nullptr, "grid or block is null");
    NEED(ctx, grid[0] && grid[1] && grid[2] && block[0] && block[1] && block[2], "grid and block dimensions must be positive");
    NEED(ctx, (uint64_t)block[0] * block[1] * block[2] <= 1024, "a block holds at most 1024 threads");
    CU(ctx, cudaLaunchKernel(k->fn, dim3(grid[0], grid[1], grid[2]), dim3(block[0], block[1], block[2]), args, shared_bytes, pick(ctx, stream)));
    ctx->launches += 1;
    return DCB_OK;
}

extern "C" dcb_status dcb_kernel_destroy(dcb_kernel* k) {
    if (!k) return set_err(nullptr, DCB_ERR_INVALID_ARGUMENT, "kernel is null");
    cudaSetDevice(k->ctx->device);
    if (k->lib) cudaLibraryUnload(k->lib);
    delete k;
    return DCB_OK;
}

// ============================================================================================ timing
extern "C" dcb_status dcb_event_create(dcb_ctx* ctx, void** out_event) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_event != nullptr, "out_event is null");
    cudaEvent_t e;
    CU(ctx, cudaEventCreate(&e));
    *out_event = (void*)e;
    return DCB_OK;
}

extern "C" dcb_status dcb_event_record(dcb_ctx* ctx, void* event, void* stream) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, event != nullptr, "event is null");
    CU(ctx, cudaEventRecord((cudaEvent_t)event, pick(ctx, stream)));
    return DCB_OK;
}

extern "C" dcb_status dcb_event_elapsed_ms(dcb_ctx* ctx, void* start, void* stop, float* out_ms) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, start && stop && out_ms, "null argument");
    CU(ctx, cudaEventSynchronize((cudaEvent_t)stop));
    CU(ctx, cudaEventElapsedTime(out_ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return DCB_OK;
}

extern "C" dcb_status dcb_event_destroy(dcb_ctx* ctx, void* event) {
    dcb_status st = use(ctx);
    if (st) return st;
    if (event) CU(ctx, cudaEventDestroy((cudaEvent_t)event));
    return DCB_OK;
}

extern "C" dcb_status dcb_launch_count(dcb_ctx* ctx, int64_t* out_launches) {
    dcb_status st = use(ctx);
    if (st) return st;
    NEED(ctx, out_launches != nullptr, "out_launches is null");
    *out_launches = ctx->launches;
    return DCB_OK;
}
