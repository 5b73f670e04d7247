/*
 * dcb200.h — C ABI of libdcb200.so, the B200 (sm_100a) engine behind DotCompute's
 * data-parallel LINQ hot path: fused Select / Zip / Where pipelines ending in
 * ToArray, Sum, Min, Max, Average or Count.
 *
 * The managed side binds these entry points with [LibraryImport("dcb200")]. Each
 * declaration names the reference code (path inside the DotCompute source tree,
 * file:line) whose job it takes over.
 *
 * Conventions
 *   - Every function returns a dcb_status (int32). 0 is success. No exception and no
 *     callback crosses this boundary. The text of the last failure on a context is
 *     read with dcb_last_error().
 *   - One dcb_ctx drives one GPU. Every entry point makes that GPU current itself, so
 *     it may be called from any thread (managed continuations hop threads; the
 *     reference calls cuCtxSetCurrent before each native call for the same reason,
 *     src/Backends/DotCompute.Backends.CUDA/Kernels/CudaKernelLauncher.cs:220). A compiled
 *     pipeline may be run from several threads and streams at once: the library
 *     serialises what they share and keeps device scratch per (pipeline, stream).
 *   - Sizes and element counts are int64_t / size_t throughout. The reference uses
 *     int lengths (src/Core/DotCompute.Abstractions/Interfaces/IUnifiedMemoryBuffer.cs:20,
 *     src/Extensions/DotCompute.Linq/CodeGeneration/RuntimeExecutor.cs:275), which
 *     overflow at 2^28 floats; this ABI does not.
 *   - A `stream` argument is a cudaStream_t passed as void*; NULL means the context's
 *     own stream.
 *   - There is no CPU fallback behind any of these calls. If the GPU, the driver or
 *     NVRTC is missing the call fails with a status; it never computes on the host.
 */
#ifndef DCB200_H
#define DCB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DCB_ABI_VERSION 1

/* ------------------------------------------------------------------------- status */

typedef int32_t dcb_status;

/* Status codes. The hundreds digit is the class, mirroring CudaErrorClass
 * (src/Backends/DotCompute.Backends.CUDA/ErrorHandling/CudaErrorClassification.cs:17-46):
 * 1xx transient, 2xx resource, 3xx programmer, 4xx fatal, 5xx query semantics. */
enum {
    DCB_OK = 0,
    DCB_ERR_NOT_READY = 101,        /* transient: work still in flight */
    DCB_ERR_TIMEOUT = 102,          /* transient: a bounded device-side wait ran out */
    DCB_ERR_OUT_OF_MEMORY = 201,    /* resource: device or pinned allocation failed */
    DCB_ERR_OUTPUT_TOO_SMALL = 202, /* resource: ToArray output capacity below survivor count */
    DCB_ERR_INVALID_ARGUMENT = 301, /* programmer: null / negative / mismatched argument (ArgumentException) */
    DCB_ERR_NOT_SUPPORTED = 302,    /* programmer: lambda or type outside the translator's grammar (NotSupportedException) */
    DCB_ERR_COMPILE = 303,          /* programmer: NVRTC rejected generated or user source */
    DCB_ERR_DISPOSED = 304,         /* programmer: handle used after destroy (ObjectDisposedException) */
    DCB_ERR_NO_DEVICE = 401,        /* fatal: no usable CUDA device / driver */
    DCB_ERR_CUDA = 402,             /* fatal: a CUDA call failed; text in dcb_last_error */
    DCB_ERR_EMPTY_SEQUENCE = 501,   /* Min/Max/Average of zero elements (InvalidOperationException in System.Linq) */
    DCB_ERR_OVERFLOW = 502,         /* checked integer Sum left its type's range, or int.MinValue / -1 in a lambda (OverflowException) */
    DCB_ERR_DIVIDE_BY_ZERO = 503    /* an integer / or % in a lambda met a zero divisor (DivideByZeroException) */
};

enum { DCB_CLASS_NONE = 0, DCB_CLASS_TRANSIENT = 1, DCB_CLASS_RESOURCE = 2,
       DCB_CLASS_PROGRAMMER = 3, DCB_CLASS_FATAL = 4, DCB_CLASS_QUERY = 5 };

/* Replaces CudaErrorClassification.Classify (ErrorHandling/CudaErrorClassification.cs:17-46). */
int32_t dcb_status_class(dcb_status s);
const char* dcb_status_name(dcb_status s);
int32_t dcb_abi_version(void);

/* -------------------------------------------------------------------------- types */

/* Element types: the unmanaged primitives the reference maps to CUDA C
 * (src/Extensions/DotCompute.Linq/CodeGeneration/CudaKernelGenerator.cs:1399-1416). */
enum {
    DCB_T_NONE = 0,
    DCB_T_I8 = 1,  /* sbyte  */
    DCB_T_U8 = 2,  /* byte   */
    DCB_T_I16 = 3, /* short  */
    DCB_T_U16 = 4, /* ushort */
    DCB_T_I32 = 5, /* int    */
    DCB_T_U32 = 6, /* uint   */
    DCB_T_I64 = 7, /* long   */
    DCB_T_U64 = 8, /* ulong  */
    DCB_T_F32 = 9, /* float  */
    DCB_T_F64 = 10, /* double */
    DCB_T_BOOL = 11 /* bool, one byte */
};
int32_t dcb_type_size(int32_t type);

/* Operators of a query, in call order. Same vocabulary as the reference's expression
 * visitor (src/Extensions/DotCompute.Linq/Compilation/ExpressionTreeVisitor.cs:234-272),
 * plus Zip, which the reference rejects (ExpressionTreeVisitor.cs:268). */
enum {
    DCB_OP_SELECT = 1,   /* lambda: one parameter, any result type                 */
    DCB_OP_WHERE = 2,    /* lambda: one parameter, bool result; order is preserved  */
    DCB_OP_ZIP = 3,      /* lambda: two parameters; must be the first operator      */
    DCB_OP_TOARRAY = 16, /* terminal: materialise the surviving elements in order   */
    DCB_OP_SUM = 17,     /* terminal: int / long (checked) or float / double (fp64 accumulation) */
    DCB_OP_MIN = 18,
    DCB_OP_MAX = 19,
    DCB_OP_AVERAGE = 20,
    DCB_OP_COUNT = 21,   /* also LongCount */
    DCB_OP_FIRST_INDEX = 22, /* terminal: index (in the source sequence) of the first element that passes every Where, -1 if none.
                                TakeWhile / SkipWhile (with the negated predicate) and First(predicate) are built on it;
                                the reference lists them in its visitor (ExpressionTreeVisitor.cs:249,263-265)            */
    DCB_OP_LAST_INDEX = 23   /* terminal: index of the last such element, -1 if none (Last / LastOrDefault)              */
};

typedef struct dcb_op {
    int32_t kind;       /* DCB_OP_* */
    const char* lambda; /* C# lambda text, e.g. "x => x * x + 3f"; NULL for terminals */
} dcb_op;

typedef struct dcb_pipeline_desc {
    int32_t elem_type0; /* element type of the source sequence                     */
    int32_t elem_type1; /* element type of Zip's second sequence, else DCB_T_NONE   */
    int32_t n_ops;
    const dcb_op* ops;  /* zero or more SELECT/WHERE/ZIP followed by one terminal   */
    uint32_t flags;     /* DCB_PIPE_* */
} dcb_pipeline_desc;

enum {
    DCB_PIPE_FORCE_JIT = 1u /* ignore the precompiled kernel table, always go through NVRTC */
};

typedef struct dcb_pipeline_info {
    int32_t terminal;     /* DCB_OP_* of the terminal                              */
    int32_t out_type;     /* element type reaching the terminal (ToArray element type) */
    int32_t result_type;  /* type of the scalar a reduction returns (Average(int) is double) */
    int32_t has_filter;   /* 1 if any Where is present                             */
    int32_t n_inputs;     /* 1, or 2 with Zip                                      */
    int32_t precompiled;  /* 1 if served from the ahead-of-time kernel table, 0 if NVRTC built it */
    int64_t tile_elems;   /* elements one compaction tile covers (0 if not a compaction) */
    double  compile_ms;   /* wall time dcb_pipeline_compile spent                   */
} dcb_pipeline_info;

/* What a run produced. For reductions the fields not named by the terminal are zero. */
typedef struct dcb_result {
    int64_t count;     /* elements that reached the terminal (survivors)           */
    double  f64;       /* Sum / Average / Min / Max when result_type is F32 or F64 (already rounded to
                          float precision for F32) */
    int64_t i64;       /* Sum / Min / Max / Count when result_type is an integer type up to I64 */
    uint64_t u64;      /* the same for U64                                          */
    uint32_t flags;    /* DCB_RES_* */
    uint32_t launches; /* kernels launched by this call                             */
    float   kernel_ms; /* device time of those kernels (CUDA events), 0 if not timed */
    float   total_ms;  /* device time including copies for the *_host call, else kernel_ms */
} dcb_result;

enum {
    DCB_RES_SAW_NAN = 1u,
    DCB_RES_TRUNCATED = 2u,
    DCB_RES_TIMEOUT = 4u,
    DCB_RES_OVERFLOW = 8u,
    DCB_RES_PREFIX_RANGE = 32u,     /* record only: slots DCB_SLOT_PREFIX_MIN_LO.. hold the range of the running sum */
    DCB_RES_DIVIDE_BY_ZERO = 64u,   /* an integer division or remainder in a lambda had a zero divisor */
    DCB_RES_DIVIDE_OVERFLOW = 128u  /* ... or was MinValue / -1 */
};

/* Raw per-run record the kernels write in device memory: 16 eight-byte slots. A sharded
 * query combines these across GPUs with NCCL before dcb_result_finalize(). */
enum {
    DCB_SLOT_FSUM = 0,   /* double: floating Sum accumulator                       */
    DCB_SLOT_COUNT_F = 1,/* double: count (exact below 2^53), so {sum,count} is one fp64 all-reduce */
    DCB_SLOT_ISUM_LO = 2,/* int64: low word of the integer Sum                     */
    DCB_SLOT_ISUM_HI = 3,/* int64: high word (sign-extended), non-trivial only for 64-bit elements */
    DCB_SLOT_COUNT = 4,  /* int64: survivors                                        */
    DCB_SLOT_FMIN = 5,   /* double                                                  */
    DCB_SLOT_FMAX = 6,   /* double                                                  */
    DCB_SLOT_IMIN = 7,   /* int64 (raw bits of the element for U64)                 */
    DCB_SLOT_IMAX = 8,   /* int64                                                   */
    DCB_SLOT_FLAGS = 9,  /* uint64: DCB_RES_* bits plus NaN bookkeeping             */
    DCB_SLOT_OFFSET = 10,/* int64: after dcb_peer_exchange_async, the sum of the counts of all lower ranks, i.e. where this
                            GPU's compacted output starts in the global, rank-ordered result; 0 without an exchange */
    DCB_SLOT_LOCAL_COUNT = 11, /* int64: this GPU's own count (after an exchange DCB_SLOT_COUNT holds the global total) */
    DCB_SLOT_PREFIX_MIN_LO = 12, /* Sum over int / long (checked like Enumerable.Sum: the call fails with DCB_ERR_OVERFLOW as  */
    DCB_SLOT_PREFIX_MIN_HI = 13, /* soon as a running sum, taken in source order, leaves the element type's range): smallest and */
    DCB_SLOT_PREFIX_MAX_LO = 14, /* largest running sum, empty prefix included, as 128-bit two's complement (low, high word).    */
    DCB_SLOT_PREFIX_MAX_HI = 15, /* Records of adjacent ranges combine as (s1+s2, min(lo1, s1+lo2), max(hi1, s1+hi2)), in order. */
    DCB_SLOT_NSLOTS = 16
};
#define DCB_DEVICE_RESULT_BYTES 128

typedef struct dcb_ctx dcb_ctx;
typedef struct dcb_buf dcb_buf;
typedef struct dcb_pipeline dcb_pipeline;
typedef struct dcb_kernel dcb_kernel;

/* ---------------------------------------------------------------------- lifecycle */

/* Opens GPU `device`, creates its stream and scratch. Replaces `new CudaAccelerator(deviceId: 0)`
 * + CudaContext (src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:184-194,
 * src/Backends/DotCompute.Backends.CUDA/CudaAccelerator.cs:59,192-195). */
dcb_status dcb_init(int32_t device, dcb_ctx** out_ctx);
dcb_status dcb_shutdown(dcb_ctx* ctx);
/* Copies the last error text of `ctx` (or of the calling thread when ctx is NULL) into buf. */
dcb_status dcb_last_error(dcb_ctx* ctx, char* buf, size_t cap);
/* Number of CUDA devices visible; 0 with DCB_ERR_NO_DEVICE when there is none. */
dcb_status dcb_device_count(int32_t* out_count);
/* Name, SM count, memory in bytes of the context's GPU. Replaces IComputeOrchestrator.GetDeviceInfo
 * (src/Core/DotCompute.Abstractions/Interfaces/IComputeOrchestrator.cs:21-104). */
dcb_status dcb_device_info(dcb_ctx* ctx, char* name, size_t name_cap, int32_t* sm_count,
                           int64_t* total_mem, int32_t* cc_major, int32_t* cc_minor);
/* Use `stream` (a cudaStream_t) as the context's stream from now on; NULL restores its own. */
dcb_status dcb_set_stream(dcb_ctx* ctx, void* stream);
dcb_status dcb_stream_sync(dcb_ctx* ctx, void* stream);
/* Upper bound on polls of one device-side wait (a look-back wait inside the compaction kernel, a wait for a peer's
 * partial in the exchange kernel) before it gives up and reports DCB_ERR_TIMEOUT (defaults 1<<22 and 1<<20). */
dcb_status dcb_set_spin_limit(dcb_ctx* ctx, uint32_t max_polls);

/* Per-context switches. Their initial values are read from the environment once, at dcb_init (DCB200_COMPACT_KERNEL,
 * DCB200_FORCE_SCALAR, DCB200_BLOCKS_PER_SM, DCB200_CACHE_MAX_ENTRIES); nothing reads the environment at launch time.
 * They stand where the reference has CompilationOptions / KernelCache settings
 * (src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:132, new KernelCache(maxEntries: 100)). */
enum {
    DCB_OPT_COMPACT_KERNEL = 1,       /* 0 = automatic (the streamed kernel where the query allows), 1 = always the
                                         one-tile-per-block look-back kernel                                          */
    DCB_OPT_FORCE_SCALAR = 2,         /* 1 = scalar kernel variants even for 16-byte aligned buffers                   */
    DCB_OPT_BLOCKS_PER_SM = 3,        /* cap on resident blocks per SM used to size persistent grids; 0 = what fits    */
    DCB_OPT_WITHHOLD_FIRST_COUNT = 4, /* test switch for the time-out path, driven from the host: the next compactions keep
                                         the survivor count of their first tile to themselves, so every bounded look-back
                                         wait for it runs out and the run ends with DCB_ERR_TIMEOUT (no fault, no trap)   */
    DCB_OPT_CACHE_MAX_ENTRIES = 5,    /* compiled pipelines kept per context (default 100, least recently used first out) */
    DCB_OPT_CACHE_ENTRIES = 6,        /* read-only: compiled pipelines in the cache now                                 */
    DCB_OPT_OVERLAP_LAUNCHES = 7      /* 1 = reductions are launched with programmatic stream serialisation: a query may start
                                         reading its input while the kernel before it on the same stream is still finishing
                                         (scratch and record are touched only after the grid-dependency wait). The caller
                                         thereby states that a query's INPUT is not written by the work enqueued just before it
                                         on that stream. Hides launch latency and ramp-up between back-to-back queries.   */
};
dcb_status dcb_set_option(dcb_ctx* ctx, int32_t option, int64_t value);
dcb_status dcb_get_option(dcb_ctx* ctx, int32_t option, int64_t* out_value);

/* ------------------------------------------------------------------------- memory */

/* Device buffers. Replace CudaMemoryManager.AllocateAsync / FreeAsync
 * (src/Backends/DotCompute.Backends.CUDA/Memory/CudaMemoryManager.cs:140-292) and back the
 * IUnifiedMemoryBuffer<T> contract (src/Core/DotCompute.Abstractions/Interfaces/IUnifiedMemoryBuffer.cs:13-261).
 * Allocation comes from the device's stream-ordered pool, not one cudaMalloc per buffer. */
dcb_status dcb_alloc(dcb_ctx* ctx, size_t bytes, dcb_buf** out_buf);
dcb_status dcb_free(dcb_ctx* ctx, dcb_buf* buf);
/* Wrap memory somebody else owns (for instance a tensor) without taking ownership. */
dcb_status dcb_buf_wrap(dcb_ctx* ctx, void* device_ptr, size_t bytes, dcb_buf** out_buf);
/* Zero-copy sub-range: Slice(offset,length) / AsType<T>() of IUnifiedMemoryBuffer (IUnifiedMemoryBuffer.cs:13-200). */
dcb_status dcb_buf_slice(dcb_ctx* ctx, dcb_buf* parent, size_t byte_offset, size_t bytes, dcb_buf** out_buf);
void*  dcb_devptr(const dcb_buf* buf);
size_t dcb_buf_bytes(const dcb_buf* buf);

/* Copies. Replace the blocking cudaMemcpy calls of CudaMemoryManager (CudaMemoryManager.cs:605-664)
 * with stream-ordered ones; `host` should be pinned for the copy to be truly asynchronous. */
dcb_status dcb_h2d_async(dcb_ctx* ctx, dcb_buf* dst, size_t dst_off, const void* host, size_t bytes, void* stream);
dcb_status dcb_d2h_async(dcb_ctx* ctx, void* host, const dcb_buf* src, size_t src_off, size_t bytes, void* stream);
dcb_status dcb_d2d_async(dcb_ctx* ctx, dcb_buf* dst, size_t dst_off, const dcb_buf* src, size_t src_off, size_t bytes, void* stream);
/* FillAsync of IUnifiedMemoryBuffer<T>: repeats a 1/2/4/8-byte pattern. */
dcb_status dcb_fill_async(dcb_ctx* ctx, dcb_buf* dst, size_t dst_off, const void* pattern, int32_t pattern_bytes, size_t count, void* stream);

/* Pinned host memory. Replace CudaPinnedMemoryAllocator (src/Backends/DotCompute.Backends.CUDA/Memory/CudaPinnedMemoryAllocator.cs:104). */
dcb_status dcb_host_alloc_pinned(dcb_ctx* ctx, size_t bytes, void** out_host);
dcb_status dcb_host_free_pinned(dcb_ctx* ctx, void* host);
dcb_status dcb_pin_host(dcb_ctx* ctx, void* host, size_t bytes);   /* cudaHostRegister of caller memory */
dcb_status dcb_unpin_host(dcb_ctx* ctx, void* host);

/* Bytes currently allocated / peak / number of allocations served (CudaMemoryManager.Analytics.cs). */
dcb_status dcb_memory_stats(dcb_ctx* ctx, int64_t* bytes_in_use, int64_t* peak_bytes, int64_t* n_allocs);

/* ------------------------------------------------------------------------ compile */

/* Translate one C# lambda to the CUDA C statements it becomes inside a fused kernel. Replaces
 * CudaKernelGenerator.ExpressionToCode / FormatConstant / GetOperator / GenerateMethodCall
 * (src/Extensions/DotCompute.Linq/CodeGeneration/CudaKernelGenerator.cs:1254-1391) and covers the wider
 * vocabulary of GpuExpressionTranslator (bitwise, shifts, ?:, casts, Math.*). `param_types` gives the
 * DCB_T_* type of each lambda parameter. On success *result_type is the C# type of the body. */
dcb_status dcb_translate_lambda(const char* lambda, const int32_t* param_types, int32_t n_params,
                                char* out_code, size_t out_cap, int32_t* result_type,
                                char* err, size_t err_cap);

/* Translate one [Kernel] method (C# source of a `static void` method over Span<T> / ReadOnlySpan<T> / T[] buffers and scalars)
 * to CUDA C. Replaces KernelExecutionMetadataEmitter.GenerateCuda / DetectDimensions
 * (src/Runtime/DotCompute.Generators/Kernel/Generation/KernelExecutionMetadataEmitter.cs:31-105, 275-436). Statements: local
 * declarations, assignments (also compound, ++, --), blocks, if / else, for, while, bare return; expressions as in lambdas plus
 * buffer[i], buffer.Length (becomes a trailing `const unsigned int __length` parameter, as in the reference) and
 * KernelContext.{ThreadId,BlockId,BlockDim,GridDim}.{X,Y,Z}. A body that names only ThreadId gets the global index for it, which is
 * what the reference's CPU invoker gives it (KernelExecutionMetadataEmitter.cs:117-170). meta_json receives
 * {"name", "needs_length", "dimensions", "params": [{"name", "is_buffer", "is_readonly", "element_type"}]}, the fields of the
 * reference's generated registry entry (KernelRegistrationEmitter.cs:56-192). Needs no GPU. */
dcb_status dcb_translate_kernel_method(const char* csharp_method, char* cuda_out, size_t cuda_cap, size_t* cuda_needed,
                                       char* meta_json, size_t meta_cap, char* err, size_t err_cap);

/* Build the fused kernels of a query. Replaces CompilationPipeline.CompileToGpuKernelAsync ->
 * CudaRuntimeKernelCompiler.CompileFromGraphAsync -> CudaKernelGenerator.GenerateCudaKernel -> NVRTC
 * (src/Extensions/DotCompute.Linq/CodeGeneration/CompilationPipeline.cs:914-965,
 * src/Extensions/DotCompute.Linq/Compilation/CudaRuntimeKernelCompiler.cs:80-189,
 * src/Extensions/DotCompute.Linq/CodeGeneration/CudaKernelGenerator.cs:81-125,
 * src/Backends/DotCompute.Backends.CUDA/Compilation/PTXCompiler.cs:83-273). Compiled pipelines are cached per
 * context under a key that contains the full lambda text (the reference's key leaves it out,
 * src/Extensions/DotCompute.Linq/CodeGeneration/KernelCache.cs:297-351). */
dcb_status dcb_pipeline_compile(dcb_ctx* ctx, const dcb_pipeline_desc* desc, dcb_pipeline** out_pipeline);
/* Gives back one reference obtained from dcb_pipeline_compile. The pipeline stays cached; once nobody holds it, it is a
 * candidate for eviction when the cache is full (DCB_OPT_CACHE_MAX_ENTRIES; KernelCache.cs:297-351 has the same bound). */
dcb_status dcb_pipeline_destroy(dcb_pipeline* p);
dcb_status dcb_pipeline_info_get(const dcb_pipeline* p, dcb_pipeline_info* out_info);
/* The generated CUDA source (the text NVRTC saw, or would see for a precompiled pipeline). */
dcb_status dcb_pipeline_source(const dcb_pipeline* p, char* buf, size_t cap, size_t* needed);
/* Generate that source without a GPU or a context (used to test the generator on any machine). */
dcb_status dcb_pipeline_generate_source(const dcb_pipeline_desc* desc, char* buf, size_t cap, size_t* needed,
                                        char* err, size_t err_cap);

/* ---------------------------------------------------------------------------- run */

/* Run a compiled query on device-resident inputs. Replaces RuntimeExecutor.ExecuteGpuOnCudaAsync's launch
 * (src/Extensions/DotCompute.Linq/CodeGeneration/RuntimeExecutor.cs:245-312) and
 * CudaCompiledKernel.ExecuteAsync / CudaKernelLauncher (src/Backends/DotCompute.Backends.CUDA/Kernels/CudaCompiledKernel.cs:495-547,
 * Kernels/CudaKernelLauncher.cs:204-347).
 *   in0, in1   device pointers to n elements each (in1 NULL unless Zip)
 *   out        device pointer with room for out_cap elements of out_type (ToArray only, else NULL)
 *   d_result   device pointer to DCB_DEVICE_RESULT_BYTES the kernels fill; NULL uses context scratch
 *   d_prev     device pointer to an earlier run's record whose count is the output offset of this run
 *              (chains chunked compactions without a host round trip); normally NULL
 * The call only enqueues work on `stream`. */
dcb_status dcb_pipeline_run_async(dcb_pipeline* p, const void* in0, const void* in1, int64_t n,
                                  void* out, int64_t out_cap, void* d_result, const void* d_prev, void* stream);
/* Same, then waits, reads the record back and applies the terminal's semantics
 * (empty-sequence and overflow errors, Average division, rounding to float). */
dcb_status dcb_pipeline_run(dcb_pipeline* p, const void* in0, const void* in1, int64_t n,
                            void* out, int64_t out_cap, dcb_result* result, void* stream);
/* The same with flags. DCB_RUN_TAKE: the query is `...Where(...)...Take(k)` and out_cap is k. The compaction stops reading
 * its input soon after k survivors are known (persistent blocks stop drawing tiles once a tile starts at or beyond k), more
 * survivors than k is not an error, and result->count is the number of elements written (at most k). The reference's visitor
 * lists Take (src/Extensions/DotCompute.Linq/Compilation/ExpressionTreeVisitor.cs:263-265); System.Linq stops iterating at k. */
enum { DCB_RUN_TAKE = 1u };
dcb_status dcb_pipeline_run_ex(dcb_pipeline* p, const void* in0, const void* in1, int64_t n,
                               void* out, int64_t out_cap, uint32_t flags, dcb_result* result, void* stream);
/* Turn a (possibly NCCL-combined) 16-slot record held in HOST memory into a dcb_result: applies what System.Linq's
 * terminal does after its loop (the scalar branch of ComputeQueryProvider.Execute,
 * src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:240-267). */
dcb_status dcb_result_finalize(const dcb_pipeline* p, const void* host_record, dcb_result* result);
/* The same without a pipeline or a GPU: terminal is a DCB_OP_*, out_type the element type that reached it. */
dcb_status dcb_record_finalize(int32_t terminal, int32_t out_type, const void* host_record, dcb_result* result);

/* The call a host-array user makes: inputs and output are HOST buffers (pinned for full speed). Copies go
 * through the chunked, double-buffered staging path overlapped with the kernels. Replaces the whole of
 * RuntimeExecutor.ExecuteGpuOnCudaAsync (alloc, H2D, launch, D2H, free; RuntimeExecutor.cs:245-312) and
 * BaseMemoryManager.AllocateAndCopyAsync (src/Core/DotCompute.Core/Memory/BaseMemoryManager.cs:104-112).
 * For ToArray, host_out receives result->count elements (capacity host_out_cap). */
dcb_status dcb_pipeline_run_host(dcb_pipeline* p, const void* host_in0, const void* host_in1, int64_t n,
                                 void* host_out, int64_t host_out_cap, dcb_result* result);
/* The same with DCB_RUN_* flags; with DCB_RUN_TAKE no further chunk is uploaded once k survivors have come back. */
dcb_status dcb_pipeline_run_host_ex(dcb_pipeline* p, const void* host_in0, const void* host_in1, int64_t n,
                                    void* host_out, int64_t host_out_cap, uint32_t flags, dcb_result* result);

/* ------------------------------------------------------------------ peer exchange */

/* Exchange of partials for sharded reductions (one process per GPU), without NCCL: dcb_peer_exchange_async enqueues a
 * one-warp kernel that stores this GPU's partial (the record a reduction just wrote) into an exchange area in each peer's
 * memory over NVLink, waits (bounded) for the peers' partials in its own area, folds all of them in rank order, so every GPU
 * computes the bit-identical total, and rewrites the record with the global result. Enqueue it on a side stream behind the
 * reduction (an event) and it runs beside the next query's reduce kernel, so neither NVLink latency nor the skew between GPUs
 * is on the critical path of a stream of queries; dcb_pipeline_run (the blocking call) enqueues it on its own stream. All
 * ranks must issue the same sequence of exchanges. A peer that never arrives ends the wait with DCB_RES_TIMEOUT in the record.
 * The reference has no multi-GPU LINQ path (device 0 only, src/Extensions/DotCompute.Linq/ComputeQueryableExtensions.cs:188);
 * its P2P manager only copies buffers (src/Backends/DotCompute.Backends.CUDA/P2P/CudaP2PManager.cs:137-242).
 *   dcb_peer_area_create     allocates this GPU's 2 KiB exchange area and writes its 64-byte CUDA IPC handle to handle_out
 *   dcb_peer_connect         handles = world handles, handle_stride bytes apart, gathered from all ranks (index = rank)
 *   dcb_peer_area_ptr / dcb_peer_connect_local   the same for a host that drives several GPUs from ONE process (as the
 *                            reference does): exchange plain device pointers of the areas (peer access enabled by the caller)
 *   dcb_peer_exchange_async  d_record: the 128-byte device record of the reduction; out_type: DCB_T_* that reached its terminal
 *   dcb_peer_disconnect      back to single-GPU behaviour */
dcb_status dcb_peer_area_create(dcb_ctx* ctx, void* handle_out, size_t handle_cap);
dcb_status dcb_peer_connect(dcb_ctx* ctx, int32_t world, int32_t rank, const void* handles, size_t handle_stride);
dcb_status dcb_peer_area_ptr(dcb_ctx* ctx, void** out_area, size_t* out_bytes);
dcb_status dcb_peer_connect_local(dcb_ctx* ctx, int32_t world, int32_t rank, void* const* areas);
dcb_status dcb_peer_exchange_async(dcb_ctx* ctx, void* d_record, int32_t out_type, void* stream);
dcb_status dcb_peer_disconnect(dcb_ctx* ctx);

/* ------------------------------------------------------- OrderBy, GroupBy, Join (multi-block) */

/* The three relational operators of the reference's generators, which emit single-block or direct-index kernels
 * (src/Extensions/DotCompute.Linq/CodeGeneration/CudaKernelGenerator.cs:613-751 OrderBy, :753-825 GroupBy, :827-900 Join;
 * OrderByKernelGenerator.cs:108, GroupByKernelGenerator.cs:152, JoinKernelGenerator.cs:140-239) with the CPU semantics of
 * CpuKernelGenerator.cs:475-723. All three work on KEYS the caller has already computed with a fused Select pipeline (the key
 * selector) and return INDICES into the source, which the caller gathers or feeds to another pipeline (the result selector).
 * Sizes are limited to 2^32 - 1 elements (indices and counts are 32-bit). Scratch comes from the context's stream-ordered pool.
 *
 *   dcb_sort_indices     stable argsort of n keys of type key_type (DCB_T_*; floating keys order as .NET's comparer does: NaN
 *                        first, -0 equal to +0); descending != 0 sorts descending, ties still in source order. A least-
 *                        significant-digit radix sort, 8 bits a pass, over any number of blocks. Passes whose digit is the
 *                        same in every key are skipped (keys below 1000: two passes of four); to know them the call reads
 *                        the keys once and synchronises the stream once (not while the stream is being captured).
 *   dcb_sort_by_key      the same sort with the elements travelling beside their keys instead of their positions:
 *                        d_sorted_values = d_values in stable key order, with no gather afterwards (a gather reads one
 *                        32-byte sector per element from all over the source: a quarter of OrderBy's time). value_bytes must
 *                        be 4; DCB_ERR_NOT_SUPPORTED otherwise (use dcb_sort_indices + dcb_gather). d_values may be d_keys.
 *   dcb_gather           dst[i] = src[indices[i]] for elements of 1, 2, 4 or 8 bytes.
 *   dcb_prefix_sum       d_out[i] = d_in[0] + ... + d_in[i] (inclusive != 0) or ... + d_in[i-1] (exclusive) for int, long, float
 *                        or double columns of any length (the reference's scan kernel, CudaKernelGenerator.cs:499-576,
 *                        covers one block of 256). Integers add in their own width and wrap, as that kernel does; floats
 *                        add in fp64 and each output is rounded once. d_out may be d_in.
 *   dcb_group_aggregate  groups n (key, value) pairs by key; aggregate = DCB_AGG_*. One output per group, in order of first
 *                        occurrence of the key (the order a Dictionary enumerates in, CpuKernelGenerator.cs:620-633):
 *                        d_out_first[g] = index of the group's first element (its key is keys[that]), d_out_counts[g], and
 *                        the aggregate as double in d_out_f64[g] (Sum / Min / Max / Average; integer values also exactly in
 *                        d_out_i64[g] for Sum / Min / Max). Floating sums accumulate in fp64. *out_groups = number of groups;
 *                        DCB_ERR_OUTPUT_TOO_SMALL if it exceeds out_cap (then call again with larger outputs).
 *   dcb_join_indices     equi-join of outer and inner keys. DCB_JOIN_INNER: one (outer index, inner index) pair per match,
 *                        ordered by outer index, then inner index (the order of Enumerable.Join); DCB_JOIN_SEMI / ANTI: the
 *                        outer indices with at least one / with no match (d_inner_out may be NULL). With d_outer_out NULL
 *                        only *out_pairs is computed (to size the outputs). */
enum { DCB_AGG_COUNT = 0, DCB_AGG_SUM = 1, DCB_AGG_MIN = 2, DCB_AGG_MAX = 3, DCB_AGG_AVERAGE = 4 };
enum { DCB_JOIN_INNER = 0, DCB_JOIN_SEMI = 2, DCB_JOIN_ANTI = 3 };   /* values of JoinKernelGenerator.JoinType (:67-77) */
dcb_status dcb_sort_indices(dcb_ctx* ctx, int32_t key_type, const void* d_keys, int64_t n, int32_t descending,
                            uint32_t* d_indices, void* stream);
dcb_status dcb_sort_by_key(dcb_ctx* ctx, int32_t key_type, const void* d_keys, int64_t n, int32_t descending,
                           int32_t value_bytes, const void* d_values, void* d_sorted_values, void* stream);
dcb_status dcb_prefix_sum(dcb_ctx* ctx, int32_t elem_type, const void* d_in, int64_t n, int32_t inclusive, void* d_out, void* stream);
dcb_status dcb_gather(dcb_ctx* ctx, int32_t elem_bytes, const void* d_src, const uint32_t* d_indices, int64_t n, void* d_dst, void* stream);
dcb_status dcb_group_aggregate(dcb_ctx* ctx, int32_t key_type, const void* d_keys, int32_t value_type, const void* d_values, int64_t n,
                               int32_t aggregate, int64_t out_cap, uint32_t* d_out_first, int64_t* d_out_counts, double* d_out_f64,
                               int64_t* d_out_i64, int64_t* out_groups, void* stream);
dcb_status dcb_join_indices(dcb_ctx* ctx, int32_t key_type, const void* d_outer_keys, int64_t n_outer, const void* d_inner_keys,
                            int64_t n_inner, int32_t join_kind, int64_t out_cap, uint32_t* d_outer_out, uint32_t* d_inner_out,
                            int64_t* out_pairs, void* stream);

/* ------------------------------------------------------------- no device allocation */

/* Tiles the fixed scratch of dcb_compact_noalloc holds. With every pointer 16-byte aligned a tile is 8192 elements for
 * 4-byte inputs and outputs (4096 for 8-byte ones), so float queries up to 2^29 elements fit; with an unaligned pointer
 * the scalar kernel runs, whose tile is 2048 elements (2^27 elements per call). The refusal's text names the limit. */
#define DCB_NOALLOC_MAX_TILES 65536

/* Stable Where [-> Select] -> ToArray for callers that must not allocate device memory. (No counterpart in the
 * reference: its backend allocates per call.) Think of a host process that handed all of HBM to its own buffer pool
 * at start-up, where a cudaMalloc from inside a native library fails or falsifies the pool's accounting, or of a
 * latency-critical loop that cannot afford the implicit synchronisation of an allocation.
 *
 * This call allocates nothing: no cudaMalloc / cudaFree / pool allocation, no NVRTC, no module load. The look-back
 * descriptors live in a fixed device array inside the library image (DCB_NOALLOC_MAX_TILES * 8 + 256 bytes, held by
 * every GPU that loads the library until the process exits). Therefore:
 *   - only queries of the precompiled table are accepted (others: DCB_ERR_NOT_SUPPORTED);
 *   - n may not need more than DCB_NOALLOC_MAX_TILES tiles (else DCB_ERR_INVALID_ARGUMENT, text via dcb_last_error(NULL,..));
 *   - all calls on one GPU share the array, which still holds the previous call's contents (the call clears what must
 *     start at zero on `stream` itself); calls that overlap on the same GPU race and must be serialised by the caller;
 *   - the first call on each device looks up the array's device address; make that first call outside any stream
 *     capture.
 * in0 / in1 / out / d_record are device pointers supplied by the caller; d_record receives DCB_DEVICE_RESULT_BYTES
 * (survivor count in slot DCB_SLOT_COUNT, DCB_RES_* bits in slot DCB_SLOT_FLAGS). The call only enqueues work on `stream`
 * (NULL = the default stream). There is no dcb_ctx: `device` is the CUDA device ordinal; the call makes it current while
 * it works and puts the caller's current device back before it returns. */
dcb_status dcb_compact_noalloc(int32_t device, const dcb_pipeline_desc* desc, const void* in0, const void* in1,
                               int64_t n, void* out, int64_t out_cap, void* d_record, void* stream);

/* ---------------------------------------------------------- [Kernel] source kernels */

/* Compile CUDA C text produced by the [Kernel] generator and launch it. Replace
 * CudaAccelerator.CompileKernelAsync + CudaCompiledKernel.LoadModule + cuLaunchKernel as used by
 * KernelExecutionService.ExecuteAsync (src/Runtime/DotCompute.Runtime/Services/KernelExecutionService.cs:291-328,
 * src/Backends/DotCompute.Backends.CUDA/Kernels/CudaCompiledKernel.cs:151-225). NVRTC runs with
 * --gpu-architecture=sm_100a and without --use_fast_math (the reference passes it, PTXCompiler.cs:263-264). */
dcb_status dcb_kernel_compile(dcb_ctx* ctx, const char* cuda_source, const char* entry_point, dcb_kernel** out_kernel);
dcb_status dcb_kernel_launch(dcb_kernel* k, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_bytes,
                             void** args, void* stream);
dcb_status dcb_kernel_destroy(dcb_kernel* k);

/* ------------------------------------------------------------------------- timing */

/* CUDA events on the context's stream. Replace the ExecutionMetrics timers of the LINQ executor
 * (src/Extensions/DotCompute.Linq/CodeGeneration/ExecutionMetrics.cs:11-60). */
dcb_status dcb_event_create(dcb_ctx* ctx, void** out_event);
dcb_status dcb_event_record(dcb_ctx* ctx, void* event, void* stream);
dcb_status dcb_event_elapsed_ms(dcb_ctx* ctx, void* start, void* stop, float* out_ms);
dcb_status dcb_event_destroy(dcb_ctx* ctx, void* event);
/* Kernels launched by this context since dcb_init (the library's own counter). */
dcb_status dcb_launch_count(dcb_ctx* ctx, int64_t* out_launches);

#ifdef __cplusplus
}
#endif
#endif /* DCB200_H */
