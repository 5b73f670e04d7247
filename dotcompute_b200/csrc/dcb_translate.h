// dcb_translate.h — C# lambda text -> CUDA C "chain" functor.
//
// Takes the place of the reference's expression-to-CUDA printers
// (src/Extensions/DotCompute.Linq/CodeGeneration/CudaKernelGenerator.cs:1254-1416 and the wider vocabulary of
// src/Extensions/DotCompute.Linq/CodeGeneration/GpuExpressionTranslator.cs:130-342). The reference prints the
// operators as written and lets C++ typing rules decide the arithmetic; this translator types every
// sub-expression by the C# rules (binary numeric promotion, constant-expression narrowing, shift-count
// masking, wrapping integer arithmetic) and prints the conversions explicitly, so the kernel computes what the
// C# lambda computes.
#ifndef DCB_TRANSLATE_H
#define DCB_TRANSLATE_H

#include <string>
#include <vector>

namespace dcbt {

// Values equal DCB_T_* of the C ABI.
enum Type { T_NONE = 0, T_I8, T_U8, T_I16, T_U16, T_I32, T_U32, T_I64, T_U64, T_F32, T_F64, T_BOOL };

const char* cuda_name(int type);    // "float", "long long", ...
const char* csharp_name(int type);  // "float", "long", ...
int type_size(int type);
bool is_numeric(int type);

// Translate `lambda` ("x => x * 2f + 1f", "(a, b) => a * b"). `args[i]` is the CUDA expression that stands for
// parameter i and `arg_types[i]` its type. Returns false and fills `err` when the text is outside the grammar.
bool translate_lambda(const std::string& lambda, const std::vector<std::string>& args, const std::vector<int>& arg_types,
                      std::string* code, int* result_type, std::string* err);

// A [Kernel] method (C# source text of one static void method) translated to CUDA C. Takes the place of
// KernelExecutionMetadataEmitter.GenerateCuda / DetectDimensions
// (src/Runtime/DotCompute.Generators/Kernel/Generation/KernelExecutionMetadataEmitter.cs:31-105, 275-436).
struct KernelParam { std::string name; bool is_buffer = false; bool is_readonly = false; int elem_type = T_NONE; };
struct KernelMethod {
    std::string name;            // also the CUDA entry point
    std::string cuda_source;     // extern "C" __global__ void name(...) { ... }
    bool needs_length = false;   // the body read a buffer's .Length: a trailing `const unsigned int __length` was added
    int dimensions = 1;          // 1, 2 or 3 (highest KernelContext axis used)
    std::vector<KernelParam> params;
};
bool translate_kernel_method(const std::string& csharp, KernelMethod* out, std::string* err);

struct OpSpec { int kind; std::string lambda; };   // kind = DCB_OP_*

struct ChainInfo {
    int in0 = T_NONE, in1 = T_NONE;   // input element types
    int n_in = 1;
    int out_type = T_NONE;            // element type reaching the terminal
    int terminal = 0;                 // DCB_OP_*
    int result_type = T_NONE;         // scalar type a reduction returns
    int red_mask = 0;                 // RED_* bits the kernel needs
    bool checked_div = false;         // a lambda divides integers by something that may be zero: the module has a fault word
    bool checked_sum = false;         // Sum over int / long: the kernel tracks the range of the running sum (checked arithmetic)
    bool has_filter = false;
    bool is_identity = false;         // no Select/Where/Zip at all
    std::string chain_src;            // struct dcb_chain { ... };
    std::string key;                  // canonical text identifying the pipeline (types + ops + translated code)
};

// Build the chain of a whole query. Checks operator order and the terminal's type rules.
bool build_chain(int elem_type0, int elem_type1, const std::vector<OpSpec>& ops, ChainInfo* info, std::string* err, int* status);

// Complete translation unit for NVRTC or nvcc: prelude + chain + extern "C" kernels whose names end in `suffix`.
// `kernels_header` is the text of dcb_kernels.cuh, or empty to emit an #include of it instead.
struct Tuning {
    int block = 256;            // threads per block (the kernels assume 256)
    int unroll = 4;             // 16-byte loads in flight per thread in map / reduce
    int reduce_min_blocks = 0;  // second argument of __launch_bounds__ for the reduce kernels; 0 = 6 (one input) / 4 (Zip)
    int compact_block = 256;    // threads per block of the compaction kernels
    int compact_rows = 0;       // rows per warp in the compaction tile; 0 = automatic (dcb::compact_rows_for)
    int compact_min_blocks = 4; // second argument of __launch_bounds__ for the compaction kernels; 0 = none
    // streamed compaction kernel (dcb::compact_stream_body)
    int stream = 1;             // 1 = build it (as dcb_compact_stream) when the query allows
    int stream_warps = 4;       // worker warps per block (the block has two more warps: offsets and loader)
    int stream_rows = 0;        // rows of 32 packs per worker and tile; 0 = automatic (stream_rows_for)
    int stream_lag = 3;         // rounds between ranking a tile and writing it (its offset is ready after two)
    int stream_copy_warps = 2;  // warps that only write ranked tiles out (0: every worker writes its own run after ranking the next tile)
    int stream_nbuf = 5;        // shared-memory slots per input: lag + 1 + tiles on their way in
    int stream_depth = 3;       // 16-byte descriptor loads per lane of the offsets warp (128 * depth tiles per window)
    int stream_ahead_mb = 12;   // distance of the L2 prefetch in front of the tile being drawn; 0 = none
    int stream_draw_ahead = 0;  // rounds the draw of a tile id may run ahead of ranking; 0 = as soon as a slot is free
    int stream_min_blocks = 2;  // second argument of __launch_bounds__; 0 = none
};

// Shape of the streamed compaction kernel (dcb::compact_stream_body): rows per worker warp such that one slot (a
// tile of every input) holds at most 16 KB (six slots, two blocks per SM), or 0 when the query cannot use the kernel (no Where, or an output element
// wider than the first input's, which rules out staging in place).
int stream_rows_for(const ChainInfo& info, int warps);
long long stream_tile_elems(const ChainInfo& info, int rows, int warps);
long long stream_smem_bytes(const ChainInfo& info, int rows, int warps, int nbuf);
int stream_block_threads(int warps, int copy_warps);
std::string build_program(const ChainInfo& info, const std::string& suffix, const std::string& kernels_header,
                          const Tuning& tuning, bool with_prelude);

unsigned long long fnv1a(const std::string& s);

}  // namespace dcbt
#endif
