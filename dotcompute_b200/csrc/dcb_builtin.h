// dcb_builtin.h — table of pipelines compiled ahead of time by nvcc from the same templates and the same
// translator output that NVRTC would see. A query whose canonical key is in the table starts without a JIT step.
#ifndef DCB_BUILTIN_H
#define DCB_BUILTIN_H

struct dcb_builtin_entry {
    const char* key;        // canonical pipeline key (dcbt::ChainInfo::key)
    const void* k_vec;      // kernel taking 16-byte aligned pointers
    const void* k_scalar;   // kernel for any alignment
    int unroll;             // packs per thread per tile the kernels were built with
    int compact_block;      // threads per block of the compaction kernels
    const void* k_stream;   // streamed compaction kernel, or null when the query has none
    int stream_rows;        // rows per worker warp it was built with
    int stream_warps;       // worker warps per block
    int stream_nbuf;        // shared-memory slots per input
    int stream_copy_warps;  // warps per block that only write tiles out
};

const dcb_builtin_entry* dcb_builtin_find(const char* key);
int dcb_builtin_count();
const dcb_builtin_entry* dcb_builtin_at(int i);

#endif
