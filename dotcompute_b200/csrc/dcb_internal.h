// dcb_internal.h - helpers shared by the library's own translation units (not part of the C ABI).
#ifndef DCB_INTERNAL_H
#define DCB_INTERNAL_H

// Sets the calling thread's last-error text, the one dcb_last_error(NULL, ...) returns.
void dcb_set_thread_error(const char* msg);

struct dcb_ctx;
// Makes the context's GPU current for the calling thread (0 = ok, else a dcb_status) / the stream an entry point should
// use for a caller-supplied `stream` argument (NULL = the context's own) / counts kernels launched on the context's behalf.
int dcb_ctx_make_current(dcb_ctx* ctx);
void* dcb_ctx_pick_stream(dcb_ctx* ctx, void* stream);
void dcb_ctx_count_launches(dcb_ctx* ctx, int n);

#endif
