// dcb_internal.h - helpers shared by the library's own translation units (not part of the C ABI).
#ifndef DCB_INTERNAL_H
#define DCB_INTERNAL_H

// Sets the calling thread's last-error text, the one dcb_last_error(NULL, ...) returns.
void dcb_set_thread_error(const char* msg);

#endif
