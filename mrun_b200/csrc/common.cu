// Error string of the kernel library and its version query.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

int mrun_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
    return 1;
}

// The message of the last failed call on this thread.
MRUN_API const char* mrun_last_error() { return g_error; }

// 100 for sm_100a builds; lets the loader check that it opened the right library.
MRUN_API int mrun_target_arch() { return 100; }
