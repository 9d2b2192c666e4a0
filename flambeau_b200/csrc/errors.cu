// Error channel of the kernel library: the last message per host thread.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_last_error[1024] = "";

int g_fb_pdl = 1;

// Switches programmatic dependent launch on (1, the default) or off (0) for all later launches.
FB_API void fb_set_pdl(int on) { g_fb_pdl = on ? 1 : 0; }

int fb_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

int fb_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fb_fail(-2, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

FB_API const char* fb_last_error() { return g_last_error; }

// Version stamp checked by the Python loader against the sources it compiled.
FB_API int fb_abi_version() { return 1; }
