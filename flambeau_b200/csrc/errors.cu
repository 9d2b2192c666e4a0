// Error channel of the kernel library: the last message per host thread.
#include "common.cuh"

#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

static thread_local char g_last_error[1024] = "";

int g_fb_pdl = 1;
// Kernels that fill a multiprocessor by themselves (the two-SM product, the tcgen05 attention and the 256-token
// tile of the one-SM product: about 193 KB of shared memory and all of tensor memory) are launched plainly.  With
// hundreds of launches queued ahead of the device (a deep model's step of several hundred rows), programmatic
// launches of these kernels stopped the device: no kernel of the queue made progress any more, although no wait
// of any kernel here depends on a later one; launched plainly they run.  They run for tens of microseconds and
// more, so the overlap of their prologue with the tail of the kernel before them is what they give up.
long g_fb_pdl_max_smem = 128 * 1024;

// Switches programmatic dependent launch on (1, the default) or off (0) for all later launches.
FB_API void fb_set_pdl(int on) { g_fb_pdl = on ? 1 : 0; }

// Kernels that ask for more than `bytes` of dynamic shared memory are launched plainly (they wait for all earlier
// work and are not overlapped with the kernel before them) even while programmatic dependent launch is on.
FB_API void fb_set_pdl_max_smem(long long bytes) { g_fb_pdl_max_smem = (long)bytes; }

FbPrefetch fb_make_prefetch(const void* base, long long rows, long long row_stride_bytes, int bytes_per_row) {
    FbPrefetch pf = {nullptr, 0, 0, 0};
    const bool ok = base && rows > 0 && rows < (1LL << 31) && bytes_per_row >= 16 && row_stride_bytes >= bytes_per_row &&
                    ((uintptr_t)base & 15) == 0 && row_stride_bytes % 16 == 0;
    if (!ok) return pf;
    pf.base = (const char*)base;
    pf.rows = (int)rows;
    pf.row_stride = (long)row_stride_bytes;
    pf.bytes = bytes_per_row & ~15;
    return pf;
}

int fb_device_ordinal() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    return dev < FB_MAX_DEVICES ? dev : FB_MAX_DEVICES - 1;
}

int fb_sm_count() {
    static int sms[FB_MAX_DEVICES] = {};
    const int dev = fb_device_ordinal();
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

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
