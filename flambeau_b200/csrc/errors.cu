// Error channel of the kernel library: the last message per host thread.
#include "common.cuh"

#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

static thread_local char g_last_error[1024] = "";

int g_fb_pdl = 1;
// The two-SM product (a cluster kernel) is launched plainly, and with it the 256-token tile of the one-SM product,
// its stand-in.  With hundreds of launches queued ahead of the device (a deep model's step of several hundred rows
// whose products do not fill every SM pair), programmatic launches of the cluster kernel stopped the device: no
// kernel of the queue made progress any more, although no wait in any kernel here depends on a later kernel;
// with that one kernel launched plainly the same queue runs.  The tcgen05 attention kernel and everything else
// keep their programmatic launches.  The products concerned run for tens of microseconds and more; what they give
// up is the overlap of their prologue with the tail of the kernel before them.
int g_fb_plain_classes = FB_LAUNCH_GEMM_PAIR | FB_LAUNCH_GEMM_WIDE;

// Switches programmatic dependent launch on (1, the default) or off (0) for all later launches.
FB_API void fb_set_pdl(int on) { g_fb_pdl = on ? 1 : 0; }

// Which kernel classes (a bit set of FbLaunchClass) are launched plainly while programmatic dependent launch is on.
FB_API void fb_set_plain_launch_classes(int classes) { g_fb_plain_classes = classes; }

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

// `rows` rows of `width_bytes` from pinned host memory to the device, each side with its own distance between rows
// (one asynchronous 2-d copy on the stream: a step's descriptor is a few rows of a wider staging buffer).
FB_API int fb_copy_rows_to_device(void* dst, long long dst_pitch, const void* src, long long src_pitch,
                                  long long width_bytes, long long rows, cudaStream_t stream) {
    if (width_bytes <= 0 || rows <= 0) return 0;
    const cudaError_t e = cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width_bytes,
                                            (size_t)rows, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fb_fail(-2, "copy of a step's descriptor to the device failed: %s", cudaGetErrorString(e));
    return 0;
}

FB_API const char* fb_last_error() { return g_last_error; }

// Version stamp checked by the Python loader against the sources it compiled.
FB_API int fb_abi_version() { return 1; }
