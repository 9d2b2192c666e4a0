// Shared vocabulary of the kernel library: dtype codes, typed loads and
// stores, the error channel, and warp/block reductions.
//
// Every exported launcher is `extern "C"`, takes raw device pointers, sizes
// and a stream, validates its arguments on the host, and returns 0 or a
// negative code after recording a message that `fb_last_error()` returns.
// The reference validates every launch the same way before it reaches the
// device (crates/forward/src/core/composites/standard_attn.rs:74-119).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define FB_API extern "C" __attribute__((visibility("default")))

enum FbDtype : int { FB_F32 = 0, FB_BF16 = 1 };

// Status word bits that kernels may set (never trap, never spin forever).
enum FbStatus : int {
    FB_STATUS_BAD_TOKEN = 1,      // embedding id outside the table
    FB_STATUS_BAD_PAGE = 2,       // block table entry missing for a live key
    FB_STATUS_WAIT_TIMEOUT = 4,   // a bounded barrier wait ran out
};

int fb_fail(int code, const char* fmt, ...);   // records the message, returns code
int fb_check_launch(const char* what);          // cudaGetLastError -> fb_fail

#define FB_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) return fb_fail(-1, __VA_ARGS__);           \
    } while (0)

// ---- the device ---------------------------------------------------------------
constexpr int FB_MAX_DEVICES = 64;
int fb_device_ordinal();    // the current device, clamped into [0, FB_MAX_DEVICES)
int fb_sm_count();          // multiprocessors of the current device (asked once per device)

// Set-up that a launcher does once per device (raising a kernel's shared-memory limit): `flags` is the
// launcher's own static array of FB_MAX_DEVICES zeros.  Two host threads may both see "not yet" and both do the
// set-up, which is harmless because the set-up is idempotent.
inline bool fb_needs_setup(const bool* flags) { return !flags[fb_device_ordinal()]; }
inline void fb_setup_done(bool* flags) { flags[fb_device_ordinal()] = true; }

// Weights of the launchers' cost models (how many shares of K pay off): about what one device streams from
// memory and what one multiprocessor's tensor pipe multiplies.  They rank choices; nothing is sized by them.
constexpr double FB_MODEL_HBM_BYTES_PER_S = 6.0e12;
constexpr double FB_MODEL_SM_FLOPS = 9.0e12;

// ---- activations of gated feed-forwards -----------------------------------------
// out = act(gate) * up.  The code travels as a launcher argument (0 = no gating where that is an option).
enum FbAct : int { FB_ACT_SILU = 1, FB_ACT_GELU_TANH = 2 };
inline bool fb_act_known(int act) { return act == FB_ACT_SILU || act == FB_ACT_GELU_TANH; }
__device__ __forceinline__ float fb_gate_times(int act, float g, float u) {
    if (act == FB_ACT_GELU_TANH) {
        // 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))
        const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
        return 0.5f * g * (1.0f + t) * u;
    }
    return g / (1.0f + expf(-g)) * u;             // SiLU (crates/model-ops/src/ops/activation.rs:107-118)
}

// ---- launches ---------------------------------------------------------------
// Kernels of a step run back to back on one stream.  With programmatic dependent launch the next kernel of the
// stream may be scheduled while this one is still draining: every kernel begins with fb_pdl_launch_dependents()
// (which lets the kernel after it start being placed once all of this kernel's blocks have begun) and calls
// fb_pdl_wait() before its first read of what the kernel before it produced and before its first global write.
// fb_pdl_wait() returns once all earlier kernels of the stream have completed and their writes are visible, so
// the order of results is that of ordinary stream launches; only launch latency and prologues overlap.
extern int g_fb_pdl;        // 1: launch with the programmatic-serialization attribute; 0: plain launches
// Kernel classes that are launched plainly even while programmatic dependent launch is on (a bit set of FbLaunchClass).
enum FbLaunchClass : int { FB_LAUNCH_OTHER = 0, FB_LAUNCH_GEMM_PAIR = 1, FB_LAUNCH_ATTENTION_TC = 2, FB_LAUNCH_GEMM_WIDE = 4 };
extern int g_fb_plain_classes;

__device__ __forceinline__ void fb_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void fb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline void fb_launch_class(int launch_class, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (g_fb_pdl && !(launch_class & g_fb_plain_classes)) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);     // an error shows in fb_check_launch()
}
template <typename... KArgs, typename... Args>
inline void fb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      Args... args) {
    fb_launch_class(FB_LAUNCH_OTHER, kernel, grid, block, smem, stream, args...);
}

// ---- a running start for the product that follows ---------------------------
// The first `bytes` of every row of a weight matrix, fetched into L2 by a kernel that has the memory system to
// spare (the split-key attention kernel when its stream of cache ends), so that the product after it finds its
// first k-blocks there.  It travels in the launcher's arguments; a hint, nothing depends on it.
struct FbPrefetch {
    const char* base;      // nullptr: nothing to do
    int rows;
    long row_stride;       // bytes
    int bytes;             // per row, a multiple of 16
};
// The hint for `rows` rows `row_stride_bytes` apart from `base`, `bytes_per_row` of each; an empty hint when the
// arguments cannot be used (no base, unaligned rows, too few bytes).
FbPrefetch fb_make_prefetch(const void* base, long long rows, long long row_stride_bytes, int bytes_per_row);

__device__ __forceinline__ void fb_prefetch_issue(const FbPrefetch& pf, long worker, long n_workers) {
    if (!pf.base) return;
    for (long r = worker; r < pf.rows; r += n_workers)
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf.base + r * pf.row_stride), "r"(pf.bytes) : "memory");
}

// ---- typed access -----------------------------------------------------------
__device__ __forceinline__ float fb_to_float(float v) { return v; }
__device__ __forceinline__ float fb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T fb_from_float(float v);
template <> __device__ __forceinline__ float fb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 fb_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// ---- reductions -------------------------------------------------------------
__device__ __forceinline__ float fb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float fb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `scratch` holds at least 32 floats of shared memory.
// Every thread of the block must call it; every thread gets the result.
__device__ __forceinline__ float fb_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = fb_warp_sum(v);
    __syncthreads();                       // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = fb_warp_sum(r);
    return r;
}
__device__ __forceinline__ float fb_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = fb_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = fb_warp_max(r);
    return r;
}

// Dispatch a dtype code to a template parameter.
#define FB_DISPATCH_DTYPE(code, T, ...)                                   \
    do {                                                                  \
        if ((code) == FB_F32) { using T = float; __VA_ARGS__; }           \
        else if ((code) == FB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return fb_fail(-1, "unknown dtype code %d", (int)(code));    \
    } while (0)
