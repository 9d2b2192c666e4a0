/* An entry point of the kernel library that allocates nothing.
 *
 * It has no counterpart in the reference (arte-fact/flambeau); it exists for
 * callers of this library that may not allocate device memory at the moment
 * they need a matrix product.  Two kinds of caller are meant.  A host program
 * that sized everything at start-up and handed all remaining device memory to
 * its own pool: for it a cudaMalloc inside a library call can simply fail.
 * And a serving loop that must not stall: cudaMalloc and cudaFree synchronise
 * the whole device, so a call that allocates, even rarely, puts a pause of
 * unknown length into a loop that is otherwise only stream-ordered.
 *
 * The ordinary split-K product (fb_gemm_tc) takes its scratch from the caller:
 * float32 partial tiles and one arrival counter per output tile.
 * fb_gemm_tc_noalloc is the same kernel with that scratch in a fixed array
 * inside the library's device image.  The caller still passes the operands
 * and the output; nothing else is needed.
 *
 * Limits
 *   - at most FB_NOALLOC_MAX_ROWS rows of X (the shapes of a decode step) and at
 *     most FB_NOALLOC_MAX_TILES * 128 output features; larger calls are refused
 *     with an error (fb_last_error() says which limit), never shrunk silently;
 *   - the array takes FB_NOALLOC_SCRATCH_BYTES of device memory on every GPU
 *     that loads the library, from load until the process exits.
 *
 * Sharing
 *   Every call on a device uses the same array, and the array keeps what the
 *   last call left in it.  Each call therefore clears the arrival counters (a
 *   stream-ordered memset) before its kernel; the partial tiles need no
 *   clearing because every element read was written by the same call.  Two
 *   calls whose kernels overlap on the GPU (different streams, or the same
 *   call from two host threads) race on the array and give wrong results:
 *   keep calls on one device on one stream, or order them with events.
 *
 * Set-up
 *   The first call on a device looks up the array's device address
 *   (cudaGetSymbolAddress, with that device current), raises the kernel's
 *   shared-memory limit and resolves the driver's tensor-map encoder.  Make
 *   that first call before any stream capture.  Later calls do no set-up.
 *
 * The call returns 0, or a negative code after recording a message.
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FB_NOALLOC_MAX_ROWS 64
#define FB_NOALLOC_MAX_TILES 4096
#define FB_NOALLOC_PARTIAL_BYTES (24u << 20)
#define FB_NOALLOC_SCRATCH_BYTES (FB_NOALLOC_PARTIAL_BYTES + FB_NOALLOC_MAX_TILES * 4u)

/* out[M,N] = X[M,K] * W[N,K]^T; X and W bfloat16 with row strides lda, ldw in elements (multiples of 8,
 * 16-byte aligned bases); out float32 (o_dtype 0) or bfloat16 (o_dtype 1) with row stride ldo; `status` is
 * a device int that receives fault bits (a bounded wait that ran out); all pointers are device pointers of
 * the current device; the work is queued on `stream`. */
__attribute__((visibility("default")))
int fb_gemm_tc_noalloc(const void* X, long long lda, const void* W, long long ldw, void* out, int o_dtype,
                       long long ldo, int M, int N, int K, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
