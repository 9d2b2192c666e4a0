// What the tensor pipe of one SM takes per tcgen05.mma (M = 128, bfloat16, accumulator in tensor memory) when one
// thread issues them back to back, and what commits and mbarrier waits in that thread's stream add: the figures the
// loops of the MMA-issuing warps in attention_tc.cu and gemm_tc*.cu were laid out by.  A program of its own (one CTA,
// operands and tensor memory initialised, every wait bounded); prints a table of cycles per instruction.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I flambeau_b200/csrc -o mma_issue_rate \
//        flambeau_b200/csrc/probes/mma_issue_rate.cu && ./mma_issue_rate
#include <cstdio>
#include <cuda_runtime.h>

#include "umma.cuh"

namespace {

constexpr int PATTERNS = 9;
const char* const NAMES[PATTERNS] = {
    "S-shaped, N = 64 (A, B from shared memory, one accumulator)",
    "S-shaped, N = 128",
    "S-shaped, N = 256",
    "PV-shaped, N = 128 (A from tensor memory, B MN-major)",
    "attention key tile: 2 x (4 PV + 8 S of N = 64)",
    "... with commits at 4 points of the tile",
    "... with commits at 4 points and 6 waits (flag + try_wait)",
    "... with 1 wait and 3 commits at 1 point",
    "key tile of 128: 2 x (1 wait, 8 PV + 8 S of N = 128, 2 commits)",
};

__global__ void __launch_bounds__(128, 1) rate_kernel(long long* out, int* status, int reps) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    __shared__ uint64_t bar, passed, dummy[3];
    __shared__ uint32_t slot;
    __shared__ int flag;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < 192 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x3f803f80u;   // bf16 1.0
    if (tid == 0) {
        flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_init(smem_u32(&passed), 1);          // never arrived on: a wait for parity 1 passes at once
        for (int i = 0; i < 3; ++i) mbar_init(smem_u32(&dummy[i]), 1 << 20);   // commits land here; nobody waits
        mbar_fence_init();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) tmem_alloc(&slot, 512);
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tm = slot;
    {   // every thread fills its lane of tensor memory (values that are neither denormal nor NaN as bf16 or f32)
        uint32_t z[32];
        for (int i = 0; i < 32; ++i) z[i] = 0x3c003c00u;
        for (int c = 0; c < 512; c += 32) tmem_st32(tm + ((uint32_t)(warp * 32) << 16) + c, z);
        tmem_wait_st();
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    if (tid == 32) {
        const uint32_t A = smem_u32(smem), B = smem_u32(smem + 64 * 1024), V = smem_u32(smem + 128 * 1024);
        auto s_mma = [&](int t, int kk, int n, int acc) {     // row tile t, K step kk of 8, N columns
            umma_bf16(tm + t * 128, umma_desc(A + t * 32768 + (kk / 4) * 16384 + (kk % 4) * 32),
                      umma_desc(B + (kk / 4) * (n * 128) + (kk % 4) * 32), umma_idesc(n), acc);
        };
        auto pv_mma = [&](int t, int kk, int keys) {          // 16 keys of a V tile of `keys` keys
            umma_bf16_ts(tm + 256 + t * 128, tm + t * 128 + kk * 8, umma_desc_mn(V + kk * 16 * 128, keys * 128, 1024),
                         umma_idesc(128, true), 1);
        };
        auto wait_passed = [&](bool with_flag) {
            if (with_flag && *(volatile int*)&flag) return;
            mbar_wait(smem_u32(&passed), 1, status);
        };
        uint32_t phase = 0;
        for (int pat = 0; pat < PATTERNS; ++pat) {
            const long long t0 = clock64();
            int n = 0;
            for (int r = 0; r < reps; ++r) {
                if (pat <= 2) {
                    for (int kk = 0; kk < 8; ++kk, ++n) s_mma(0, kk, 64 << pat, 1);
                } else if (pat == 3) {
                    for (int kk = 0; kk < 8; ++kk, ++n) pv_mma(0, kk, 128);
                } else if (pat <= 6) {
                    for (int t = 0; t < 2; ++t) {
                        if (pat == 6) { wait_passed(true); wait_passed(true); tmem_fence_after(); }
                        for (int kk = 0; kk < 4; ++kk, ++n) pv_mma(t, kk, 64);
                        if (pat >= 5) { umma_commit(smem_u32(&dummy[0])); umma_commit(smem_u32(&dummy[1])); }
                        if (pat == 6) { wait_passed(true); tmem_fence_after(); }
                        for (int kk = 0; kk < 8; ++kk, ++n) s_mma(t, kk, 64, kk > 0);
                        if (pat >= 5) { umma_commit(smem_u32(&dummy[2])); umma_commit(smem_u32(&dummy[1])); }
                    }
                } else if (pat == 7) {
                    wait_passed(false);
                    tmem_fence_after();
                    for (int t = 0; t < 2; ++t)
                        for (int kk = 0; kk < 4; ++kk, ++n) pv_mma(t, kk, 64);
                    for (int t = 0; t < 2; ++t)
                        for (int kk = 0; kk < 8; ++kk, ++n) s_mma(t, kk, 64, kk > 0);
                    for (int i = 0; i < 3; ++i) umma_commit(smem_u32(&dummy[i]));
                } else {
                    for (int t = 0; t < 2; ++t) {
                        wait_passed(false);
                        tmem_fence_after();
                        for (int kk = 0; kk < 8; ++kk, ++n) pv_mma(t, kk, 128);
                        for (int kk = 0; kk < 8; ++kk, ++n) s_mma(t, kk, 128, kk > 0);
                        umma_commit(smem_u32(&dummy[0]));
                        umma_commit(smem_u32(&dummy[1]));
                    }
                }
            }
            const long long t_issued = clock64();
            umma_commit(smem_u32(&bar));
            mbar_wait(smem_u32(&bar), phase, status);
            phase ^= 1;
            const long long t1 = clock64();
            out[3 * pat] = t1 - t0;
            out[3 * pat + 1] = n;
            out[3 * pat + 2] = t_issued - t0;
        }
    }
    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        tmem_dealloc(tm, 512);
    }
}

}  // namespace

int main() {
    long long* out;
    int* status;
    if (cudaMalloc(&out, 3 * PATTERNS * sizeof(long long)) != cudaSuccess || cudaMalloc(&status, 16) != cudaSuccess) {
        fprintf(stderr, "mma_issue_rate: no CUDA device\n");
        return 1;
    }
    cudaMemset(out, 0, 3 * PATTERNS * sizeof(long long));
    cudaMemset(status, 0, 16);
    cudaFuncSetAttribute(rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    for (int rep = 0; rep < 2; ++rep) rate_kernel<<<1, 128, 200 * 1024>>>(out, status, 32);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h[3 * PATTERNS];
    int st[4];
    cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
    cudaMemcpy(st, status, 16, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess || st[0] != 0) {
        fprintf(stderr, "mma_issue_rate: %s, status word %d\n", cudaGetErrorString(e), st[0]);
        return 1;
    }
    printf("%-64s %10s %8s %12s %12s\n", "instruction stream", "cycles", "MMAs", "cycles each", "issue each");
    for (int p = 0; p < PATTERNS; ++p)
        printf("%-64s %10lld %8lld %12.1f %12.1f\n", NAMES[p], h[3 * p], h[3 * p + 1], (double)h[3 * p] / (double)h[3 * p + 1],
               (double)h[3 * p + 2] / (double)h[3 * p + 1]);
    return 0;
}
