// The two-SM form of the tensor-core product (gemm_tc_pair.cu), chosen by the launchers in gemm_tc.cu.
#pragma once

#include "tensor_map.cuh"
#include "common.cuh"

// 0 if the one-SM kernel should take this shape; else the number of shares of K the two-SM kernel would use
// (1 = the whole sum; more only if the caller has that many float32 slabs, max_slabs > 1).
int fb_gemm_pair_plan(int M, int N, int K, int max_slabs);
// out[M,N] (or act(g)*u of alternating features into [M,N/2] when `gated` is an FbAct code) = X[M,K] * W[N,K]^T; with splits > 1
// share s of K goes to out + s * slab_stride (float32) and the caller adds the slabs.  accumulate: the whole float32
// product is added to what `out` holds instead of replacing it.
int fb_launch_gemm_pair(const void* X, long lda, const void* W, long ldw, void* out, int o_dtype, long ldo,
                        long slab_stride, int splits, int M, int N, int K, int gated, int accumulate, int* status,
                        cudaStream_t stream);
