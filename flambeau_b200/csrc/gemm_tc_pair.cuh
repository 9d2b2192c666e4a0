// The two-SM form of the tensor-core product (gemm_tc_pair.cu), chosen by the launchers in gemm_tc.cu.
#pragma once

#include "tensor_map.cuh"
#include "common.cuh"

// Pairs of SMs that run at a time.
int fb_gemm_pair_slots();
// Whether the two-SM kernel is the better choice for this shape (hundreds of rows, enough tiles for every pair).
bool fb_gemm_pair_takes(int M, int N, int K);
// out[M,N] (or silu(g)*u of alternating features into [M,N/2] when gated) = X[M,K] * W[N,K]^T, the whole sum.
int fb_launch_gemm_pair(const void* X, long lda, const void* W, long ldw, void* out, int o_dtype, long ldo, int M,
                        int N, int K, int gated, int* status, cudaStream_t stream);
