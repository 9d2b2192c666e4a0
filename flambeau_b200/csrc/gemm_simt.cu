// out[M,N] = A[M,K] * W[N,K]^T with float32 FMA accumulation on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores: the
// tensor pipes have no float32 x float32 mode) and the fallback of the
// bfloat16 path for shapes the tensor-core kernel refuses.  Each output
// element sums its K products in ascending k in one thread, so the result of
// a row does not depend on how many rows the call has.
// Weight layout as in the reference: rows = outputs, columns = inputs
// (crates/kernels-hip/src/kernels/mmq_f16_tile.cu:34-39).
#include "common.cuh"

template <typename TA, typename TW, typename TO, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const TA* __restrict__ A, long lda, const TW* __restrict__ W, long ldw,
                 TO* __restrict__ out, long ldo, int M, int N, int K) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = tid; e < BM * BK; e += THREADS) {
            const int row = e / BK, kk = e - row * BK;
            const int m = m0 + row, k = k0 + kk;
            As[kk][row] = (m < M && k < K) ? fb_to_float(A[(size_t)m * lda + k]) : 0.0f;
        }
#pragma unroll
        for (int e = tid; e < BN * BK; e += THREADS) {
            const int row = e / BK, kk = e - row * BK;
            const int n = n0 + row, k = k0 + kk;
            Ws[kk][row] = (n < N && k < K) ? fb_to_float(W[(size_t)n * ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) out[(size_t)m * ldo + n] = fb_from_float<TO>(acc[i][j]);
        }
    }
}

template <typename TA, typename TW, typename TO>
static int launch_gemm_simt(const void* A, long lda, const void* W, long ldw, void* out, long ldo, int M, int N,
                            int K, cudaStream_t stream) {
    if (M >= 256 && N >= 128) {
        constexpr int BM = 128, BN = 128, BK = 8, TM = 8, TN = 8;
        dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
        fb_launch((gemm_simt_kernel<TA, TW, TO, BM, BN, BK, TM, TN>), grid, (BM / TM) * (BN / TN), 0, stream, 
            (const TA*)A, lda, (const TW*)W, ldw, (TO*)out, ldo, M, N, K);
    } else if (M > 16) {
        constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
        dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
        fb_launch((gemm_simt_kernel<TA, TW, TO, BM, BN, BK, TM, TN>), grid, (BM / TM) * (BN / TN), 0, stream, 
            (const TA*)A, lda, (const TW*)W, ldw, (TO*)out, ldo, M, N, K);
    } else {
        constexpr int BM = 16, BN = 64, BK = 32, TM = 2, TN = 2;
        dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
        fb_launch((gemm_simt_kernel<TA, TW, TO, BM, BN, BK, TM, TN>), grid, (BM / TM) * (BN / TN), 0, stream, 
            (const TA*)A, lda, (const TW*)W, ldw, (TO*)out, ldo, M, N, K);
    }
    return fb_check_launch("gemm_simt");
}

FB_API int fb_gemm_simt(const void* A, int a_dtype, long long lda, const void* W, int w_dtype, long long ldw,
                        void* out, int o_dtype, long long ldo, int M, int N, int K, cudaStream_t stream) {
    FB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    FB_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm: a row stride is shorter than its row");
    if (M == 0) return 0;
    FB_REQUIRE((N + 15) / 16 <= 2147483647 && (M + 15) / 16 <= 65535, "gemm: too many rows (M=%d)", M);
    FB_DISPATCH_DTYPE(a_dtype, TA, FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(o_dtype, TO,
        return (launch_gemm_simt<TA, TW, TO>(A, (long)lda, W, (long)ldw, out, (long)ldo, M, N, K, stream)))));
    return 0;
}
