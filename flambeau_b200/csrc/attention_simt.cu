// Paged causal (sliding-window) attention on the CUDA cores, float32 math.
//
// One warp owns one (query row, query head).  It walks the visible keys
// [t0, p] in ascending position, 32 at a time: each lane scores one key
// (dot product over the head), the warp agrees on the running maximum, and
// the lanes then split the head dimensions to accumulate P*V.  Masked keys
// are never touched (crates/kernels-hip/src/kernels/
// attention_prefill_flash_tile_f16.cu:181-200 skips them the same way; the
// online-softmax update is the one of attention_prefill_f16_paged.cu:69-149).
//
// The same kernel serves prompt portions and decoded tokens in one launch: a
// row only needs its position and the block table of its sequence (whose row starts
// at logical page table_base[sequence], or at page 0 without table_base).  It is the
// attention of the true 32-bit path and the reference for the faster kernels.
#include "common.cuh"

template <typename T, int NDR>   // NDR = ceil(head_dim / 32) accumulator registers per lane
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                            const T* __restrict__ k_pool, const T* __restrict__ v_pool, int page_size,
                            int n_pages, const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ table_base,
                            const int* __restrict__ positions, const int* __restrict__ row_seq, int n, int nh,
                            int nkv, int hd, int window, float scale, const float* __restrict__ score_slopes,
                            int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ float q_sh[];                    // [4 warps][hd]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + warp;
    const bool active = item < (long)n * nh;
    const int row = active ? (int)(item / nh) : 0;
    const int head = active ? (int)(item - (long)row * nh) : 0;
    const int kvh = head / (nh / nkv);
    float* qs = q_sh + warp * hd;
    if (active) {
        const T* qp = q + (size_t)row * q_stride + (size_t)head * hd;
        for (int d = lane; d < hd; d += 32) qs[d] = fb_to_float(qp[d]);
    }
    __syncwarp();
    if (!active) return;

    const int p = positions[row];
    const float slope = score_slopes ? score_slopes[head] : 0.0f;
    const int t0 = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int* table = block_table + (size_t)row_seq[row] * table_stride;
    const int base_page = table_base ? table_base[row_seq[row]] : 0;     // the table row starts at this logical page

    float m = -INFINITY, l = 0.0f;
    float acc[NDR];
#pragma unroll
    for (int r = 0; r < NDR; ++r) acc[r] = 0.0f;

    for (int base = t0; base <= p; base += 32) {
        const int t = base + lane;
        const bool valid = t <= p;
        float s = -INFINITY;
        int my_page = -1;
        if (valid) {
            const int entry = t / page_size - base_page;
            my_page = (entry >= 0 && entry < table_stride) ? table[entry] : -1;
            if (my_page < 0 || my_page >= n_pages) {
                atomicOr(status, FB_STATUS_BAD_PAGE);
                my_page = -1;
            } else {
                const T* kr = k_pool + (((size_t)my_page * nkv + kvh) * page_size + (t % page_size)) * hd;
                float dot = 0.0f;
                for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], fb_to_float(kr[d]), dot);
                s = dot * scale + slope * (float)(t - p);
            }
        }
        const float tile_max = fb_warp_max(s);
        if (tile_max == -INFINITY) continue;            // nothing readable in this tile
        const float m_new = fmaxf(m, tile_max);
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        const float pr = (s == -INFINITY) ? 0.0f : expf(s - m_new);
        l = l * corr + fb_warp_sum(pr);
#pragma unroll
        for (int r = 0; r < NDR; ++r) acc[r] *= corr;
        const int count = min(32, p - base + 1);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const int page_j = __shfl_sync(0xffffffffu, my_page, j);
            if (page_j < 0) continue;
            const int tj = base + j;
            const T* vr = v_pool + (((size_t)page_j * nkv + kvh) * page_size + (tj % page_size)) * hd;
#pragma unroll
            for (int r = 0; r < NDR; ++r) {
                const int d = lane + 32 * r;
                if (d < hd) acc[r] = fmaf(pj, fb_to_float(vr[d]), acc[r]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    T* op = out + (size_t)row * out_stride + (size_t)head * hd;
#pragma unroll
    for (int r = 0; r < NDR; ++r) {
        const int d = lane + 32 * r;
        if (d < hd) op[d] = fb_from_float<T>(acc[r] * inv);
    }
}

template <typename T, int NDR>
static int launch_attention_simt(const void* q, long q_stride, void* out, long out_stride, const void* k_pool,
                                 const void* v_pool, int page_size, int n_pages, const int* block_table,
                                 int table_stride, const int* table_base, const int* positions, const int* row_seq,
                                 int n, int nh,
                                 int nkv, int hd, int window, float scale, const float* score_slopes, int* status,
                                 cudaStream_t stream) {
    const long items = (long)n * nh;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    fb_launch((paged_attention_simt_kernel<T, NDR>), blocks, 128, 4 * hd * sizeof(float), stream, 
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pool, (const T*)v_pool, page_size, n_pages,
        block_table, table_stride, table_base, positions, row_seq, n, nh, nkv, hd, window, scale, score_slopes, status);
    return fb_check_launch("paged_attention_simt");
}

FB_API int fb_paged_attention_simt(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                   const void* k_pool, const void* v_pool, int page_size, int n_pages,
                                   const int* block_table, int table_stride, const int* table_base,
                                   const int* positions, const int* row_seq, int n, int nh, int nkv, int hd,
                                   int window, float scale, const float* score_slopes, int* status,
                                   cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && hd > 0, "attention: bad sizes n=%d heads=%d kv=%d hd=%d", n, nh, nkv, hd);
    FB_REQUIRE(nh % nkv == 0, "attention: %d query heads are not a multiple of %d key/value heads", nh, nkv);
    FB_REQUIRE(hd <= 512, "attention: head size %d is larger than 512", hd);
    FB_REQUIRE(page_size > 0 && n_pages > 0 && window >= 0, "attention: bad cache geometry");
    if (n == 0) return 0;
#define FB_ATTN_CASE(NDR)                                                                                      \
    FB_DISPATCH_DTYPE(dtype, T, return (launch_attention_simt<T, NDR>(q, (long)q_stride, out, (long)out_stride,     \
        k_pool, v_pool, page_size, n_pages, block_table, table_stride, table_base, positions, row_seq, n, nh, \
        nkv, hd, window, scale, score_slopes, status, stream)))
    if (hd <= 32) { FB_ATTN_CASE(1); }
    else if (hd <= 64) { FB_ATTN_CASE(2); }
    else if (hd <= 128) { FB_ATTN_CASE(4); }
    else if (hd <= 256) { FB_ATTN_CASE(8); }
    else { FB_ATTN_CASE(16); }
#undef FB_ATTN_CASE
    return 0;
}
