// Row-wise kernels between the matrix products: embedding gather, fused
// residual add + RMSNorm, rotary tables, rotary + paged cache write, act(gate)*up.
// All arithmetic is float32 whatever the storage type; the residual stream
// itself is float32 in both engine modes.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: x[t,:] = E[ids[t],:]  (crates/forward/src/core/composites/embed.rs:26-62)
// ---------------------------------------------------------------------------
template <typename TT>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ x, int H, int V, int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(status, FB_STATUS_BAD_TOKEN);
        id = 0;
    }
    const TT* src = table + (size_t)id * H;
    float* dst = x + (size_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = fb_to_float(src[c]);
}

FB_API int fb_embedding(const void* table, int table_dtype, const int* ids, float* x, int n, int H,
                        int V, int* status, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && H > 0 && V > 0, "embedding: bad sizes n=%d H=%d V=%d", n, H, V);
    if (n == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    FB_DISPATCH_DTYPE(table_dtype, TT,
        fb_launch((embedding_kernel<TT>), n, threads, 0, stream, (const TT*)table, ids, x, H, V, status));
    return fb_check_launch("embedding");
}

// ---------------------------------------------------------------------------
// Fused residual add + RMSNorm.
//   r = rows ? rows[j] : j
//   v = x[r] + sum_p delta[p][r]        (delta optional; n_partials slabs, slab stride given)
//   if (!rows && delta) x[r] = v        (the stream is updated in place)
//   out[j] = v * (w + w_offset) / sqrt(mean(v^2) + eps)      (w_offset 0 for a plain weight, 1 for a "1 + w" norm)
// crates/kernels-hip/src/kernels/rmsnorm_f16_add_residual.cu; rmsnorm_f16.cu:41-85.
// The row lives in shared memory between the two passes.
// ---------------------------------------------------------------------------
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_partials,
                                   size_t partial_stride, const TW* __restrict__ w,
                                   TO* __restrict__ out, const int* __restrict__ rows, int H, float eps,
                                   float w_offset) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ float row[];
    __shared__ float red[32];
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    float* xr = x + (size_t)r * H;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (delta) {
            for (int p = 0; p < n_partials; ++p)
                v += fb_to_float(delta[(size_t)p * partial_stride + (size_t)r * H + c]);
            if (!rows) xr[c] = v;
        }
        row[c] = v;
        ss += v * v;
    }
    ss = fb_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)j * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        o[c] = fb_from_float<TO>(row[c] * (fb_to_float(w[c]) + w_offset) * inv);
}

// Fast path: width a multiple of 4 and at most 4 * VPT * blockDim: every thread keeps its part of the row in
// registers and issues all of its loads before the first use, so a row costs one round trip to memory.
template <typename T> struct Vec4 {};
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TD, typename TW, typename TO, int VPT>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_partials,
                                       size_t partial_stride, const TW* __restrict__ w, TO* __restrict__ out,
                                       const int* __restrict__ rows, int H, float eps, float w_offset) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    __shared__ float red[32];
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    float* xr = x + (size_t)r * H;
    const int nvec = H >> 2;
    float4 v[VPT], wv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nvec) {
            v[i] = Vec4<float>::load(xr + 4 * c);
            wv[i] = Vec4<TW>::load(w + 4 * c);
            wv[i].x += w_offset; wv[i].y += w_offset; wv[i].z += w_offset; wv[i].w += w_offset;
        } else {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            wv[i] = v[i];
        }
    }
    if (delta) {
        // the slabs are independent loads: issue them four slabs at a time, add in slab order
        for (int p0 = 0; p0 < n_partials; p0 += 4) {
            float4 d[4][VPT];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const TD* dp = delta + (size_t)(p0 + q) * partial_stride + (size_t)r * H;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int c = threadIdx.x + i * blockDim.x;
                    d[q][i] = (p0 + q < n_partials && c < nvec) ? Vec4<TD>::load(dp + 4 * c)
                                                                : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    v[i].x += d[q][i].x; v[i].y += d[q][i].y; v[i].z += d[q][i].z; v[i].w += d[q][i].w;
                }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    if (delta && !rows) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < nvec) Vec4<float>::store(xr + 4 * c, v[i]);
        }
    }
    ss = fb_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)j * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nvec)
            Vec4<TO>::store(o + 4 * c, make_float4(v[i].x * wv[i].x * inv, v[i].y * wv[i].y * inv,
                                                   v[i].z * wv[i].z * inv, v[i].w * wv[i].w * inv));
    }
}

// Many rows with one delta each, or with none (a prompt's portion): R rows per CTA and V vectors per thread and row,
// every load of the CTA's rows issued before the first use.  One row per CTA leaves too few loads in flight to fill
// the memory pipe when each thread has only one vector of the row.  Without a delta (the stream already holds the
// sum) nothing is written back to the stream.
template <typename TD, typename TW, typename TO, int R, int V, bool HAS_DELTA>
__global__ void __launch_bounds__(1024)
add_rmsnorm_rows_kernel(float* __restrict__ x, const TD* __restrict__ delta, const TW* __restrict__ w,
                        TO* __restrict__ out, int n, int H, float eps, float w_offset) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    __shared__ float red[R][32];
    const int r0 = R * blockIdx.x;
    float4 a[R][V], d[R][V], wv[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        wv[v] = Vec4<TW>::load(w + 4 * (threadIdx.x + v * blockDim.x));
        wv[v].x += w_offset; wv[v].y += w_offset; wv[v].z += w_offset; wv[v].w += w_offset;
    }
#pragma unroll
    for (int r = 0; r < R; ++r)                     // a row past the end reads the last row again and stores nothing
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const size_t at = (size_t)min(r0 + r, n - 1) * H + 4 * (threadIdx.x + v * blockDim.x);
            a[r][v] = Vec4<float>::load(x + at);
            if (HAS_DELTA) d[r][v] = Vec4<TD>::load(delta + at);
        }
    if (HAS_DELTA) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int v = 0; v < V; ++v) {
                a[r][v].x += d[r][v].x; a[r][v].y += d[r][v].y; a[r][v].z += d[r][v].z; a[r][v].w += d[r][v].w;
                if (r0 + r < n) Vec4<float>::store(x + (size_t)(r0 + r) * H + 4 * (threadIdx.x + v * blockDim.x), a[r][v]);
            }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float s = 0.0f;
#pragma unroll
        for (int v = 0; v < V; ++v)
            s += a[r][v].x * a[r][v].x + a[r][v].y * a[r][v].y + a[r][v].z * a[r][v].z + a[r][v].w * a[r][v].w;
        s = fb_warp_sum(s);
        if (lane == 0) red[r][warp] = s;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float s = lane < nw ? red[r][lane] : 0.0f;
        ss[r] = fb_warp_sum(s);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (r0 + r >= n) break;
        const float inv = 1.0f / sqrtf(ss[r] / (float)H + eps);
#pragma unroll
        for (int v = 0; v < V; ++v)
            Vec4<TO>::store(out + (size_t)(r0 + r) * H + 4 * (threadIdx.x + v * blockDim.x),
                            make_float4(a[r][v].x * wv[v].x * inv, a[r][v].y * wv[v].y * inv,
                                        a[r][v].z * wv[v].z * inv, a[r][v].w * wv[v].w * inv));
    }
}

template <typename TD, typename TW, typename TO>
static int launch_add_rmsnorm(float* x, const void* delta, int n_partials, size_t partial_stride,
                              const void* w, void* out, const int* rows, int n_out, int H, float eps,
                              float w_offset, cudaStream_t stream) {
    const bool aligned = H % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                         ((uintptr_t)out % 16 == 0) && (!delta || ((uintptr_t)delta % 16 == 0 && partial_stride % 4 == 0));
    const int nvec4 = H / 4, per_thread = (nvec4 + 1023) / 1024;
    if (aligned && !rows && (delta ? n_partials == 1 : true) && n_out > 256 && per_thread <= 2 &&
        nvec4 % (32 * per_thread) == 0) {
        const int threads = nvec4 / per_thread;
#define FB_NORM_ROWS(R_, V_)                                                                                  \
        do {                                                                                                  \
            if (delta)                                                                                        \
                fb_launch((add_rmsnorm_rows_kernel<TD, TW, TO, R_, V_, true>), (n_out + R_ - 1) / R_, threads, 0, \
                          stream, x, (const TD*)delta, (const TW*)w, (TO*)out, n_out, H, eps, w_offset);      \
            else                                                                                              \
                fb_launch((add_rmsnorm_rows_kernel<TD, TW, TO, R_, V_, false>), (n_out + R_ - 1) / R_, threads, 0, \
                          stream, x, (const TD*)delta, (const TW*)w, (TO*)out, n_out, H, eps, w_offset);      \
        } while (0)
        if (!delta && nvec4 >= 512 && nvec4 % 128 == 0) {
            // Nothing to add: half the loads a row, and CTAs of a quarter of the threads with four vectors each keep
            // more of them in flight (2,048 x 4,096: 8.6 us against 11.8 us with 1,024 threads a row).
            fb_launch((add_rmsnorm_rows_kernel<TD, TW, TO, 2, 4, false>), (n_out + 1) / 2, nvec4 / 4, 0, stream, x,
                      (const TD*)delta, (const TW*)w, (TO*)out, n_out, H, eps, w_offset);
            return fb_check_launch("add_rmsnorm");
        }
        if (per_thread == 2) FB_NORM_ROWS(1, 2); else if (nvec4 <= 256) FB_NORM_ROWS(4, 1); else FB_NORM_ROWS(2, 1);
#undef FB_NORM_ROWS
        return fb_check_launch("add_rmsnorm");
    }
    if (aligned && H <= 16384) {
        const int nvec = H / 4;
        int threads = nvec >= 1024 ? 1024 : ((nvec + 31) / 32) * 32;
        // hundreds of rows (a portion whose product left shares of K): a quarter of the threads with four vectors
        // each, as for the rows kernel above; a few rows (decoding) keep one vector a thread
        if (n_out >= 128 && nvec >= 512 && nvec <= 4096 && nvec % 128 == 0) threads = nvec / 4;
        const int vpt = (nvec + threads - 1) / threads;
#define FB_NORM_VEC(V)                                                                                        \
        fb_launch((add_rmsnorm_vec_kernel<TD, TW, TO, V>), n_out, threads, 0, stream, x, (const TD*)delta, n_partials,  \
            partial_stride, (const TW*)w, (TO*)out, rows, H, eps, w_offset)
        if (vpt == 1) FB_NORM_VEC(1); else if (vpt == 2) FB_NORM_VEC(2); else FB_NORM_VEC(4);
#undef FB_NORM_VEC
        return fb_check_launch("add_rmsnorm");
    }
    const size_t smem = (size_t)H * sizeof(float);
    auto kern = add_rmsnorm_kernel<TD, TW, TO>;
    if (smem > 48 * 1024) {
        if (smem > 220 * 1024) return fb_fail(-1, "add_rmsnorm: width %d does not fit in shared memory", H);
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    fb_launch((kern), n_out, threads, smem, stream, x, (const TD*)delta, n_partials, partial_stride, (const TW*)w,
                                           (TO*)out, rows, H, eps, w_offset);
    return fb_check_launch("add_rmsnorm");
}

FB_API int fb_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_partials,
                          long long partial_stride, const void* w, int w_dtype, void* out, int out_dtype,
                          const int* rows, int n_out, int H, float eps, float w_offset, cudaStream_t stream) {
    FB_REQUIRE(n_out >= 0 && H > 0, "add_rmsnorm: bad sizes n=%d H=%d", n_out, H);
    FB_REQUIRE(eps > 0.0f, "add_rmsnorm: eps must be positive");
    if (n_out == 0) return 0;
    if (!delta) { delta_dtype = FB_F32; n_partials = 0; }
    FB_DISPATCH_DTYPE(delta_dtype, TD, FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, TO,
        return (launch_add_rmsnorm<TD, TW, TO>(x, delta, n_partials, (size_t)partial_stride, w, out, rows,
                                               n_out, H, eps, w_offset, stream)))));
    return 0;
}

// ---------------------------------------------------------------------------
// Rotary tables for one step: cos/sin [n, half] of pos * inv_freq[i].
// The angle is formed and reduced in double precision so that it is right to
// float32 rounding at any position; the tables are float32.
// Formula: crates/kernels-hip/src/kernels/rope_neox_partial_f16.cu:39-46.
// ---------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t, int n, int half) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * half) return;
    const int t = idx / half, i = idx - t * half;
    double s, c;
    sincos((double)positions[t] * inv_freq[i], &s, &c);
    cos_t[idx] = (float)c;
    sin_t[idx] = (float)s;
}

FB_API int fb_rope_table(const int* positions, const double* inv_freq, float* cos_t, float* sin_t, int n,
                         int half, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && half > 0, "rope_table: bad sizes n=%d half=%d", n, half);
    if (n == 0) return 0;
    const int total = n * half;
    fb_launch((rope_table_kernel), (total + 255) / 256, 256, 0, stream, positions, inv_freq, cos_t, sin_t, n, half);
    return fb_check_launch("rope_table");
}

// ---------------------------------------------------------------------------
// Rotary (split-half pairs (i, i+half)) on q in place and on k on its way into
// the cache; v is copied into the cache.  One block per token.
// Cache layout: [page][kv head][slot in page][head_dim]; the physical page of
// logical position p of sequence s is block_table[s*table_stride + p/page_size - table_base[s]]: a table row
// starts at the sequence's first live page (table_base == nullptr: at page 0).
// crates/kernels-hip/src/kernels/rope_neox_partial_f16.cu:39-52 (rotation),
// kv_append_f16_paged_prefill.cu (row placement).
// ---------------------------------------------------------------------------
// Element j of a row that is stored as `n_partials` slabs `partial_stride` elements apart (split-K shares).
template <typename TI>
__device__ __forceinline__ float slab_sum(const TI* __restrict__ row, int j, int n_partials, long partial_stride) {
    float acc = fb_to_float(row[j]);
    for (int p = 1; p < n_partials; p += 8) {         // eight independent loads in flight, added in slab order
        float a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            a[u] = p + u < n_partials ? fb_to_float(row[(size_t)(p + u) * partial_stride + j]) : 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += a[u];
    }
    return acc;
}

template <typename TI, typename T>
__global__ void rope_kv_write_kernel(const TI* __restrict__ q_in, long q_in_stride, int n_partials,
                                     long partial_stride, T* __restrict__ q_out,
                                     long q_out_stride, const TI* __restrict__ k, long k_stride,
                                     const TI* __restrict__ v, long v_stride, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, int half,
                                     const int* __restrict__ positions, const int* __restrict__ row_seq,
                                     const int* __restrict__ block_table, int table_stride,
                                     const int* __restrict__ table_base,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool, int page_size, int n_pages,
                                     int nh, int nkv, int hd, int write_kv, int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    // grid (tokens, nh + nkv): blocks y < nh rotate one query head; the others rotate one key head into the
    // cache and copy the value head beside it.
    const int t = blockIdx.x, hy = blockIdx.y;
    const int per_head = hd - half;                 // `half` rotated pairs + (hd - 2*half) untouched dims
    const float* ct = cos_t ? cos_t + (size_t)t * half : nullptr;
    const float* st = sin_t ? sin_t + (size_t)t * half : nullptr;
    if (hy < nh) {
        // q_out may be q_in itself: a thread reads both halves of its pair before it writes them
        const TI* src = q_in + (size_t)t * q_in_stride + (size_t)hy * hd;
        T* dst = q_out + (size_t)t * q_out_stride + (size_t)hy * hd;
        for (int j = threadIdx.x; j < per_head; j += blockDim.x) {
            if (j < half) {
                const float a = slab_sum(src, j, n_partials, partial_stride), b = slab_sum(src, j + half, n_partials, partial_stride);
                const float c = ct[j], s = st[j];
                dst[j] = fb_from_float<T>(a * c - b * s);
                dst[j + half] = fb_from_float<T>(a * s + b * c);
            } else {
                dst[j + half] = fb_from_float<T>(slab_sum(src, j + half, n_partials, partial_stride));
            }
        }
        return;
    }
    if (!write_kv) return;
    const int h = hy - nh;
    const int pos = positions[t];
    const int seq = row_seq[t];
    const int entry = pos / page_size - (table_base ? table_base[seq] : 0);
    const int page = (entry >= 0 && entry < table_stride) ? block_table[(size_t)seq * table_stride + entry] : -1;
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0) atomicOr(status, FB_STATUS_BAD_PAGE);
        return;
    }
    const int slot = pos % page_size;
    const TI* ksrc = k + (size_t)t * k_stride + (size_t)h * hd;
    const TI* vsrc = v + (size_t)t * v_stride + (size_t)h * hd;
    const size_t base = (((size_t)page * nkv + h) * page_size + slot) * hd;
    T* kdst = k_pool + base;
    T* vdst = v_pool + base;
    for (int j = threadIdx.x; j < per_head; j += blockDim.x) {
        if (j < half) {
            const float a = slab_sum(ksrc, j, n_partials, partial_stride), b = slab_sum(ksrc, j + half, n_partials, partial_stride);
            const float c = ct[j], s = st[j];
            kdst[j] = fb_from_float<T>(a * c - b * s);
            kdst[j + half] = fb_from_float<T>(a * s + b * c);
        } else {
            kdst[j + half] = fb_from_float<T>(slab_sum(ksrc, j + half, n_partials, partial_stride));
        }
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) vdst[d] = fb_from_float<T>(slab_sum(vsrc, d, n_partials, partial_stride));
}

// The same work four elements at a time (all strides, the head size and the rotary half multiples of 4,
// 16-byte aligned rows): one item = four consecutive pairs of one head, or four untouched dimensions, or four
// values.  Items of a token: (nh + nkv) * (hd - half) / 4 rotary items, then nkv * hd / 4 value items.
template <typename TI>
__device__ __forceinline__ float4 slab_sum4(const TI* __restrict__ p, int n_partials, long partial_stride) {
    float4 acc = Vec4<TI>::load(p);
    for (int s = 1; s < n_partials; s += 8) {         // eight independent loads in flight, added in slab order
        float4 a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            a[u] = s + u < n_partials ? Vec4<TI>::load(p + (size_t)(s + u) * partial_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) { acc.x += a[u].x; acc.y += a[u].y; acc.z += a[u].z; acc.w += a[u].w; }
    }
    return acc;
}

// TOK tokens per thread (the same item of each): every load of the thread's tokens is issued before the first
// use, which is what fills the memory pipe when a prompt's portion brings thousands of tokens.  A token past the
// end reads the last token again and stores nothing.
template <typename TI, typename T, int TOK>
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(const TI* __restrict__ q_in, long q_in_stride, int n_partials, long partial_stride,
                         T* __restrict__ q_out, long q_out_stride, const TI* __restrict__ k, long k_stride,
                         const TI* __restrict__ v, long v_stride, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, int half, const int* __restrict__ positions,
                         const int* __restrict__ row_seq, const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ table_base, T* __restrict__ k_pool, T* __restrict__ v_pool,
                         int page_size, int n_pages, int n, int nh, int nkv, int hd, int write_kv, int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int t0 = blockIdx.x * TOK;
    const int per_head = (hd - half) >> 2;                  // items per head
    const int rot_items = half >> 2;
    const int q_items = nh * per_head, k_items = write_kv ? nkv * per_head : 0;
    const int v_items = write_kv ? nkv * (hd >> 2) : 0;
    const int item = blockIdx.y * blockDim.x + threadIdx.x;
    if (item >= q_items + k_items + v_items) return;

    int tok[TOK];
    bool live[TOK];
    size_t cache_row[TOK];
#pragma unroll
    for (int i = 0; i < TOK; ++i) {
        live[i] = t0 + i < n;
        tok[i] = min(t0 + i, n - 1);
        cache_row[i] = 0;
    }
    if (item >= q_items) {
        int pos[TOK], page[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i) pos[i] = positions[tok[i]];
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            const int seq = row_seq[tok[i]];
            const int entry = pos[i] / page_size - (table_base ? table_base[seq] : 0);
            page[i] = (entry >= 0 && entry < table_stride) ? block_table[(size_t)seq * table_stride + entry] : -1;
        }
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            if (page[i] < 0 || page[i] >= n_pages) {
                if (live[i]) atomicOr(status, FB_STATUS_BAD_PAGE);
                live[i] = false;
                page[i] = 0;
            }
            cache_row[i] = ((size_t)page[i] * nkv) * page_size + (pos[i] % page_size);   // + head * page_size below
        }
    }
    if (item >= q_items + k_items) {
        const int idx = item - q_items - k_items;
        const int h = idx / (hd >> 2), d = (idx - h * (hd >> 2)) << 2;
        float4 val[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i)
            val[i] = slab_sum4(v + (size_t)tok[i] * v_stride + (size_t)h * hd + d, n_partials, partial_stride);
#pragma unroll
        for (int i = 0; i < TOK; ++i)
            if (live[i]) Vec4<T>::store(v_pool + (cache_row[i] + (size_t)h * page_size) * hd + d, val[i]);
        return;
    }
    const bool is_q = item < q_items;
    const int idx = is_q ? item : item - q_items;
    const int h = idx / per_head, j = idx - h * per_head;
    const TI* src = is_q ? q_in + (size_t)h * hd : k + (size_t)h * hd;
    const long src_stride = is_q ? q_in_stride : k_stride;
    if (j < rot_items) {
        const int d = j << 2;
        float4 a[TOK], b[TOK], c[TOK], sn[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            const TI* row = src + (size_t)tok[i] * src_stride;
            a[i] = slab_sum4(row + d, n_partials, partial_stride);
            b[i] = slab_sum4(row + d + half, n_partials, partial_stride);
            c[i] = *reinterpret_cast<const float4*>(cos_t + (size_t)tok[i] * half + d);
            sn[i] = *reinterpret_cast<const float4*>(sin_t + (size_t)tok[i] * half + d);
        }
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            if (!live[i]) continue;
            T* dst = is_q ? q_out + (size_t)tok[i] * q_out_stride + (size_t)h * hd
                          : k_pool + (cache_row[i] + (size_t)h * page_size) * hd;
            Vec4<T>::store(dst + d, make_float4(a[i].x * c[i].x - b[i].x * sn[i].x, a[i].y * c[i].y - b[i].y * sn[i].y,
                                                a[i].z * c[i].z - b[i].z * sn[i].z, a[i].w * c[i].w - b[i].w * sn[i].w));
            Vec4<T>::store(dst + d + half,
                           make_float4(a[i].x * sn[i].x + b[i].x * c[i].x, a[i].y * sn[i].y + b[i].y * c[i].y,
                                       a[i].z * sn[i].z + b[i].z * c[i].z, a[i].w * sn[i].w + b[i].w * c[i].w));
        }
    } else {
        const int d = 2 * half + ((j - rot_items) << 2);     // untouched dimensions behind the rotary part
        float4 val[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i) val[i] = slab_sum4(src + (size_t)tok[i] * src_stride + d, n_partials, partial_stride);
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            if (!live[i]) continue;
            T* dst = is_q ? q_out + (size_t)tok[i] * q_out_stride + (size_t)h * hd
                          : k_pool + (cache_row[i] + (size_t)h * page_size) * hd;
            Vec4<T>::store(dst + d, val[i]);
        }
    }
}

// q_in/k/v have dtype `in_dtype` (the projection's output, float32 in both engine modes so that q and k are
// rounded once, after the rotation); q_out and the cache have dtype `out_dtype`.  The inputs may be split-K
// shares: `n_partials` slabs `partial_stride` elements apart, which are added here.
FB_API int fb_rope_kv_write(const void* q_in, long long q_in_stride, int n_partials, long long partial_stride,
                            void* q_out, long long q_out_stride,
                            const void* k, long long k_stride, const void* v, long long v_stride, int in_dtype,
                            int out_dtype, const float* cos_t, const float* sin_t, int half,
                            const int* positions, const int* row_seq, const int* block_table,
                            int table_stride, const int* table_base, void* k_pool, void* v_pool, int page_size,
                            int n_pages, int n,
                            int nh, int nkv, int hd, int write_kv, int* status, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && nh > 0 && nkv >= 0 && hd > 0, "rope_kv_write: bad sizes");
    FB_REQUIRE(half >= 0 && 2 * half <= hd, "rope_kv_write: rotary width %d exceeds head size %d", 2 * half, hd);
    FB_REQUIRE(half == 0 || (cos_t && sin_t), "rope_kv_write: rotary tables missing");
    FB_REQUIRE(!write_kv || (page_size > 0 && n_pages > 0 && k_pool && v_pool && block_table),
               "rope_kv_write: cache arguments missing");
    FB_REQUIRE(q_in != q_out || (in_dtype == out_dtype && n_partials <= 1),
               "rope_kv_write: in-place rotation needs one dtype and one slab");
    if (n_partials < 1) n_partials = 1;
    if (n == 0) return 0;
    FB_REQUIRE(nh + nkv <= 65535, "rope_kv_write: too many heads");
    const bool aligned16 = ((uintptr_t)q_in % 16 == 0) && ((uintptr_t)q_out % 16 == 0) && ((uintptr_t)k % 16 == 0) &&
                           ((uintptr_t)v % 16 == 0) && ((uintptr_t)cos_t % 16 == 0) && ((uintptr_t)sin_t % 16 == 0) &&
                           ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0);
    const bool vec = aligned16 && hd % 4 == 0 && half % 4 == 0 && q_in_stride % 4 == 0 && q_out_stride % 4 == 0 &&
                     k_stride % 4 == 0 && v_stride % 4 == 0 && partial_stride % 4 == 0 && q_in != q_out;
    if (vec) {
        const int items = (nh + (write_kv ? nkv : 0)) * ((hd - half) / 4) + (write_kv ? nkv * (hd / 4) : 0);
        const int per = n >= 1024 ? 2 : 1;             // tokens per thread
#define FB_ROPE_VEC(TOK_)                                                                                     \
        FB_DISPATCH_DTYPE(in_dtype, TI, FB_DISPATCH_DTYPE(out_dtype, T,                                       \
            (fb_launch((rope_kv_write_vec_kernel<TI, T, TOK_>), dim3((n + TOK_ - 1) / TOK_, (items + 255) / 256), 256, \
                0, stream, (const TI*)q_in, (long)q_in_stride, n_partials, (long)partial_stride, (T*)q_out,   \
                (long)q_out_stride, (const TI*)k, (long)k_stride, (const TI*)v, (long)v_stride, cos_t, sin_t, \
                half, positions, row_seq, block_table, table_stride, table_base, (T*)k_pool, (T*)v_pool,      \
                page_size, n_pages, n, nh, nkv, hd, write_kv, status))))
        if (per == 2) FB_ROPE_VEC(2); else FB_ROPE_VEC(1);
#undef FB_ROPE_VEC
        return fb_check_launch("rope_kv_write");
    }
    FB_DISPATCH_DTYPE(in_dtype, TI, FB_DISPATCH_DTYPE(out_dtype, T,
        (fb_launch((rope_kv_write_kernel<TI, T>), dim3(n, nh + (write_kv ? nkv : 0)), hd >= 128 ? 64 : 32, 0, stream, (const TI*)q_in, q_in_stride, n_partials, (long)partial_stride, (T*)q_out, q_out_stride,
            (const TI*)k, k_stride, (const TI*)v, v_stride, cos_t, sin_t, half, positions, row_seq, block_table,
            table_stride, table_base, (T*)k_pool, (T*)v_pool, page_size, n_pages, nh, nkv, hd, write_kv, status))));
    return fb_check_launch("rope_kv_write");
}

// ---------------------------------------------------------------------------
// act(gate) * up on a fused [n, 2I] buffer whose columns alternate: column 2c is gate c, column 2c+1 is up c
// (the feed-forward stacks its gate and up weights row by row in that order, so that the tensor-core product
// can apply the activation in its epilogue with a neighbour exchange; this kernel serves the other paths).
// crates/kernels-hip/src/kernels/swiglu_f32_to_f16.cu; activation.rs:107-118.
// ---------------------------------------------------------------------------
template <typename TI, typename T>
__global__ void gate_mul_kernel(const TI* __restrict__ gu, long stride, int n_partials, long partial_stride,
                                T* __restrict__ out, int n, int I, int act) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * I) return;
    const int r = (int)(idx / I), c = (int)(idx - (size_t)r * I);
    const TI* row = gu + (size_t)r * stride;
    const float g = slab_sum(row, 2 * c, n_partials, partial_stride);
    const float u = slab_sum(row, 2 * c + 1, n_partials, partial_stride);
    out[idx] = fb_from_float<T>(fb_gate_times(act, g, u));
}

// Two outputs per thread from one 4-wide load (g0, u0, g1, u1); I even, strides multiples of 4, aligned rows.
template <typename TI, typename T>
__global__ void gate_mul_vec_kernel(const TI* __restrict__ gu, long stride, int n_partials, long partial_stride,
                                    T* __restrict__ out, int n, int I, int act) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int nvec = I >> 1;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * nvec) return;
    const int r = (int)(idx / nvec), c = (int)(idx - (size_t)r * nvec);
    const float4 v = slab_sum4(gu + (size_t)r * stride + 4 * c, n_partials, partial_stride);
    T* o = out + (size_t)r * I + 2 * c;
    o[0] = fb_from_float<T>(fb_gate_times(act, v.x, v.y));
    o[1] = fb_from_float<T>(fb_gate_times(act, v.z, v.w));
}

// gate_up has dtype in_dtype and may be split-K shares (n_partials slabs partial_stride elements apart);
// out has dtype out_dtype; `act` is an FbAct code.
FB_API int fb_gate_mul(const void* gate_up, long long stride, int in_dtype, int n_partials,
                       long long partial_stride, void* out, int out_dtype, int n, int I, int act,
                       cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && I > 0 && stride >= 2LL * I, "gate_mul: bad sizes n=%d I=%d stride=%lld", n, I, stride);
    FB_REQUIRE(fb_act_known(act), "gate_mul: unknown activation code %d", act);
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    const bool vec = I % 2 == 0 && stride % 4 == 0 && partial_stride % 4 == 0 && (uintptr_t)gate_up % 16 == 0;
    if (vec) {
        const size_t total = (size_t)n * (I / 2);
        FB_DISPATCH_DTYPE(in_dtype, TI, FB_DISPATCH_DTYPE(out_dtype, T,
            (fb_launch((gate_mul_vec_kernel<TI, T>), (unsigned)((total + 255) / 256), 256, 0, stream,
                (const TI*)gate_up, stride, n_partials, (long)partial_stride, (T*)out, n, I, act))));
        return fb_check_launch("gate_mul");
    }
    const size_t total = (size_t)n * I;
    FB_DISPATCH_DTYPE(in_dtype, TI, FB_DISPATCH_DTYPE(out_dtype, T,
        (fb_launch((gate_mul_kernel<TI, T>), (unsigned)((total + 255) / 256), 256, 0, stream,
            (const TI*)gate_up, stride, n_partials, (long)partial_stride, (T*)out, n, I, act))));
    return fb_check_launch("gate_mul");
}
