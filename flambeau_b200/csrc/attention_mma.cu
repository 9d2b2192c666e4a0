// Paged causal (sliding-window) attention for portions of prompts, bfloat16 on the tensor cores (mma.sync
// m16n8k16, float32 accumulation and softmax), and the entry point of the bfloat16 attention.
//
// A CTA owns one key/value head and a tile of up to 128 query rows = (128 / G) tokens x the G query heads that
// share the head, so every K/V tile is read once for the whole group.  Its four warps take 32 rows each (16 for
// heads wider than 128), so that every K/V fragment fetched from shared memory feeds two row blocks; each walks
// all visible key tiles with an online softmax.  CTAs are numbered heaviest first over all heads and sequences.
// Sequences of a step with at most 16 rows (decoded tokens, portions of a few tokens) go to the split-key
// arrangement instead (attention_split.cu); heads of 64 and 128 with pages that tile 64 keys go to the tcgen05
// kernel (attention_tc.cu) unless that is switched off.
//
// Keys and values come through the block table in tiles of 64 keys through a two-stage pipeline: whole pages by
// tensor-map copies (128-byte swizzle) when a tile is a whole number of pages and the head a whole number of
// 64-column blocks, single rows by bulk copies otherwise.  A key outside [t0, p] of every row of the CTA is not
// read at all, so pages that the cache manager has taken back are never touched.  Softmax runs in base 2 with
// scale*log2(e) folded into the scores.  Head sizes are padded with zeros to HD_MAX in shared memory, so any head
// size that is a multiple of 8 runs.
//
// Formulas: crates/kernels-hip/src/kernels/attention_prefill_flash_tile_f16.cu:73-213 (tile + online softmax).
#include <stdlib.h>

#include "attention_common.cuh"

namespace {

using namespace fb_attn;

constexpr int LONG_THREADS = 128;  // four warps
constexpr int NST = 2;             // K/V tiles in shared memory: a tile is reused for up to 128 rows, and two CTAs
                                   // on an SM are worth more than a third tile

// 16-row blocks per warp: two while the accumulators fit in registers.
__host__ __device__ constexpr int long_row_blocks(int hd_max) { return hd_max > 128 ? 1 : 2; }

template <int HD_MAX, bool TMA>
__global__ void __launch_bounds__(LONG_THREADS)
attention_mma_kernel(const __grid_constant__ AttnArgs a) {
    constexpr int NT = LONG_THREADS;
    fb_pdl_launch_dependents();
    // The step's descriptor was on the device before the step's first kernel: everything up to the first read of
    // Q or of the cache (the CTA's share of the work, barriers, clearing) runs ahead of the kernel before this one.
    constexpr int LDS = HD_MAX + 8;                 // row stride of Q (and of K/V when padded): 16 bytes of padding
    constexpr int TILE_ELEMS = TMA ? KT * HD_MAX : KT * LDS;
    constexpr int NKS = HD_MAX / 16;                // k-steps of Q K^T
    constexpr int NDB = HD_MAX / 8;                 // n-blocks of P V
    constexpr int R = long_row_blocks(HD_MAX);      // 16-row blocks per warp: K/V fragments are reused R times
    constexpr int ROWS = 64 * R;                    // query rows per CTA
    constexpr int NSB = KT / 8;                     // n-blocks of S

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [ROWS][LDS]
    // Q first; the K/V tiles start on a 1024-byte boundary (the swizzle pattern of TMA mode needs it).
    // Stage by stage: K tile, V tile.
    const uint32_t smem_base = smem_u32(smem_raw);
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(
        smem_raw + (((smem_base + ROWS * LDS * 2 + 1023u) & ~1023u) - smem_base));
    auto k_tile = [&](int buf) { return tiles + buf * (2 * TILE_ELEMS); };
    auto v_tile = [&](int buf) { return tiles + buf * (2 * TILE_ELEMS) + TILE_ELEMS; };
    uint8_t* tail = reinterpret_cast<uint8_t*>(tiles + NST * 2 * TILE_ELEMS);
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);                         // [NST] tile-complete barriers
    int* bail = reinterpret_cast<int*>(tail + 32);                              // a bounded wait ran out

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.nh / a.nkv;
    const int hd = a.hd, hd_chunks = hd / 8;
    // TMA mode: one copy per (K or V, page of the tile, 64-column block), issued by thread number = copy number
    const int pages_per_tile = TMA ? KT / a.page_size : 1;
    const int col_blocks = TMA ? hd / 64 : 1;
    const int tma_ops = 2 * pages_per_tile * col_blocks;

    // ---- what this CTA has to do: query tokens [tok0, tok0 + ntok) of a sequence, one key/value head ----
    // CTAs are numbered heaviest first over the whole step: the last tokens of every sequence and head (they see
    // the most keys) get the first SMs, whatever head or sequence they belong to
    const int pairs = a.nkv * portion_seqs(a);
    const int rank = blockIdx.x / pairs, pair = blockIdx.x - rank * pairs;
    const int seq = portion_seq(a, pair / a.nkv), kvh = pair % a.nkv;
    const int q_tiles = gridDim.x / pairs;
    const int q_len = a.seq_q_len[seq];
    if (q_len * G <= a.short_rows) return;                      // the split-key arrangement's
    const int TQ = ROWS / G;
    const int tok0 = (q_tiles - 1 - rank) * TQ;               // later tiles see more keys: start them first
    if (tok0 >= q_len) return;
    const int ntok = min(TQ, q_len - tok0);
    const int q_start = a.seq_q_start[seq], pos0 = a.seq_pos_start[seq];
    const int rows_valid = ntok * G;
    const KeyRange kr = key_range(pos0 + tok0, pos0 + tok0 + ntok - 1, a.window);
    const int k_begin = kr.tile_lo, k_end = kr.t_hi + 1, t_hi = kr.t_hi;
    const int n_tiles = (k_end - k_begin + KT - 1) / KT;
    const int* table = a.block_table + (size_t)seq * a.table_stride;
    const int base_page = table_base_of(a, seq);

    if (tid == 0) {
        for (int st = 0; st < NST; ++st) mbar_init(smem_u32(&full[st]), TMA ? tma_ops : 2 * KT);
        *bail = 0;
        mbar_fence_init();
    }
    // Pages that no query can see are not fetched, and a head narrower than the tile leaves padding columns:
    // clear them so that what stays there is finite.
    if (TMA) {
        for (int idx = tid; idx < 2 * NST * TILE_ELEMS / 8; idx += NT)
            *reinterpret_cast<uint4*>(tiles + idx * 8) = make_uint4(0, 0, 0, 0);
    } else if (hd < HD_MAX) {
        const int pad_chunks = HD_MAX / 8 - hd_chunks;
        for (int idx = tid; idx < 2 * NST * KT * pad_chunks; idx += NT) {
            const int r = idx / pad_chunks, c = hd_chunks + idx - r * pad_chunks;
            *reinterpret_cast<uint4*>(tiles + r * LDS + c * 8) = make_uint4(0, 0, 0, 0);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();                                  // barriers initialised, tiles cleared
    fb_pdl_wait();                                    // from here on: Q and the cache, which earlier kernels wrote

    // The page id this thread will need for the tile that starts at `tile_start`, read ahead of time so that the
    // copy can be issued without waiting for the table: -2 = nothing to fetch there (no query of this CTA sees
    // it), -1 = the table has no page although one is needed (flagged when the tile is issued).
    auto lookup = [&](int tile_start) -> int {
        int t_first, span;
        if constexpr (TMA) {
            if (tid >= tma_ops) return -2;
            t_first = tile_start + ((tid >> 1) / col_blocks) * a.page_size;
            span = a.page_size;
        } else {
            if (tid >= 2 * KT) return -2;
            t_first = tile_start + (tid & (KT - 1));
            span = 1;
        }
        if (!(t_first + span > kr.t_lo && t_first < k_end)) return -2;
        const int page = table_page(a, table, base_page, t_first / a.page_size);
        return (page < 0 || page >= a.n_pages) ? -1 : page;
    };

    // TMA mode: thread number = copy number: (K or V, page of the tile, 64-column block), one tensor-map copy each.
    // Otherwise: one row of 64 keys (threads 0..63) or 64 values (threads 64..127) per thread: a bulk copy of the
    // row's hd*2 bytes.  Copies are counted on the tile's barrier.  What no query of this CTA may see (before the
    // window or past the last position) is not read.
    auto load_tile = [&](int buf, int tile_start, int page) {
        const uint32_t bar = smem_u32(&full[buf]);
        if constexpr (TMA) {
            if (tid >= tma_ops) return;
            const bool is_v = tid & 1;
            const int rest = tid >> 1;
            const int cb = rest % col_blocks, pj = rest / col_blocks;
            if (page >= 0) {
                __nv_bfloat16* dst = (is_v ? v_tile(buf) : k_tile(buf)) + cb * (KT * 64) + pj * a.page_size * 64;
                mbar_expect_tx(bar, (uint32_t)(a.page_size * 128));
                tma_load_2d(smem_u32(dst), is_v ? &a.map_v : &a.map_k, bar, cb * 64,
                            (page * a.nkv + kvh) * a.page_size);
            } else {
                if (page == -1) atomicOr(a.status, FB_STATUS_BAD_PAGE);
                mbar_arrive(bar);                     // stale (finite) data stays in the slot; it is masked
            }
            return;
        }
        if (tid >= 2 * KT) return;
        const int r = tid & (KT - 1);
        const bool is_v = tid >= KT;
        const int t = tile_start + r;
        __nv_bfloat16* dst = (is_v ? v_tile(buf) : k_tile(buf)) + r * LDS;
        if (page >= 0) {
            const size_t off = (((size_t)page * a.nkv + kvh) * a.page_size + (t % a.page_size)) * hd;
            mbar_expect_tx(bar, (uint32_t)(hd * 2));
            bulk_copy_g2s(smem_u32(dst), (is_v ? a.v_pool : a.k_pool) + off, (uint32_t)(hd * 2), bar);
        } else {
            if (page == -1) atomicOr(a.status, FB_STATUS_BAD_PAGE);
            for (int c = 0; c < hd_chunks; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
            // order these generic stores before a later bulk copy into the same row
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar);
        }
    };

    // prologue: NST - 1 tiles in flight; the page id for the tile after them is already on its way
    int next_page = lookup(k_begin);
#pragma unroll
    for (int st = 0; st < NST - 1; ++st)
        if (st < n_tiles) {
            load_tile(st, k_begin + st * KT, next_page);
            next_page = lookup(k_begin + (st + 1) * KT);
        }

    // ---- stage Q (zero-padded) ----
    for (int idx = tid; idx < ROWS * (HD_MAX / 8); idx += NT) {
        const int r = idx / (HD_MAX / 8), c = idx - r * (HD_MAX / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_valid && c < hd_chunks) {
            const int token = q_start + tok0 + r / G, head = kvh * G + r % G;
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)token * a.q_stride + (size_t)head * hd + c * 8);
        }
        *reinterpret_cast<uint4*>(Qs + r * LDS + c * 8) = v;
    }
    __syncthreads();                                  // Q staged

    const int row_base = warp * (16 * R);           // first row of this warp within the CTA
    // per-thread rows of row block rb: row_base + 16*rb + lane/4 and that + 8
    int p_row[R][2], t0_row[R][2];
    float slope_row[R][2];                          // the row's head's penalty on distance, in base-2 units
#pragma unroll
    for (int rb = 0; rb < R; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = row_base + 16 * rb + (lane >> 2) + 8 * h;
            slope_row[rb][h] = a.score_slopes && r < rows_valid ? a.score_slopes[kvh * G + r % G] * 1.4426950408889634f : 0.0f;
            if (r < rows_valid) {
                p_row[rb][h] = pos0 + tok0 + r / G;
                t0_row[rb][h] = (a.window > 0 && p_row[rb][h] - a.window + 1 > 0) ? p_row[rb][h] - a.window + 1 : 0;
            } else {
                p_row[rb][h] = -1;                    // sees nothing
                t0_row[rb][h] = 0;
            }
        }
    float m_run[R][2], l_run[R][2];
    float o[R][NDB][4];
#pragma unroll
    for (int rb = 0; rb < R; ++rb) {
        m_run[rb][0] = m_run[rb][1] = -INFINITY;
        l_run[rb][0] = l_run[rb][1] = 0.0f;
#pragma unroll
        for (int d = 0; d < NDB; ++d)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[rb][d][e] = 0.0f;
    }

    for (int it = 0; it < n_tiles; ++it) {
        const int buf = it % NST;
        const int tile_start = k_begin + it * KT;
        if (!mbar_wait(smem_u32(&full[buf]), (uint32_t)(it / NST) & 1u, a.status)) *bail = 1;
        __syncthreads();                              // every thread is past tile it-1: its buffer is free
        if (*bail) break;
        if (it + NST - 1 < n_tiles) {
            load_tile((it + NST - 1) % NST, tile_start + (NST - 1) * KT, next_page);
            next_page = lookup(tile_start + NST * KT);    // consumed one iteration from now
        }
        if constexpr (TMA) {
            // Whole pages arrive, the slots behind the last position included, and what a page holds there was
            // never written by this request.  Scores of such keys are masked by assignment, but their values
            // would be multiplied by a probability of 0, and 0 * NaN is NaN: clear those value rows.
            if (tile_start + KT > t_hi + 1) {
                const int first_dead = t_hi + 1 - tile_start;               // >= 0 because tile_start <= t_hi
                __nv_bfloat16* vz = v_tile(buf);
                const int chunks = (KT - first_dead) * 8;                    // 16-byte chunks per 64-column block
                for (int idx = tid; idx < chunks * (HD_MAX / 64); idx += NT) {
                    const int cb = idx / chunks, rest = idx - cb * chunks;
                    *reinterpret_cast<uint4*>(vz + cb * (KT * 64) + (first_dead + rest / 8) * 64 + (rest & 7) * 8) =
                        make_uint4(0, 0, 0, 0);
                }
                __syncthreads();
            }
        }
        const __nv_bfloat16* kt = k_tile(buf);
        const __nv_bfloat16* vt = v_tile(buf);

        // ---- S = Q K^T for this warp's rows and keys: every K fragment serves all R row blocks ----
        float s[R][NSB][4];
#pragma unroll
        for (int rb = 0; rb < R; ++rb)
#pragma unroll
            for (int nb = 0; nb < NSB; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[rb][nb][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < NKS; ks += 2) {
            uint32_t qa[R][4], qb[R][4];
#pragma unroll
            for (int rb = 0; rb < R; ++rb) {
                const __nv_bfloat16* qrow = Qs + (row_base + 16 * rb + (lane & 15)) * LDS + 8 * (lane >> 4);
                ldmatrix_x4(qa[rb], qrow + ks * 16);
                ldmatrix_x4(qb[rb], qrow + (ks + 1) * 16);
            }
#pragma unroll
            for (int nb = 0; nb < NSB; ++nb) {
                uint32_t b[4];     // (b0,b1): dims ks*16..+15, (b2,b3): dims (ks+1)*16..+15, keys nb*8..+7
                ldmatrix_x4(b, tile_at<HD_MAX, TMA>(kt, nb * 8 + (lane & 7), ks * 16 + 8 * (lane >> 3)));
#pragma unroll
                for (int rb = 0; rb < R; ++rb) {
                    mma_bf16(s[rb][nb], qa[rb], b[0], b[1]);
                    mma_bf16(s[rb][nb], qb[rb], b[2], b[3]);
                }
            }
        }
        // ---- scale, mask, online softmax ----
        uint32_t pa[R][KT / 16][4];            // the probabilities as A fragments of P V
#pragma unroll
        for (int rb = 0; rb < R; ++rb) {
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < NSB; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int t = tile_start + nb * 8 + 2 * (lane & 3) + (e & 1);
                    const bool ok = t >= t0_row[rb][h] && t <= p_row[rb][h] && t < k_end;
                    const float v = ok ? fmaf(slope_row[rb][h], (float)(t - p_row[rb][h]), s[rb][nb][e] * a.scale_log2e) : -INFINITY;
                    s[rb][nb][e] = v;
                    tile_max[h] = fmaxf(tile_max[h], v);
                }
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float tm = tile_max[h];
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
                const float m_new = fmaxf(m_run[rb][h], tm);
                const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;     // a row that has seen nothing yet
                corr[h] = exp2f(m_run[rb][h] - m_use);
                m_run[rb][h] = m_new;
                float sum = 0.0f;
#pragma unroll
                for (int nb = 0; nb < NSB; ++nb) {
                    const float p0 = exp2f(s[rb][nb][2 * h] - m_use), p1 = exp2f(s[rb][nb][2 * h + 1] - m_use);
                    s[rb][nb][2 * h] = p0;
                    s[rb][nb][2 * h + 1] = p1;
                    sum += p0 + p1;
                }
                l_run[rb][h] = l_run[rb][h] * corr[h] + sum;
            }
#pragma unroll
            for (int d = 0; d < NDB; ++d) {
                o[rb][d][0] *= corr[0]; o[rb][d][1] *= corr[0];
                o[rb][d][2] *= corr[1]; o[rb][d][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < KT / 16; ++kk) {
                pa[rb][kk][0] = pack_bf16(s[rb][2 * kk][0], s[rb][2 * kk][1]);
                pa[rb][kk][1] = pack_bf16(s[rb][2 * kk][2], s[rb][2 * kk][3]);
                pa[rb][kk][2] = pack_bf16(s[rb][2 * kk + 1][0], s[rb][2 * kk + 1][1]);
                pa[rb][kk][3] = pack_bf16(s[rb][2 * kk + 1][2], s[rb][2 * kk + 1][3]);
            }
        }
        // ---- O += P V: every V fragment serves all R row blocks ----
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
            for (int d = 0; d < NDB; d += 2) {
                uint32_t b[4];     // (b0,b1): dims d*8..+7, (b2,b3): dims (d+1)*8..+7, keys kk*16..+15
                ldmatrix_x4_trans(b, tile_at<HD_MAX, TMA>(vt, kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1),
                                                          d * 8 + 8 * (lane >> 4)));
#pragma unroll
                for (int rb = 0; rb < R; ++rb) {
                    mma_bf16(o[rb][d], pa[rb][kk], b[0], b[1]);
                    mma_bf16(o[rb][d + 1], pa[rb][kk], b[2], b[3]);
                }
            }
        }
    }
    __syncthreads();                                  // every warp is done with the tiles
    if (*bail) return;
#pragma unroll
    for (int rb = 0; rb < R; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[rb][h] += __shfl_xor_sync(0xffffffffu, l_run[rb][h], 1);
            l_run[rb][h] += __shfl_xor_sync(0xffffffffu, l_run[rb][h], 2);
        }

    // ---- normalise and write ----
#pragma unroll
    for (int rb = 0; rb < R; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = row_base + 16 * rb + (lane >> 2) + 8 * h;
            if (r >= rows_valid) continue;
            const float inv = l_run[rb][h] > 0.0f ? 1.0f / l_run[rb][h] : 0.0f;
            const int token = q_start + tok0 + r / G, head = kvh * G + r % G;
            __nv_bfloat16* dst = a.out + (size_t)token * a.out_stride + (size_t)head * hd;
#pragma unroll
            for (int d = 0; d < NDB; ++d) {
                const int col = d * 8 + 2 * (lane & 3);
                if (col < hd)
                    *reinterpret_cast<__nv_bfloat162*>(dst + col) =
                        __floats2bfloat162_rn(o[rb][d][2 * h] * inv, o[rb][d][2 * h + 1] * inv);
            }
        }
}

__host__ __device__ constexpr size_t long_smem_bytes(int hd_max, bool tma) {
    return (size_t)64 * long_row_blocks(hd_max) * (hd_max + 8) * 2 + 1024 /* alignment */ +
           (size_t)2 * NST * KT * (tma ? hd_max : hd_max + 8) * 2 + 64 /* barriers */;
}

template <int HD_MAX, bool TMA>
int launch_long(const AttnArgs& a, int n_seqs, int max_q_len, cudaStream_t stream) {
    constexpr size_t smem = long_smem_bytes(HD_MAX, TMA);
    auto kern = attention_mma_kernel<HD_MAX, TMA>;
    static bool configured[FB_MAX_DEVICES] = {};
    if (smem > 48 * 1024 && fb_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fb_fail(-2, "attention_mma: cannot reserve %d bytes of shared memory: %s",
                                             (int)smem, cudaGetErrorString(e));
        fb_setup_done(configured);
    }
    const int TQ = 64 * long_row_blocks(HD_MAX) / (a.nh / a.nkv);
    const dim3 grid(((max_q_len + TQ - 1) / TQ) * a.nkv * portion_seqs(a));
    fb_launch((kern), grid, LONG_THREADS, smem, stream, a);
    return fb_check_launch("attention_mma");
}

int launch_long(const AttnArgs& a, int hd_max, bool tma, int n_seqs, int max_q_len, cudaStream_t stream) {
    switch (hd_max) {
        case 32: return launch_long<32, false>(a, n_seqs, max_q_len, stream);
        case 64: return tma ? launch_long<64, true>(a, n_seqs, max_q_len, stream)
                            : launch_long<64, false>(a, n_seqs, max_q_len, stream);
        case 128: return tma ? launch_long<128, true>(a, n_seqs, max_q_len, stream)
                             : launch_long<128, false>(a, n_seqs, max_q_len, stream);
        default: return tma ? launch_long<256, true>(a, n_seqs, max_q_len, stream)
                            : launch_long<256, false>(a, n_seqs, max_q_len, stream);
    }
}

int g_attention_tc = -1;           // -1: not decided yet (the environment decides), 0: off, 1: on

bool attention_tc_enabled() {
    if (g_attention_tc < 0) {
        const char* env = getenv("FLAMBEAU_ATTN_TC");
        g_attention_tc = (env && env[0] == '0') ? 0 : 1;
    }
    return g_attention_tc == 1;
}

}  // namespace

// Portions of prompts run on the tcgen05 kernel where it takes the geometry (1, the default) or always on the
// mma.sync kernel (0).
FB_API void fb_set_attention_tc(int on) { g_attention_tc = on ? 1 : 0; }

// q, out: bfloat16 [rows, heads*hd]; pools bfloat16 [pages][kv heads][page size][hd].
// seq_*: per sequence of the step (device int32); table_base (may be null): the logical page that column 0 of each
// sequence's table row stands for; multi_seqs (may be null: all sequences): the n_multi sequences that bring more
// than one token, which is all that the arrangements for portions lay their grid over.  max_q_len / max_kv_len / any_short / any_long come from the host's copy of the
// step descriptor.  `scratch` holds the arrival counters and partial results of the split-key arrangement.
// prefetch_*: the first prefetch_bytes_per_row bytes of each of prefetch_rows rows (prefetch_row_stride bytes
// apart, from prefetch_base) are fetched into L2 when the split-key kernel's stream of cache ends: the matrix of
// the product that follows (a hint; null base: none).
FB_API int fb_paged_attention_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* k_pool, const void* v_pool, int page_size, int n_pages,
                                  const int* block_table, int table_stride, const int* table_base,
                                  const int* seq_q_start, const int* seq_q_len, const int* seq_pos_start,
                                  const int* multi_seqs, int n_multi, int n_seqs, int max_q_len, int max_kv_len, int any_short, int any_long, int nh, int nkv, int hd,
                                  int window, float scale, const float* score_slopes, float* scratch,
                                  long long scratch_floats,
                                  const void* prefetch_base, long long prefetch_rows, long long prefetch_row_stride,
                                  int prefetch_bytes_per_row, int* status, cudaStream_t stream) {
    FB_REQUIRE(n_seqs >= 0 && nh > 0 && nkv > 0 && hd > 0, "attention_mma: bad sizes");
    FB_REQUIRE(!multi_seqs || (n_multi >= 0 && n_multi <= n_seqs), "attention_mma: bad list of multi-token sequences");
    FB_REQUIRE(nh % nkv == 0, "attention_mma: %d query heads are not a multiple of %d key/value heads", nh, nkv);
    FB_REQUIRE(hd % 8 == 0 && hd <= 256, "attention_mma: head size %d must be a multiple of 8 and at most 256", hd);
    const int G = nh / nkv;
    FB_REQUIRE(G <= 64, "attention_mma: %d query heads per key/value head exceed 64", G);
    FB_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0, "attention_mma: q rows must be 16-byte aligned");
    FB_REQUIRE(out_stride % 2 == 0 && ((uintptr_t)out & 3) == 0, "attention_mma: out rows must be 4-byte aligned");
    FB_REQUIRE(page_size > 0 && n_pages > 0 && window >= 0, "attention_mma: bad cache geometry");
    if (n_seqs == 0) return 0;
    const int HD_MAX = hd <= 32 ? 32 : hd <= 64 ? 64 : hd <= 128 ? 128 : 256;
    AttnArgs a;
    a.q = (const __nv_bfloat16*)q; a.q_stride = (long)q_stride;
    a.out = (__nv_bfloat16*)out; a.out_stride = (long)out_stride;
    a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
    a.page_size = page_size; a.n_pages = n_pages;
    a.block_table = block_table; a.table_stride = table_stride; a.table_base = table_base;
    a.seq_q_start = seq_q_start; a.seq_q_len = seq_q_len; a.seq_pos_start = seq_pos_start;
    a.multi_seqs = multi_seqs; a.n_multi = n_multi;
    a.nh = nh; a.nkv = nkv; a.hd = hd; a.window = window;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.score_slopes = score_slopes;
    a.status = status;
    a.short_rows = G <= 16 ? 16 : 0;               // with more than 16 heads per group even one token is "long"
    if (a.short_rows == 0) {                       // then single tokens run in the arrangement for portions as well,
        any_long = any_long || any_short;          // whose grid must cover every sequence
        any_short = 0;
        a.multi_seqs = nullptr;
    }
    // whole pages fetched by tensor-map copies when a 64-key tile is a whole number of pages and the head a whole
    // number of 64-column blocks; single rows by bulk copies otherwise
    const bool tma = hd % 64 == 0 && page_size >= 8 && page_size <= KT && KT % page_size == 0;
    if (tma) {
        const long pool_rows = (long)n_pages * nkv * page_size;
        int rc = fb_tensor_map_bf16(&a.map_k, k_pool, pool_rows, hd, hd, 64, page_size);
        if (rc) return rc;
        rc = fb_tensor_map_bf16(&a.map_v, v_pool, pool_rows, hd, hd, 64, page_size);
        if (rc) return rc;
    }
    a.n_seqs = n_seqs;
    a.short_ctas = 0; a.min_tiles = 1;
    a.prefetch = fb_make_prefetch(prefetch_base, prefetch_rows, prefetch_row_stride, prefetch_bytes_per_row);
    a.part_o = nullptr; a.part_ml = nullptr; a.part_cnt = nullptr;
    if (any_long) {
        const int rc = (attention_tc_enabled() && fb_attention_tc_takes(a, tma))
                           ? fb_launch_attention_tc(a, n_seqs, max_q_len, stream)
                           : launch_long(a, HD_MAX, tma, n_seqs, max_q_len, stream);
        if (rc) return rc;
    }
    if (any_short) return fb_launch_attention_split(a, HD_MAX, tma, n_seqs, scratch, scratch_floats, stream);
    return 0;
}
