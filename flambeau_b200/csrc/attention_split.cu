// Paged attention for decoded tokens and portions of a few tokens (rows = tokens x G <= 16), bfloat16 on the
// tensor cores (mma.sync m16n8k16, float32 accumulation and softmax): the split-key arrangement.
//
// All key tiles of all (sequence, key/value head) pairs form one line, pair after pair (pairs of one sequence side
// by side), and the CTAs of the launch cut that line into equal stretches: CTA c owns tiles [c * per, (c + 1) * per).
// A stretch may end inside a pair and go on into the next ones, so every CTA has the same amount of cache to stream
// whatever the number and the lengths of the sequences.  Each (CTA, pair) segment of a pair that is cut leaves a
// partial result in slot (CTA index + pair index), which is unique and needs no table, and counts itself on the
// pair; the CTA that arrives last adds the pair's segments, in their order.
//
// One warp fetches, four warps score.  The fetching warp walks the CTA's stretch of key tiles, segment after
// segment, and keeps NST tiles in flight (page ids looked up one tile ahead, a tile's slot refilled as soon as its
// four readers have left it), so the stream of cache never stops at a tile's or a segment's end; when the stretch
// is through, it fetches its share of the start of the next product's weights into L2, if the caller said which.
// Each scoring warp takes 16 of a tile's 64 keys and keeps its own running maximum, sum and output for the
// segment's rows; nothing synchronises the four between tiles.  At a segment's end the four are added up in shared
// memory; where a pair was cut, the sum goes to scratch and the CTA that arrives last at the pair adds the partials
// of all its segments, in their order.
//
// Keys and values come through the block table in tiles of 64 keys: whole pages by tensor-map copies (128-byte
// swizzle) when a tile is a whole number of pages and the head a whole number of 64-column blocks, single rows by
// bulk copies otherwise.  A key outside [t0, p] of every row of a segment is not read at all, so pages that the
// cache manager has taken back are never touched.  Softmax runs in base 2 with scale*log2(e) folded into the
// scores.  Head sizes are padded with zeros to HD_MAX in shared memory, so any head size that is a multiple of 8
// runs.
//
// Formulas: crates/kernels-hip/src/kernels/attention_decode_f16_splitk.cu:215-256 (merge of chunks),
// attention_prefill_flash_tile_f16.cu:73-213 (tile + online softmax).
#include <stdlib.h>

#include "attention_common.cuh"

namespace {

using namespace fb_attn;

__device__ __forceinline__ int short_tiles_of(const AttnArgs& a, int q_len, int pos0, int G) {
    if (q_len * G > a.short_rows) return 0;                 // belongs to the arrangement for portions
    const KeyRange kr = key_range(pos0, pos0 + q_len - 1, a.window);
    return (kr.t_hi - kr.tile_lo) / KT + 1;
}

// Per-sequence facts in shared memory: five arrays of n_seqs (+1) ints.
struct ShortSeqs {
    int *tiles, *prefix, *q_len, *pos0, *q_start;
    __device__ __forceinline__ explicit ShortSeqs(int* base, int n)
        : tiles(base), prefix(base + n), q_len(base + 2 * n + 1), pos0(base + 3 * n + 1), q_start(base + 4 * n + 1) {}
};
__host__ __device__ constexpr size_t short_seqs_bytes(size_t n) { return 4 * (5 * n + 1); }

// prefix[s] = tiles of one key/value head over sequences [0, s).  Every CTA computes it for itself from the step's
// descriptor (one round of loads, a warp scan), so that the host has nothing to prepare and a captured graph stays
// valid as the sequences grow.
__device__ __forceinline__ void short_prefix(const AttnArgs& a, int G, const ShortSeqs& ss, int tid, int nt) {
    const int n = a.n_seqs;
    for (int s = tid; s < n; s += nt) {
        const int q_len = a.seq_q_len[s], pos0 = a.seq_pos_start[s];
        ss.q_len[s] = q_len;
        ss.pos0[s] = pos0;
        ss.q_start[s] = a.seq_q_start[s];
        ss.tiles[s] = short_tiles_of(a, q_len, pos0, G);
    }
    __syncthreads();
    if (tid < 32) {
        int carry = 0;
        for (int base = 0; base < n; base += 32) {
            const int s = base + tid;
            const int v = s < n ? ss.tiles[s] : 0;
            int inc = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, off);
                if (tid >= off) inc += t;
            }
            if (s < n) ss.prefix[s] = carry + inc - v;
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (tid == 0) ss.prefix[n] = carry;
    }
    __syncthreads();
}

// Adds the segments of one row of a pair: out = sum_c 2^(m_c - m) o_c / sum_c 2^(m_c - m) l_c, segments in slots
// slot0 .. slot0 + n_chunks - 1.  One warp: a lane first takes a segment (its maximum, sum and weight), then a share
// of the head's columns.  The partials were written by other SMs: they are read past the L1.
template <int HD_MAX>
__device__ __forceinline__ void merge_row(const AttnArgs& a, size_t slot0, int n_chunks, int r, int lane,
                                          __nv_bfloat16* dst) {
    constexpr int U = HD_MAX <= 128 ? 16 : 8;          // partials whose loads are in flight together
    float acc[HD_MAX / 32];
#pragma unroll
    for (int i = 0; i < HD_MAX / 32; ++i) acc[i] = 0.0f;
    float m = -INFINITY;
    for (int ch = lane + 32; ch < n_chunks; ch += 32) m = fmaxf(m, __ldcg(a.part_ml + ((slot0 + ch) * 16 + r) * 2));
    float2 mine = make_float2(-INFINITY, 0.0f);       // segment `lane` of the first 32
    if (lane < n_chunks) mine = __ldcg(reinterpret_cast<const float2*>(a.part_ml + ((slot0 + lane) * 16 + r) * 2));
    m = fb_warp_max(fmaxf(m, mine.x));
    float l = 0.0f;
    if (m > -INFINITY) {
        for (int c0 = 0; c0 < n_chunks; c0 += 32) {
            if (c0 > 0) {
                mine = make_float2(-INFINITY, 0.0f);
                if (c0 + lane < n_chunks)
                    mine = __ldcg(reinterpret_cast<const float2*>(a.part_ml + ((slot0 + c0 + lane) * 16 + r) * 2));
            }
            const float wgt = exp2f(mine.x - m);          // 0 for a segment that saw nothing or does not exist
            l += wgt * mine.y;
            const int cnt = min(32, n_chunks - c0);
            for (int j0 = 0; j0 < cnt; j0 += U) {
                float v[U][HD_MAX / 32];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int j = j0 + u < cnt ? j0 + u : cnt - 1;
                    const float* po = a.part_o + ((slot0 + c0 + j) * 16 + r) * HD_MAX;
#pragma unroll
                    for (int i = 0; i < HD_MAX / 32; ++i) v[u][i] = __ldcg(po + lane + 32 * i);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float wj = j0 + u < cnt ? __shfl_sync(0xffffffffu, wgt, (j0 + u) & 31) : 0.0f;
#pragma unroll
                    for (int i = 0; i < HD_MAX / 32; ++i) acc[i] = fmaf(wj, v[u][i], acc[i]);
                }
            }
        }
    }
    l = fb_warp_sum(l);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < HD_MAX / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < a.hd) dst[d] = __float2bfloat16_rn(acc[i] * inv);
    }
}

// K/V tiles in shared memory: three while two CTAs still fit on an SM.
__host__ __device__ constexpr int split_stages(int hd_max) { return hd_max <= 128 ? 3 : 2; }

constexpr int SPLIT_SCORERS = 4;
constexpr int SPLIT_THREADS = 32 * (SPLIT_SCORERS + 1);
constexpr int SPLIT_COUNTERS = 1 << 16;      // arrival counters at the start of the scratch buffer

__device__ __forceinline__ void scorer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(32 * SPLIT_SCORERS) : "memory"); }

__host__ __device__ constexpr size_t split_smem_bytes(int hd_max, bool tma, size_t n_seqs) {
    return (size_t)16 * (hd_max + 8) * 2 + 1024 /* alignment */ +
           (size_t)2 * split_stages(hd_max) * KT * (tma ? hd_max : hd_max + 8) * 2 + 96 /* barriers, flags */ +
           (size_t)16 * hd_max * 4 + 512 /* the segment's sum over the four warps; their maxima and sums */ +
           short_seqs_bytes(n_seqs) + 16;
}

template <int HD_MAX, bool TMA>
__global__ void __launch_bounds__(SPLIT_THREADS, HD_MAX <= 128 ? 2 : 1)
attention_split_kernel(const __grid_constant__ AttnArgs a) {
    constexpr int NT = SPLIT_THREADS;
    fb_pdl_launch_dependents();
    // The step's descriptor was on the device before the step's first kernel: everything up to the first read of
    // Q or of the cache (the CTA's share of the work, barriers, clearing) runs ahead of the kernel before this one.
    constexpr int LDS = HD_MAX + 8;                 // row stride of Q (and of K/V when padded): 16 bytes of padding
    constexpr int TILE_ELEMS = TMA ? KT * HD_MAX : KT * LDS;
    constexpr int NKS = HD_MAX / 16;                // k-steps of Q K^T
    constexpr int NDB = HD_MAX / 8;                 // n-blocks of P V
    constexpr bool Q_IN_REGS = HD_MAX <= 128;
    constexpr int NST = split_stages(HD_MAX);  // K/V tiles in shared memory

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [16][LDS]
    const uint32_t smem_base = smem_u32(smem_raw);
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(
        smem_raw + (((smem_base + 16 * LDS * 2 + 1023u) & ~1023u) - smem_base));   // stage by stage: K tile, V tile
    auto k_tile = [&](int buf) { return tiles + buf * (2 * TILE_ELEMS); };
    auto v_tile = [&](int buf) { return tiles + buf * (2 * TILE_ELEMS) + TILE_ELEMS; };
    uint8_t* tail = reinterpret_cast<uint8_t*>(tiles + NST * 2 * TILE_ELEMS);
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);                         // [NST] a tile has landed
    uint64_t* empty = reinterpret_cast<uint64_t*>(tail + 32);                   // [NST] its four readers have left
    volatile int* flags = reinterpret_cast<volatile int*>(tail + 64);           // [0] a wait ran out, [1] last arriver
    float* o_sum = reinterpret_cast<float*>(tail + 96);                         // [16][HD_MAX] sum over the warps
    float* sml = o_sum + 16 * HD_MAX;                                           // [4 warps][16][2] maxima and sums
    const ShortSeqs ss(reinterpret_cast<int*>(sml + SPLIT_SCORERS * 32), a.n_seqs);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.nh / a.nkv;
    const int hd = a.hd, hd_chunks = hd / 8;
    const int pages_per_tile = TMA ? KT / a.page_size : 1;
    const int col_blocks = TMA ? hd / 64 : 1;

    // ---- the CTA's stretch of the line of tiles ----
    short_prefix(a, G, ss, tid, NT);
    const long total = (long)a.nkv * ss.prefix[a.n_seqs];
    const int per = max((int)((total + gridDim.x - 1) / gridDim.x), a.min_tiles);
    int g = (int)min((long)blockIdx.x * per, total);                            // the next tile of the stretch
    const int seg_hi = (int)min((long)g + per, total);
    if (g >= seg_hi) return;
    int cur_seq = 0;

    struct Seg {
        int seq, kvh, q_len, q_start, pos0, t_lo, t_hi, k_begin, k_end, n_tiles;
        int c_first, n_chunks;             // the first CTA with a segment of this pair, and how many have one
        const int* table;
        int base_page;                     // the logical page that column 0 of the table row stands for
    };
    auto next_seg = [&]() {                // the segment that starts at tile g; moves g past it
        while ((long)a.nkv * ss.prefix[cur_seq + 1] <= g) ++cur_seq;
        Seg sg;
        const int seq = cur_seq, n = ss.tiles[seq];
        const int within = g - a.nkv * ss.prefix[seq];                          // tiles into this sequence's pairs
        const int kvh = within / n, tile_a = within - kvh * n;
        const int tile_b = min(n, tile_a + (seg_hi - g));
        g += tile_b - tile_a;
        sg.seq = seq; sg.kvh = kvh; sg.q_len = ss.q_len[seq]; sg.q_start = ss.q_start[seq]; sg.pos0 = ss.pos0[seq];
        const KeyRange kr = key_range(sg.pos0, sg.pos0 + sg.q_len - 1, a.window);
        sg.t_lo = kr.t_lo; sg.t_hi = kr.t_hi;
        sg.k_begin = kr.tile_lo + tile_a * KT;
        sg.k_end = min(kr.t_hi + 1, kr.tile_lo + tile_b * KT);
        sg.n_tiles = tile_b - tile_a;
        sg.table = a.block_table + (size_t)seq * a.table_stride;
        sg.base_page = table_base_of(a, seq);
        const long first_tile = (long)a.nkv * ss.prefix[seq] + (long)kvh * n;   // of the pair, in the line of tiles
        sg.c_first = (int)(first_tile / per);
        sg.n_chunks = (int)((first_tile + n - 1) / per) - sg.c_first + 1;
        return sg;
    };

    if (tid == 0) {
        for (int st = 0; st < NST; ++st) {
            mbar_init(smem_u32(&full[st]), TMA ? 2 * pages_per_tile * col_blocks : 2 * KT);
            mbar_init(smem_u32(&empty[st]), SPLIT_SCORERS);
        }
        flags[0] = flags[1] = 0;
        mbar_fence_init();
    }
    // Pages that no query can see are not fetched, and a head narrower than the tile leaves padding columns:
    // clear the tiles once so that what stays there is finite.
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
    // Q and the cache rows of this step's own tokens come from the kernel before this one: the scoring warps wait
    // for it before they read Q, the fetching warp before the first tile that reaches a new position.  Tiles of
    // older keys were written by earlier steps and are fetched at once, while that kernel may still be running.

    // A wait that ran out anywhere makes every later wait of the CTA return at once: nobody is left behind at a
    // barrier, and the status word tells the host.
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        if (flags[0]) return false;
        if (mbar_wait(smem_u32(bar), parity, a.status)) return true;
        flags[0] = 1;
        return false;
    };

    if (warp == SPLIT_SCORERS) {
        // ================= the fetching warp =================
        // Copies of a tile: TMA mode: (K or V, page of the tile, 64-column block), one tensor-map copy each;
        // otherwise one bulk copy per row of K and of V.  Lane l issues copies l, l + 32, ...
        constexpr int OPL = TMA ? 2 : 4;                                        // copies per lane and tile at most
        const int n_ops = TMA ? 2 * pages_per_tile * col_blocks : 2 * KT;
        int pages[OPL];
        // -2 = nothing to fetch (no query of the segment sees it), -1 = the table has no page although one is needed
        auto lookup = [&](const Seg& sg, int tile_start) {
#pragma unroll
            for (int u = 0; u < OPL; ++u) {
                const int op = lane + 32 * u;
                pages[u] = -2;
                if (op >= n_ops) continue;
                int t_first, span;
                if (TMA) { t_first = tile_start + ((op >> 1) / col_blocks) * a.page_size; span = a.page_size; }
                else { t_first = tile_start + (op & (KT - 1)); span = 1; }
                if (!(t_first + span > sg.t_lo && t_first < sg.k_end)) continue;
                const int page = table_page(a, sg.table, sg.base_page, t_first / a.page_size);
                pages[u] = (page < 0 || page >= a.n_pages) ? -1 : page;
            }
        };
        auto issue = [&](const Seg& sg, int buf, int tile_start) {
            const uint32_t bar = smem_u32(&full[buf]);
#pragma unroll
            for (int u = 0; u < OPL; ++u) {
                const int op = lane + 32 * u;
                if (op >= n_ops) continue;
                const int page = pages[u];
                if (page == -1) atomicOr(a.status, FB_STATUS_BAD_PAGE);
                if (TMA) {
                    const bool is_v = op & 1;
                    const int rest = op >> 1;
                    const int cb = rest % col_blocks, pj = rest / col_blocks;
                    if (page >= 0) {
                        __nv_bfloat16* dst = (is_v ? v_tile(buf) : k_tile(buf)) + cb * (KT * 64) + pj * a.page_size * 64;
                        mbar_expect_tx(bar, (uint32_t)(a.page_size * 128));
                        tma_load_2d(smem_u32(dst), is_v ? &a.map_v : &a.map_k, bar, cb * 64,
                                    (page * a.nkv + sg.kvh) * a.page_size);
                    } else {
                        mbar_arrive(bar);             // stale (finite) data stays in the slot; it is masked
                    }
                } else {
                    const int r = op & (KT - 1);
                    const bool is_v = op >= KT;
                    __nv_bfloat16* dst = (is_v ? v_tile(buf) : k_tile(buf)) + r * LDS;
                    if (page >= 0) {
                        const int t = tile_start + r;
                        const size_t off = (((size_t)page * a.nkv + sg.kvh) * a.page_size + (t % a.page_size)) * hd;
                        mbar_expect_tx(bar, (uint32_t)(hd * 2));
                        bulk_copy_g2s(smem_u32(dst), (is_v ? a.v_pool : a.k_pool) + off, (uint32_t)(hd * 2), bar);
                    } else {
                        for (int c = 0; c < hd_chunks; ++c)
                            *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
                        // order these generic stores before a later bulk copy into the same row
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        mbar_arrive(bar);
                    }
                }
            }
        };
        Seg sg = next_seg();
        int it = 0;
        bool waited = false;
        lookup(sg, sg.k_begin);
        for (uint32_t count = 0;; ++count) {
            const int buf = (int)(count % NST);
            if (count >= NST && !wait(&empty[buf], ((count / NST) - 1) & 1u)) return;
            if (!waited && sg.k_begin + (it + 1) * KT > sg.pos0) {
                fb_pdl_wait();
                waited = true;
            }
            issue(sg, buf, sg.k_begin + it * KT);
            if (++it == sg.n_tiles) {
                if (g >= seg_hi) {
                    // the stream of cache ends here: the memory system is free for the product that follows
                    fb_prefetch_issue(a.prefetch, (long)blockIdx.x * 32 + lane, (long)gridDim.x * 32);
                    return;
                }
                sg = next_seg();
                it = 0;
            }
            lookup(sg, sg.k_begin + it * KT);         // in flight while this warp waits for the slot
        }
    }

    // ================= the scoring warps =================
    fb_pdl_wait();
    const int key0 = warp * 16;                       // this warp's keys within a tile
    uint32_t count = 0;                               // tiles consumed: slot and barrier phase follow from it
    Seg cur = next_seg();
    for (;;) {
        const int kvh = cur.kvh, q_start = cur.q_start, pos0 = cur.pos0, k_begin = cur.k_begin, k_end = cur.k_end;
        const int rows_valid = cur.q_len * G;
        // ---- stage Q (zero-padded) ----
        for (int idx = tid; idx < 16 * (HD_MAX / 8); idx += 32 * SPLIT_SCORERS) {
            const int r = idx / (HD_MAX / 8), c = idx - r * (HD_MAX / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < rows_valid && c < hd_chunks) {
                const int token = q_start + r / G, head = kvh * G + r % G;
                v = *reinterpret_cast<const uint4*>(a.q + (size_t)token * a.q_stride + (size_t)head * hd + c * 8);
            }
            *reinterpret_cast<uint4*>(Qs + r * LDS + c * 8) = v;
        }
        scorer_barrier();
        uint32_t qf[Q_IN_REGS ? NKS : 1][4];
        if (Q_IN_REGS) {
#pragma unroll
            for (int ks = 0; ks < NKS; ++ks)
                ldmatrix_x4(qf[ks], Qs + (lane & 15) * LDS + ks * 16 + 8 * (lane >> 4));
        }
        // this thread's rows: lane/4 and that + 8
        int p_row[2], t0_row[2];
        float slope_row[2];                           // the row's head's penalty on distance, in base-2 units
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (lane >> 2) + 8 * h;
            slope_row[h] = a.score_slopes && r < rows_valid ? a.score_slopes[kvh * G + r % G] * 1.4426950408889634f : 0.0f;
            if (r < rows_valid) {
                p_row[h] = pos0 + r / G;
                t0_row[h] = (a.window > 0 && p_row[h] - a.window + 1 > 0) ? p_row[h] - a.window + 1 : 0;
            } else {
                p_row[h] = -1;                        // sees nothing
                t0_row[h] = 0;
            }
        }
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
        float o[NDB][4];
#pragma unroll
        for (int d = 0; d < NDB; ++d)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[d][e] = 0.0f;

        for (int it = 0; it < cur.n_tiles; ++it) {
            const uint32_t seen = count + (uint32_t)it;
            const int buf = (int)(seen % NST);
            const int tile_start = k_begin + it * KT;
            if (wait(&full[buf], (seen / NST) & 1u)) {
                const __nv_bfloat16* kt = k_tile(buf);
                __nv_bfloat16* vt = v_tile(buf);
                if constexpr (TMA) {
                    // Whole pages arrive, the slots behind the last position included, and what a page holds there
                    // was never written by this request.  Scores of such keys are masked by assignment, but their
                    // values would be multiplied by a probability of 0, and 0 * NaN is NaN: clear those value rows
                    // (each warp its own 16).
                    const int first_dead = max(cur.t_hi + 1 - tile_start, key0);
                    if (first_dead < key0 + 16) {
                        const int chunks = (key0 + 16 - first_dead) * 8;        // 16-byte chunks per 64-column block
                        for (int idx = lane; idx < chunks * (HD_MAX / 64); idx += 32) {
                            const int cb = idx / chunks, rest = idx - cb * chunks;
                            *reinterpret_cast<uint4*>(vt + cb * (KT * 64) + (first_dead + rest / 8) * 64 + (rest & 7) * 8) =
                                make_uint4(0, 0, 0, 0);
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                    }
                }
                // ---- S = Q K^T for the 16 rows and this warp's 16 keys ----
                float s[2][4];
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nb][e] = 0.0f;
#pragma unroll
                for (int ks = 0; ks < NKS; ks += 2) {
                    uint32_t qa[4], qb[4];
                    if (Q_IN_REGS) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) { qa[e] = qf[ks][e]; qb[e] = qf[ks + 1][e]; }
                    } else {
                        const __nv_bfloat16* qrow = Qs + (lane & 15) * LDS + 8 * (lane >> 4);
                        ldmatrix_x4(qa, qrow + ks * 16);
                        ldmatrix_x4(qb, qrow + (ks + 1) * 16);
                    }
#pragma unroll
                    for (int nb = 0; nb < 2; ++nb) {
                        uint32_t b[4];     // (b0,b1): dims ks*16..+15, (b2,b3): dims (ks+1)*16..+15, keys nb*8..+7
                        ldmatrix_x4(b, tile_at<HD_MAX, TMA>(kt, key0 + nb * 8 + (lane & 7), ks * 16 + 8 * (lane >> 3)));
                        mma_bf16(s[nb], qa, b[0], b[1]);
                        mma_bf16(s[nb], qb, b[2], b[3]);
                    }
                }
                // ---- scale, mask, online softmax ----
                float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int h = e >> 1;
                        const int t = tile_start + key0 + nb * 8 + 2 * (lane & 3) + (e & 1);
                        const bool ok = t >= t0_row[h] && t <= p_row[h] && t < k_end;
                        const float v = ok ? fmaf(slope_row[h], (float)(t - p_row[h]), s[nb][e] * a.scale_log2e) : -INFINITY;
                        s[nb][e] = v;
                        tile_max[h] = fmaxf(tile_max[h], v);
                    }
                float corr[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float tm = tile_max[h];
                    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
                    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
                    const float m_new = fmaxf(m_run[h], tm);
                    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;     // a row that has seen nothing yet
                    corr[h] = exp2f(m_run[h] - m_use);
                    m_run[h] = m_new;
                    float sum = 0.0f;
#pragma unroll
                    for (int nb = 0; nb < 2; ++nb) {
                        const float p0 = exp2f(s[nb][2 * h] - m_use), p1 = exp2f(s[nb][2 * h + 1] - m_use);
                        s[nb][2 * h] = p0;
                        s[nb][2 * h + 1] = p1;
                        sum += p0 + p1;
                    }
                    l_run[h] = l_run[h] * corr[h] + sum;
                }
#pragma unroll
                for (int d = 0; d < NDB; ++d) {
                    o[d][0] *= corr[0]; o[d][1] *= corr[0];
                    o[d][2] *= corr[1]; o[d][3] *= corr[1];
                }
                uint32_t pa[4];                       // the probabilities as the A fragment of P V
                pa[0] = pack_bf16(s[0][0], s[0][1]);
                pa[1] = pack_bf16(s[0][2], s[0][3]);
                pa[2] = pack_bf16(s[1][0], s[1][1]);
                pa[3] = pack_bf16(s[1][2], s[1][3]);
                // ---- O += P V ----
#pragma unroll
                for (int d = 0; d < NDB; d += 2) {
                    uint32_t b[4];     // (b0,b1): dims d*8..+7, (b2,b3): dims (d+1)*8..+7, this warp's 16 keys
                    ldmatrix_x4_trans(b, tile_at<HD_MAX, TMA>(vt, key0 + (lane & 7) + 8 * ((lane >> 3) & 1),
                                                              d * 8 + 8 * (lane >> 4)));
                    mma_bf16(o[d], pa, b[0], b[1]);
                    mma_bf16(o[d + 1], pa, b[2], b[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty[buf]));
        }
        count += (uint32_t)cur.n_tiles;

        // ---- the segment's result: the four warps (they saw different keys of the same rows) added up ----
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
            if ((lane & 3) == 0)
                *reinterpret_cast<float2*>(sml + (warp * 16 + (lane >> 2) + 8 * h) * 2) = make_float2(m_run[h], l_run[h]);
        }
        scorer_barrier();
        float m_all[2], l_all[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (lane >> 2) + 8 * h;
            m_all[h] = -INFINITY;
#pragma unroll
            for (int w = 0; w < SPLIT_SCORERS; ++w) m_all[h] = fmaxf(m_all[h], sml[(w * 16 + r) * 2]);
            l_all[h] = 0.0f;
            float mine = 0.0f;                        // this warp's weight on the common scale
            if (m_all[h] > -INFINITY) {
#pragma unroll
                for (int w = 0; w < SPLIT_SCORERS; ++w)
                    l_all[h] += exp2f(sml[(w * 16 + r) * 2] - m_all[h]) * sml[(w * 16 + r) * 2 + 1];
                mine = exp2f(m_run[h] - m_all[h]);
            }
#pragma unroll
            for (int d = 0; d < NDB; ++d) { o[d][2 * h] *= mine; o[d][2 * h + 1] *= mine; }
        }
        // warp 0 lays its rows down, warps 1 and 2 add theirs, warp 3 adds its own and writes the result out
        const int pair = cur.seq * a.nkv + kvh;
        const bool cut = cur.n_chunks > 1;            // other CTAs hold segments of this pair too
        const size_t slot = (size_t)blockIdx.x + pair;                           // CTA index + pair index
        for (int w = 0; w < SPLIT_SCORERS; ++w) {
            if (warp == w) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = (lane >> 2) + 8 * h;
                    if (r >= rows_valid) continue;
                    float* row = o_sum + r * HD_MAX + 2 * (lane & 3);
                    if (w == 0) {
#pragma unroll
                        for (int d = 0; d < NDB; ++d)
                            *reinterpret_cast<float2*>(row + d * 8) = make_float2(o[d][2 * h], o[d][2 * h + 1]);
                    } else if (w < SPLIT_SCORERS - 1) {
#pragma unroll
                        for (int d = 0; d < NDB; ++d) {
                            float2 v = *reinterpret_cast<float2*>(row + d * 8);
                            v.x += o[d][2 * h]; v.y += o[d][2 * h + 1];
                            *reinterpret_cast<float2*>(row + d * 8) = v;
                        }
                    } else if (cut) {
                        float* po = a.part_o + (slot * 16 + r) * HD_MAX + 2 * (lane & 3);
#pragma unroll
                        for (int d = 0; d < NDB; ++d) {
                            const float2 v = *reinterpret_cast<float2*>(row + d * 8);
                            *reinterpret_cast<float2*>(po + d * 8) = make_float2(v.x + o[d][2 * h], v.y + o[d][2 * h + 1]);
                        }
                        if ((lane & 3) == 0)
                            *reinterpret_cast<float2*>(a.part_ml + (slot * 16 + r) * 2) = make_float2(m_all[h], l_all[h]);
                    } else {                          // the whole pair was this CTA's: the result itself
                        const float inv = l_all[h] > 0.0f ? 1.0f / l_all[h] : 0.0f;
                        const int token = q_start + r / G, head = kvh * G + r % G;
                        __nv_bfloat16* dst = a.out + (size_t)token * a.out_stride + (size_t)head * hd + 2 * (lane & 3);
#pragma unroll
                        for (int d = 0; d < NDB; ++d) {
                            if (d * 8 + 2 * (lane & 3) >= hd) continue;
                            const float2 v = *reinterpret_cast<float2*>(row + d * 8);
                            *reinterpret_cast<__nv_bfloat162*>(dst + d * 8) =
                                __floats2bfloat162_rn((v.x + o[d][2 * h]) * inv, (v.y + o[d][2 * h + 1]) * inv);
                        }
                    }
                }
                if (w == SPLIT_SCORERS - 1 && cut) __threadfence();    // the partial is visible before the CTA counts itself
            }
            scorer_barrier();
        }
        if (cut) {
            if (tid == 0) {
                const int arrived = atomicAdd(a.part_cnt + pair, 1);
                flags[1] = arrived == cur.n_chunks - 1;
                if (arrived == cur.n_chunks - 1) atomicExch(a.part_cnt + pair, 0);   // at rest for the next launch
            }
            scorer_barrier();
            if (flags[1] && !flags[0]) {              // the last of the pair's segments: add them all, in their order
                __threadfence();
                const size_t slot0 = (size_t)cur.c_first + pair;                     // consecutive CTAs, consecutive slots
                for (int r = warp; r < rows_valid; r += SPLIT_SCORERS) {
                    const int token = q_start + r / G, head = kvh * G + r % G;
                    merge_row<HD_MAX>(a, slot0, cur.n_chunks, r, lane,
                                      a.out + (size_t)token * a.out_stride + (size_t)head * hd);
                }
            }
        }
        if (g >= seg_hi) return;
        cur = next_seg();
    }
}

// Launches the split-key kernel with as many CTAs as are resident at once on this device (one equal stretch
// each); fills in what depends on that number.
template <int HD_MAX, bool TMA>
int launch_split(AttnArgs& a, int n_seqs, long long scratch_floats, cudaStream_t stream) {
    auto kern = attention_split_kernel<HD_MAX, TMA>;
    static int per_sm = 0, per_sm_for = -1;
    static bool configured[FB_MAX_DEVICES] = {};
    const size_t smem = split_smem_bytes(HD_MAX, TMA, (size_t)n_seqs);
    if (fb_needs_setup(configured)) {
        const size_t room = split_smem_bytes(HD_MAX, TMA, 1024);             // up to 1024 sequences in a step
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)room);
        if (e != cudaSuccess) return fb_fail(-2, "attention_split: cannot reserve %d bytes of shared memory: %s",
                                             (int)room, cudaGetErrorString(e));
        fb_setup_done(configured);
        per_sm_for = -1;
    }
    const int sms = fb_sm_count();
    if (per_sm_for != (n_seqs + 31) / 32) {           // the per-sequence arrays grow with the step
        per_sm_for = (n_seqs + 31) / 32;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
            &per_sm, kern, SPLIT_THREADS, split_smem_bytes(HD_MAX, TMA, (size_t)per_sm_for * 32));
        if (e != cudaSuccess || per_sm < 1) per_sm = 1;
    }
    a.short_ctas = sms * per_sm;
    static int min_tiles = 0;
    if (!min_tiles) {
        const char* env = getenv("FLAMBEAU_ATTN_MIN_TILES");
        min_tiles = env && atoi(env) > 0 ? atoi(env) : 3;
    }
    a.min_tiles = min_tiles;
    const long slots = a.short_ctas + (long)n_seqs * a.nkv;                 // CTA index + pair index < slots
    const long parts = slots;
    // The arrival counters come first, at a place that does not depend on the step's shape: they are zero between
    // launches, which partial results of another shape written over them would break.
    FB_REQUIRE((long)n_seqs * a.nkv <= SPLIT_COUNTERS, "attention_split: %d sequences x %d key/value heads exceed %d",
               n_seqs, a.nkv, SPLIT_COUNTERS);
    FB_REQUIRE(SPLIT_COUNTERS + parts * (16L * HD_MAX + 32) <= scratch_floats,
               "attention_split: the scratch buffer (%lld floats) is too small for %d sequences", scratch_floats,
               n_seqs);
    a.part_cnt = reinterpret_cast<int*>(a.part_o);
    a.part_o += SPLIT_COUNTERS;
    a.part_ml = a.part_o + (size_t)parts * 16 * HD_MAX;
    fb_launch((kern), dim3(a.short_ctas), SPLIT_THREADS, smem, stream, a);
    return fb_check_launch("attention_split");
}

}  // namespace

int fb_launch_attention_split(AttnArgs& a, int hd_max, bool tma, int n_seqs, float* scratch, long long scratch_floats,
                              cudaStream_t stream) {
    FB_REQUIRE(n_seqs <= 1024, "attention_split: %d sequences in one step exceed 1024", n_seqs);
    a.n_seqs = n_seqs;
    a.part_o = scratch;
    switch (hd_max) {
        case 32: return launch_split<32, false>(a, n_seqs, scratch_floats, stream);
        case 64: return tma ? launch_split<64, true>(a, n_seqs, scratch_floats, stream)
                            : launch_split<64, false>(a, n_seqs, scratch_floats, stream);
        case 128: return tma ? launch_split<128, true>(a, n_seqs, scratch_floats, stream)
                             : launch_split<128, false>(a, n_seqs, scratch_floats, stream);
        default: return tma ? launch_split<256, true>(a, n_seqs, scratch_floats, stream)
                            : launch_split<256, false>(a, n_seqs, scratch_floats, stream);
    }
}
