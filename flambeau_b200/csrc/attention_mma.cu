// Paged causal (sliding-window) attention for bfloat16 on the tensor cores
// (mma.sync m16n8k16, float32 accumulation and softmax), one kernel in two
// arrangements:
//
//   LONG  (prompt portions): a CTA owns one key/value head and a tile of up to 128
//         query rows = (128 / G) tokens x the G query heads that share the head, so
//         every K/V tile is read once for the whole group.  Its four warps take 32
//         rows each, so that every K/V fragment fetched from shared memory feeds two
//         row blocks; each walks all visible key tiles with an online softmax.
//   SHORT (decoded tokens and portions of a few tokens, rows = tokens x G <= 16):
//         the key tiles of all (sequence, key/value head) pairs of the step form one
//         line that a fixed grid of CTAs cuts into equal stretches, so that every SM
//         streams the same amount of cache whatever the batch looks like.  A CTA's
//         four warps share the 16 rows and split every 64-key tile; their partial
//         (m, l, o) are merged in shared memory.  Where a pair was cut, each of its
//         segments goes to scratch and the CTA that arrives last adds them up.
//
// Keys and values come through the block table in tiles of 64 keys with
// bulk copies through a 2-3 stage pipeline; a key outside [t0, p] of every row of the CTA is
// not read at all (its slot in shared memory is zero-filled), so pages that the
// cache manager has taken back are never touched.  Softmax runs in base 2 with
// scale*log2(e) folded into the scores.  Head sizes are padded with zeros to
// HD_MAX in shared memory, so any head size that is a multiple of 8 runs.
//
// Formulas: crates/kernels-hip/src/kernels/attention_prefill_flash_tile_f16.cu:73-213
// (tile + online softmax), attention_decode_f16_splitk.cu:215-256 (merge of chunks).
#include "async_copy.cuh"
#include "tensor_map.cuh"

namespace {

constexpr int KT = 64;             // keys per tile
constexpr int ATT_THREADS = 128;   // SHORT arrangement: four warps that split each tile's keys
constexpr int LONG_THREADS = 128;  // LONG arrangement: four warps of 32 query rows

// 16-row blocks per warp of the LONG arrangement: two while the accumulators fit in registers.
__host__ __device__ constexpr int long_row_blocks(int hd_max, bool short_rows) {
    return (short_rows || hd_max > 128) ? 1 : 2;
}
__host__ __device__ constexpr int attn_stages(int hd_max, bool short_rows) {
    // SHORT streams the cache once: three tiles (two in flight).  LONG reuses a tile for 128 rows and wants two
    // CTAs on an SM more than it wants a third tile.
    return (short_rows && hd_max <= 128) ? 3 : 2;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return smem_u32(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnArgs {
    CUtensorMap map_k, map_v;          // TMA mode: the pools as [pages * kv heads * page size, hd] matrices
    const __nv_bfloat16* q; long q_stride;
    __nv_bfloat16* out; long out_stride;
    const __nv_bfloat16* k_pool; const __nv_bfloat16* v_pool;
    int page_size, n_pages;
    const int* block_table; int table_stride;
    const int* seq_q_start; const int* seq_q_len; const int* seq_pos_start;
    int nh, nkv, hd, window;
    float scale_log2e;
    float* part_o; float* part_ml;     // SHORT: partial results, [slot][16 rows][HD_MAX] and [slot][16][2]
    int* part_cnt;                     // SHORT: per (sequence, key/value head), segments that have arrived; 0 at rest
    int n_seqs;                        // sequences of the step
    int short_ctas;                    // SHORT: CTAs of the split-key launch
    int short_rows;                    // sequences with q_len * G <= short_rows belong to the SHORT arrangement
    int* status;
};

// The keys a group of consecutive query tokens [first, last] of a sequence can see, and where tiles start.
struct KeyRange { int t_lo, t_hi, tile_lo; };
__device__ __forceinline__ KeyRange key_range(int p_first, int p_last, int window) {
    KeyRange r;
    r.t_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    r.t_hi = p_last;
    r.tile_lo = (r.t_lo / KT) * KT;
    return r;
}

// SHORT arrangement.  All key tiles of all (sequence, key/value head) pairs form one line, pair after pair (pairs
// of one sequence side by side), and the CTAs of the launch cut that line into equal stretches: CTA c owns tiles
// [c * per, (c + 1) * per).  A stretch may end inside a pair and go on into the next ones, so every CTA has the
// same amount of cache to stream whatever the number and the lengths of the sequences.  Each (CTA, pair) segment
// of a pair that is cut leaves a partial result in slot (CTA index + pair index), which is unique and needs no
// table, and counts itself on the pair; the CTA that arrives last adds the pair's segments, in their order.
__device__ __forceinline__ int short_tiles_of(const AttnArgs& a, int q_len, int pos0, int G) {
    if (q_len * G > a.short_rows) return 0;                 // belongs to the LONG arrangement
    const KeyRange kr = key_range(pos0, pos0 + q_len - 1, a.window);
    return (kr.t_hi - kr.tile_lo) / KT + 1;
}

// Per-sequence facts of the SHORT arrangement in shared memory: five arrays of n_seqs (+1) ints.
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

// Where element (row, dim) of a K/V tile lives in shared memory (dim a multiple of 8).
//   padded:  rows of HD_MAX + 8 elements (the per-row bulk copies land here);
//   swizzled (TMA mode): HD_MAX / 64 column blocks of [64 rows][128 bytes], the 16-byte chunks of a row
//   XOR-ed with (row & 7), which is how a tensor-map copy with the 128-byte swizzle stores a box.
template <int HD_MAX, bool TMA>
__device__ __forceinline__ const __nv_bfloat16* tile_at(const __nv_bfloat16* tile, int row, int dim) {
    if (TMA) return tile + (dim >> 6) * (KT * 64) + row * 64 + ((((dim & 63) >> 3) ^ (row & 7)) << 3);
    return tile + row * (HD_MAX + 8) + dim;
}

// Adds the segments of one row of a pair: out = sum_c 2^(m_c - m) o_c / sum_c 2^(m_c - m) l_c, segments in slots
// slot0 .. slot0 + n_chunks - 1.  One warp: a lane first takes a segment (its maximum, sum and weight), then a share
// of the head's columns.  The partials were written by other SMs: they are read past the L1.
template <int HD_MAX>
__device__ __forceinline__ void merge_row(const AttnArgs& a, size_t slot0, int n_chunks, int r, int lane,
                                          __nv_bfloat16* dst) {
    constexpr int U = 8;                               // segments whose loads are in flight together
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

template <int HD_MAX, bool SHORT, bool TMA>
__global__ void __launch_bounds__(SHORT ? ATT_THREADS : LONG_THREADS)
attention_mma_kernel(const __grid_constant__ AttnArgs a) {
    constexpr int NT = SHORT ? ATT_THREADS : LONG_THREADS;
    fb_pdl_launch_dependents();
    // The step's descriptor was on the device before the step's first kernel: everything up to the first read of
    // Q or of the cache (the CTA's share of the work, barriers, clearing) runs ahead of the kernel before this one.
    constexpr int LDS = HD_MAX + 8;                 // row stride of Q (and of K/V when padded): 16 bytes of padding
    constexpr int TILE_ELEMS = TMA ? KT * HD_MAX : KT * LDS;
    constexpr int NKS = HD_MAX / 16;                // k-steps of Q K^T
    constexpr int NDB = HD_MAX / 8;                 // n-blocks of P V
    constexpr int ROWS = SHORT ? 16 : 64 * long_row_blocks(HD_MAX, SHORT);   // query rows per CTA
    constexpr int WARP_KEYS = SHORT ? 16 : KT;      // keys of a tile that one warp scores
    constexpr int NSB = WARP_KEYS / 8;              // n-blocks of S per warp
    constexpr int R = long_row_blocks(HD_MAX, SHORT);   // 16-row blocks per warp: K/V fragments are reused R times
    constexpr bool Q_IN_REGS = SHORT && HD_MAX <= 128;
    constexpr int NST = attn_stages(HD_MAX, SHORT);    // K/V tiles in shared memory (NST - 1 in flight)

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
    float* sml = reinterpret_cast<float*>(tail + 64);                           // SHORT: [4 warps][16][2]
    const ShortSeqs ss(reinterpret_cast<int*>(tail + 64 + 512), a.n_seqs);      // SHORT: per-sequence facts

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.nh / a.nkv;
    const int hd = a.hd, hd_chunks = hd / 8;
    // TMA mode: one copy per (K or V, page of the tile, 64-column block), issued by thread number = op number
    const int pages_per_tile = TMA ? KT / a.page_size : 1;
    const int col_blocks = TMA ? hd / 64 : 1;
    const int tma_ops = 2 * pages_per_tile * col_blocks;

    // One piece of work: query tokens [tok0, tok0 + ntok) of a sequence, one key/value head, keys [k_begin, k_end).
    // LONG: the CTA's only one.  SHORT: a segment of the CTA's stretch.
    struct Seg {
        int seq, kvh, q_start, pos0, tok0, ntok, t_lo, t_hi, k_begin, k_end, n_tiles;
        int c_first, n_chunks;             // SHORT: the first CTA with a segment of this pair, and how many have one
        const int* table;
    };
    auto make_seg = [&](int seq, int kvh, int q_start, int pos0, int tok0, int ntok, int tile_a, int tile_b) {
        Seg sg;
        sg.seq = seq; sg.kvh = kvh; sg.q_start = q_start; sg.pos0 = pos0; sg.tok0 = tok0; sg.ntok = ntok;
        const KeyRange kr = key_range(pos0 + tok0, pos0 + tok0 + ntok - 1, a.window);
        sg.t_lo = kr.t_lo; sg.t_hi = kr.t_hi;
        sg.k_begin = kr.tile_lo + tile_a * KT;
        sg.k_end = tile_b < 0 ? kr.t_hi + 1 : min(kr.t_hi + 1, kr.tile_lo + tile_b * KT);
        sg.n_tiles = (sg.k_end - sg.k_begin + KT - 1) / KT;
        sg.table = a.block_table + (size_t)seq * a.table_stride;
        sg.c_first = 0; sg.n_chunks = 1;
        return sg;
    };

    // ---- what this CTA has to do ----
    int g = 0, seg_hi = 0, cur_seq = 0;    // SHORT: the next tile of its stretch, the stretch's end, the sequence of g
    int per = 1;                           // SHORT: tiles per CTA
    if (SHORT) {
        short_prefix(a, G, ss, tid, NT);
        const long total = (long)a.nkv * ss.prefix[a.n_seqs];
        per = (int)((total + gridDim.x - 1) / gridDim.x);
        g = (int)min((long)blockIdx.x * per, total);
        seg_hi = (int)min((long)g + per, total);
        if (g >= seg_hi) return;
    }
    auto next_seg = [&]() {                // SHORT: the segment that starts at tile g; moves g past it
        while ((long)a.nkv * ss.prefix[cur_seq + 1] <= g) ++cur_seq;
        const int seq = cur_seq, n = ss.tiles[seq];
        const int within = g - a.nkv * ss.prefix[seq];                          // tiles into this sequence's pairs
        const int kvh = within / n, tile_a = within - kvh * n;
        const int tile_b = min(n, tile_a + (seg_hi - g));
        g += tile_b - tile_a;
        Seg sg = make_seg(seq, kvh, ss.q_start[seq], ss.pos0[seq], 0, ss.q_len[seq], tile_a, tile_b);
        const long first_tile = (long)a.nkv * ss.prefix[seq] + (long)kvh * n;   // of the pair, in the line of tiles
        sg.c_first = (int)(first_tile / per);
        sg.n_chunks = (int)((first_tile + n - 1) / per) - sg.c_first + 1;
        return sg;
    };
    Seg cur;
    if (SHORT) {
        cur = next_seg();
    } else {
        const int seq = blockIdx.z, q_len = a.seq_q_len[seq];
        if (q_len * G <= a.short_rows) return;
        const int TQ = ROWS / G;
        const int tok0 = (gridDim.x - 1 - blockIdx.x) * TQ;       // later tiles see more keys: start them first
        if (tok0 >= q_len) return;
        cur = make_seg(seq, blockIdx.y, a.seq_q_start[seq], a.seq_pos_start[seq], tok0, min(TQ, q_len - tok0), 0, -1);
    }

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
    // copy can be issued without waiting for the table: -2 = nothing to fetch there (no query of this piece sees
    // it), -1 = the table has no page although one is needed (flagged when the tile is issued).
    auto lookup = [&](const Seg& sg, int tile_start) -> int {
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
        if (!(t_first + span > sg.t_lo && t_first < sg.k_end)) return -2;
        const int page = sg.table[t_first / a.page_size];
        return (page < 0 || page >= a.n_pages) ? -1 : page;
    };

    // TMA mode: thread number = copy number: (K or V, page of the tile, 64-column block), one tensor-map copy each.
    // Otherwise: one row of 64 keys (threads 0..63) or 64 values (threads 64..127) per thread: a bulk copy of the
    // row's hd*2 bytes.  Copies are counted on the tile's barrier.  What no query of this piece may see (before the
    // window, past the last position, or in another segment) is not read.
    auto load_tile = [&](const Seg& sg, int buf, int tile_start, int page) {
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
                            (page * a.nkv + sg.kvh) * a.page_size);
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
            const size_t off = (((size_t)page * a.nkv + sg.kvh) * a.page_size + (t % a.page_size)) * hd;
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

    // Puts the first NST - 1 tiles of a piece in flight (`count` tiles went through the buffers before it) and
    // returns the page id for the tile after them, already on its way.
    auto prologue = [&](const Seg& sg, uint32_t count) -> int {
        int page = lookup(sg, sg.k_begin);
#pragma unroll
        for (int st = 0; st < NST - 1; ++st)
            if (st < sg.n_tiles) {
                load_tile(sg, (int)((count + st) % NST), sg.k_begin + st * KT, page);
                page = lookup(sg, sg.k_begin + (st + 1) * KT);
            }
        return page;
    };

    uint32_t tiles_done = 0;               // tiles this CTA has consumed: buffer and barrier phase follow from it
    int next_page = prologue(cur, 0);

  for (;;) {                               // one pass per piece; LONG: exactly one
    const int kvh = cur.kvh, q_start = cur.q_start, pos0 = cur.pos0, tok0 = cur.tok0;
    const int rows_valid = cur.ntok * G;
    const int k_begin = cur.k_begin, k_end = cur.k_end, n_tiles = cur.n_tiles, t_hi = cur.t_hi;

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
    __syncthreads();                                  // Q staged (and, after a segment, its merge buffer cleared)

    const int row_base = SHORT ? 0 : warp * (16 * R);   // first row of this warp within the CTA
    const int key0 = SHORT ? warp * 16 : 0;             // first key of this warp within a tile
    uint32_t qf[Q_IN_REGS ? NKS : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int ks = 0; ks < NKS; ++ks)
            ldmatrix_x4(qf[ks], Qs + (row_base + (lane & 15)) * LDS + ks * 16 + 8 * (lane >> 4));
    }
    // per-thread rows of row block rb: row_base + 16*rb + lane/4 and that + 8
    int p_row[R][2], t0_row[R][2];
#pragma unroll
    for (int rb = 0; rb < R; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = row_base + 16 * rb + (lane >> 2) + 8 * h;
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
        const uint32_t seen = tiles_done + (uint32_t)it;
        const int buf = (int)(seen % NST);
        const int tile_start = k_begin + it * KT;
        if (!mbar_wait(smem_u32(&full[buf]), (seen / NST) & 1u, a.status)) *bail = 1;
        __syncthreads();                              // every thread is past tile it-1: its buffer is free
        if (*bail) break;
        if (it + NST - 1 < n_tiles) {
            load_tile(cur, (int)((seen + NST - 1) % NST), tile_start + (NST - 1) * KT, next_page);
            next_page = lookup(cur, tile_start + NST * KT);    // consumed one iteration from now
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
                if (Q_IN_REGS) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) { qa[rb][e] = qf[ks][e]; qb[rb][e] = qf[ks + 1][e]; }
                } else {
                    const __nv_bfloat16* qrow = Qs + (row_base + 16 * rb + (lane & 15)) * LDS + 8 * (lane >> 4);
                    ldmatrix_x4(qa[rb], qrow + ks * 16);
                    ldmatrix_x4(qb[rb], qrow + (ks + 1) * 16);
                }
            }
#pragma unroll
            for (int nb = 0; nb < NSB; ++nb) {
                uint32_t b[4];     // (b0,b1): dims ks*16..+15, (b2,b3): dims (ks+1)*16..+15, keys nb*8..+7
                ldmatrix_x4(b, tile_at<HD_MAX, TMA>(kt, key0 + nb * 8 + (lane & 7), ks * 16 + 8 * (lane >> 3)));
#pragma unroll
                for (int rb = 0; rb < R; ++rb) {
                    mma_bf16(s[rb][nb], qa[rb], b[0], b[1]);
                    mma_bf16(s[rb][nb], qb[rb], b[2], b[3]);
                }
            }
        }
        // ---- scale, mask, online softmax ----
        uint32_t pa[R][WARP_KEYS / 16][4];            // the probabilities as A fragments of P V
#pragma unroll
        for (int rb = 0; rb < R; ++rb) {
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < NSB; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int t = tile_start + key0 + nb * 8 + 2 * (lane & 3) + (e & 1);
                    const bool ok = t >= t0_row[rb][h] && t <= p_row[rb][h] && t < k_end;
                    const float v = ok ? s[rb][nb][e] * a.scale_log2e : -INFINITY;
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
            for (int kk = 0; kk < WARP_KEYS / 16; ++kk) {
                pa[rb][kk][0] = pack_bf16(s[rb][2 * kk][0], s[rb][2 * kk][1]);
                pa[rb][kk][1] = pack_bf16(s[rb][2 * kk][2], s[rb][2 * kk][3]);
                pa[rb][kk][2] = pack_bf16(s[rb][2 * kk + 1][0], s[rb][2 * kk + 1][1]);
                pa[rb][kk][3] = pack_bf16(s[rb][2 * kk + 1][2], s[rb][2 * kk + 1][3]);
            }
        }
        // ---- O += P V: every V fragment serves all R row blocks ----
#pragma unroll
        for (int kk = 0; kk < WARP_KEYS / 16; ++kk) {
#pragma unroll
            for (int d = 0; d < NDB; d += 2) {
                uint32_t b[4];     // (b0,b1): dims d*8..+7, (b2,b3): dims (d+1)*8..+7, keys kk*16..+15
                ldmatrix_x4_trans(b, tile_at<HD_MAX, TMA>(vt, key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1),
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
    tiles_done += (uint32_t)n_tiles;
#pragma unroll
    for (int rb = 0; rb < R; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[rb][h] += __shfl_xor_sync(0xffffffffu, l_run[rb][h], 1);
            l_run[rb][h] += __shfl_xor_sync(0xffffffffu, l_run[rb][h], 2);
        }

    if (!SHORT) {
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
        return;
    }

    // ---- SHORT: the next segment's first tiles go on their way, then the four warps (they saw different keys of
    // the same rows) are merged into one partial.  The merge buffer is the stage used last, which the next
    // segment's first NST - 1 tiles do not touch.
    const bool more = g < seg_hi;
    Seg nxt = cur;
    if (more) {
        nxt = next_seg();
        next_page = prologue(nxt, tiles_done);
    }
    float* so = reinterpret_cast<float*>(k_tile((int)((tiles_done + NST - 1) % NST)));      // [4 warps][16][HD_MAX]
    static_assert(!SHORT || 4 * 16 * HD_MAX * 4 <= 2 * KT * HD_MAX * 2, "the merge buffer fits in one stage");
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + 8 * h;
#pragma unroll
        for (int d = 0; d < NDB; ++d) {
            const int col = d * 8 + 2 * (lane & 3);
            *reinterpret_cast<float2*>(so + (warp * 16 + r) * HD_MAX + col) = make_float2(o[0][d][2 * h], o[0][d][2 * h + 1]);
        }
        if ((lane & 3) == 0) {
            sml[(warp * 16 + r) * 2] = m_run[0][h];
            sml[(warp * 16 + r) * 2 + 1] = l_run[0][h];
        }
    }
    __syncthreads();
    const int pair = cur.seq * a.nkv + kvh;
    const bool cut = cur.n_chunks > 1;                // other CTAs hold segments of this pair too
    float* po = a.part_o + ((size_t)blockIdx.x + pair) * 16 * HD_MAX;        // slot = CTA index + pair index
    float* pml = a.part_ml + ((size_t)blockIdx.x + pair) * 16 * 2;
    for (int idx = tid; idx < rows_valid * HD_MAX; idx += NT) {
        const int r = idx / HD_MAX, c = idx - r * HD_MAX;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, sml[(w * 16 + r) * 2]);
        float acc = 0.0f, l = 0.0f;
        if (m > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float wgt = exp2f(sml[(w * 16 + r) * 2] - m);
                acc += wgt * so[(w * 16 + r) * HD_MAX + c];
                l += wgt * sml[(w * 16 + r) * 2 + 1];
            }
        }
        if (cut) {
            po[idx] = acc;
            if (c == 0) { pml[r * 2] = m; pml[r * 2 + 1] = l; }
        } else if (c < hd) {                          // the whole pair was this CTA's: the result itself
            const int token = q_start + r / G, head = kvh * G + r % G;
            a.out[(size_t)token * a.out_stride + (size_t)head * hd + c] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
        }
    }
    if (cut) __threadfence();                         // the partial is visible before this CTA counts itself
    __syncthreads();                                  // every thread has read the merge buffer
    if (cut) {
        if (tid == 0) {
            const int arrived = atomicAdd(a.part_cnt + pair, 1);
            bail[1] = arrived == cur.n_chunks - 1;
            if (bail[1]) atomicExch(a.part_cnt + pair, 0);                     // at rest again for the next launch
        }
        __syncthreads();
        if (bail[1]) {                                // the last of the pair's segments: add them all
            __threadfence();
            const size_t slot0 = (size_t)cur.c_first + pair;                   // consecutive CTAs, consecutive slots
            for (int r = warp; r < rows_valid; r += NT / 32) {
                const int token = q_start + r / G, head = kvh * G + r % G;
                merge_row<HD_MAX>(a, slot0, cur.n_chunks, r, lane,
                                  a.out + (size_t)token * a.out_stride + (size_t)head * hd);
            }
        }
    }
    if (!more) return;
    // that stage receives the next segment's tile NST - 1: make it finite again (see the clearing above)
    if (TMA) {
        for (int idx = tid; idx < 2 * TILE_ELEMS / 8; idx += NT)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(so) + idx * 8) = make_uint4(0, 0, 0, 0);
    } else if (hd < HD_MAX) {
        const int pad_chunks = HD_MAX / 8 - hd_chunks;
        for (int idx = tid; idx < 2 * KT * pad_chunks; idx += NT) {
            const int r = idx / pad_chunks, c = hd_chunks + idx - r * pad_chunks;
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(so) + r * LDS + c * 8) = make_uint4(0, 0, 0, 0);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    cur = nxt;
  }
}

// (plus 16 + short_seqs_bytes(sequences) for the SHORT arrangement's per-sequence facts, added at launch)
__host__ __device__ constexpr size_t attn_smem_bytes(int hd_max, bool short_rows, bool tma) {
    return (size_t)(short_rows ? 16 : 64 * long_row_blocks(hd_max, false)) * (hd_max + 8) * 2 + 1024 /* alignment */ +
           (size_t)2 * attn_stages(hd_max, short_rows) * KT * (tma ? hd_max : hd_max + 8) * 2 + 64 /* barriers */ +
           (short_rows ? 512 : 0) /* merge maxima and sums */;
}

template <int HD_MAX, bool SHORT, bool TMA>
int launch_one(const AttnArgs& a, dim3 grid, const char* what, cudaStream_t stream) {
    constexpr size_t base = attn_smem_bytes(HD_MAX, SHORT, TMA);
    constexpr size_t room = base + 16 + short_seqs_bytes(1024);      // up to 1024 sequences in the SHORT arrangement
    const size_t smem = base + 16 + (SHORT ? short_seqs_bytes(a.n_seqs) : 0);
    auto kern = attention_mma_kernel<HD_MAX, SHORT, TMA>;
    static bool configured = false;
    if (!configured && room > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)room);
        if (e != cudaSuccess) return fb_fail(-2, "%s: cannot reserve %d bytes of shared memory: %s", what, (int)room,
                                             cudaGetErrorString(e));
        configured = true;
    }
    fb_launch((kern), grid, SHORT ? ATT_THREADS : LONG_THREADS, smem, stream, a);
    return fb_check_launch(what);
}

// CTAs of the SHORT arrangement that are resident at once on this device (its grid: one equal stretch each).
template <int HD_MAX, bool TMA>
int short_resident_ctas(int n_seqs) {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const size_t smem = attn_smem_bytes(HD_MAX, true, TMA) + 16 + short_seqs_bytes(n_seqs);
    int per_sm = (int)(227 * 1024 / (smem + 1024));           // shared memory is what limits them
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    return sms * per_sm;
}

template <int HD_MAX>
int launch_attention_mma(const AttnArgs& args, bool tma, int n_seqs, int max_q_len, int any_short, int any_long,
                         long long scratch_floats, cudaStream_t stream) {
    AttnArgs a = args;
    const int G = a.nh / a.nkv;
    if (any_short) {
        if constexpr (HD_MAX >= 64) a.short_ctas = tma ? short_resident_ctas<HD_MAX, true>(n_seqs)
                                                       : short_resident_ctas<HD_MAX, false>(n_seqs);
        else a.short_ctas = short_resident_ctas<HD_MAX, false>(n_seqs);
        const long slots = a.short_ctas + (long)n_seqs * a.nkv;          // CTA index + pair index < slots
        FB_REQUIRE(slots * (16L * HD_MAX + 32) + (long)n_seqs * a.nkv <= scratch_floats,
                   "attention_mma: the scratch buffer (%lld floats) is too small for %d sequences", scratch_floats,
                   n_seqs);
        a.part_ml = a.part_o + (size_t)slots * 16 * HD_MAX;
        a.part_cnt = reinterpret_cast<int*>(a.part_ml + (size_t)slots * 32);
    }
    if (any_long) {
        const int TQ = 64 * long_row_blocks(HD_MAX, false) / G;
        const dim3 grid((max_q_len + TQ - 1) / TQ, a.nkv, n_seqs);
        int rc;
        if constexpr (HD_MAX >= 64) {
            rc = tma ? launch_one<HD_MAX, false, true>(a, grid, "attention_mma (long)", stream)
                     : launch_one<HD_MAX, false, false>(a, grid, "attention_mma (long)", stream);
        } else {
            rc = launch_one<HD_MAX, false, false>(a, grid, "attention_mma (long)", stream);
        }
        if (rc) return rc;
    }
    if (any_short) {
        const dim3 grid(a.short_ctas, 1, 1);
        int rc;
        if constexpr (HD_MAX >= 64) {
            rc = tma ? launch_one<HD_MAX, true, true>(a, grid, "attention_mma (short)", stream)
                     : launch_one<HD_MAX, true, false>(a, grid, "attention_mma (short)", stream);
        } else {
            rc = launch_one<HD_MAX, true, false>(a, grid, "attention_mma (short)", stream);
        }
        if (rc) return rc;
    }
    return 0;
}

}  // namespace

// q, out: bfloat16 [rows, heads*hd]; pools bfloat16 [pages][kv heads][page size][hd].
// seq_*: per sequence of the step (device int32).  max_q_len / max_kv_len / any_short / any_long come from the
// host's copy of the step descriptor.  `scratch` holds the partials of the SHORT arrangement.
FB_API int fb_paged_attention_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* k_pool, const void* v_pool, int page_size, int n_pages,
                                  const int* block_table, int table_stride, const int* seq_q_start,
                                  const int* seq_q_len, const int* seq_pos_start, int n_seqs, int max_q_len,
                                  int max_kv_len, int any_short, int any_long, int nh, int nkv, int hd, int window,
                                  float scale, float* scratch, long long scratch_floats, int* status,
                                  cudaStream_t stream) {
    FB_REQUIRE(n_seqs >= 0 && nh > 0 && nkv > 0 && hd > 0, "attention_mma: bad sizes");
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
    a.block_table = block_table; a.table_stride = table_stride;
    a.seq_q_start = seq_q_start; a.seq_q_len = seq_q_len; a.seq_pos_start = seq_pos_start;
    a.nh = nh; a.nkv = nkv; a.hd = hd; a.window = window;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.status = status;
    a.short_rows = G <= 16 ? 16 : 0;               // with more than 16 heads per group even one token is "long"
    if (a.short_rows == 0) { any_long = any_long || any_short; any_short = 0; }
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
    a.short_ctas = 0;
    a.part_o = scratch;
    a.part_ml = nullptr;
    a.part_cnt = nullptr;
    FB_REQUIRE(!any_short || n_seqs <= 1024, "attention_mma: %d sequences in one step exceed 1024", n_seqs);
    switch (HD_MAX) {
        case 32: return launch_attention_mma<32>(a, tma, n_seqs, max_q_len, any_short, any_long, scratch_floats, stream);
        case 64: return launch_attention_mma<64>(a, tma, n_seqs, max_q_len, any_short, any_long, scratch_floats, stream);
        case 128: return launch_attention_mma<128>(a, tma, n_seqs, max_q_len, any_short, any_long, scratch_floats, stream);
        default: return launch_attention_mma<256>(a, tma, n_seqs, max_q_len, any_short, any_long, scratch_floats, stream);
    }
}
