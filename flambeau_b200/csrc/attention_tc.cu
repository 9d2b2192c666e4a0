// Paged causal (sliding-window) attention for portions of prompts on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), for heads of 64 or 128 bfloat16 and pages that tile 64 keys.
//
// A CTA owns one key/value head and 256 query rows = (256 / G) tokens x the G query heads that share the head, as
// two row tiles of 128 that use every K/V tile fetched (one row tile when two would leave SMs without work), and
// walks the visible keys in tiles of 64.  CTAs are numbered heaviest first over all heads and sequences.
//
//   S = Q K^T      tcgen05.mma, Q and K K-major in shared memory (128-byte swizzle), S in tensor memory, two
//                  buffers per row tile: the scores run two key tiles ahead of the softmax;
//   softmax        one thread per row (the row = its tensor-memory lane): the row's 64 scores in one tcgen05.ld
//                  round trip, base-2 online softmax in float32, P rounded to bfloat16 and stored with tcgen05.st
//                  over the scores it came from;
//   O += P V       tcgen05.mma with P read from tensor memory and V as it lies in the cache ([key][dim], the
//                  MN-major operand); O in tensor memory.
//
// O is rescaled only when a row's maximum has grown by more than 2^8 since the exponentials' reference point was
// last moved (the sum l is kept against the same reference, so O / l is exact either way); the first tile sets
// the reference.  Warps: 0 fetches K and V pages with tensor-map copies through four-slot rings of their own (page
// ids read from the block table 32 at a time); 1 owns tensor memory; 1 and 2 issue the MMAs of row tiles 0 and 1;
// 4..7 and 8..11 are the softmax of the two row tiles (a warp reads the quarter of the lanes given by its index
// modulo 4).  A wait names a phase of an mbarrier only by its parity, so every barrier here is waited on for the
// phase that is current or just completed: one barrier per buffer, and one of its own for the last product.  Every
// wait is bounded in time; when one runs out the kernel flags it, leaves its loops, frees its tensor memory and
// returns.
//
// Formulas: crates/kernels-hip/src/kernels/attention_prefill_flash_tile_f16.cu:73-213 (tile + online softmax).
#include "attention_common.cuh"
#include "umma.cuh"

namespace {

using namespace fb_attn;

constexpr int BM = 128;            // query rows per row tile (the M of the MMAs)
constexpr int BN = 64;             // keys per tile
// Threads of a CTA with RT row tiles: warp 0 fetches, warps 1 and 2 issue the MMAs of row tiles 0 and 1 (warp 3 has no
// work), warps 4..7 (and 8..11) are the softmax of row tile 0 (and 1).
__host__ __device__ constexpr int tc_threads(int rt) { return 128 + BM * rt; }
constexpr int NKV = 4;             // K slots and V slots
constexpr int TMEM_COLS = 512;     // S/P buffer b of row tile t at (2t + b) * 64; O of row tile t at RT * 128 + t * 128
constexpr float RESCALE_STEP = 8.0f;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD, int RT> struct TcSmem {
    static constexpr int Q_BYTES = BM * HD * 2;                 // one row tile: [HD/64 column blocks][128 rows][128 bytes]
    static constexpr int KV_BYTES = BN * HD * 2;                // one K or V tile: [HD/64][64 keys][128 bytes]
    static constexpr int TAIL_BYTES = 256;                      // barriers, tensor-memory address, flag
    static constexpr int USED = RT * Q_BYTES + NKV * 2 * KV_BYTES + TAIL_BYTES + 1024 /* alignment */;
    // one CTA per SM: two would both want all of tensor memory
    static constexpr int BYTES = USED > 120 * 1024 ? USED : 120 * 1024;
};

// RT row tiles of 128 rows per CTA: with two, both use every K/V tile that is fetched and the tensor pipe works for
// one under the softmax of the other; with one, a short portion still spreads over enough CTAs.
template <int HD, int RT>
__global__ void __launch_bounds__(tc_threads(RT), 1)
attention_tc_kernel(const __grid_constant__ AttnArgs a) {
    fb_pdl_launch_dependents();
    using SM = TcSmem<HD, RT>;
    constexpr int CB = HD / 64;                                 // 64-column blocks of a head
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    uint8_t* Qs = smem;                                         // [RT] row tiles
    uint8_t* Ks = Qs + RT * SM::Q_BYTES;                        // [NKV] tiles
    uint8_t* Vs = Ks + NKV * SM::KV_BYTES;                      // [NKV] tiles
    uint8_t* tail = Vs + NKV * SM::KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
    uint64_t* k_full = bars;                                    // [NKV] a K tile has landed
    uint64_t* k_empty = bars + NKV;                             // [NKV] both row tiles' scores are computed
    uint64_t* v_full = bars + 2 * NKV;                          // [NKV] a V tile has landed
    uint64_t* v_empty = bars + 3 * NKV;                         // [NKV] both row tiles' products are computed
    uint64_t* s_full = bars + 4 * NKV;                          // [RT][2] S of a row tile is in tensor memory (two buffers)
    uint64_t* p_full = bars + 4 * NKV + 2 * RT;                 // [RT][2] P of a row tile is in tensor memory, per buffer:
                                                                //       the softmax may be two tiles ahead of the products
    uint64_t* pv_done = bars + 4 * NKV + 4 * RT;                // [RT]  O of a row tile holds the key tile's product
    uint64_t* o_done = bars + 4 * NKV + 5 * RT;                 // [RT]  O of a row tile holds all products (used once)
    uint64_t* q_full = bars + 4 * NKV + 6 * RT;                 //       Q is staged
    uint64_t* v_clean = bars + 4 * NKV + 6 * RT + 1;            //       row tile 0 has cleared a V tile's unseen rows (at most twice)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * NKV + 6 * RT + 2);
    int* bail = reinterpret_cast<int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.nh / a.nkv, hd = a.hd;

    // ---- what this CTA has to do: query tokens [tok0, tok0 + ntok) of a sequence, one key/value head ----
    // CTAs are numbered heaviest first over the whole step: the last tokens of every sequence and head (they see
    // the most keys) get the first SMs, whatever head or sequence they belong to
    const int pairs = a.nkv * portion_seqs(a);
    const int rank = blockIdx.x / pairs, pair = blockIdx.x - rank * pairs;
    const int seq = portion_seq(a, pair / a.nkv), kvh = pair % a.nkv;
    const int q_tiles = gridDim.x / pairs;
    const int q_len = a.seq_q_len[seq];
    if (q_len * G <= a.short_rows) return;                      // the split-key arrangement's
    const int TQ = RT * BM / G;
    const int tok0 = (q_tiles - 1 - rank) * TQ;               // later tokens see more keys: start them first
    if (tok0 >= q_len) return;
    const int ntok = min(TQ, q_len - tok0);
    const int q_start = a.seq_q_start[seq], pos0 = a.seq_pos_start[seq];
    const int rows_valid = ntok * G;                            // of the CTA's RT * 128 rows
    const int p_first = pos0 + tok0, p_last = pos0 + tok0 + ntok - 1;
    const int t_lo = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;
    const int t_hi = p_last;
    const int k_begin = (t_lo / BN) * BN, k_end = t_hi + 1;
    const int n_tiles = (k_end - k_begin + BN - 1) / BN;        // both row tiles walk all of them
    const int* table = a.block_table + (size_t)seq * a.table_stride;
    const int pages_per_tile = BN / a.page_size;
    const int n_ops = pages_per_tile * CB;                      // copies per K or V tile: (page, column block)
    // Value rows no query of the CTA sees: pages of the first tile wholly before the window, keys of the last tile
    // behind the last position.  Whole pages arrive, the slots behind the last position included, and what a page
    // holds there was never written by this request; pages wholly before the window or behind the last position do
    // not arrive at all, and their slots hold whatever was there.  The probabilities of such keys are 0, but
    // 0 * NaN is NaN: the softmax of row tile 0 clears those rows, 128 bytes per key and column block, before it
    // lets its product start, and says so on a barrier that the thread of row tile 1's products waits for.
    const int dead_lo_first = ((t_lo - k_begin) / a.page_size) * a.page_size;      // rows [0, dead_lo_first) of tile 0
    const int dead_hi_last = k_end - (k_begin + (n_tiles - 1) * BN);               // rows [dead_hi_last, BN) of the last tile
    auto dead_lo_of = [&](int j) { return j == 0 ? dead_lo_first : 0; };
    auto dead_hi_of = [&](int j) { return j == n_tiles - 1 ? dead_hi_last : BN; };
    auto has_dead = [&](int j) { return dead_lo_of(j) > 0 || dead_hi_of(j) < BN; };

    if (tid == 0) {
        for (int s = 0; s < NKV; ++s) {
            mbar_init(smem_u32(&k_full[s]), n_ops);
            mbar_init(smem_u32(&k_empty[s]), RT);
            mbar_init(smem_u32(&v_full[s]), n_ops);
            mbar_init(smem_u32(&v_empty[s]), RT);
        }
        for (int t = 0; t < RT; ++t) {
            mbar_init(smem_u32(&s_full[2 * t]), 1);
            mbar_init(smem_u32(&s_full[2 * t + 1]), 1);
            mbar_init(smem_u32(&p_full[2 * t]), BM);
            mbar_init(smem_u32(&p_full[2 * t + 1]), BM);
            mbar_init(smem_u32(&pv_done[t]), 1);
            mbar_init(smem_u32(&o_done[t]), 1);
        }
        mbar_init(smem_u32(q_full), RT * BM);
        mbar_init(smem_u32(v_clean), BM);
        *bail = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    fb_pdl_wait();                                              // from here on: Q and the cache

    // a wait that ran out anywhere ends every loop of the CTA
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        if (mbar_try_wait(smem_u32(bar), parity)) return true;  // a wait that passes costs one round trip to shared memory
        if (*(volatile int*)bail) return false;
        if (mbar_wait(smem_u32(bar), parity, a.status)) return true;
        *(volatile int*)bail = 1;
        return false;
    };

    if (warp == 0) {
        // ================= fetch: lane l copies (page l / CB, column block l % CB) of every K and V tile ==========
        // K tiles and V tiles run through rings of their own: a K slot is free as soon as its scores are computed
        // (a tile ahead of the softmax), a V slot after the tile's products, so a copy has two tiles' time to land.
        // Page ids come from the block table 32 at a time (one per lane, the next 32 already on their way), so a
        // tile does not wait for the table: -2 = nothing to fetch (no query of the CTA sees the page), -1 = the
        // table has no page although one is needed.
        const int first_entry = k_begin / a.page_size - table_base_of(a, seq);   // the table entry of tile 0's first page
        auto entries = [&](int block) -> int {                  // table entries first_entry + 32 * block + lane
            const int e = first_entry + 32 * block + lane;      // (below 0: a page before the row's first, never needed)
            return (e >= 0 && e < a.table_stride) ? table[e] : -1;
        };
        int ids_block = 0, ids_cur = entries(0), ids_next = entries(1);
        auto lookup = [&](int j) -> int {
            const int rel = j * pages_per_tile + lane / CB;     // this lane's page of tile j, counted from tile 0
            const int block = (j * pages_per_tile) / 32;        // the same for all lanes: a tile's pages share a block
            if (block != ids_block) {                           // tiles come in order: the next block
                ids_cur = ids_next;
                ids_next = entries(block + 1);
                ids_block = block;
            }
            const int page = __shfl_sync(0xffffffffu, ids_cur, rel & 31);
            if (lane >= n_ops || j >= n_tiles) return -2;
            const int t_first = k_begin + rel * a.page_size;
            if (!(t_first + a.page_size > t_lo && t_first < k_end)) return -2;
            return (page < 0 || page >= a.n_pages) ? -1 : page;
        };
        auto issue = [&](uint8_t* tile, const CUtensorMap* map, uint64_t* full, int page) {
            if (lane >= n_ops) return;
            const uint32_t bar = smem_u32(full);
            if (page >= 0) {
                const int cb = lane % CB, pj = lane / CB;
                mbar_expect_tx(bar, (uint32_t)(a.page_size * 128));
                tma_load_2d(smem_u32(tile + cb * (BN * 128) + pj * a.page_size * 128), map, bar, cb * 64,
                            (page * a.nkv + kvh) * a.page_size);
            } else {
                if (page == -1) atomicOr(a.status, FB_STATUS_BAD_PAGE);
                mbar_arrive(bar);                               // whatever lies in the slot stays; it is masked
            }
        };
        int page = lookup(0);
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j % NKV;
            const uint32_t reuse = (uint32_t)(j / NKV - 1) & 1u;
            if (j >= NKV && !wait(&k_empty[s], reuse)) break;
            issue(Ks + s * SM::KV_BYTES, &a.map_k, &k_full[s], page);
            if (j >= NKV && !wait(&v_empty[s], reuse)) break;
            issue(Vs + s * SM::KV_BYTES, &a.map_v, &v_full[s], page);
            page = lookup(j + 1);                               // in flight while this warp waits for the next slot
        }
    } else if (warp < 4) {
        // ================= MMA issue: warp 1 for row tile 0, warp 2 for row tile 1 =================
        // Scores run two key tiles ahead of the softmax (two buffers per row tile), so a row tile's softmax never
        // waits for the tensor pipe.  Per key tile: O += P V, then the scores of the tile after next into the
        // columns P lay in (the MMAs of one thread run in the order of their issue, so the product has read P by
        // then), then every commit of the step at one point.  Measured on one SM with back-to-back instructions:
        // a thread that issues MMAs runs in step with the tensor pipe (its queue is a few instructions deep), so
        // the pipe stands still while that thread waits for a barrier, and every point of the instruction stream
        // where tcgen05.commit stands costs the pipe about 170 cycles, however many commits stand there.  Hence a
        // thread for each row tile (the pipe has the other's MMAs meanwhile), the waits for K and V ahead of the
        // wait for P (they pass at once unless the cache is late), and one point of commits per key tile.
        const int t = warp - 1;
        if (t < RT && elect_one()) {
            constexpr uint32_t idesc_s = umma_idesc(BN);
            constexpr uint32_t idesc_o = umma_idesc(HD, true);
            const uint32_t q_addr = smem_u32(Qs + t * SM::Q_BYTES);
            auto issue_s = [&](int j) {                         // S buffer j & 1 of the row tile = Q_t K_j^T
                const uint32_t k_addr = smem_u32(Ks + (j % NKV) * SM::KV_BYTES);
                const uint32_t d = tmem_base + (uint32_t)((2 * t + (j & 1)) * BN);
#pragma unroll
                for (int kk = 0; kk < HD / UMMA_K; ++kk)
                    umma_bf16(d, umma_desc(q_addr + (uint32_t)((kk / 4) * (BM * 128) + (kk % 4) * 32)),
                              umma_desc(k_addr + (uint32_t)((kk / 4) * (BN * 128) + (kk % 4) * 32)), idesc_s,
                              kk > 0 ? 1u : 0u);
            };
            bool ok = wait(q_full, 0);
            for (int j = 0; ok && j < 2 && j < n_tiles; ++j) {
                ok = wait(&k_full[j % NKV], (uint32_t)(j / NKV) & 1u);
                if (!ok) break;
                tmem_fence_after();
                issue_s(j);
                umma_commit(smem_u32(&s_full[2 * t + (j & 1)]));
                umma_commit(smem_u32(&k_empty[j % NKV]));
            }
            for (int j = 0; ok && j < n_tiles; ++j) {
                const bool more = j + 2 < n_tiles;              // there are scores left to compute
                ok = wait(&v_full[j % NKV], (uint32_t)(j / NKV) & 1u);
                if (ok && more) ok = wait(&k_full[(j + 2) % NKV], (uint32_t)((j + 2) / NKV) & 1u);
                // (the barrier's first phase is tile 0's clearing if tile 0 has rows to clear, else the last tile's)
                if (ok && t > 0 && has_dead(j)) ok = wait(v_clean, (j > 0 && has_dead(0)) ? 1u : 0u);
                if (ok) ok = wait(&p_full[2 * t + (j & 1)], (uint32_t)(j >> 1) & 1u);
                if (!ok) break;
                tmem_fence_after();
                const uint32_t v_addr = smem_u32(Vs + (j % NKV) * SM::KV_BYTES);
                const uint32_t p_addr = tmem_base + (uint32_t)((2 * t + (j & 1)) * BN);     // bf16 pairs over the scores
                const uint32_t d = tmem_base + (uint32_t)(RT * 128 + t * 128);
#pragma unroll
                for (int kk = 0; kk < BN / UMMA_K; ++kk) {      // 16 keys = 8 columns of P each
                    const uint64_t db = umma_desc_mn(v_addr + (uint32_t)(kk * 16 * 128), BN * 128, 1024);
                    umma_bf16_ts(d, p_addr + (uint32_t)(kk * 8), db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                if (more) issue_s(j + 2);
                umma_commit(smem_u32(&pv_done[t]));
                if (j == n_tiles - 1) umma_commit(smem_u32(&o_done[t]));
                umma_commit(smem_u32(&v_empty[j % NKV]));
                if (more) {
                    umma_commit(smem_u32(&s_full[2 * t + (j & 1)]));
                    umma_commit(smem_u32(&k_empty[(j + 2) % NKV]));
                }
            }
        }
        __syncwarp();
    } else {
        // ================= softmax: thread = query row = tensor-memory lane; warps 4..7 row tile 0, 8..11 row tile 1 =====
        const int quarter = warp & 3;                           // the lanes this warp may read
        const int t = (warp - 4) >> 2;                          // its row tile
        const int r = t * BM + quarter * 32 + lane;             // row of the CTA
        const bool valid = r < rows_valid;
        const int token = q_start + tok0 + r / G, head = kvh * G + r % G;
        // ---- stage Q (zero rows beyond the CTA's share) ----
        {
            const __nv_bfloat16* src = a.q + (size_t)token * a.q_stride + (size_t)head * hd;
            uint8_t* qrow = Qs + t * SM::Q_BYTES + (r - t * BM) * 128;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
                *reinterpret_cast<uint4*>(qrow + (c / 8) * (BM * 128) + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(q_full));
        }
        const int p_row = valid ? pos0 + tok0 + r / G : -1;     // a row beyond the share sees nothing
        const int t0_row = (a.window > 0 && p_row - a.window + 1 > 0) ? p_row - a.window + 1 : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t o_addr = lane_addr + (uint32_t)(RT * 128 + t * 128); // O of this row
        float m_ref = -INFINITY;                                // reference point of the exponentials (scaled, base 2)
        float l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int tile_start = k_begin + j * BN;
            const uint32_t s_addr = lane_addr + (uint32_t)((2 * t + (j & 1)) * BN);   // S, and P over it, of this row
            ok = ok && __all_sync(0xffffffffu, wait(&s_full[2 * t + (j & 1)], (uint32_t)(j >> 1) & 1u));
            if (!ok) continue;
            tmem_fence_after();
            // every key of the tile is visible to every row of the warp, or each is compared
            const bool plain = __all_sync(0xffffffffu, tile_start + BN - 1 <= p_row && tile_start >= t0_row);
            // ---- the row's 64 scores into registers (one round trip), masked where needed; their maximum ----
            uint32_t v[BN / 32][32];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) tmem_ld32_nowait(s_addr + (uint32_t)(c * 32), v[c]);
            tmem_wait_ld();
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (plain) {
#pragma unroll
                for (int c = 0; c < BN / 32; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[c][i]));
            } else {
#pragma unroll
                for (int c = 0; c < BN / 32; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = tile_start + c * 32 + i;
                        if (!(key >= t0_row && key <= p_row)) v[c][i] = 0xff800000u;      // -inf
                        mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[c][i]));
                    }
            }
            const float m_new = fmaxf(m_ref, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2e);
            if (j == 0) {
                m_ref = m_new;                                  // O is overwritten by the first product
            } else if (__any_sync(0xffffffffu, m_new > m_ref + RESCALE_STEP || (m_ref == -INFINITY && m_new > m_ref))) {
                // move the reference point: O *= 2^(old - new), for the whole warp at once.  (The product of tile
                // j - 2 is complete, that of tile j cannot start before this thread is through: the phase asked
                // for is the current one or the one just completed.)
                ok = __all_sync(0xffffffffu, wait(&pv_done[t], (uint32_t)(j - 1) & 1u));
                if (!ok) continue;
                tmem_fence_after();
                const float f = m_new == -INFINITY ? 1.0f : exp2f(m_ref - m_new);
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t w[32];
                    tmem_ld32_nowait(o_addr + (uint32_t)(c * 32), w);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * f);
                    tmem_st32(o_addr + (uint32_t)(c * 32), w);
                }
                tmem_wait_st();
                l *= f;
                m_ref = m_new;
            }
            // ---- P = 2^(s - reference), rounded to bfloat16, over the scores it came from: keys 32c .. 32c + 31
            // go to columns 16c .. 16c + 15 ----
            const float neg_ref = m_ref == -INFINITY ? 0.0f : -m_ref;
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    // a masked score is -inf: 2^-inf = 0
                    const float p0 = fast_exp2(fmaf(__uint_as_float(v[c][2 * i]), a.scale_log2e, neg_ref));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(v[c][2 * i + 1]), a.scale_log2e, neg_ref));
                    sum4[i & 3] += p0 + p1;
                    pk[i] = pack_bf16(p0, p1);
                }
                tmem_st16(s_addr + (uint32_t)(c * 16), pk);
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if (t == 0 && has_dead(j)) {                        // (only the first and the last tile can)
                const int dead_lo = dead_lo_of(j), dead_hi = dead_hi_of(j);
                ok = __all_sync(0xffffffffu, wait(&v_full[j % NKV], (uint32_t)(j / NKV) & 1u));
                if (!ok) continue;
                uint8_t* vt = Vs + (j % NKV) * SM::KV_BYTES;
                const int n_dead = dead_lo + (BN - dead_hi);
                for (int idx = tid - 128; idx < n_dead * 8 * CB; idx += BM) {
                    const int cb = idx / (n_dead * 8), rest = idx - cb * (n_dead * 8);
                    const int k = rest / 8, row = k < dead_lo ? k : dead_hi + (k - dead_lo);
                    *reinterpret_cast<uint4*>(vt + cb * (BN * 128) + row * 128 + (rest & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                if (RT > 1) mbar_arrive(smem_u32(v_clean));
            }
            tmem_wait_st();
            tmem_fence_before();
            mbar_arrive(smem_u32(&p_full[2 * t + (j & 1)]));
        }
        // ---- O / l, written as bfloat16 ----
        // (a barrier of its own: pv_done may be one or two phases on by now, and a wait names a phase by its parity)
        if (ok) ok = __all_sync(0xffffffffu, wait(&o_done[t], 0));
        if (ok) {
            tmem_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = a.out + (size_t)token * a.out_stride + (size_t)head * hd;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32_nowait(o_addr + (uint32_t)(c * 32), v);
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            w[e] = pack_bf16(__uint_as_float(v[8 * q4 + 2 * e]) * inv,
                                             __uint_as_float(v[8 * q4 + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int HD, int RT>
int launch_tc(const AttnArgs& a, int n_seqs, int max_q_len, cudaStream_t stream) {
    auto kern = attention_tc_kernel<HD, RT>;
    using SM = TcSmem<HD, RT>;
    static bool configured[FB_MAX_DEVICES] = {};
    if (fb_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::BYTES);
        if (e != cudaSuccess) return fb_fail(-2, "attention_tc: cannot reserve %d bytes of shared memory: %s",
                                             SM::BYTES, cudaGetErrorString(e));
        fb_setup_done(configured);
    }
    const int TQ = RT * BM / (a.nh / a.nkv);
    const dim3 grid(((max_q_len + TQ - 1) / TQ) * a.nkv * portion_seqs(a));
    fb_launch_class(FB_LAUNCH_ATTENTION_TC, (kern), grid, tc_threads(RT), (size_t)SM::BYTES, stream, a);
    return fb_check_launch("attention_tc");
}

// Two row tiles per CTA when that still gives every SM a CTA, else one.
template <int HD>
int launch_tc(const AttnArgs& a, int n_seqs, int max_q_len, cudaStream_t stream) {
    const int sms = fb_sm_count();
    const int TQ2 = 2 * BM / (a.nh / a.nkv);
    const long ctas2 = (long)((max_q_len + TQ2 - 1) / TQ2) * a.nkv * portion_seqs(a);   // an upper bound: short ones leave early
    return ctas2 >= sms ? launch_tc<HD, 2>(a, n_seqs, max_q_len, stream) : launch_tc<HD, 1>(a, n_seqs, max_q_len, stream);
}

}  // namespace

bool fb_attention_tc_takes(const AttnArgs& a, bool tma) {
    const int G = a.nh / a.nkv;
    return tma && !a.score_slopes && (a.hd == 64 || a.hd == 128) && G <= BM && BN % a.page_size == 0 &&
           a.out_stride % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
}

int fb_launch_attention_tc(const AttnArgs& a, int n_seqs, int max_q_len, cudaStream_t stream) {
    return a.hd == 64 ? launch_tc<64>(a, n_seqs, max_q_len, stream) : launch_tc<128>(a, n_seqs, max_q_len, stream);
}
