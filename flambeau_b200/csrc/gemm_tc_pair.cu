// out[M,N] = X[M,K] * W[N,K]^T in bfloat16 with two SMs on one tile (tcgen05.mma cta_group::2), for products with
// hundreds of rows (portions of prompts).
//
// A cluster of two CTAs owns 256 output features x 256 tokens.  Each CTA stages its own 128 weight rows and its
// own 128 of the 256 tokens, so a CTA fetches and holds half of what the one-CTA kernel (gemm_tc.cu) does for
// the token operand; the even CTA of the pair issues one MMA of M = 256, N = 256 that reads both CTAs' shared
// memory and writes both CTAs' tensor memory (128 features x 256 tokens in each).  Otherwise it is the
// arrangement of gemm_tc.cu: swap-AB, K-major operands with the 128-byte swizzle, 64 elements of K a stage,
// two accumulators so that the epilogue of one tile overlaps the products of the next, persistent pairs.
//
// Barriers.  full[s] lives in the even CTA and counts the bytes of both CTAs' copies (the copies carry
// cta_group::2, which lets them signal the peer's barrier).  empty[s] and acc_full[b] exist in both CTAs and are
// signalled in both by one tcgen05.commit with a CTA mask.  acc_empty[b] lives in the even CTA and takes one
// arrival from each CTA's epilogue.  No copy is multicast.  Every wait on an mbarrier is bounded in time as in
// gemm_tc.cu; the two cluster barriers (after set-up, before the tensor memory is freed) are reached by every
// thread on every path.
#include "gemm_tc_pair.cuh"
#include "umma.cuh"

#include <stdlib.h>

namespace {

constexpr int PBM = 128;               // output features per CTA
constexpr int PBN = 256;               // tokens per pair (UMMA N)
constexpr int PBNH = PBN / 2;          // tokens staged by one CTA
constexpr int PBK = 64;
constexpr int P_THREADS = 320;         // warp 0: copies, warp 1: tensor memory and MMA, warps 2..9: epilogue
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = PBM * PBK * 2;
constexpr int P_STAGE_BYTES = P_A_BYTES + PBNH * PBK * 2;
constexpr int P_TMEM_COLS = 2 * PBN;
// The epilogue's way out: 16 tokens x this CTA's 128 features (float32 at most), two buffers for each of its two
// groups of four warps (one is filled while a tensor-map store empties the other).
constexpr int P_OUT_TOKENS = 16;
constexpr int P_OUT_BYTES = P_OUT_TOKENS * PBM * 4;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256 + 4 * P_OUT_BYTES;
// Pairs that run at a time: one per two SMs of the current device.
inline int pair_slots() { return fb_sm_count() / 2 > 0 ? fb_sm_count() / 2 : 1; }

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t in_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A box of a tensor map into this CTA's shared memory; its bytes are counted on `bar`, which may lie in the peer.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// One arrival on the barrier at this offset in both CTAs when the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// One box of an output map (x = feature, y = token, z = slab) from shared memory to global memory; the store joins
// the thread's current bulk group.
__device__ __forceinline__ void tma_store_3d(const void* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
// The same, added to what global memory holds (float32 adds, done by the memory system: each element of the output
// gets exactly one such add from this kernel, so the result does not depend on any order).
__device__ __forceinline__ void tma_add_3d(const void* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until all but the last of this thread's groups of stores have read their shared memory (which may then be written
// again) / until all of them are complete.
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// One unit of work: output tile (nt, mt) and share `split` of its K range.  Token tiles vary fastest, so pairs
// that run together share weight tiles through L2; shares of K vary slowest.  The last token tile of a product
// whose rows do not fill it is multiplied at its own width: n_tok = the tile's rows rounded up to 32 (the N of
// the MMA; each CTA supplies n_tok / 2 tokens), so a step of 2,048 + 32 rows pays for 32 rows more, not for 256.
struct PairUnit { int mt, nt, split, kb_begin, n_kb, n_tok; };
__device__ __forceinline__ PairUnit pair_unit(int u, int tiles_m, int tiles, int splits, int kb_total, int M) {
    PairUnit w;
    const int t = u % tiles;
    w.split = u / tiles;
    w.mt = t % tiles_m;
    w.nt = t / tiles_m;
    w.kb_begin = (int)((long)w.split * kb_total / splits);
    w.n_kb = (int)((long)(w.split + 1) * kb_total / splits) - w.kb_begin;
    const int rows_left = M - w.mt * PBN;
    w.n_tok = rows_left >= PBN ? PBN : ((rows_left + 31) / 32) * 32;
    return w;
}

template <typename TO>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_o, int boxed_out,
                    TO* __restrict__ out, long ldo, long slab_stride, int M, int N, int K, int tiles_m, int tiles,
                    int splits, int n_units, int gated, int accumulate, int* status) {
    constexpr int S = P_STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + S * P_STAGE_BYTES);
    // bars[0..S): stage full (even CTA's are used), [S..2S): stage empty, [2S..2S+2): accumulator full,
    // [2S+2..2S+4): accumulator empty (even CTA's are used)
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * S + 4);
    int* bail = (int*)(tmem_slot + 1);
    uint8_t* out_stage = smem + S * P_STAGE_BYTES + 256;     // [2 groups of warps][2 buffers][16 tokens][128 features]

    fb_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int kb_total = (K + PBK - 1) / PBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[S + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * S]), 1);
        mbar_init(smem_u32(&bars[2 * S + 1]), 1);
        mbar_init(smem_u32(&bars[2 * S + 2]), 2);
        mbar_init(smem_u32(&bars[2 * S + 3]), 2);
        *bail = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)P_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                          // both CTAs' barriers exist before either signals the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- copies: this CTA's weight rows and its half of the tokens ----------------
        if (elect_one()) {
            uint32_t it = 0;
            bool first = true;
            for (int u = pair; u < n_units && !*(volatile int*)bail; u += n_pairs) {
                const PairUnit w = pair_unit(u, tiles_m, tiles, splits, kb_total, M);
                const int n0 = w.nt * (2 * PBM) + (int)rank * PBM;
                const int m0 = w.mt * PBN + (int)rank * (w.n_tok / 2);    // this CTA's half of the tile's tokens
                int i = 0;
                if (first) {
                    // weights do not depend on the kernel before this one; the activations do
                    first = false;
                    const int pre = w.n_kb < S ? w.n_kb : S;
                    for (int j = 0; j < pre; ++j) {
                        if (rank == 0) mbar_expect_tx(smem_u32(&bars[j]), 2u * P_STAGE_BYTES);
                        tma_load_2d_pair(smem_u32(smem + (size_t)j * P_STAGE_BYTES), &map_w,
                                         in_cta(smem_u32(&bars[j]), 0), (w.kb_begin + j) * PBK, n0);
                    }
                    fb_pdl_wait();
                    for (int j = 0; j < pre; ++j)
                        tma_load_2d_pair(smem_u32(smem + (size_t)j * P_STAGE_BYTES + P_A_BYTES), &map_x,
                                         in_cta(smem_u32(&bars[j]), 0), (w.kb_begin + j) * PBK, m0);
                    i = pre;
                    it = (uint32_t)pre;
                }
                for (; i < w.n_kb; ++i, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t round = it / S;
                    if (!mbar_wait(smem_u32(&bars[S + s]), (round & 1u) ^ 1u, status)) { *bail = 1; break; }
                    if (rank == 0) mbar_expect_tx(smem_u32(&bars[s]), 2u * P_STAGE_BYTES);
                    const uint32_t full = in_cta(smem_u32(&bars[s]), 0);
                    uint8_t* stage = smem + (size_t)s * P_STAGE_BYTES;
                    tma_load_2d_pair(smem_u32(stage), &map_w, full, (w.kb_begin + i) * PBK, n0);
                    tma_load_2d_pair(smem_u32(stage + P_A_BYTES), &map_x, full, (w.kb_begin + i) * PBK, m0);
                }
            }
            if (first) fb_pdl_wait();
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA: the even CTA issues for the pair ----------------
        if (rank == 0 && elect_one()) {
            uint32_t it = 0;
            int j = 0;
            for (int u = pair; u < n_units && !*(volatile int*)bail; u += n_pairs, ++j) {
                const PairUnit w = pair_unit(u, tiles_m, tiles, splits, kb_total, M);
                const int n_kb = w.n_kb;
                const uint32_t idesc = umma_idesc(w.n_tok, false, 2 * PBM);
                const int b = j & 1;
                const uint32_t use = (uint32_t)(j >> 1);
                // both CTAs' epilogues must have drained this accumulator (two units ago)
                if (!mbar_wait(smem_u32(&bars[2 * S + 2 + b]), (use & 1u) ^ 1u, status)) { *bail = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * PBN);
                bool ok = true;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t round = it / S;
                    ok = mbar_wait(smem_u32(&bars[s]), round & 1u, status);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint8_t* stage = smem + (size_t)s * P_STAGE_BYTES;
                    const uint64_t da = umma_desc(smem_u32(stage));
                    const uint64_t db = umma_desc(smem_u32(stage + P_A_BYTES));
#pragma unroll
                    for (int k = 0; k < PBK / UMMA_K; ++k)
                        umma_bf16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                                       (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(smem_u32(&bars[S + s]));       // the stage is free in both CTAs
                }
                if (!ok) { *bail = 1; break; }
                umma_commit_pair(smem_u32(&bars[2 * S + b]));       // the accumulator is complete in both CTAs
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: this CTA's 128 features x 256 tokens ----------------
        fb_pdl_wait();
        const int quarter = warp & 3;
        const int half_id = (warp - 2) >> 2;
        const int row_local = quarter * 32 + lane;
        uint32_t boxes = 0;                                     // boxes this group of warps has staged: the buffers take turns
        int j = 0;
        for (int u = pair; u < n_units; u += n_pairs, ++j) {
            const PairUnit w = pair_unit(u, tiles_m, tiles, splits, kb_total, M);
            const int m0 = w.mt * PBN;
            const int n = w.nt * (2 * PBM) + (int)rank * PBM + row_local;
            TO* dst = out + (size_t)w.split * (size_t)slab_stride;     // this share's slab (the whole sum: slab 0)
            const int b = j & 1;
            const uint32_t use = (uint32_t)(j >> 1);
            const bool mine = !*(volatile int*)bail && mbar_wait(smem_u32(&bars[2 * S + b]), use & 1u, status);
            if (!mine) *bail = 1;
            // all or none: the turns below meet at barriers of their own
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const bool got = !*(volatile int*)bail;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * PBN);
            if (got) {
                // Sixteen tokens of the CTA's 128 features a turn, by each of the two groups of four warps.  Where the
                // output's strides allow a tensor map the values go to shared memory as [token][feature] and one
                // thread sends the box on its way (rows and columns beyond the output's edge are not written): a
                // thousand 128-byte stores a tile from the warps themselves keep the epilogue waiting for the memory
                // system's acknowledgements (7 us a tile against 2 to 3 us this way).
                const int width = gated ? PBM / 2 : PBM;        // features of a staged row
                const bool leader = quarter == 0 && lane == 0;
#pragma unroll 1
                for (int c = half_id * 16; c < w.n_tok; c += 32) {
                    if (m0 + c >= M) break;
                    TO* stage = reinterpret_cast<TO*>(out_stage + (half_id * 2 + (boxes & 1)) * P_OUT_BYTES);
                    ++boxes;
                    float v[16];
                    if (w.n_kb > 0) {
                        tmem_ld16(taddr + (uint32_t)c, v);
                    } else {
#pragma unroll
                        for (int q = 0; q < 16; ++q) v[q] = 0.0f;
                    }
                    if (boxed_out) {
                        if (leader) bulk_wait_read();           // the box sent from this buffer, the one before last, has left it
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + half_id) : "memory");
                    }
                    if (gated) {
                        // features alternate gate, up: the even lane writes act(gate) * up to column n / 2
                        float r[16];
#pragma unroll
                        for (int q = 0; q < 16; ++q) {
                            const float up = __shfl_xor_sync(0xffffffffu, v[q], 1);
                            r[q] = fb_gate_times(gated, v[q], up);
                        }
                        if (boxed_out) {
                            if (!(lane & 1)) {
#pragma unroll
                                for (int q = 0; q < 16; ++q) stage[q * width + (row_local >> 1)] = fb_from_float<TO>(r[q]);
                            }
                        } else {
                            const bool writes = !(lane & 1) && n + 1 < N;
#pragma unroll
                            for (int q = 0; q < 16; ++q)
                                if (writes && m0 + c + q < M)
                                    dst[(size_t)(m0 + c + q) * ldo + (n >> 1)] = fb_from_float<TO>(r[q]);
                        }
                    } else if (boxed_out) {
#pragma unroll
                        for (int q = 0; q < 16; ++q) stage[q * width + row_local] = fb_from_float<TO>(v[q]);
                    } else if (n < N) {
#pragma unroll
                        for (int q = 0; q < 16; ++q)
                            if (m0 + c + q < M) {
                                TO* at = dst + (size_t)(m0 + c + q) * ldo + n;     // (no other thread has this element)
                                *at = fb_from_float<TO>(accumulate ? fb_to_float(*at) + v[q] : v[q]);
                            }
                    }
                    if (boxed_out) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + half_id) : "memory");
                        if (leader) {
                            const int x = (w.nt * (2 * PBM) + (int)rank * PBM) >> (gated ? 1 : 0);
                            if (accumulate) tma_add_3d(&map_o, smem_u32(stage), x, m0 + c, w.split);
                            else tma_store_3d(&map_o, smem_u32(stage), x, m0 + c, w.split);
                            bulk_commit();
                        }
                    }
                }
            }
            // this CTA's half of the accumulator may be overwritten: one arrival per CTA at the even CTA
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (warp == 2 && lane == 0) mbar_arrive_remote(in_cta(smem_u32(&bars[2 * S + 2 + b]), 0));
            if (*(volatile int*)bail) break;
        }
    }
    if (warp >= 2 && (warp & 3) == 0 && lane == 0) bulk_wait_all();   // the boxes this thread sent are in memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                          // neither CTA leaves while the other may still reach into it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)P_TMEM_COLS) : "memory");
    }
}

template <typename TO>
int launch_pair(const void* X, long lda, const void* W, long ldw, void* out, long ldo, long slab_stride, int splits,
                int M, int N, int K, int gated, int accumulate, int* status, cudaStream_t stream) {
    CUtensorMap mw, mx;
    int rc = fb_tensor_map_bf16(&mw, W, N, K, ldw, PBK, PBM);
    if (rc) return rc;
    rc = fb_tensor_map_bf16(&mx, X, M, K, lda, PBK, PBNH);
    if (rc) return rc;
    // the output as boxes of 16 tokens x a CTA's features (half as many where the epilogue folds gate and up)
    CUtensorMap mo;
    const int boxed = fb_tensor_map_out(&mo, out, (int)sizeof(TO), M, gated ? N / 2 : N, ldo, splits, slab_stride,
                                        gated ? PBM / 2 : PBM, P_OUT_TOKENS);
    if (boxed < 0) return boxed;
    auto kern = gemm_tc_pair_kernel<TO>;
    static bool configured[FB_MAX_DEVICES] = {};
    if (fb_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
        if (e != cudaSuccess) return fb_fail(-2, "gemm_tc_pair: cannot reserve %d bytes of shared memory: %s",
                                             P_SMEM_BYTES, cudaGetErrorString(e));
        fb_setup_done(configured);
    }
    const int tiles_m = (M + PBN - 1) / PBN, tiles_n = (N + 2 * PBM - 1) / (2 * PBM);
    const long tiles = (long)tiles_m * tiles_n;
    const long n_units = tiles * splits;
    if (n_units > 2000000000L) return fb_fail(-1, "gemm_tc_pair: too many tiles (M=%d N=%d)", M, N);
    const int pairs = (int)(n_units < pair_slots() ? n_units : pair_slots());
    fb_launch_class(FB_LAUNCH_GEMM_PAIR, (kern), 2 * pairs, P_THREADS, P_SMEM_BYTES, stream, mw, mx, mo,
                    boxed == 0 ? 1 : 0, (TO*)out, ldo, slab_stride, M, N, K, tiles_m, (int)tiles, splits, (int)n_units,
                    gated, accumulate, status);
    return fb_check_launch("gemm_tc_pair");
}

}  // namespace

static int g_pair_on = -1;                       // -1: not yet read from the environment
FB_API void fb_set_gemm_pair(int on) { g_pair_on = on ? 1 : 0; }

// Shares of K for the pairs: as many as make the rounds of the resident pairs shortest, each share beyond the first
// costing one more float32 copy of the output (written here, added by the consumer), counted in k-block times.
static int pair_splits(long tiles, int kb_total, int max_splits, int M, int N) {
    const double kb_seconds = 2.0 * PBM * PBN * PBK / FB_MODEL_SM_FLOPS;
    const double share_cost_kb = ((double)M * N * 8.0 / FB_MODEL_HBM_BYTES_PER_S) / kb_seconds;
    const int slots = pair_slots();
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= max_splits && s <= kb_total; ++s) {
        const long units = tiles * s;
        const long rounds = (units + slots - 1) / slots;
        const double cost = rounds * ((double)((kb_total + s - 1) / s) + 0.5) + (s - 1) * share_cost_kb;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

int fb_gemm_pair_plan(int M, int N, int K, int max_slabs) {
    if (g_pair_on < 0) g_pair_on = (getenv("FLAMBEAU_GEMM_PAIR") && atoi(getenv("FLAMBEAU_GEMM_PAIR")) == 0) ? 0 : 1;
    if (!g_pair_on || K <= 0 || M <= PBNH) return 0;
    const long tiles = (long)((M + PBN - 1) / PBN) * ((N + 2 * PBM - 1) / (2 * PBM));
    const int kb_total = (K + PBK - 1) / PBK;
    const int splits = pair_splits(tiles, kb_total, max_slabs < 1 ? 1 : (max_slabs > 16 ? 16 : max_slabs), M, N);
    // A long K on few tiles needs shares of K; where the caller has no slabs for them, the one-SM kernel, whose
    // shares meet in scratch, is the better choice.
    if (splits == 1 && tiles < 48 && kb_total >= 128) return 0;
    return splits;
}

int fb_launch_gemm_pair(const void* X, long lda, const void* W, long ldw, void* out, int o_dtype, long ldo,
                        long slab_stride, int splits, int M, int N, int K, int gated, int accumulate, int* status,
                        cudaStream_t stream) {
    if (splits < 1 || (splits > 1 && (slab_stride <= 0 || o_dtype != FB_F32 || gated)))
        return fb_fail(-1, "gemm_tc_pair: %d shares of K need float32 slabs", splits);
    if (accumulate && (o_dtype != FB_F32 || splits != 1 || gated))
        return fb_fail(-1, "gemm_tc_pair: only a whole float32 product can be added to its output");
    if (o_dtype == FB_F32)
        return launch_pair<float>(X, lda, W, ldw, out, ldo, slab_stride, splits, M, N, K, gated, accumulate, status,
                                  stream);
    if (o_dtype == FB_BF16)
        return launch_pair<__nv_bfloat16>(X, lda, W, ldw, out, ldo, 0, 1, M, N, K, gated, 0, status, stream);
    return fb_fail(-1, "gemm_tc_pair: unknown output dtype code %d", o_dtype);
}
