// out[M,N] = X[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores.
//
// The weight is the 128-row operand of tcgen05.mma and the tokens are its N
// dimension ("swap-AB"): one CTA owns 128 output features x BN tokens, with
// BN in {16, 32, 64, 128, 256} chosen from the number of rows, so a decode step of a few
// tokens streams the weights at full width instead of padding the token side
// to 128.  Both operands are K-major in shared memory, staged by TMA with the
// 128-byte swizzle, 64 elements of K per stage; the float32 accumulator
// lives in tensor memory and is read back with tcgen05.ld by four epilogue
// warps whose lanes are the output features, so that a warp stores 32
// consecutive features of one token.
//
// Warps: 0 = TMA producer, 1 = tensor-memory owner and MMA issuer, 2..9 = epilogue (a warp may only read the
// quarter of the tensor-memory lanes given by its index modulo 4; two warps share a quarter and split the columns).
// Split-K: grid.z CTAs share one output tile; each writes its float32 partial
// to scratch, and the CTA that arrives last (an atomic counter per tile, no
// waiting) adds the partials in split order and writes the result, so the sum
// does not depend on the order of arrival.
//
// Every wait on an mbarrier is bounded in time: when it runs out the kernel
// sets FB_STATUS_WAIT_TIMEOUT in the status word, leaves its loops, frees its
// tensor memory and returns.
//
// The reference multiplies with scalar-FMA tiles of 64 outputs x 8 rows
// (crates/kernels-hip/src/kernels/mmq_f16_tile.cu:32-107); the weight layout
// (rows = outputs) is the same.
#include "gemm_tc_pair.cuh"
#include "tensor_map.cuh"
#include "umma.cuh"

#include <mutex>
#include <stdlib.h>

namespace {

constexpr int BM = 128;          // output features per CTA (UMMA M)
constexpr int BK = 64;           // K elements per stage: 128 bytes, one swizzle row
constexpr int GEMM_THREADS = 320;      // warp 0: TMA, warp 1: MMA, warps 2..9: epilogue (two per lane quarter)
constexpr int EPI_THREADS = 256;

template <int BN> struct TileCfg {
    // A stage holds KA swizzle atoms of K (64 elements each) of both operands.  (Two atoms a stage, which make
    // every visit to a weight row 256 contiguous bytes, were measured for the 16-token tile: no gain over one.)
    static constexpr int KA = 1;
    static constexpr int KSTEP = KA * BK;                   // elements of K per stage
    static constexpr int ATOM_BYTES = BM * BK * 2 + BN * BK * 2;
    static constexpr int STAGE_BYTES = KA * ATOM_BYTES;
    static constexpr int STAGES = BN == 16 ? 6 : BN == 32 ? 5 : BN == 64 ? 4 : BN == 128 ? 3 : 4;
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;      // tensor-memory columns of one accumulator
    static constexpr int TMEM_COLS = 2 * ACC_COLS;          // two accumulators: the epilogue of one unit of work
                                                            // overlaps the products of the next
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// One unit of work: output tile (m_tile, n_tile) and one share `split` of its K range.  Token tiles vary
// fastest, so CTAs that run together share weight tiles through L2; shares of K vary slowest.
struct Unit { int m0, n0, split, kb_begin, n_kb, tile_id; };
__device__ __forceinline__ Unit unit_of(int u, int tiles_m, int tiles_n, int splits, int kb_total) {
    Unit w;
    const int mt = u % tiles_m;
    const int r = u / tiles_m;
    const int nt = r % tiles_n;
    w.split = r / tiles_n;
    w.m0 = mt;                                   // scaled by the caller (BN is a template parameter there)
    w.n0 = nt * BM;
    w.tile_id = nt * tiles_m + mt;
    w.kb_begin = (int)((long)w.split * kb_total / splits);
    w.n_kb = (int)((long)(w.split + 1) * kb_total / splits) - w.kb_begin;
    return w;
}

// Persistent: the grid is at most one or two CTAs per SM; CTA c takes units c, c + grid, c + 2*grid, ...
// The TMA pipeline runs on across units, and the accumulator alternates between two regions of tensor memory.
template <int BN, typename TO>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               TO* __restrict__ out, long ldo, long slab_stride, float* __restrict__ partials,
               int* __restrict__ tile_counters, int M, int N, int K, int splits, int tiles_m, int tiles_n,
               int n_units, int gated, int* status) {
    using Cfg = TileCfg<BN>;
    constexpr int S = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + S * Cfg::STAGE_BYTES);
    // bars[0..S): stage full, [S..2S): stage empty, [2S..2S+2): accumulator full, [2S+2..2S+4): accumulator empty
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * S + 4);
    int* last_flag = (int*)(tmem_slot + 1);
    int* bail = last_flag + 1;                   // a bounded wait ran out somewhere in this CTA

    fb_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_total = (K + Cfg::KSTEP - 1) / Cfg::KSTEP;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[S + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * S]), 1);
        mbar_init(smem_u32(&bars[2 * S + 1]), 1);
        mbar_init(smem_u32(&bars[2 * S + 2]), EPI_THREADS);
        mbar_init(smem_u32(&bars[2 * S + 3]), EPI_THREADS);
        *bail = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            uint32_t it = 0;                     // stages issued so far, over all units
            bool first = true;
            for (int u = blockIdx.x; u < n_units && !*(volatile int*)bail; u += gridDim.x) {
                const Unit w = unit_of(u, tiles_m, tiles_n, splits, kb_total);
                const int m0 = w.m0 * BN;
                int i = 0;
                if (first) {
                    // The weights do not depend on the kernel before this one: the first tiles are requested
                    // while that kernel may still be running; the activations follow the dependency wait.
                    first = false;
                    const int pre = w.n_kb < S ? w.n_kb : S;
                    for (int j = 0; j < pre; ++j) {
                        const uint32_t full = smem_u32(&bars[j]);
                        mbar_expect_tx(full, (uint32_t)Cfg::STAGE_BYTES);
#pragma unroll
                        for (int a = 0; a < Cfg::KA; ++a)
                            tma_load_2d(smem_u32(smem + (size_t)j * Cfg::STAGE_BYTES + a * Cfg::ATOM_BYTES), &map_w, full,
                                        (w.kb_begin + j) * Cfg::KSTEP + a * BK, w.n0);
                    }
                    fb_pdl_wait();
                    for (int j = 0; j < pre; ++j)
#pragma unroll
                        for (int a = 0; a < Cfg::KA; ++a)
                            tma_load_2d(smem_u32(smem + (size_t)j * Cfg::STAGE_BYTES + a * Cfg::ATOM_BYTES + BM * BK * 2),
                                        &map_x, smem_u32(&bars[j]), (w.kb_begin + j) * Cfg::KSTEP + a * BK, m0);
                    i = pre;
                    it = (uint32_t)pre;
                }
                for (; i < w.n_kb; ++i, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t round = it / S;
                    if (!mbar_wait(smem_u32(&bars[S + s]), (round & 1u) ^ 1u, status)) { *bail = 1; break; }
                    const uint32_t full = smem_u32(&bars[s]);
                    mbar_expect_tx(full, (uint32_t)Cfg::STAGE_BYTES);
                    uint8_t* stage = smem + (size_t)s * Cfg::STAGE_BYTES;
                    const int k0 = (w.kb_begin + i) * Cfg::KSTEP;
#pragma unroll
                    for (int a = 0; a < Cfg::KA; ++a) {
                        tma_load_2d(smem_u32(stage + a * Cfg::ATOM_BYTES), &map_w, full, k0 + a * BK, w.n0);
                        tma_load_2d(smem_u32(stage + a * Cfg::ATOM_BYTES + BM * BK * 2), &map_x, full, k0 + a * BK, m0);
                    }
                }
            }
            if (first) fb_pdl_wait();
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc(BN);
            uint32_t it = 0;
            int j = 0;                           // units done by this CTA
            for (int u = blockIdx.x; u < n_units && !*(volatile int*)bail; u += gridDim.x, ++j) {
                const Unit w = unit_of(u, tiles_m, tiles_n, splits, kb_total);
                const int b = j & 1;
                const uint32_t use = (uint32_t)(j >> 1);
                // the epilogue must have drained this accumulator (two units ago)
                if (!mbar_wait(smem_u32(&bars[2 * S + 2 + b]), (use & 1u) ^ 1u, status)) { *bail = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * Cfg::ACC_COLS);
                bool ok = true;
                for (int i = 0; i < w.n_kb; ++i, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t round = it / S;
                    ok = mbar_wait(smem_u32(&bars[s]), round & 1u, status);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint8_t* stage = smem + (size_t)s * Cfg::STAGE_BYTES;
#pragma unroll
                    for (int a = 0; a < Cfg::KA; ++a) {
                        const uint64_t da = umma_desc(smem_u32(stage + a * Cfg::ATOM_BYTES));
                        const uint64_t db = umma_desc(smem_u32(stage + a * Cfg::ATOM_BYTES + BM * BK * 2));
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // 16 elements of K = 32 bytes further along the swizzled row
                            umma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                                      (i > 0 || a > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(smem_u32(&bars[S + s]));            // frees the stage when the MMAs have read it
                }
                if (!ok) { *bail = 1; break; }
                umma_commit(smem_u32(&bars[2 * S + b]));            // accumulator complete
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warps 2..9, lane quarter = warp % 4, column half = (warp - 2) / 4 ----------
        fb_pdl_wait();                                              // before any global write of this kernel
        const int quarter = warp & 3;
        const int half_id = (warp - 2) >> 2;                        // which 16-column chunks this warp takes
        const int row_local = quarter * 32 + lane;                  // output feature within the tile
        int j = 0;
        for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++j) {
            const Unit w = unit_of(u, tiles_m, tiles_n, splits, kb_total);
            const int m0 = w.m0 * BN, n0 = w.n0, split = w.split, n_kb = w.n_kb;
            const int n = n0 + row_local;
            const int b = j & 1;
            const uint32_t use = (uint32_t)(j >> 1);
            const bool got = !*(volatile int*)bail && mbar_wait(smem_u32(&bars[2 * S + b]), use & 1u, status);
            if (!got) *bail = 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * Cfg::ACC_COLS);
            if (splits == 1 || slab_stride > 0) {
                // the whole sum, or this split's share of it written to its own slab (the consumer adds the slabs)
                TO* dst = out + (size_t)split * (size_t)slab_stride;
                if (got) {
#pragma unroll 1
                    for (int c = half_id * 16; c < BN; c += 32) {
                        if (m0 + c >= M) break;
                        float v[16];
                        if (n_kb > 0) {
                            tmem_ld16(taddr + (uint32_t)c, v);
                        } else {
#pragma unroll
                            for (int q = 0; q < 16; ++q) v[q] = 0.0f;
                        }
                        if (gated) {
                            // output features alternate gate, up: even lanes hold a gate, their odd neighbour its
                            // up; the even lane writes act(gate) * up to column n / 2 of a half-as-wide output
                            // (`gated` is the activation's code).
                            // Every lane computes (straight-line code, sixteen independent chains); odd lanes'
                            // results are dropped.
                            float r[16];
#pragma unroll
                            for (int q = 0; q < 16; ++q) {
                                const float up = __shfl_xor_sync(0xffffffffu, v[q], 1);
                                r[q] = fb_gate_times(gated, v[q], up);
                            }
                            const bool writes = !(lane & 1) && n + 1 < N;
#pragma unroll
                            for (int q = 0; q < 16; ++q)
                                if (writes && m0 + c + q < M)
                                    dst[(size_t)(m0 + c + q) * ldo + (n >> 1)] = fb_from_float<TO>(r[q]);
                        } else if (n < N) {
#pragma unroll
                            for (int q = 0; q < 16; ++q)
                                if (m0 + c + q < M) dst[(size_t)(m0 + c + q) * ldo + n] = fb_from_float<TO>(v[q]);
                        }
                    }
                }
            } else {
                const int tile_id = w.tile_id;
                float* mine = partials + ((size_t)tile_id * splits + split) * (size_t)(BN * BM);
#pragma unroll 1
                for (int c = half_id * 16; c < BN; c += 32) {
                    if (m0 + c >= M) break;
                    float v[16];
                    if (got && n_kb > 0) {
                        tmem_ld16(taddr + (uint32_t)c, v);
                    } else {
#pragma unroll
                        for (int q = 0; q < 16; ++q) v[q] = 0.0f;
                    }
#pragma unroll
                    for (int q = 0; q < 16; ++q) mine[(size_t)(c + q) * BM + row_local] = v[q];
                }
                __threadfence();
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int arrived = atomicAdd(&tile_counters[tile_id], 1);
                    *last_flag = (arrived == splits - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
                    const float* base = partials + (size_t)tile_id * splits * (size_t)(BN * BM);
#pragma unroll 1
                    for (int c = half_id * 4; c < BN && m0 + c < M; c += 8) {
                        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        for (int s = 0; s < splits; ++s) {
                            float v[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) v[q] = __ldcg(base + ((size_t)s * BN + c + q) * BM + row_local);
#pragma unroll
                            for (int q = 0; q < 4; ++q) acc[q] += v[q];
                        }
                        if (n < N) {
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                if (m0 + c + q < M) out[(size_t)(m0 + c + q) * ldo + n] = fb_from_float<TO>(acc[q]);
                        }
                    }
                    if (warp == 2 && lane == 0) tile_counters[tile_id] = 0;  // ready for the next launch
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");                // last_flag may be rewritten
            }
            // this accumulator may be overwritten now
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(smem_u32(&bars[2 * S + 2 + b]));
            if (*(volatile int*)bail) break;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

// How many shares of K per output tile.  CTA c of a grid of `grid` takes units c, c + grid, ...; a unit costs its
// k-blocks plus a little for switching accumulators; every share beyond the first costs the traffic of one more
// copy of the output (written here, read by whoever adds the shares), counted in k-block times.
int pick_splits(int tiles, int kb_total, int slots, int max_splits, double share_cost_kb) {
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= max_splits && s <= kb_total; ++s) {
        const long units = (long)tiles * s;
        const long grid = units < slots ? units : slots;
        const long rounds = (units + grid - 1) / grid;
        const double cost = rounds * ((double)((kb_total + s - 1) / s) + 0.5) + (s - 1) * share_cost_kb;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

template <int BN, typename TO>
int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, void* out, long ldo, long slab_stride, int max_slabs,
              int* splits_used, float* partials, long partial_floats, int* counters, int n_counters, int M, int N,
              int K, int force_splits, int* status, cudaStream_t stream, int gated = 0) {
    using Cfg = TileCfg<BN>;
    const int tiles_n = (N + BM - 1) / BM, tiles_m = (M + BN - 1) / BN;
    const int tiles = tiles_n * tiles_m;
    const int kb_total = (K + Cfg::KSTEP - 1) / Cfg::KSTEP;
    const int per_sm = Cfg::SMEM_BYTES <= 113 * 1024 ? 2 : 1;
    const int slots = fb_sm_count() * per_sm;
    // One more share = one more float32 copy of the output, written and read once at about HBM speed.  A k-block
    // of one CTA takes its stage bytes at the CTA's part of that speed when the weights stream from DRAM (few
    // rows), or its flops at an SM's tensor rate when the tile is large enough to be bound by them.
    const double kb_seconds = BN <= 64 ? (double)Cfg::STAGE_BYTES / (FB_MODEL_HBM_BYTES_PER_S / slots)
                                       : 2.0 * BM * BN * BK / FB_MODEL_SM_FLOPS;
    const double share_cost_kb = ((double)M * N * 8.0 / FB_MODEL_HBM_BYTES_PER_S) / kb_seconds;
    int splits = force_splits > 0 ? force_splits : pick_splits(tiles, kb_total, slots, 16, share_cost_kb);
    if (gated) splits = 1;                       // the activation needs the whole sum
    if (splits > kb_total) splits = kb_total;
    if (slab_stride > 0) {
        if (splits > max_slabs) splits = max_slabs;
    } else {
        while (splits > 1 && ((long)tiles * splits * BN * BM > partial_floats || tiles > n_counters)) --splits;
    }
    if (splits_used) *splits_used = splits;
    const long n_units = (long)tiles * splits;
    if (n_units > 2000000000L) return fb_fail(-1, "gemm_tc: too many tiles (M=%d N=%d)", M, N);
    auto kern = gemm_tc_kernel<BN, TO>;
    static bool configured[FB_MAX_DEVICES] = {};
    if (fb_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return fb_fail(-2, "gemm_tc: cannot reserve %d bytes of shared memory: %s",
                                             Cfg::SMEM_BYTES, cudaGetErrorString(e));
        fb_setup_done(configured);
    }
    const int grid = (int)(n_units < slots ? n_units : slots);
    fb_launch_class(BN >= 256 ? FB_LAUNCH_GEMM_WIDE : FB_LAUNCH_OTHER, (kern), grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream, mw, mx, (TO*)out, ldo, slab_stride, partials,
              counters, M, N, K, splits, tiles_m, tiles_n, (int)n_units, gated, status);
    return fb_check_launch("gemm_tc");
}

}  // namespace

// X [M,K] and W [N,K] are bfloat16 with row strides lda, ldw (elements); out is float32 or bfloat16.
// Split-K has two forms.  With slab_stride == 0 the splits meet in `partials` (float32 scratch) and the CTA that
// arrives last at `counters` (int32, zero before the first call; the kernel leaves them zero) writes the sum.
// With slab_stride > 0 (float32 out only) split s writes its share to out + s * slab_stride and the caller's
// next kernel adds the `*splits_used` slabs (at most max_slabs), which costs no second pass here.
// Shapes the TMA path cannot take are refused with an error, never computed wrongly.
FB_API int fb_gemm_tc(const void* X, long long lda, const void* W, long long ldw, void* out, int o_dtype,
                      long long ldo, long long slab_stride, int max_slabs, int* splits_used, int M, int N, int K,
                      float* partials, long long partial_floats, int* counters, int n_counters, int force_splits,
                      int* status, cudaStream_t stream) {
    FB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    FB_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm_tc: a row stride is shorter than its row");
    FB_REQUIRE(lda % 8 == 0 && ldw % 8 == 0, "gemm_tc: row strides must be multiples of 8 elements (16 bytes)");
    FB_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    FB_REQUIRE(partials && counters && n_counters > 0, "gemm_tc: split-K scratch missing");
    FB_REQUIRE(slab_stride == 0 || (o_dtype == FB_F32 && max_slabs >= 1 && slab_stride >= (long long)M * ldo),
               "gemm_tc: slabs must be float32, at least one, and not overlap");
    if (splits_used) *splits_used = 1;
    if (M == 0) return 0;
    const int BN = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if (BN == 256 && force_splits <= 1 && (o_dtype == FB_F32 || o_dtype == FB_BF16)) {
        const int slabs = (slab_stride > 0 && o_dtype == FB_F32 && force_splits == 0) ? max_slabs : 1;
        if (const int shares = fb_gemm_pair_plan(M, N, K, slabs)) {
            if (splits_used) *splits_used = shares;
            return fb_launch_gemm_pair(X, (long)lda, W, (long)ldw, out, o_dtype, (long)ldo, (long)slab_stride, shares,
                                       M, N, K, 0, 0, status, stream);
        }
    }
    CUtensorMap mw, mx;
    int rc = fb_tensor_map_bf16(&mw, W, N, K, (long)ldw, BK, BM);
    if (rc) return rc;
    rc = fb_tensor_map_bf16(&mx, X, M, K, (long)lda, BK, BN);
    if (rc) return rc;
#define FB_TC_CASE(BN_)                                                                                         \
    case BN_:                                                                                                   \
        if (o_dtype == FB_F32)                                                                                  \
            return launch_tc<BN_, float>(mw, mx, out, (long)ldo, (long)slab_stride, max_slabs, splits_used,     \
                                         partials, (long)partial_floats, counters, n_counters, M, N, K,         \
                                         force_splits, status, stream);                                         \
        else if (o_dtype == FB_BF16)                                                                            \
            return launch_tc<BN_, __nv_bfloat16>(mw, mx, out, (long)ldo, 0, 1, splits_used, partials,           \
                                                 (long)partial_floats, counters, n_counters, M, N, K,           \
                                                 force_splits, status, stream);                                 \
        break;
    switch (BN) {
        FB_TC_CASE(16)
        FB_TC_CASE(32)
        FB_TC_CASE(64)
        FB_TC_CASE(128)
        FB_TC_CASE(256)
    }
#undef FB_TC_CASE
    return fb_fail(-1, "gemm_tc: unknown output dtype code %d", o_dtype);
}

// acc[M,N] += X[M,K] * W[N,K]^T in float32 where the product is one that leaves in whole tiles through the two-SM
// kernel (hundreds of rows, and no shares of K would be chosen although the caller has `max_slabs` slabs for them):
// each element gets one float32 add, so a residual stream takes a part's output without a pass of its own.
// Returns 1 if the product was added, 0 if this is not such a product (nothing was done: the caller takes the
// other way), negative on an error.
FB_API int fb_gemm_tc_add(const void* X, long long lda, const void* W, long long ldw, float* acc, long long ldacc,
                          int max_slabs, int M, int N, int K, int* status, cudaStream_t stream) {
    FB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc_add: bad sizes M=%d N=%d K=%d", M, N, K);
    FB_REQUIRE(lda >= K && ldw >= K && ldacc >= N, "gemm_tc_add: a row stride is shorter than its row");
    FB_REQUIRE(lda % 8 == 0 && ldw % 8 == 0, "gemm_tc_add: row strides must be multiples of 8 elements (16 bytes)");
    FB_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tc_add: operands must be 16-byte aligned");
    if (M <= 128) return 0;
    if (fb_gemm_pair_plan(M, N, K, max_slabs < 1 ? 1 : max_slabs) != 1) return 0;
    const int rc = fb_launch_gemm_pair(X, (long)lda, W, (long)ldw, acc, FB_F32, (long)ldacc, 0, 1, M, N, K, 0, 1, status,
                                       stream);
    return rc ? rc : 1;
}

// out[M, N/2] = act(g) * u with [g_0, u_0, g_1, u_1, ...] = X[M,K] * W[N,K]^T: W stacks gate and up rows
// alternately, and the activation `act` (an FbAct code) is applied in the epilogue (the whole sum in one CTA, so
// K is not split).
FB_API int fb_gemm_tc_gated(const void* X, long long lda, const void* W, long long ldw, void* out, int o_dtype,
                            long long ldo, int M, int N, int K, int act, float* partials, long long partial_floats,
                            int* counters, int n_counters, int* status, cudaStream_t stream) {
    FB_REQUIRE(M >= 0 && N > 0 && K > 0 && N % 2 == 0, "gemm_tc_gated: bad sizes M=%d N=%d K=%d", M, N, K);
    FB_REQUIRE(fb_act_known(act), "gemm_tc_gated: unknown activation code %d", act);
    FB_REQUIRE(lda >= K && ldw >= K && ldo >= N / 2, "gemm_tc_gated: a row stride is shorter than its row");
    FB_REQUIRE(lda % 8 == 0 && ldw % 8 == 0, "gemm_tc_gated: row strides must be multiples of 8 elements");
    FB_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tc_gated: operands must be 16-byte aligned");
    if (M == 0) return 0;
    const int BN = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if (BN == 256 && (o_dtype == FB_F32 || o_dtype == FB_BF16) && fb_gemm_pair_plan(M, N, K, 1))
        return fb_launch_gemm_pair(X, (long)lda, W, (long)ldw, out, o_dtype, (long)ldo, 0, 1, M, N, K, act, 0, status,
                                   stream);
    CUtensorMap mw, mx;
    int rc = fb_tensor_map_bf16(&mw, W, N, K, (long)ldw, BK, BM);
    if (rc) return rc;
    rc = fb_tensor_map_bf16(&mx, X, M, K, (long)lda, BK, BN);
    if (rc) return rc;
#define FB_TCG_CASE(BN_)                                                                                        \
    case BN_:                                                                                                   \
        if (o_dtype == FB_F32)                                                                                  \
            return launch_tc<BN_, float>(mw, mx, out, (long)ldo, 0, 1, nullptr, partials, (long)partial_floats, \
                                         counters, n_counters, M, N, K, 1, status, stream, act);                \
        else if (o_dtype == FB_BF16)                                                                            \
            return launch_tc<BN_, __nv_bfloat16>(mw, mx, out, (long)ldo, 0, 1, nullptr, partials,               \
                                                 (long)partial_floats, counters, n_counters, M, N, K, 1, status, \
                                                 stream, act);                                                  \
        break;
    switch (BN) {
        FB_TCG_CASE(16)
        FB_TCG_CASE(32)
        FB_TCG_CASE(64)
        FB_TCG_CASE(128)
        FB_TCG_CASE(256)
    }
#undef FB_TCG_CASE
    return fb_fail(-1, "gemm_tc_gated: unknown output dtype code %d", o_dtype);
}

// ---------------------------------------------------------------------------
// The product for callers that must not allocate (declared and described in no_alloc.h; no counterpart in the
// reference).  Same kernel and launcher as fb_gemm_tc in its meet-in-scratch form; the scratch is this array.
// ---------------------------------------------------------------------------
#include "no_alloc.h"

// Partial tiles (float32) followed by one arrival counter per output tile.  Held by every GPU that loads the
// library until the process exits.  In host code this name is only a handle for cudaGetSymbolAddress: it is not
// a device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char fb_noalloc_scratch[FB_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
void* g_noalloc_base[NOALLOC_MAX_DEVICES] = {};      // device address of the array, per device ordinal
std::mutex g_noalloc_mu;

// Once per device, with that device current: the array's device address.
int noalloc_scratch(unsigned char** base) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fb_fail(-2, "gemm_tc_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES)
        return fb_fail(-1, "gemm_tc_noalloc: device ordinal %d is outside [0, %d)", dev, NOALLOC_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_base[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, fb_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return fb_fail(-2, "gemm_tc_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                           cudaGetErrorString(e));
        g_noalloc_base[dev] = p;
    }
    *base = (unsigned char*)g_noalloc_base[dev];
    return 0;
}
}  // namespace

int fb_gemm_tc_noalloc(const void* X, long long lda, const void* W, long long ldw, void* out, int o_dtype,
                       long long ldo, int M, int N, int K, int* status, cudaStream_t stream) {
    FB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc_noalloc: bad sizes M=%d N=%d K=%d", M, N, K);
    FB_REQUIRE(M <= FB_NOALLOC_MAX_ROWS, "gemm_tc_noalloc: %d rows exceed the maximum of %d", M, FB_NOALLOC_MAX_ROWS);
    const int tiles_n = (N + BM - 1) / BM;
    FB_REQUIRE(tiles_n <= FB_NOALLOC_MAX_TILES, "gemm_tc_noalloc: %d output features exceed the maximum of %d", N,
               FB_NOALLOC_MAX_TILES * BM);
    FB_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm_tc_noalloc: a row stride is shorter than its row");
    FB_REQUIRE(lda % 8 == 0 && ldw % 8 == 0, "gemm_tc_noalloc: row strides must be multiples of 8 elements");
    FB_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tc_noalloc: operands must be 16-byte aligned");
    FB_REQUIRE(status != nullptr, "gemm_tc_noalloc: the status word is missing");
    if (M == 0) return 0;
    unsigned char* base = nullptr;
    int rc = noalloc_scratch(&base);
    if (rc) return rc;
    float* partials = (float*)base;
    int* counters = (int*)(base + FB_NOALLOC_PARTIAL_BYTES);
    // the array keeps the last call's contents: the counters must start at zero (stream-ordered, no allocation)
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)FB_NOALLOC_MAX_TILES * sizeof(int), stream);
    if (e != cudaSuccess) return fb_fail(-2, "gemm_tc_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
    const int BN = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    CUtensorMap mw, mx;
    rc = fb_tensor_map_bf16_uncached(&mw, W, N, K, (long)ldw, BK, BM);
    if (rc) return rc;
    rc = fb_tensor_map_bf16_uncached(&mx, X, M, K, (long)lda, BK, BN);
    if (rc) return rc;
    const long partial_floats = (long)(FB_NOALLOC_PARTIAL_BYTES / sizeof(float));
#define FB_NA_CASE(BN_)                                                                                          \
    case BN_:                                                                                                    \
        if (o_dtype == FB_F32)                                                                                   \
            return launch_tc<BN_, float>(mw, mx, out, (long)ldo, 0, 1, nullptr, partials, partial_floats,        \
                                         counters, FB_NOALLOC_MAX_TILES, M, N, K, 0, status, stream);            \
        else if (o_dtype == FB_BF16)                                                                             \
            return launch_tc<BN_, __nv_bfloat16>(mw, mx, out, (long)ldo, 0, 1, nullptr, partials,                \
                                                 partial_floats, counters, FB_NOALLOC_MAX_TILES, M, N, K, 0,     \
                                                 status, stream);                                                \
        break;
    switch (BN) {
        FB_NA_CASE(16)
        FB_NA_CASE(32)
        FB_NA_CASE(64)
    }
#undef FB_NA_CASE
    return fb_fail(-1, "gemm_tc_noalloc: unknown output dtype code %d", o_dtype);
}
