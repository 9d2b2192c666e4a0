// What the two arrangements of the bfloat16 tensor-core attention share: the argument block, the key range a group
// of query tokens can see, the layout of a K/V tile in shared memory and the mma.sync / ldmatrix wrappers.
#pragma once

#include "async_copy.cuh"
#include "tensor_map.cuh"

namespace fb_attn {

constexpr int KT = 64;             // keys per tile

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
    const int* table_base;             // per sequence: the logical page that column 0 of its table row stands for
                                       // (nullptr: page 0); released leading pages are not in the table
    const int* seq_q_start; const int* seq_q_len; const int* seq_pos_start;
    const int* multi_seqs; int n_multi;   // the sequences that bring more than one token, in step order: the grid of
                                          // the arrangements for portions covers only these (nullptr: all n_seqs)
    int nh, nkv, hd, window;
    float scale_log2e;
    const float* score_slopes;         // per query head, or nullptr: slope * (key position - query position) is added
                                       // to the scaled score (a linear penalty on distance; <= 0 for the keys a
                                       // query sees when the slope is >= 0)
    float* part_o; float* part_ml;     // split-key: partial results, [slot][16 rows][HD_MAX] and [slot][16][2]
    int* part_cnt;                     // split-key: per (sequence, key/value head), segments that have arrived; 0 at rest
    int n_seqs;                        // sequences of the step
    int short_ctas;                    // split-key: CTAs of the split-key launch
    int min_tiles;                     // split-key: a CTA's stretch is at least this long
    int short_rows;                    // sequences with q_len * G <= short_rows belong to the split-key arrangement
    FbPrefetch prefetch;               // split-key: rows to fetch into L2 when a CTA has issued its last tile
    int* status;
};

// The page id of logical page `logical` of a sequence whose table row `table` starts at logical page `base_page`
// (-1 where the row has no such column).
__device__ __forceinline__ int table_page(const AttnArgs& a, const int* table, int base_page, int logical) {
    const int e = logical - base_page;
    return (e >= 0 && e < a.table_stride) ? table[e] : -1;
}
__device__ __forceinline__ int table_base_of(const AttnArgs& a, int seq) { return a.table_base ? a.table_base[seq] : 0; }
// Sequences that the arrangements for portions lay their grid over, and the j-th of them.
__host__ __device__ __forceinline__ int portion_seqs(const AttnArgs& a) { return a.multi_seqs ? a.n_multi : a.n_seqs; }
__device__ __forceinline__ int portion_seq(const AttnArgs& a, int j) { return a.multi_seqs ? a.multi_seqs[j] : j; }

// The keys a group of consecutive query tokens [first, last] of a sequence can see, and where tiles start.
struct KeyRange { int t_lo, t_hi, tile_lo; };
__device__ __forceinline__ KeyRange key_range(int p_first, int p_last, int window) {
    KeyRange r;
    r.t_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    r.t_hi = p_last;
    r.tile_lo = (r.t_lo / KT) * KT;
    return r;
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

}  // namespace fb_attn

// The split-key arrangement (attention_split.cu): sequences with q_len * G <= a.short_rows.  Fills in what depends
// on its grid, launches, returns 0 or an error code with the message set.
int fb_launch_attention_split(fb_attn::AttnArgs& a, int hd_max, bool tma, int n_seqs, float* scratch,
                              long long scratch_floats, cudaStream_t stream);

// The tcgen05 arrangement for portions of prompts (attention_tc.cu): whether it takes this geometry, and its launch.
bool fb_attention_tc_takes(const fb_attn::AttnArgs& a, bool tma);
int fb_launch_attention_tc(const fb_attn::AttnArgs& a, int n_seqs, int max_q_len, cudaStream_t stream);
