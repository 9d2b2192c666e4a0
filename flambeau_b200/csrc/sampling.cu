// Token choice on the device: penalties and logit bias, then per row either
// argmax (temperature <= 0; the lowest index wins a tie) or a draw from
// softmax(logits / T), optionally restricted by top-k, top-p and min-p.
//
// Order of operations and formulas follow the reference's host sampler
// (crates/runtime/src/sampling.rs:306-335 order; :486-496 argmax tie rule;
// :575-607 penalties; :610-746 softmax with max subtraction, filters,
// inverse-CDF pick with u * sum of the kept mass).  The filters are applied as
// a threshold on the (unnormalised) probabilities found by radix selection
// instead of a sort: the kept set is {i : z_i >= tau}, tau the largest of the
// k-th largest value, the value that closes the top-p prefix, and
// min_p * z_max.  Entries that tie with tau are all kept.  The draw walks the
// kept entries in index order.
#include "common.cuh"

#define SAMPLE_THREADS 1024

// (token, count) pairs per row: logits[row][tok] gets the three penalties.
__global__ void penalties_kernel(float* __restrict__ logits, long stride, int V, const int* __restrict__ rows,
                                 const int* __restrict__ tokens, const int* __restrict__ counts,
                                 const float* __restrict__ repetition, const float* __restrict__ presence,
                                 const float* __restrict__ frequency, int n_pairs) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int r = rows[i], tok = tokens[i];
    if (tok < 0 || tok >= V) return;
    float* l = logits + (size_t)r * stride + tok;
    float v = *l;
    const float rep = repetition[r];
    if (rep != 1.0f && rep > 0.0f) v = v > 0.0f ? v / rep : v * rep;
    if (presence[r] != 0.0f) v -= presence[r];
    if (frequency[r] != 0.0f) v -= frequency[r] * (float)counts[i];
    *l = v;
}

FB_API int fb_apply_penalties(float* logits, long long stride, int V, const int* rows, const int* tokens,
                              const int* counts, const float* repetition, const float* presence,
                              const float* frequency, int n_pairs, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    fb_launch((penalties_kernel), (n_pairs + 255) / 256, 256, 0, stream, logits, (long)stride, V, rows, tokens, counts,
                                                               repetition, presence, frequency, n_pairs);
    return fb_check_launch("apply_penalties");
}

// (row, token, bias) triples: logits[row][tok] += bias.  Pairs must be unique.
__global__ void logit_bias_kernel(float* __restrict__ logits, long stride, int V, const int* __restrict__ rows,
                                  const int* __restrict__ tokens, const float* __restrict__ bias, int n) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int tok = tokens[i];
    if (tok < 0 || tok >= V) return;
    logits[(size_t)rows[i] * stride + tok] += bias[i];
}

FB_API int fb_apply_logit_bias(float* logits, long long stride, int V, const int* rows, const int* tokens,
                               const float* bias, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    fb_launch((logit_bias_kernel), (n + 255) / 256, 256, 0, stream, logits, (long)stride, V, rows, tokens, bias, n);
    return fb_check_launch("apply_logit_bias");
}

struct SampleShared {
    float red[32];
    int red_i[32];
    float hist[256];
    float scan[SAMPLE_THREADS];
    float f_bcast;
    int i_bcast;
    unsigned u_bcast;
};

// Radix selection over the bit patterns of the non-negative values z_i.
// by_mass == 0: the `target`-th largest value (target counts entries).
// by_mass == 1: the value at which the mass summed from the largest value down
// first reaches `target`.  Returns 0 when the whole row does not reach it.
template <typename ZF>
__device__ float radix_threshold(SampleShared& sh, ZF z_of, int c0, int c1, int by_mass, float target) {
    unsigned prefix = 0, mask = 0;
    float remaining = target;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.hist[b] = 0.0f;
        __syncthreads();
        for (int i = c0; i < c1; ++i) {
            const float z = z_of(i);
            const unsigned bits = __float_as_uint(z);
            if ((bits & mask) == prefix) atomicAdd(&sh.hist[(bits >> shift) & 255u], by_mass ? z : 1.0f);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float acc = 0.0f;
            int chosen = -1;
            for (int b = 255; b >= 0; --b) {
                if (acc + sh.hist[b] >= remaining && sh.hist[b] > 0.0f) { chosen = b; break; }
                acc += sh.hist[b];
            }
            sh.i_bcast = chosen;
            sh.f_bcast = remaining - acc;
        }
        __syncthreads();
        const int chosen = sh.i_bcast;
        if (chosen < 0) return 0.0f;
        remaining = sh.f_bcast;
        prefix |= (unsigned)chosen << shift;
        mask |= 255u << shift;
    }
    return __uint_as_float(prefix);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long stride, int V, const float* __restrict__ temperature,
              const float* __restrict__ uniform, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p, int* __restrict__ out) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    __shared__ SampleShared sh;
    const int row = blockIdx.x;
    const float* l = logits + (size_t)row * stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);

    // ---- argmax, lowest index on ties ----
    // (consecutive threads read consecutive entries; a thread meets its entries in rising order, so `>` keeps the
    // lowest index among equals, and the reduction below compares indices)
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    {
        int i = tid;
        for (; i + 3 * SAMPLE_THREADS < V; i += 4 * SAMPLE_THREADS) {
            const float v0 = l[i], v1 = l[i + SAMPLE_THREADS], v2 = l[i + 2 * SAMPLE_THREADS], v3 = l[i + 3 * SAMPLE_THREADS];
            if (v0 > best) { best = v0; best_i = i; }
            if (v1 > best) { best = v1; best_i = i + SAMPLE_THREADS; }
            if (v2 > best) { best = v2; best_i = i + 2 * SAMPLE_THREADS; }
            if (v3 > best) { best = v3; best_i = i + 3 * SAMPLE_THREADS; }
        }
        for (; i < V; i += SAMPLE_THREADS) {
            const float v = l[i];
            if (v > best) { best = v; best_i = i; }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { sh.red[warp] = best; sh.red_i[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = sh.red[lane];
        best_i = sh.red_i[lane];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { sh.f_bcast = best; sh.i_bcast = best_i == 0x7fffffff ? 0 : best_i; }
    }
    __syncthreads();
    const float row_max = sh.f_bcast;
    const int row_argmax = sh.i_bcast;
    const float T = temperature ? temperature[row] : 0.0f;
    if (!(T > 0.0f)) {
        if (tid == 0) out[row] = row_argmax;
        return;
    }
    const float inv_t = 1.0f / T;
    const float max_scaled = row_max * inv_t;
    auto z_of = [&](int i) { return expf(l[i] * inv_t - max_scaled); };

    // ---- threshold from the filters ----
    float tau = 0.0f;
    const int k = top_k ? top_k[row] : 0;
    const float tp = top_p ? top_p[row] : 0.0f;
    const float mp = min_p ? min_p[row] : 0.0f;
    if (k > 0 && k < V) tau = fmaxf(tau, radix_threshold(sh, z_of, c0, c1, 0, (float)k));
    if (tp > 0.0f && tp < 1.0f) {
        float part = 0.0f;
        for (int i = c0; i < c1; ++i) part += z_of(i);
        const float total = fb_block_sum(part, sh.red);
        tau = fmaxf(tau, radix_threshold(sh, z_of, c0, c1, 1, tp * total));
    }
    if (mp > 0.0f) tau = fmaxf(tau, mp);               // z_max is exp(0) = 1

    // ---- inverse-CDF pick over the kept entries, in index order ----
    float part = 0.0f;
    int last_kept = -1;
    for (int i = c0; i < c1; ++i) {
        const float z = z_of(i);
        if (z >= tau) { part += z; last_kept = i; }
    }
    __syncthreads();
    sh.scan[tid] = part;
    __syncthreads();
    // inclusive scan over the 1024 per-thread sums (Hillis-Steele in shared memory)
    for (int o = 1; o < SAMPLE_THREADS; o <<= 1) {
        const float add = tid >= o ? sh.scan[tid - o] : 0.0f;
        __syncthreads();
        sh.scan[tid] += add;
        __syncthreads();
    }
    const float kept_sum = sh.scan[SAMPLE_THREADS - 1];
    const float before = sh.scan[tid] - part;
    const float target = uniform[row] * kept_sum;
    if (tid == 0) { sh.i_bcast = 0x7fffffff; sh.u_bcast = 0; }
    __syncthreads();
    if (part > 0.0f && before <= target && target <= before + part) atomicMin(&sh.i_bcast, tid);
    atomicMax(&sh.u_bcast, (unsigned)(last_kept + 1));
    __syncthreads();
    if (sh.i_bcast == 0x7fffffff) {
        if (tid == 0) out[row] = (int)sh.u_bcast > 0 ? (int)sh.u_bcast - 1 : row_argmax;
        return;
    }
    if (tid == sh.i_bcast) {
        float r = target - before;
        int pick = last_kept;
        for (int i = c0; i < c1; ++i) {
            const float z = z_of(i);
            if (z >= tau) {
                r -= z;
                if (r <= 0.0f) { pick = i; break; }
            }
        }
        out[row] = pick;
    }
}

FB_API int fb_sample(const float* logits, long long stride, int n, int V, const float* temperature,
                     const float* uniform, const int* top_k, const float* top_p, const float* min_p, int* out,
                     cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && V > 0 && stride >= V, "sample: bad sizes n=%d V=%d", n, V);
    FB_REQUIRE(!temperature || uniform, "sample: a temperature needs uniform numbers");
    if (n == 0) return 0;
    fb_launch((sample_kernel), n, SAMPLE_THREADS, 0, stream, logits, (long)stride, V, temperature, uniform, top_k, top_p,
                                                    min_p, out);
    return fb_check_launch("sample");
}
