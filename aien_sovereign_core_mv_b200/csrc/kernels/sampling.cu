// Token choice from float32 logits: greedy (first maximum wins) and temperature sampling with
// optional top-k and top-p, one block per row.
//
// Rules restated from the reference sampler (crates/aien-inference-abi/src/transformer_backend.rs:
// 104-172; top-k from src/qwen3_moe_omega.rs:3246-3272):
//   * temperature <= 0.001 is greedy; ties go to the lower token id (src/tensor.rs:299-318);
//   * top-k keeps the k largest logits, ties to the lower id;
//   * probabilities are softmax(l / T) with the maximum subtracted;
//   * top-p keeps the smallest prefix, in order of falling probability (ties to the lower id),
//     whose mass reaches top_p;
//   * one uniform number u in [0,1), scaled to the kept mass, picks the token.
// Own design: u comes from Philox4x32-10 keyed by the request's seed with counter
// (request id, position), so a draw depends on nothing else in the batch; the kept set is
// walked in token-id order.  Thresholds are found by bisection on an order-preserving integer
// image of the floats, which needs no sort.  `probs` is scratch of V floats per row.
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int SM_THREADS = 1024;

__device__ __forceinline__ uint32_t ordered_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ double block_sum_f64(double v, double* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < nwarps; ++w) total += red[w];
    return total;
}
__device__ __forceinline__ long long block_sum_i64(long long v, double* red) {
    long long* r = reinterpret_cast<long long*>(red);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) r[warp] = v;
    __syncthreads();
    long long total = 0;
    for (int w = 0; w < nwarps; ++w) total += r[w];
    return total;
}

// argmax with ties to the lower index; returns to every thread
__device__ int block_argmax(const float* __restrict__ row, int V, float* best_val_out, double* red) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    float* rv = reinterpret_cast<float*>(red);
    int* ri = reinterpret_cast<int*>(red) + 64;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { rv[warp] = bv; ri[warp] = bi; }
    __syncthreads();
    bv = rv[0]; bi = ri[0];
    for (int w = 1; w < nwarps; ++w) {
        if (rv[w] > bv || (rv[w] == bv && ri[w] < bi)) { bv = rv[w]; bi = ri[w]; }
    }
    *best_val_out = bv;
    return bi;
}

// Smallest id c such that #{i <= c : pred(i)} >= need, pred(i) = (key(row[i]) == thr) [&& extra]
template <typename Pred>
__device__ int id_cutoff(int V, long long need, Pred pred, double* red) {
    int lo = 0, hi = V - 1;                       // answer in [lo, hi]
    while (lo < hi) {
        const int mid = lo + (hi - lo) / 2;
        long long c = 0;
        for (int i = threadIdx.x; i <= mid; i += blockDim.x) c += pred(i) ? 1 : 0;
        c = block_sum_i64(c, red);
        if (c >= need) hi = mid; else lo = mid + 1;
    }
    return lo;
}

__global__ void __launch_bounds__(SM_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const float* __restrict__ top_p, const int* __restrict__ top_k,
                   const unsigned long long* __restrict__ seeds, const long long* __restrict__ request_ids,
                   const int* __restrict__ positions, float* __restrict__ probs_scratch,
                   int* __restrict__ out_ids) {
    __shared__ double red[64];
    __shared__ double scan[SM_THREADS];
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * V;
    float maxv;
    const int amax = block_argmax(row, V, &maxv, red);
    const float T = temperature ? temperature[r] : 0.f;
    if (!(T > 0.001f)) {                           // greedy threshold of the reference
        if (tid == 0) out_ids[r] = amax;
        return;
    }
    float* probs = probs_scratch + (size_t)r * V;

    // ---- top-k: allowed(i) = key > thr_k || (key == thr_k && i <= cut_k)
    const int k = top_k ? top_k[r] : 0;
    uint32_t thr_k = 0; int cut_k = V - 1;
    if (k > 0 && k < V) {
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            long long c = 0;
            for (int i = tid; i < V; i += SM_THREADS) c += ordered_key(row[i]) >= cand ? 1 : 0;
            c = block_sum_i64(c, red);
            if (c >= k) prefix = cand;
        }
        thr_k = prefix;
        long long gt = 0;
        for (int i = tid; i < V; i += SM_THREADS) gt += ordered_key(row[i]) > thr_k ? 1 : 0;
        gt = block_sum_i64(gt, red);
        const uint32_t tk = thr_k;
        cut_k = id_cutoff(V, (long long)k - gt, [&](int i) { return ordered_key(row[i]) == tk; }, red);
    }

    // ---- unnormalised probabilities e_i = exp((l_i - max) / T) of the allowed tokens
    const double inv_t = 1.0 / (double)T;
    double z = 0.0;
    for (int i = tid; i < V; i += SM_THREADS) {
        const uint32_t key = ordered_key(row[i]);
        const bool allowed = key > thr_k || (key == thr_k && i <= cut_k);
        const float e = allowed ? (float)exp(((double)row[i] - (double)maxv) * inv_t) : 0.f;
        probs[i] = e;
        z += (double)e;
    }
    z = block_sum_f64(z, red);

    // ---- top-p: kept(i) = e_i > 0 && (key > thr_p || (key == thr_p && i <= cut_p))
    const float tp = top_p ? top_p[r] : 1.f;
    uint32_t thr_p = 0; int cut_p = V - 1;
    double kept_mass = z;
    if (tp > 0.f && tp < 1.f) {
        const double target = (double)tp * z;
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            double mass = 0.0;
            for (int i = tid; i < V; i += SM_THREADS)
                if (ordered_key(row[i]) >= cand) mass += (double)probs[i];
            mass = block_sum_f64(mass, red);
            if (mass >= target) prefix = cand;
        }
        thr_p = prefix;
        double m_gt = 0.0; long long n_eq = 0;
        for (int i = tid; i < V; i += SM_THREADS) {
            const uint32_t key = ordered_key(row[i]);
            if (key > thr_p) m_gt += (double)probs[i];
            else if (key == thr_p && probs[i] > 0.f) n_eq += 1;
        }
        m_gt = block_sum_f64(m_gt, red);
        n_eq = block_sum_i64(n_eq, red);
        const double p_thr = (double)(float)exp(((double)key_value(thr_p) - (double)maxv) * inv_t);
        long long need = 1;
        if (p_thr > 0.0) {
            need = (long long)ceil((target - m_gt) / p_thr);
            if (need < 1) need = 1;
        }
        if (need > n_eq) need = n_eq;
        if (need < 1) need = 1;
        const uint32_t tpk = thr_p;
        cut_p = id_cutoff(V, need, [&](int i) { return ordered_key(row[i]) == tpk && probs[i] > 0.f; }, red);
        kept_mass = m_gt + (double)need * p_thr;
    }

    // ---- draw: walk the kept set in id order
    uint32_t rnd[4];
    const unsigned long long seed = seeds ? seeds[r] : 0ull;
    const unsigned long long rid = request_ids ? (unsigned long long)request_ids[r] : 0ull;
    const uint32_t posn = positions ? (uint32_t)positions[r] : 0u;
    philox4x32_10(posn, 0u, (uint32_t)rid, (uint32_t)(rid >> 32), (uint32_t)seed, (uint32_t)(seed >> 32), rnd);
    const double u = (double)((((unsigned long long)rnd[0] << 32) | rnd[1]) >> 11) * (1.0 / 9007199254740992.0);

    const int per = (V + SM_THREADS - 1) / SM_THREADS;
    const int lo = tid * per, hi = min(V, lo + per);
    double local = 0.0;
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = ordered_key(row[i]);
        if (probs[i] > 0.f && (key > thr_p || (key == thr_p && i <= cut_p))) local += (double)probs[i];
    }
    scan[tid] = local;
    __syncthreads();
    __shared__ int chosen;
    __shared__ int last_kept_thread;
    if (tid == 0) {
        double total = 0.0;
        for (int w = 0; w < SM_THREADS; ++w) total += scan[w];
        const double rr = u * total;
        double cum = 0.0;
        int pick = -1, last = 0;
        for (int w = 0; w < SM_THREADS; ++w) {
            const double s = scan[w];
            if (s > 0.0) last = w;
            if (pick < 0 && rr < cum + s) { pick = w; scan[w] = rr - cum; }   // remainder to walk inside w
            cum += s;
        }
        if (pick < 0) { pick = last; scan[last] = INFINITY; }
        chosen = pick;
        last_kept_thread = last;
    }
    __syncthreads();
    (void)kept_mass; (void)last_kept_thread;
    if (tid == chosen) {
        const double rem = scan[tid];
        double cum = 0.0;
        int pick = -1, last = lo;
        for (int i = lo; i < hi; ++i) {
            const uint32_t key = ordered_key(row[i]);
            if (probs[i] > 0.f && (key > thr_p || (key == thr_p && i <= cut_p))) {
                cum += (double)probs[i];
                last = i;
                if (rem < cum) { pick = i; break; }
            }
        }
        out_ids[r] = pick >= 0 ? pick : last;
    }
}

__global__ void __launch_bounds__(SM_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ out_ids) {
    __shared__ double red[64];
    float mv;
    const int a = block_argmax(logits + (size_t)blockIdx.x * V, V, &mv, red);
    if (threadIdx.x == 0) out_ids[blockIdx.x] = a;
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_argmax_rows(const float* logits, int R, int V, int* out_ids, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return AIEN_E_SHAPE;
    argmax_rows_kernel<<<R, SM_THREADS, 0, stream>>>(logits, V, out_ids);
    return launch_status();
}

// `probs_scratch` holds R*V floats (only rows with temperature > 0.001 touch it).
AIEN_API int aien_sample_rows(const float* logits, int R, int V, const float* temperature, const float* top_p,
                              const int* top_k, const unsigned long long* seeds, const long long* request_ids,
                              const int* positions, float* probs_scratch, int* out_ids, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return AIEN_E_SHAPE;
    sample_rows_kernel<<<R, SM_THREADS, 0, stream>>>(logits, V, temperature, top_p, top_k, seeds, request_ids,
                                                     positions, probs_scratch, out_ids);
    return launch_status();
}
