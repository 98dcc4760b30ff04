// Token choice from float32 logits: greedy (first maximum wins) and temperature sampling with
// optional top-k and top-p, one block per row, or a cluster of eight blocks per row when the rows are few.
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
// image of the floats, which needs no sort.  The nucleus bisects over the few tokens that can
// belong to it, gathered in shared memory (tokens too light to matter are left out by a bound
// that is exact); a flat distribution with more than 4,096 such tokens bisects over the row (pass by pass
// in one CTA; in a cluster with every thread's tokens in registers).  The draw walks the kept tokens in id
// order with integer masses: a thread sums a run of consecutive tokens, the runs are added up in order.
// Masses are summed as integers, so no result depends on an order of summation.  Temperature alone
// (every token drawable) sums runs of consecutive tokens per thread and walks the run that holds the draw.
// `probs` is scratch of V floats per row.
#include "common.cuh"
#include <cooperative_groups.h>
#include <math.h>
#include <cstdlib>

namespace aien {

namespace cg = cooperative_groups;

constexpr int SM_THREADS = 1024;
// A step of few rows shares each row among the CTAs of a cluster: every CTA takes an eighth of the row in
// the passes over it (maximum, counts, the gathering of the tokens that can matter), the first CTA collects
// what the others found through distributed shared memory and goes on as one CTA alone does.  What is
// collected are sets and integer sums, so the token drawn is the same one.
constexpr int SM_CLUSTER = 8;
struct SmClusterSlot {             // what a CTA of the cluster tells the others
    float val; int idx;            // its part's maximum
    int count;                     // tokens it gathered
    int pad;
    unsigned long long z;          // its part's mass, in units
};

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

__device__ __forceinline__ long long warp_sum_i64(long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) { return (unsigned long long)warp_sum_i64((long long)v); }

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, double* red) {
    return (unsigned long long)block_sum_i64((long long)v, red);
}

// Calls f(i, row[i]) for every i < V.  Which thread visits which elements, and in which order, is
// fixed by V and the block size alone.  16-byte loads, four in flight per thread, when the row allows.
template <typename F>
__device__ __forceinline__ void scan_row(const float* __restrict__ row, int V, F f) {
    const int nt = blockDim.x, tid = threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        const int V4 = V >> 2;
        const float4* r4 = reinterpret_cast<const float4*>(row);
        int i = tid;
        for (; i + 3 * nt < V4; i += 4 * nt) {
            const float4 a = r4[i], b = r4[i + nt], c = r4[i + 2 * nt], d = r4[i + 3 * nt];
            f(4 * i, a.x); f(4 * i + 1, a.y); f(4 * i + 2, a.z); f(4 * i + 3, a.w);
            f(4 * (i + nt), b.x); f(4 * (i + nt) + 1, b.y); f(4 * (i + nt) + 2, b.z); f(4 * (i + nt) + 3, b.w);
            f(4 * (i + 2 * nt), c.x); f(4 * (i + 2 * nt) + 1, c.y); f(4 * (i + 2 * nt) + 2, c.z); f(4 * (i + 2 * nt) + 3, c.w);
            f(4 * (i + 3 * nt), d.x); f(4 * (i + 3 * nt) + 1, d.y); f(4 * (i + 3 * nt) + 2, d.z); f(4 * (i + 3 * nt) + 3, d.w);
        }
        for (; i < V4; i += nt) {
            const float4 a = r4[i];
            f(4 * i, a.x); f(4 * i + 1, a.y); f(4 * i + 2, a.z); f(4 * i + 3, a.w);
        }
        for (int j = (V4 << 2) + tid; j < V; j += nt) f(j, row[j]);
    } else {
        for (int j = tid; j < V; j += nt) f(j, row[j]);
    }
}

// The same over the elements lo <= i < hi (lo a multiple of 4, so that an aligned row stays aligned).
template <typename F>
__device__ __forceinline__ void scan_range(const float* __restrict__ row, int lo, int hi, F f) {
    if (hi > lo) scan_row(row + lo, hi - lo, [&](int i, float v) { f(i + lo, v); });
}

// argmax over lo <= i < hi with ties to the lower index; returns to every thread (index 0x7fffffff over an empty range)
__device__ int block_argmax(const float* __restrict__ row, int lo, int hi, float* best_val_out, double* red) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    scan_range(row, lo, hi, [&](int i, float v) {
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    });
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

// Smallest id c such that #{i <= c : pred(i, vals[i])} >= need (need >= 1 and at most the number
// of hits): every thread counts a run of consecutive ids, the runs are added up in order.
template <typename Pred>
__device__ int id_cutoff(const float* __restrict__ vals, int V, long long need, Pred pred, long long* run_count, int* result) {
    const int tid = threadIdx.x, per = (V + blockDim.x - 1) / blockDim.x;
    const int lo = tid * per, hi = min(V, lo + per);
    long long c = 0;
    for (int i = lo; i < hi; ++i) c += pred(i, vals[i]) ? 1 : 0;
    __syncthreads();
    run_count[tid] = c;
    if (tid == 0) *result = V - 1;
    __syncthreads();
    long long before = 0;
    for (int w = 0; w < tid; ++w) before += run_count[w];
    if (before < need && before + c >= need) {               // the need-th hit lies in this thread's run
        long long seen = before;
        for (int i = lo; i < hi; ++i)
            if (pred(i, vals[i]) && ++seen == need) { *result = i; break; }
    }
    __syncthreads();
    return *result;
}

// Probabilities are summed as integers (units of 2^-40 of the largest one), so that a sum does not
// depend on the order of its terms: the candidates of the nucleus are gathered in no fixed order.
__device__ __forceinline__ unsigned long long prob_units(float e) { return __float2ull_rz(e * 1099511627776.0f); }   // the scaling by 2^40 is exact

constexpr int SM_CAND = 4096;

// Exclusive sums over the block of one value per thread, in thread order (within a warp by shuffles, the
// warps' totals through `wt`, 32 values of shared memory); *block_total receives the sum.
__device__ __forceinline__ unsigned long long block_exclusive_u64(unsigned long long mine, unsigned long long* wt,
                                                                  unsigned long long* block_total) {
    const int tid = threadIdx.x;
    unsigned long long incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += up;
    }
    __syncthreads();
    if ((tid & 31) == 31) wt[tid >> 5] = incl;
    __syncthreads();
    unsigned long long before = 0, all = 0;
    for (int w = 0; w < SM_THREADS / 32; ++w) {
        if (w < (tid >> 5)) before += wt[w];
        all += wt[w];
    }
    *block_total = all;
    return before + incl - mine;
}

// Two sums over the ranks of a cluster, of values that every thread of a rank holds alike, and the sum of
// v0 over the ranks before this one.  `xs`: two pairs of shared memory per rank, used in turn (`it` counts the
// exchanges), so that one cluster barrier per exchange is enough: a rank can write a pair again only after the
// barrier of the exchange between, which every rank reaches after it has read that pair.  ACROSS false: one rank alone.
template <bool ACROSS>
__device__ __forceinline__ void cluster_sums(unsigned long long v0, unsigned long long v1, unsigned long long (*xs)[2], int& it, int rank,
                                             unsigned long long* t0, unsigned long long* t1, unsigned long long* before0) {
    if (!ACROSS) { *t0 = v0; *t1 = v1; *before0 = 0; return; }
    cg::cluster_group cluster = cg::this_cluster();
    const int slot = it & 1;
    ++it;
    if (threadIdx.x == 0) { xs[slot][0] = v0; xs[slot][1] = v1; }
    cluster.sync();
    unsigned long long a0 = 0, a1 = 0, b0 = 0;
    for (int rk = 0; rk < SM_CLUSTER; ++rk) {
        const unsigned long long* o = cluster.map_shared_rank(&xs[slot][0], rk);
        const unsigned long long x0 = o[0], x1 = o[1];
        if (rk < rank) b0 += x0;
        a0 += x0; a1 += x1;
    }
    *t0 = a0; *t1 = a1; *before0 = b0;
}

// The draw among the tokens lo <= i < hi of this rank (and of the other ranks' parts when ACROSS), in id order,
// masses in integer units: units_of(i) is what token i weighs (0: not kept).  A thread sums a run of consecutive
// tokens, the runs are added up in order, the thread whose run holds the draw walks it.  Every thread calls this.
template <bool ACROSS, typename UnitsOf>
__device__ __forceinline__ void draw_by_runs(int lo, int hi, double u, UnitsOf units_of, unsigned long long* wt,
                                             unsigned long long (*xs)[2], int& it, int rank, int r, int fallback_id,
                                             int* __restrict__ out_ids, float* __restrict__ out_logprob) {
    const int tid = threadIdx.x;
    const int run = (hi - lo + SM_THREADS - 1) / SM_THREADS;
    const int a = min(hi, lo + tid * run), b = min(hi, a + run);
    unsigned long long mine = 0;
    for (int i = a; i < b; ++i) mine += units_of(i);
    unsigned long long part = 0, total = 0, unused = 0, part_before = 0;
    const unsigned long long before = block_exclusive_u64(mine, wt, &part);
    cluster_sums<ACROSS>(part, 0ull, xs, it, rank, &total, &unused, &part_before);
    if (total == 0) {                                   // nothing kept weighs a unit: cannot be, but never leave the id unset
        if (rank == 0 && tid == 0) { out_ids[r] = fallback_id; if (out_logprob != nullptr) out_logprob[r] = 0.f; }
        return;
    }
    unsigned long long rr = (unsigned long long)(u * (double)total);
    if (rr >= total) rr = total - 1;
    const unsigned long long first = part_before + before;          // this thread's run owns the units [first, first + mine)
    if (rr >= first && rr < first + mine) {
        unsigned long long cum = first;
        for (int i = a; i < b; ++i) {
            const unsigned long long w = units_of(i);
            if (rr < cum + w) {
                out_ids[r] = i;
                if (out_logprob != nullptr) out_logprob[r] = (float)log((double)w / (double)total);   // within the kept set
                break;
            }
            cum += w;
        }
    }
}

// The nucleus of a row whose tokens that can matter do not fit in shared memory (a flat distribution), by all
// ranks of the cluster: a thread keeps the probabilities of its run of consecutive tokens in registers, the
// bisection for the threshold adds the masses over block and cluster (integers: no order), ties at the threshold
// go to the lower ids, and the draw walks the kept tokens in id order (draw_by_runs).  The same threshold, the
// same kept set and the same token as the pass-by-pass way of one CTA.  Needs runs of SM_RUN_MAX tokens at most.
constexpr int SM_RUN_MAX = 20;
__device__ __forceinline__ void nucleus_across_cluster(const float* __restrict__ row, int lo, int hi, int V, float maxv, float inv_t,
                                                       float tp, unsigned long long z, double u, unsigned long long* wt, double* red,
                                                       unsigned long long (*xs)[2], int& it, int rank, int r, int fallback_id,
                                                       int* __restrict__ out_ids, float* __restrict__ out_logprob) {
    const int tid = threadIdx.x;
    const int run = (hi - lo + SM_THREADS - 1) / SM_THREADS;
    const int a = min(hi, lo + tid * run), b = min(hi, a + run);
    uint32_t eb[SM_RUN_MAX];
#pragma unroll
    for (int j = 0; j < SM_RUN_MAX; ++j) eb[j] = (a + j < b) ? __float_as_uint(expf((row[a + j] - maxv) * inv_t)) : 0u;
    unsigned long long target = (unsigned long long)ceil((double)tp * (double)z);
    if (target > z) target = z;
    if (target < 1) target = 1;
    unsigned long long t0 = 0, t1 = 0, before = 0;
    uint32_t prefix = 0;
    for (int bit = 30; bit >= 0; --bit) {                                   // bit 31 is the sign: never set
        const uint32_t cand = prefix | (1u << bit);
        unsigned long long m = 0;
#pragma unroll
        for (int j = 0; j < SM_RUN_MAX; ++j) m += eb[j] >= cand ? prob_units(__uint_as_float(eb[j])) : 0ull;
        m = block_sum_u64(m, red);
        cluster_sums<true>(m, 0ull, xs, it, rank, &t0, &t1, &before);
        if (t0 >= target) prefix = cand;
    }
    if (prefix == 0) prefix = 1;
    unsigned long long m_gt = 0, n_eq = 0;
#pragma unroll
    for (int j = 0; j < SM_RUN_MAX; ++j) {
        if (eb[j] > prefix) m_gt += prob_units(__uint_as_float(eb[j]));
        else if (eb[j] == prefix) n_eq += 1;
    }
    const unsigned long long mine_eq = n_eq;
    m_gt = block_sum_u64(m_gt, red);
    n_eq = block_sum_u64(n_eq, red);
    cluster_sums<true>(m_gt, n_eq, xs, it, rank, &t0, &t1, &before);
    m_gt = t0; n_eq = t1;
    const unsigned long long q_thr = prob_units(__uint_as_float(prefix));
    unsigned long long need = 1;
    if (q_thr > 0 && target > m_gt) need = (target - m_gt + q_thr - 1) / q_thr;
    if (need > n_eq) need = n_eq;
    if (need < 1) need = 1;
    int cut = V - 1;
    if (need < n_eq) {                                                      // ties at the threshold: the lower ids
        unsigned long long part = 0, part_before = 0;
        const unsigned long long first = block_exclusive_u64(mine_eq, wt, &part);
        cluster_sums<true>(part, 0ull, xs, it, rank, &t0, &t1, &part_before);
        const unsigned long long mine_first = part_before + first;         // ties before this thread's run
        unsigned long long found = 0;                                      // id + 1 of the need-th tie, in the one thread that holds it
        if (mine_first < need && need <= mine_first + mine_eq) {
            unsigned long long seen = mine_first;
#pragma unroll
            for (int j = 0; j < SM_RUN_MAX; ++j)
                if (eb[j] == prefix && ++seen == need) found = (unsigned long long)(a + j) + 1;
        }
        found = block_sum_u64(found, red);
        cluster_sums<true>(found, 0ull, xs, it, rank, &t0, &t1, &before);
        if (t0 > 0) cut = (int)(t0 - 1);
    }
    const uint32_t thr = prefix;
    draw_by_runs<true>(lo, hi, u, [&](int i) {
        const float e = expf((row[i] - maxv) * inv_t);
        const uint32_t bits = __float_as_uint(e);
        return (e > 0.f && (bits > thr || (bits == thr && i <= cut))) ? prob_units(e) : 0ull;
    }, wt, xs, it, rank, r, fallback_id, out_ids, out_logprob);
    cg::this_cluster().sync();                                              // nobody leaves while its pairs may still be read
}

// The candidate lists of a cluster's ranks put together in rank 0 (in no particular order: what is made of
// them are sets and integer sums), with the sum of the ranks' masses in *z when z is given.  A rank's count
// may exceed SM_CAND (its list is then cut short): the total does too and the caller takes another way.
// Returns the total (SM_CAND + 1 at most) to every rank; every thread of every rank calls this.
__device__ __forceinline__ int collect_candidates(SmClusterSlot& cl, uint32_t* cand_bits, int* cand_id, int* cand_count,
                                                  unsigned long long* z, int rank) {
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x;
    if (tid == 0) { cl.count = min(*cand_count, SM_CAND + 1); cl.z = z ? *z : 0ull; }
    cluster.sync();
    int total = 0;
    unsigned long long zsum = 0;
    bool fits = true;
    for (int rk = 0; rk < SM_CLUSTER; ++rk) {                        // rank 0's own list stays where it is, the others follow it
        const SmClusterSlot* o = cluster.map_shared_rank(&cl, rk);
        const int n = o->count;
        zsum += o->z;
        if (total + n > SM_CAND) fits = false;
        if (rank == 0 && rk > 0 && fits) {
            const uint32_t* rb = cluster.map_shared_rank(cand_bits, rk);
            const int* ri = cluster.map_shared_rank(cand_id, rk);
            for (int j = tid; j < n; j += blockDim.x) { cand_bits[total + j] = rb[j]; cand_id[total + j] = ri[j]; }
        }
        total = min(total + n, SM_CAND + 1);
    }
    if (rank == 0) {
        __syncthreads();
        if (tid == 0) *cand_count = total;
        __syncthreads();
    }
    if (z) *z = zsum;
    cluster.sync();                                    // rank 0 has read the others' lists
    return total;
}

// One row.  CL: the CTA is rank `rank` of a cluster of SM_CLUSTER that shares the row; ranks other than 0
// return once nothing more is asked of them.  Every rank passes the same cluster barriers: what decides
// the way is the same in all of them (the row's options and sums over the whole row).
template <bool CL>
__device__ __forceinline__ void sample_row(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const float* __restrict__ top_p, const int* __restrict__ top_k,
                   const unsigned long long* __restrict__ seeds, const long long* __restrict__ request_ids,
                   const int* __restrict__ positions, float* __restrict__ probs_scratch,
                   int* __restrict__ out_ids, float* __restrict__ out_logprob, const int r, const int rank) {
    __shared__ double red[64];
    __shared__ double scan[SM_THREADS];
    __shared__ uint32_t cand_bits[SM_CAND];         // nucleus candidates: their probabilities, as bit patterns,
    __shared__ int cand_id[SM_CAND];                // and (one-pass case) their token ids
    __shared__ int cand_count, cut_result;
    __shared__ SmClusterSlot cl;
    __shared__ uint32_t s_prefix;                   // what the first warp found for the block
    __shared__ int s_tie;
    __shared__ long long s_count;
    __shared__ unsigned long long s_total;
    __shared__ unsigned long long cl_x[2][2];       // pairs the ranks of a cluster exchange (cluster_sums)
    int cl_it = 0;
    const int tid = threadIdx.x;
    const float* row = logits + (size_t)r * V;
    // this rank's part of the row in the shared passes
    const int per = CL ? (((V + SM_CLUSTER - 1) / SM_CLUSTER + 3) & ~3) : V;
    const int lo = CL ? min(V, rank * per) : 0, hi = CL ? min(V, lo + per) : V;
    float maxv;
    int amax = block_argmax(row, lo, hi, &maxv, red);
    if (CL) {
        cg::cluster_group cluster = cg::this_cluster();
        if (tid == 0) { cl.val = maxv; cl.idx = amax; }
        cluster.sync();
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int rk = 0; rk < SM_CLUSTER; ++rk) {
            const SmClusterSlot* o = cluster.map_shared_rank(&cl, rk);
            const float ov = o->val;
            const int oi = o->idx;
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        maxv = bv; amax = bi;
        cluster.sync();                            // everybody has read: the slots may be written again
    }
    const float T = temperature ? temperature[r] : 0.f;
    if (!(T > 0.001f)) {                           // greedy threshold of the reference
        if (CL && rank != 0) return;
        if (tid == 0) out_ids[r] = amax;
        if (out_logprob != nullptr) {              // log softmax of the logits as they are, at the maximum: -ln sum exp(l - max)
            double sum = 0.0;
            scan_row(row, V, [&](int, float v) { sum += (double)expf(v - maxv); });
            sum = block_sum_f64(sum, red);
            if (tid == 0) out_logprob[r] = (float)(-log(sum));
        }
        return;
    }
    float* probs = probs_scratch + (size_t)r * V;
    long long* run_count = reinterpret_cast<long long*>(scan);

    // the uniform number of this draw
    uint32_t rnd[4];
    const unsigned long long seed = seeds ? seeds[r] : 0ull;
    const unsigned long long rid = request_ids ? (unsigned long long)request_ids[r] : 0ull;
    const uint32_t posn = positions ? (uint32_t)positions[r] : 0u;
    philox4x32_10(posn, 0u, (uint32_t)rid, (uint32_t)(rid >> 32), (uint32_t)seed, (uint32_t)(seed >> 32), rnd);
    const double u = (double)((((unsigned long long)rnd[0] << 32) | rnd[1]) >> 11) * (1.0 / 9007199254740992.0);

    // ---- the usual cases in one pass over the row: a peaked distribution with a nucleus and/or a
    // small top-k.  The pass gathers, with their ids, the tokens that can matter in shared memory:
    //   * top-k: those no further below the largest logit than the k-th largest (to a step of 0.5,
    //     found from a small histogram in a pass of its own): at least k and at most 4,096 of them;
    //     the k-th largest among them is found there, and the rest of the row is out;
    //   * nucleus alone: those of at least (1 - top_p) / (2 V) of the heaviest token's probability:
    //     all lighter tokens together weigh less than what the nucleus leaves out.
    // Thresholds and the draw then need no further look at the row.  Too many gathered, more than
    // 1,024 kept, or a tie at a threshold: the general path below.
    {
        const int k0 = top_k ? top_k[r] : 0;
        const float tp0 = top_p ? top_p[r] : 1.f;
        const bool use_k = k0 > 0 && k0 < V, use_p = tp0 > 0.f && tp0 < 1.f;
        bool listed = false;
        unsigned long long z0 = 0;
        int C = 0;
        const float inv_t0 = 1.0f / T;
        if (use_k && k0 <= SM_THREADS) {
            // how far below the largest logit the k-th largest lies, from counts in steps of 0.5 (only
            // the few tokens within 32 of the maximum are counted); then those tokens are gathered
            int* hist = reinterpret_cast<int*>(scan);
            if (tid < 64) hist[tid] = 0;
            if (tid == 0) cand_count = 0;
            __syncthreads();
            scan_range(row, lo, hi, [&](int, float v) {
                const float d = (maxv - v) * 2.0f;
                if (d < 64.0f) atomicAdd(&hist[(int)d], 1);
            });
            __syncthreads();
            if (CL) {                                                       // the counts of the whole row, in every rank
                cg::cluster_group cluster = cg::this_cluster();
                cluster.sync();
                int all = 0;
                if (tid < 64)
                    for (int rk = 0; rk < SM_CLUSTER; ++rk) all += cluster.map_shared_rank(hist, rk)[tid];
                cluster.sync();
                if (tid < 64) hist[tid] = all;
                __syncthreads();
            }
            int step_sel = -1, cum = 0;
            for (int b = 0; b < 64; ++b) {
                cum += hist[b];
                if (cum >= k0) { step_sel = b; break; }
            }
            __syncthreads();                                                // hist (in `scan`) is free again
            C = SM_CAND + 1;
            if (step_sel >= 0 && cum <= SM_CAND) {
                scan_range(row, lo, hi, [&](int i, float v) {
                    const float d = (maxv - v) * 2.0f;
                    if (d < 64.0f && (int)d <= step_sel) {
                        const int at = atomicAdd(&cand_count, 1);
                        if (at < SM_CAND) { cand_bits[at] = ordered_key(v); cand_id[at] = i; }
                    }
                });
                __syncthreads();
                if (CL) {
                    collect_candidates(cl, cand_bits, cand_id, &cand_count, nullptr, rank);      // at most `cum`: it fits
                    if (rank != 0) return;
                }
                C = cand_count;
            } else if (CL && rank != 0) {
                return;                                                     // the general path is rank 0's alone
            }
            if (C <= SM_CAND && C >= k0) {
                // the k-th largest key among the gathered: the first warp alone bisects (sums over its lanes need no
                // barrier; a block-wide sum per bit cost more than the passes over the row)
                if (tid < 32) {
                    uint32_t pfx = 0;
                    for (int bit = 31; bit >= 0; --bit) {
                        const uint32_t cand = pfx | (1u << bit);
                        long long c = 0;
                        for (int j = tid; j < C; j += 32) c += cand_bits[j] >= cand ? 1 : 0;
                        if (warp_sum_i64(c) >= k0) pfx = cand;
                    }
                    long long n = 0;
                    for (int j = tid; j < C; j += 32) n += cand_bits[j] >= pfx ? 1 : 0;
                    n = warp_sum_i64(n);
                    if (tid == 0) { s_prefix = pfx; s_count = n; }
                }
                __syncthreads();
                const uint32_t prefix = s_prefix;
                const long long n_ge = s_count;
                if (n_ge == k0) {                                           // no tie at the k-th place
                    for (int j = tid; j < C; j += SM_THREADS) {
                        const float e = cand_bits[j] >= prefix ? expf((key_value(cand_bits[j]) - maxv) * inv_t0) : 0.f;
                        cand_bits[j] = __float_as_uint(e);                  // from here on: probabilities; 0 = not allowed
                        z0 += prob_units(e);
                    }
                    z0 = block_sum_u64(z0, red);
                    listed = true;
                }
            }
        } else if (!use_k && use_p) {
            const float light0 = 0.499f * (1.0f - tp0) / (float)V;
            if (tid == 0) cand_count = 0;
            __syncthreads();
            scan_range(row, lo, hi, [&](int i, float v) {
                const float e = expf((v - maxv) * inv_t0);
                z0 += prob_units(e);
                if (e >= light0 && *(volatile int*)&cand_count <= SM_CAND) {
                    const int at = atomicAdd(&cand_count, 1);
                    if (at < SM_CAND) { cand_bits[at] = __float_as_uint(e); cand_id[at] = i; }
                }
            });
            z0 = block_sum_u64(z0, red);
            if (CL) {
                const int all = collect_candidates(cl, cand_bits, cand_id, &cand_count, &z0, rank);
                if (all > SM_CAND && (hi - lo + SM_THREADS - 1) / SM_THREADS <= SM_RUN_MAX) {
                    // too many for shared memory (a flat distribution): every rank keeps its part of the row in registers
                    nucleus_across_cluster(row, lo, hi, V, maxv, inv_t0, tp0, z0, u, reinterpret_cast<unsigned long long*>(scan), red,
                                           cl_x, cl_it, rank, r, amax, out_ids, out_logprob);
                    return;
                }
                if (rank != 0) return;
            }
            C = cand_count;
            listed = C <= SM_CAND;
        } else if (!use_k && !use_p) {
            // Temperature alone: every token stays drawable, so the draw walks the whole row in id order.  Masses in
            // integer units again: a thread sums a run of consecutive tokens of its rank's part, the runs are added up
            // in order (and the ranks' parts through the cluster), the thread whose run holds the draw walks it.
            draw_by_runs<CL>(lo, hi, u, [&](int i) { return prob_units(expf((row[i] - maxv) * inv_t0)); },
                             reinterpret_cast<unsigned long long*>(scan), cl_x, cl_it, rank, r, amax, out_ids, out_logprob);
            if (CL) cg::this_cluster().sync();                              // nobody leaves while its pairs may still be read
            return;
        } else if (CL && rank != 0) {
            return;                                                         // no shared pass for these options
        }
        if (listed) {
            // thresholds and sums over the gathered, again by the first warp alone
            __syncthreads();
            if (tid < 32) {
                uint32_t pfx = 1;                                           // kept: probability bits >= pfx (0 marks what top-k left out)
                bool tie_w = false;
                if (use_p) {
                    unsigned long long target = (unsigned long long)ceil((double)tp0 * (double)z0);
                    if (target > z0) target = z0;
                    if (target < 1) target = 1;
                    pfx = 0;
                    for (int bit = 30; bit >= 0; --bit) {
                        const uint32_t cand = pfx | (1u << bit);
                        unsigned long long m = 0;
                        for (int j = tid; j < C; j += 32) m += cand_bits[j] >= cand ? prob_units(__uint_as_float(cand_bits[j])) : 0ull;
                        if (warp_sum_u64(m) >= target) pfx = cand;
                    }
                    if (pfx == 0) pfx = 1;
                    unsigned long long m_gt = 0; long long n_eq = 0;
                    for (int j = tid; j < C; j += 32) {
                        if (cand_bits[j] > pfx) m_gt += prob_units(__uint_as_float(cand_bits[j]));
                        else if (cand_bits[j] == pfx) n_eq += 1;
                    }
                    m_gt = warp_sum_u64(m_gt);
                    n_eq = warp_sum_i64(n_eq);
                    const unsigned long long q_thr = prob_units(__uint_as_float(pfx));
                    long long need = 1;
                    if (q_thr > 0 && target > m_gt) need = (long long)((target - m_gt + q_thr - 1) / q_thr);
                    tie_w = need < n_eq;                                    // only some of the tokens at the threshold are kept
                }
                unsigned long long tot = 0; long long kept_n = 0;
                for (int j = tid; j < C; j += 32)
                    if (cand_bits[j] >= pfx) { tot += prob_units(__uint_as_float(cand_bits[j])); kept_n += 1; }
                tot = warp_sum_u64(tot);
                kept_n = warp_sum_i64(kept_n);
                if (tid == 0) { s_prefix = pfx; s_tie = tie_w ? 1 : 0; s_total = tot; s_count = kept_n; }
            }
            __syncthreads();
            const uint32_t prefix = s_prefix;
            const bool tie = s_tie != 0;
            const unsigned long long total = s_total;
            const long long n_kept = s_count;
            if (!tie && n_kept <= SM_THREADS && total > 0) {
                unsigned long long rr = (unsigned long long)(u * (double)total);
                if (rr >= total) rr = total - 1;
                // the kept token j owns the units [before_j, before_j + units_j) in id order; one of them holds rr
                for (int j = tid; j < C; j += SM_THREADS) {
                    if (cand_bits[j] < prefix) continue;
                    const int my_id = cand_id[j];
                    unsigned long long before = 0;
                    for (int i = 0; i < C; ++i)
                        if (cand_bits[i] >= prefix && cand_id[i] < my_id) before += prob_units(__uint_as_float(cand_bits[i]));
                    const unsigned long long mine = prob_units(__uint_as_float(cand_bits[j]));
                    if (rr >= before && rr < before + mine) {
                        out_ids[r] = my_id;
                        if (out_logprob != nullptr) out_logprob[r] = (float)log((double)mine / (double)total);   // within the kept set
                    }
                }
                return;
            }
        }
        __syncthreads();
    }

    // ---- top-k: allowed(i) = key > thr_k || (key == thr_k && i <= cut_k)
    const int k = top_k ? top_k[r] : 0;
    uint32_t thr_k = 0; int cut_k = V - 1;
    if (k > 0 && k < V) {
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            long long c = 0;
            scan_row(row, V, [&](int, float v) { c += ordered_key(v) >= cand ? 1 : 0; });
            c = block_sum_i64(c, red);
            if (c >= k) prefix = cand;
        }
        thr_k = prefix;
        long long gt = 0, eq = 0;
        const uint32_t tk = thr_k;
        scan_row(row, V, [&](int, float v) { const uint32_t key = ordered_key(v); gt += key > tk ? 1 : 0; eq += key == tk ? 1 : 0; });
        gt = block_sum_i64(gt, red);
        eq = block_sum_i64(eq, red);
        if ((long long)k - gt < eq)                               // ties at the threshold: the lower ids
            cut_k = id_cutoff(row, V, (long long)k - gt, [&](int, float v) { return ordered_key(v) == tk; }, run_count, &cut_result);
    }

    // ---- unnormalised probabilities e_i = exp((l_i - max) / T) of the allowed tokens, and their sum
    const float inv_t = 1.0f / T;
    unsigned long long z_units = 0;
    {
        const uint32_t tk = thr_k; const int ck = cut_k;
        scan_row(row, V, [&](int i, float v) {
            const uint32_t key = ordered_key(v);
            const bool allowed = key > tk || (key == tk && i <= ck);
            const float e = allowed ? expf((v - maxv) * inv_t) : 0.f;
            probs[i] = e;
            z_units += prob_units(e);
        });
    }
    z_units = block_sum_u64(z_units, red);          // also makes every thread's probs visible to the block

    // ---- top-p: kept(i) = e_i > 0 && (bits(e_i) > thr_p || (bits(e_i) == thr_p && i <= cut_p)); probabilities
    // are not negative, so their bit patterns order like their values
    const float tp = top_p ? top_p[r] : 1.f;
    uint32_t thr_p = 0; int cut_p = V - 1;
    if (tp > 0.f && tp < 1.f) {
        unsigned long long target = (unsigned long long)ceil((double)tp * (double)z_units);
        if (target > z_units) target = z_units;
        if (target < 1) target = 1;
        // tokens of at most `small` units each cannot weigh more than z - target together, so the
        // nucleus lies among the others: gather those (few, when the distribution is peaked)
        const unsigned long long small = (z_units - target) / (unsigned long long)V;
        if (tid == 0) cand_count = 0;
        __syncthreads();
        // units(e) > small  <=>  e * 2^40 >= small + 1  <=>  e >= the smallest float not below (small + 1) / 2^40
        const float light = __double2float_ru((double)(small + 1) * (1.0 / 1099511627776.0));
        scan_row(probs, V, [&](int, float e) {
            if (e >= light && *(volatile int*)&cand_count <= SM_CAND) {   // once the list has overflowed nobody queues for it any more
                const int at = atomicAdd(&cand_count, 1);
                if (at < SM_CAND) cand_bits[at] = __float_as_uint(e);
            }
        });
        __syncthreads();
        const int C = cand_count;
        const bool in_smem = C <= SM_CAND;
        // mass of the tokens whose probability bits are >= cand (bit patterns compare as integers)
        auto mass_at_least = [&](uint32_t cand) {
            unsigned long long m = 0;
            if (in_smem) {
                for (int j = tid; j < C; j += SM_THREADS) m += cand_bits[j] >= cand ? prob_units(__uint_as_float(cand_bits[j])) : 0ull;
            } else {
                scan_row(probs, V, [&](int, float e) { m += __float_as_uint(e) >= cand ? prob_units(e) : 0ull; });
            }
            return block_sum_u64(m, red);
        };
        uint32_t prefix = 0;
        for (int bit = 30; bit >= 0; --bit) {                   // bit 31 is the sign: never set
            const uint32_t cand = prefix | (1u << bit);
            if (mass_at_least(cand) >= target) prefix = cand;
        }
        thr_p = prefix;
        const uint32_t tpk = thr_p;
        unsigned long long m_gt = 0; long long n_eq = 0;
        if (in_smem) {
            for (int j = tid; j < C; j += SM_THREADS) {
                if (cand_bits[j] > tpk) m_gt += prob_units(__uint_as_float(cand_bits[j]));
                else if (cand_bits[j] == tpk) n_eq += 1;
            }
        } else {
            scan_row(probs, V, [&](int, float e) {
                const uint32_t b = __float_as_uint(e);
                if (b > tpk) m_gt += prob_units(e); else if (b == tpk && e > 0.f) n_eq += 1;
            });
        }
        m_gt = block_sum_u64(m_gt, red);
        n_eq = block_sum_i64(n_eq, red);
        const unsigned long long q_thr = prob_units(__uint_as_float(tpk));
        long long need = 1;
        if (q_thr > 0 && target > m_gt) need = (long long)((target - m_gt + q_thr - 1) / q_thr);
        if (need > n_eq) need = n_eq;
        if (need < 1) need = 1;
        if (need < n_eq)                                           // ties at the threshold: the lower ids
            cut_p = id_cutoff(probs, V, need, [&](int, float e) { return __float_as_uint(e) == tpk && e > 0.f; }, run_count, &cut_result);
    }

    // ---- draw: the kept set in id order, masses in integer units (this CTA alone, over the whole row)
    {
        const uint32_t tp_thr = thr_p; const int tp_cut = cut_p;
        draw_by_runs<false>(0, V, u, [&](int i) {
            const float e = probs[i];
            const uint32_t b = __float_as_uint(e);
            return (e > 0.f && (b > tp_thr || (b == tp_thr && i <= tp_cut))) ? prob_units(e) : 0ull;
        }, reinterpret_cast<unsigned long long*>(scan), cl_x, cl_it, 0, r, amax, out_ids, out_logprob);
    }
}

__global__ void __launch_bounds__(SM_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const float* __restrict__ top_p, const int* __restrict__ top_k,
                   const unsigned long long* __restrict__ seeds, const long long* __restrict__ request_ids,
                   const int* __restrict__ positions, float* __restrict__ probs_scratch,
                   int* __restrict__ out_ids, float* __restrict__ out_logprob) {
    sample_row<false>(logits, V, temperature, top_p, top_k, seeds, request_ids, positions, probs_scratch, out_ids, out_logprob,
                      (int)blockIdx.x, 0);
}

// The same with a cluster of SM_CLUSTER CTAs per row (launched with that cluster dimension).
__global__ void __launch_bounds__(SM_THREADS)
sample_rows_cluster_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                           const float* __restrict__ top_p, const int* __restrict__ top_k,
                           const unsigned long long* __restrict__ seeds, const long long* __restrict__ request_ids,
                           const int* __restrict__ positions, float* __restrict__ probs_scratch,
                           int* __restrict__ out_ids, float* __restrict__ out_logprob) {
    sample_row<true>(logits, V, temperature, top_p, top_k, seeds, request_ids, positions, probs_scratch, out_ids, out_logprob,
                     (int)(blockIdx.x / SM_CLUSTER), (int)cg::this_cluster().block_rank());
}

// Up to how many rows a launch gives every row a cluster: while all clusters run at once (temperature 0.7, top-p 0.95,
// 151,936 logits, one CTA a row -> clusters: 1 row 39 -> 27 us, 8 rows 42 -> 30 us, 12 rows 42 -> 31 us, 16 rows 42 -> 41 us,
// 32 rows 42 -> 56 us).
constexpr int SM_CLUSTER_MAX_ROWS = 12;

static void launch_sample_rows(const float* logits, int R, int V, const float* temperature, const float* top_p, const int* top_k,
                               const unsigned long long* seeds, const long long* request_ids, const int* positions,
                               float* probs_scratch, int* out_ids, float* out_logprob, cudaStream_t stream) {
    static int mode = -1;                              // AIEN_B200_SAMPLE_CLUSTER=0: never, 1: whatever the number of rows
    if (mode < 0) { const char* e = getenv("AIEN_B200_SAMPLE_CLUSTER"); mode = e == nullptr ? 2 : (e[0] == '0' ? 0 : 1); }
    if (mode == 1 || (mode == 2 && R <= SM_CLUSTER_MAX_ROWS)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)R * SM_CLUSTER);
        cfg.blockDim = dim3(SM_THREADS);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = SM_CLUSTER;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, sample_rows_cluster_kernel, logits, V, temperature, top_p, top_k, seeds, request_ids, positions,
                               probs_scratch, out_ids, out_logprob) == cudaSuccess)
            return;
        (void)cudaGetLastError();                      // a device that refuses the cluster: one CTA a row draws the same tokens
    }
    sample_rows_kernel<<<R, SM_THREADS, 0, stream>>>(logits, V, temperature, top_p, top_k, seeds, request_ids, positions,
                                                     probs_scratch, out_ids, out_logprob);
}

__global__ void __launch_bounds__(SM_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ out_ids) {
    __shared__ double red[64];
    float mv;
    const int a = block_argmax(logits + (size_t)blockIdx.x * V, 0, V, &mv, red);
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
    launch_sample_rows(logits, R, V, temperature, top_p, top_k, seeds, request_ids, positions, probs_scratch, out_ids, nullptr, stream);
    return launch_status();
}

// The same, and the log-probability of each chosen token in out_logprob [R]: for a greedy row the
// log softmax of the logits at the maximum, -ln sum exp(l - max) (crates/aien-inference-abi/src/
// tensor.rs:299-318); for a sampled row ln(p / kept mass) with p = softmax(l / T), the probability
// inside the set the draw was made from (src/transformer_backend.rs:171).
AIEN_API int aien_sample_rows_logprob(const float* logits, int R, int V, const float* temperature, const float* top_p,
                                      const int* top_k, const unsigned long long* seeds, const long long* request_ids,
                                      const int* positions, float* probs_scratch, int* out_ids, float* out_logprob,
                                      cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || out_logprob == nullptr) return AIEN_E_SHAPE;
    launch_sample_rows(logits, R, V, temperature, top_p, top_k, seeds, request_ids, positions, probs_scratch, out_ids, out_logprob, stream);
    return launch_status();
}
