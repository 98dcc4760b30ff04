// Paged causal grouped-query attention, one block per (query token, query head), any head size
// up to 256, any number of heads and groups, any page size, optional window.
//
// It serves the true-32-bit engine for every kind of step (whole prompts, portions with an
// offset, single decoded tokens) and is the plain kernel the faster attention kernels are
// checked against.  A token at position p of request s sees the keys at positions
// max(0, p-window+1) .. p of that request, read through the request's block table; keys are
// visited in position order in chunks of 128 with an online softmax, so the result depends
// only on the token's own position and cache contents, never on how the step was cut or
// batched.  Scores, softmax and the weighted sum are float32
// (formulas: crates/aien-inference-abi/src/backend.rs:311-379, scale 1/sqrt(head_dim)).
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int AG_THREADS = 128;

template <typename TQ, typename TKV, typename TO>
__global__ void __launch_bounds__(AG_THREADS)
paged_attention_generic_kernel(const TQ* __restrict__ q, long q_stride,
                               const TKV* __restrict__ k_cache, const TKV* __restrict__ v_cache,
                               const int* __restrict__ block_table, int max_blocks,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               TO* __restrict__ out, long out_stride,
                               int nq, int nkv, int hd, int page_size, int window, float scale) {
    __shared__ float qs[256];
    __shared__ float p[AG_THREADS];
    __shared__ int slots[AG_THREADS];
    __shared__ float red[32];
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seq_of_token[t] * max_blocks;
    const int kvh = h / (nq / nkv);
    const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    for (int d = tid; d < hd; d += AG_THREADS) qs[d] = to_f(q[(size_t)t * q_stride + (size_t)h * hd + d]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;                      // dims tid and tid + 128
    for (int base = start; base <= pos; base += AG_THREADS) {
        const int j = base + tid;
        float score = -INFINITY;
        int slot = -1;
        if (j <= pos) {
            const int page = bt[j / page_size];
            if (page >= 0) {
                slot = page * page_size + (j % page_size);
                const TKV* kp = k_cache + ((size_t)slot * nkv + kvh) * hd;
                float dot = 0.f;
                for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f(kp[d]), dot);
                score = dot * scale;
            }
        }
        slots[tid] = slot;
        const float cmax = block_max(score, red);
        const float m_new = fmaxf(m, cmax);
        if (m_new == -INFINITY) continue;              // nothing visible yet (whole chunk masked)
        const float e = (slot >= 0) ? expf(score - m_new) : 0.f;
        p[tid] = e;
        const float csum = block_sum(e, red);           // also orders the writes to p/slots
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + csum;
        acc0 *= corr;
        acc1 *= corr;
        const int n = (pos - base + 1 < AG_THREADS) ? pos - base + 1 : AG_THREADS;
        for (int jj = 0; jj < n; ++jj) {
            const int sl = slots[jj];
            if (sl < 0) continue;
            const float pj = p[jj];
            const TKV* vp = v_cache + ((size_t)sl * nkv + kvh) * hd;
            if (tid < hd) acc0 = fmaf(pj, to_f(vp[tid]), acc0);
            if (tid + AG_THREADS < hd) acc1 = fmaf(pj, to_f(vp[tid + AG_THREADS]), acc1);
        }
        m = m_new;
        __syncthreads();
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;        // empty context gives zeros (backend.rs:320)
    TO* o = out + (size_t)t * out_stride + (size_t)h * hd;
    if (tid < hd) o[tid] = from_f<TO>(acc0 * inv);
    if (tid + AG_THREADS < hd) o[tid + AG_THREADS] = from_f<TO>(acc1 * inv);
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_paged_attention_generic(
    const void* q, long q_stride, const void* k_cache, const void* v_cache,
    const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
    void* out, long out_stride, int nq, int nkv, int hd, int page_size, int window, float scale,
    int act_dt, int kv_dt, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > 256 || nkv <= 0 || nq % nkv != 0 || page_size <= 0) return AIEN_E_SHAPE;
    if (T > 65535) return AIEN_E_SHAPE;
    dim3 grid(nq, T);
    AIEN_DISPATCH_DTYPE(act_dt, TQ, AIEN_DISPATCH_DTYPE(kv_dt, TKV,
        (paged_attention_generic_kernel<TQ, TKV, TQ><<<grid, AG_THREADS, 0, stream>>>(
            (const TQ*)q, q_stride, (const TKV*)k_cache, (const TKV*)v_cache, block_table, max_blocks,
            seq_of_token, positions, (TQ*)out, out_stride, nq, nkv, hd, page_size, window, scale))));
    return launch_status();
}
