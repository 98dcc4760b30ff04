// The merge of the per-chunk partial results of split-key decode attention, shared by the kernels
// that produce them.  Chunk c of a (token, query head) left an unnormalised weighted sum
// part_out[row][c][hd], its maximum and its denominator part_ml[row][c][2]; the merge weighs the
// chunks by exp(max_c - max) and normalises.  The order of the sums is fixed by the chunk indices
// alone, never by which CTA runs the merge or when: the denominators are added in 32 interleaved
// series (chunk index mod 32, each in chunk order) and the series by a fixed tree; the weighted sums
// in AD_MERGE_WAYS interleaved series (chunk index mod AD_MERGE_WAYS, each in chunk order), and the
// series then in order.  The series are what lets a long context be merged with many loads in flight:
// one series per warp, several chunks of each requested before the first is used (a token of 32,768
// keys has 256 chunks of 2 KB per kv head, which one thread after another took three times as long
// to read as the attention itself).
#pragma once
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int AD_MERGE_WAYS = 8;

// floats of shared-memory scratch ad_merge_chunks needs: 1 / denominator per head, a weight per chunk and
// head, and one area that holds the chunk denominators first and the series' sums afterwards
// (every area starts on a 16-byte boundary: the series' sums are written four floats at a time)
__host__ __device__ inline size_t ad_merge_round4(size_t n) { return (n + 3) & ~(size_t)3; }
__host__ __device__ inline size_t ad_merge_scratch_floats(int max_splits, int G, int hd) {
    const size_t a = ad_merge_round4((size_t)max_splits * G), b = (size_t)AD_MERGE_WAYS * hd;
    return ad_merge_round4((size_t)G) + a + (a > b ? a : b);
}

// scratch: ad_merge_scratch_floats(max_splits, G, hd) floats of shared memory.  row0: index of the kv
// head's first query head among part_out's rows; out_row: where that head's output starts.  Every one of
// the `nthreads` threads (a multiple of 32) calls this; `sync` is a barrier over exactly those threads.
// hd % 4 == 0, hd <= 128 * PER (PER: float4 a lane takes per chunk and head, 1 or 2).
template <int NH, int PER, typename Sync>
__device__ __forceinline__ void ad_merge_chunks(float* scratch, const float* __restrict__ part_out, const float* __restrict__ part_ml,
                                                __nv_bfloat16* __restrict__ out_row, size_t row0, int G, int hd, int max_splits,
                                                int s_lo, int nsp, int tid, int nthreads, Sync sync) {
    float* Fi = scratch;                                 // [G]: 1 / total denominator
    float* Fm = Fi + ad_merge_round4((size_t)G);         // [nsp][G]: chunk max, then the chunk's weight
    float* Fl = Fm + ad_merge_round4((size_t)max_splits * G);   // [nsp][G]: chunk denominator; later [AD_MERGE_WAYS][hd]: the series' sums
    float* Ps = Fl;
    // All loads of a phase are independent of one another, so a phase costs one round trip to L2.
    for (int i = tid; i < nsp * G; i += nthreads) {
        const int sp = i / G, h = i - sp * G;
        const size_t row = (row0 + h) * max_splits + s_lo + sp;
        Fm[sp * G + h] = __ldcg(part_ml + row * 2);
        Fl[sp * G + h] = __ldcg(part_ml + row * 2 + 1);
    }
    sync();
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    for (int h = warp; h < G; h += nwarps) {             // a warp per head, a lane per series of chunks
        float M = -INFINITY;
        for (int sp = lane; sp < nsp; sp += 32) M = fmaxf(M, Fm[sp * G + h]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
        for (int sp = lane; sp < nsp; sp += 32) {
            const float ms = Fm[sp * G + h];
            const float f = ms == -INFINITY ? 0.f : expf(ms - M);
            L += Fl[sp * G + h] * f;
            Fm[sp * G + h] = f;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        if (lane == 0) Fi[h] = L > 0.f ? 1.0f / L : 0.f;
    }
    sync();                                              // the denominators are used up: their place takes the series' sums
    const int hd4 = hd >> 2;                             // float4 per chunk and head: lane takes lane (and lane + 32)
    constexpr int U = 8 / PER;                           // chunks of a series requested together
    for (int h = 0; h < G; ++h) {
        const float4* src = reinterpret_cast<const float4*>(part_out + ((row0 + h) * max_splits + s_lo) * hd);
        for (int v = warp; v < AD_MERGE_WAYS; v += nwarps) {
            float4 acc[PER];
#pragma unroll
            for (int jj = 0; jj < PER; ++jj) acc[jj] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp = v; sp < nsp; sp += U * AD_MERGE_WAYS) {
                float4 t[U][PER];
                float f[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int c = sp + u * AD_MERGE_WAYS;
                    f[u] = c < nsp ? Fm[c * G + h] : 0.f;
#pragma unroll
                    for (int jj = 0; jj < PER; ++jj) {
                        const int j = lane + 32 * jj;
                        t[u][jj] = (c < nsp && j < hd4) ? __ldcg(src + (size_t)c * hd4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (sp + u * AD_MERGE_WAYS >= nsp) break;
#pragma unroll
                    for (int jj = 0; jj < PER; ++jj) {
                        acc[jj].x += t[u][jj].x * f[u]; acc[jj].y += t[u][jj].y * f[u];
                        acc[jj].z += t[u][jj].z * f[u]; acc[jj].w += t[u][jj].w * f[u];
                    }
                }
            }
#pragma unroll
            for (int jj = 0; jj < PER; ++jj) {
                const int j = lane + 32 * jj;
                if (j < hd4) reinterpret_cast<float4*>(Ps + (size_t)v * hd)[j] = acc[jj];
            }
        }
        sync();
        for (int d = tid; d < hd; d += nthreads) {
            float o = 0.f;
#pragma unroll
            for (int v = 0; v < AD_MERGE_WAYS; ++v) o += Ps[(size_t)v * hd + d];
            out_row[(size_t)h * hd + d] = __float2bfloat16_rn(o * Fi[h]);
        }
        sync();
    }
}

// The same merge as a kernel of its own, for contexts so long that one CTA per (token, kv head) would spend
// more time reading the chunks than the attention took (256 chunks at 32,768 keys).  One CTA per (token,
// query head, 32 dims of the head): warp v adds series v, a lane one dim, sixteen chunks requested at a
// time.  Every sum is made in the order ad_merge_chunks makes it, so the bits are the same.
// Launched with launch_chain behind the kernel that wrote the partial results.
constexpr int AD_MERGE_KERNEL_THREADS = AD_MERGE_WAYS * 32;
inline size_t ad_merge_kernel_smem(int max_splits) { return ((size_t)2 * max_splits + AD_MERGE_WAYS * 32 + 4) * sizeof(float); }

template <int HD>
__global__ void __launch_bounds__(AD_MERGE_KERNEL_THREADS)
paged_decode_merge_kernel(const float* __restrict__ part_out, const float* __restrict__ part_ml, const int* __restrict__ positions,
                          const int* __restrict__ token_list, __nv_bfloat16* __restrict__ out, long out_stride, int nq, int window,
                          int max_splits, int chunk) {
    extern __shared__ float adm_smem[];
    float* Fm = adm_smem;                                // [nsp]: chunk max, then the chunk's weight
    float* Fl = Fm + max_splits;                         // [nsp]: chunk denominator
    float* Ps = Fl + max_splits;                         // [AD_MERGE_WAYS][32]: the series' sums
    float* Fi = Ps + AD_MERGE_WAYS * 32;                 // 1 / total denominator
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int zt = blockIdx.x / nq, head = blockIdx.x - zt * nq;
    const int t = token_list ? token_list[zt] : zt;
    const int pos = positions[t];
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int s_lo = first / chunk, nsp = pos / chunk - s_lo + 1;
    const size_t row = (size_t)blockIdx.x;               // part rows are (token, query head)
    griddep_launch();
    griddep_wait();
    for (int i = tid; i < nsp; i += AD_MERGE_KERNEL_THREADS) {
        Fm[i] = __ldcg(part_ml + (row * max_splits + s_lo + i) * 2);
        Fl[i] = __ldcg(part_ml + (row * max_splits + s_lo + i) * 2 + 1);
    }
    __syncthreads();
    if (warp == 0) {
        float M = -INFINITY;
        for (int sp = lane; sp < nsp; sp += 32) M = fmaxf(M, Fm[sp]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
        for (int sp = lane; sp < nsp; sp += 32) {
            const float ms = Fm[sp];
            const float f = ms == -INFINITY ? 0.f : expf(ms - M);
            L += Fl[sp] * f;
            Fm[sp] = f;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        if (lane == 0) Fi[0] = L > 0.f ? 1.0f / L : 0.f;
    }
    __syncthreads();
    const int d = blockIdx.y * 32 + lane;
    const float* src = part_out + (row * max_splits + s_lo) * HD + d;
    constexpr int U = 16;
    float acc = 0.f;
    for (int sp = warp; sp < nsp; sp += U * AD_MERGE_WAYS) {
        float tv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = sp + u * AD_MERGE_WAYS;
            tv[u] = c < nsp ? __ldcg(src + (size_t)c * HD) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = sp + u * AD_MERGE_WAYS;
            if (c >= nsp) break;
            acc += tv[u] * Fm[c];
        }
    }
    Ps[warp * 32 + lane] = acc;
    __syncthreads();
    if (tid < 32) {
        float o = 0.f;
#pragma unroll
        for (int v = 0; v < AD_MERGE_WAYS; ++v) o += Ps[v * 32 + tid];
        out[(size_t)t * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(o * Fi[0]);
    }
}

// 0, or the CUDA error of the launch
template <int HD>
inline void launch_decode_merge(const float* part_out, const float* part_ml, const int* positions, const int* token_list,
                                __nv_bfloat16* out, long out_stride, int nq, int window, int max_splits, int chunk, int T,
                                cudaStream_t stream) {
    static_assert(HD % 32 == 0, "a CTA takes 32 dims of a head");
    launch_chain(paged_decode_merge_kernel<HD>, dim3((unsigned)(T * nq), HD / 32), dim3(AD_MERGE_KERNEL_THREADS),
                 ad_merge_kernel_smem(max_splits), stream, part_out, part_ml, positions, token_list, out, out_stride, nq, window,
                 max_splits, chunk);
}

}  // namespace aien
