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

}  // namespace aien
