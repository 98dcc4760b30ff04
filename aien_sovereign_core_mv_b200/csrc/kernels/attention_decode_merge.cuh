// The merge of the per-chunk partial results of split-key decode attention, shared by the kernels
// that produce them.  Chunk c of a (token, query head) left an unnormalised weighted sum
// part_out[row][c][hd], its maximum and its denominator part_ml[row][c][2]; the merge weighs the
// chunks by exp(max_c - max) in chunk order and normalises.  The order is fixed by the chunk
// index, never by which CTA runs the merge or when.
#pragma once
#include "common.cuh"
#include <math.h>

namespace aien {

// scratch: (2 * max_splits * NH + NH) floats of shared memory.  row0: index of the kv head's first
// query head among part_out's rows; out_row: where that head's output starts.  Every one of the
// `nthreads` threads calls this; `sync` is a barrier over exactly those threads.
template <int NH, typename Sync>
__device__ __forceinline__ void ad_merge_chunks(float* scratch, const float* __restrict__ part_out, const float* __restrict__ part_ml,
                                                __nv_bfloat16* __restrict__ out_row, size_t row0, int G, int hd, int max_splits,
                                                int s_lo, int nsp, int tid, int nthreads, Sync sync) {
    // All loads of a phase are independent of one another, so a phase costs one round trip to L2.
    float* Fm = scratch;                                 // [nsp][NH]: chunk max, then the chunk's weight
    float* Fl = Fm + (size_t)max_splits * NH;            // [nsp][NH]: chunk denominator
    float* Fi = Fl + (size_t)max_splits * NH;            // [NH]: 1 / total denominator
    for (int i = tid; i < nsp * G; i += nthreads) {
        const int sp = i / G, h = i - sp * G;
        const size_t row = (row0 + h) * max_splits + s_lo + sp;
        Fm[sp * NH + h] = __ldcg(part_ml + row * 2);
        Fl[sp * NH + h] = __ldcg(part_ml + row * 2 + 1);
    }
    sync();
    if (tid < G) {
        const int h = tid;
        float M = -INFINITY;
        for (int sp = 0; sp < nsp; ++sp) M = fmaxf(M, Fm[sp * NH + h]);
        float L = 0.f;
        for (int sp = 0; sp < nsp; ++sp) {
            const float ms = Fm[sp * NH + h];
            const float f = ms == -INFINITY ? 0.f : expf(ms - M);
            L += Fl[sp * NH + h] * f;
            Fm[sp * NH + h] = f;
        }
        Fi[h] = L > 0.f ? 1.0f / L : 0.f;
    }
    sync();
    for (int idx = tid; idx < G * hd; idx += nthreads) {
        const int h = idx / hd, d = idx - h * hd;
        const float* src = part_out + ((row0 + h) * max_splits + s_lo) * hd + d;
        float o = 0.f;
        int sp = 0;
        for (; sp + 4 <= nsp; sp += 4) {
            const float v0 = __ldcg(src + (size_t)(sp + 0) * hd), v1 = __ldcg(src + (size_t)(sp + 1) * hd);
            const float v2 = __ldcg(src + (size_t)(sp + 2) * hd), v3 = __ldcg(src + (size_t)(sp + 3) * hd);
            o += v0 * Fm[(sp + 0) * NH + h];
            o += v1 * Fm[(sp + 1) * NH + h];
            o += v2 * Fm[(sp + 2) * NH + h];
            o += v3 * Fm[(sp + 3) * NH + h];
        }
        for (; sp < nsp; ++sp) o += __ldcg(src + (size_t)sp * hd) * Fm[sp * NH + h];
        out_row[(size_t)h * hd + d] = __float2bfloat16_rn(o * Fi[h]);
    }
}

}  // namespace aien
