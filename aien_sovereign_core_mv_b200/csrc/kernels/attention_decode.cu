// Decode attention over the paged bfloat16 cache: one query token per request, keys split by
// absolute position into chunks of 256, one CTA per (chunk, kv head, token), then a merge.
//
// A chunk is the keys [c*256, c*256+256) of the request, so which keys are summed together is
// fixed by their positions and never by the batch or the grid.  Within a CTA eight warps take
// groups of 16 keys in turn.  Scores for a group come from mma.sync.m16n8k16 with the 16 keys as
// rows and the (up to 16) query heads that share the kv head as columns; K is read straight from
// global memory with 16-byte loads (the contraction index is permuted the same way for q and
// K, see gemv.cu).  Softmax is online and float32; the weighted sum over V is plain FMAs with
// each lane owning two adjacent dims per 64, V rows read coalesced.  Partial results
// (unnormalised sum, max, denominator) go to scratch; the merge kernel combines the chunks in
// chunk order.  Formulas: crates/aien-inference-abi/src/backend.rs:311-379 (online softmax over
// pages, scale 1/sqrt(head_dim)).
//
// Needs head_dim % 16 == 0 and <= 256, at most 16 query heads per kv head, bfloat16 q and cache.
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int AD_WARPS = 8;
constexpr int AD_CHUNK = 256;

__device__ __forceinline__ uint4 ad_ldg16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void ad_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// HS = ceil(head_dim / 32) dim steps of the score product, NT = ceil(G / 8) head tiles
template <int HS, int NT>
__global__ void __launch_bounds__(AD_WARPS * 32)
paged_decode_attention_kernel(const __nv_bfloat16* __restrict__ q, long q_stride,
                              const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                              const int* __restrict__ block_table, int max_blocks,
                              const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                              float* __restrict__ part_out, float* __restrict__ part_ml,
                              int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits) {
    constexpr int DCH = (HS + 1) / 2;            // 64-dim chunks of the output
    constexpr int NH = NT * 8;
    extern __shared__ float smem[];
    griddep_launch();
    griddep_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int G = nq / nkv;
    const int pos = positions[t];
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int lo = max(first, split * AD_CHUNK), hi = min(pos, split * AD_CHUNK + AD_CHUNK - 1);
    if (lo > hi) return;
    const int* bt = block_table + (size_t)seq_of_token[t] * max_blocks;

    float* Ps = smem + warp * (16 * NH + NH + 16);       // [16 keys][NH heads], then corr[NH], then slots[16]
    float* Cs = Ps + 16 * NH;
    int* Ss = reinterpret_cast<int*>(Cs + NH);

    // query fragments: head (nt*8 + g), dims ds*32 + c*8 .. +8
    uint4 qf[NT][HS];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int ds = 0; ds < HS; ++ds) {
            const int h = nt * 8 + g, d = ds * 32 + c * 8;
            qf[nt][ds] = (h < G && d < hd) ? ad_ldg16(q + (size_t)t * q_stride + (size_t)(kvh * G + h) * hd + d)
                                           : make_uint4(0u, 0u, 0u, 0u);
        }
    float m_run[NT][2], l_run[NT][2];
    float acc[NH][DCH][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { m_run[nt][0] = m_run[nt][1] = -INFINITY; l_run[nt][0] = l_run[nt][1] = 0.f; }
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int i = 0; i < DCH; ++i) acc[h][i][0] = acc[h][i][1] = 0.f;

    const int chunk_base = split * AD_CHUNK;
    for (int grp = warp; grp * 16 < AD_CHUNK; grp += AD_WARPS) {
        const int base = chunk_base + grp * 16;
        if (base > hi) break;
        if (base + 15 < lo) continue;
        const int kj0 = base + g, kj1 = base + g + 8;
        const bool ok0 = kj0 >= lo && kj0 <= hi, ok1 = kj1 >= lo && kj1 <= hi;
        int slot0 = -1, slot1 = -1;
        if (ok0) { const int pg = bt[kj0 / page_size]; slot0 = pg < 0 ? -1 : pg * page_size + kj0 % page_size; }
        if (ok1) { const int pg = bt[kj1 / page_size]; slot1 = pg < 0 ? -1 : pg * page_size + kj1 % page_size; }
        if (c == 0) { Ss[g] = slot0; Ss[g + 8] = slot1; }
        float S[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
        const __nv_bfloat16* k0p = k_cache + ((size_t)(slot0 < 0 ? 0 : slot0) * nkv + kvh) * hd + c * 8;
        const __nv_bfloat16* k1p = k_cache + ((size_t)(slot1 < 0 ? 0 : slot1) * nkv + kvh) * hd + c * 8;
#pragma unroll
        for (int ds = 0; ds < HS; ++ds) {
            const bool din = ds * 32 + c * 8 < hd;
            const uint4 ka = (slot0 >= 0 && din) ? ad_ldg16(k0p + ds * 32) : make_uint4(0u, 0u, 0u, 0u);
            const uint4 kb = (slot1 >= 0 && din) ? ad_ldg16(k1p + ds * 32) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                ad_mma(S[nt], ka.x, kb.x, ka.y, kb.y, qf[nt][ds].x, qf[nt][ds].y);
                ad_mma(S[nt], ka.z, kb.z, ka.w, kb.w, qf[nt][ds].z, qf[nt][ds].w);
            }
        }
        // S[nt][e]: key g, head nt*8+2c+e;  S[nt][2+e]: key g+8, same head
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float s0 = slot0 >= 0 ? S[nt][e] * scale : -INFINITY;
                const float s1 = slot1 >= 0 ? S[nt][2 + e] * scale : -INFINITY;
                float mx = fmaxf(s0, s1);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float m_new = fmaxf(m_run[nt][e], mx);
                float p0 = 0.f, p1 = 0.f, corr = 1.f;
                if (m_new != -INFINITY) {
                    p0 = slot0 >= 0 ? expf(s0 - m_new) : 0.f;
                    p1 = slot1 >= 0 ? expf(s1 - m_new) : 0.f;
                    corr = m_run[nt][e] == -INFINITY ? 0.f : expf(m_run[nt][e] - m_new);
                }
                float sum = p0 + p1;
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                sum += __shfl_xor_sync(0xffffffffu, sum, 8);
                sum += __shfl_xor_sync(0xffffffffu, sum, 16);
                l_run[nt][e] = l_run[nt][e] * corr + sum;
                m_run[nt][e] = m_new;
                const int h = nt * 8 + 2 * c + e;
                Ps[g * NH + h] = p0;
                Ps[(g + 8) * NH + h] = p1;
                if (g == 0) Cs[h] = corr;
            }
        __syncwarp();
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            if (h < G) {
                const float cr = Cs[h];
#pragma unroll
                for (int i = 0; i < DCH; ++i) { acc[h][i][0] *= cr; acc[h][i][1] *= cr; }
            }
        }
        // all V loads of the group are issued before the first use
        uint32_t vraw[16][DCH];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int sl = Ss[j];
            const __nv_bfloat16* vp = v_cache + ((size_t)(sl < 0 ? 0 : sl) * nkv + kvh) * hd;
#pragma unroll
            for (int i = 0; i < DCH; ++i) {
                const int d = i * 64 + lane * 2;
                vraw[j][i] = (sl >= 0 && d < hd) ? *reinterpret_cast<const uint32_t*>(vp + d) : 0u;
            }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float2 vv[DCH];
#pragma unroll
            for (int i = 0; i < DCH; ++i) vv[i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vraw[j][i]));
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                if (h < G) {
                    const float p = Ps[j * NH + h];
#pragma unroll
                    for (int i = 0; i < DCH; ++i) {
                        acc[h][i][0] = fmaf(p, vv[i].x, acc[h][i][0]);
                        acc[h][i][1] = fmaf(p, vv[i].y, acc[h][i][1]);
                    }
                }
            }
        }
        __syncwarp();
    }

    // ---- combine the warps in warp order
    __syncthreads();
    float* Wm = smem;                                  // [AD_WARPS][NH] max
    float* Wl = Wm + AD_WARPS * NH;                    // [AD_WARPS][NH] denominator
    float* Wa = Wl + AD_WARPS * NH;                    // [AD_WARPS][G][hd] sums
    // every lane with g == 0 holds m/l of heads 2c, 2c+1 of each tile
    if (g == 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                Wm[warp * NH + nt * 8 + 2 * c + e] = m_run[nt][e];
                Wl[warp * NH + nt * 8 + 2 * c + e] = l_run[nt][e];
            }
    }
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        if (h < G) {
#pragma unroll
            for (int i = 0; i < DCH; ++i) {
                const int d = i * 64 + lane * 2;
                if (d < hd) {
                    Wa[((size_t)warp * G + h) * hd + d] = acc[h][i][0];
                    Wa[((size_t)warp * G + h) * hd + d + 1] = acc[h][i][1];
                }
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * hd; idx += AD_WARPS * 32) {
        const int h = idx / hd, d = idx - h * hd;
        float M = -INFINITY;
        for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, Wm[w * NH + h]);
        float o = 0.f, L = 0.f;
        for (int w = 0; w < AD_WARPS; ++w) {
            const float mw = Wm[w * NH + h];
            if (mw == -INFINITY) continue;
            const float f = expf(mw - M);
            o += Wa[((size_t)w * G + h) * hd + d] * f;
            L += Wl[w * NH + h] * f;
        }
        const int head = kvh * G + h;
        const size_t row = ((size_t)t * nq + head) * max_splits + split;
        part_out[row * hd + d] = o;
        if (d == 0) { part_ml[row * 2] = M; part_ml[row * 2 + 1] = L; }
    }
}

// Combines the chunks of one (token, head) in chunk order and writes the normalised output.
__global__ void __launch_bounds__(128)
decode_attention_merge_kernel(const float* __restrict__ part_out, const float* __restrict__ part_ml,
                              const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, long out_stride,
                              int nq, int hd, int window, int max_splits) {
    griddep_launch();
    griddep_wait();
    const int h = blockIdx.x, t = blockIdx.y;
    const int pos = positions[t];
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int s_lo = first / AD_CHUNK, s_hi = pos / AD_CHUNK;
    const size_t row0 = ((size_t)t * nq + h) * max_splits;
    float M = -INFINITY;
    for (int s = s_lo; s <= s_hi; ++s) M = fmaxf(M, part_ml[(row0 + s) * 2]);
    float L = 0.f;
    for (int s = s_lo; s <= s_hi; ++s) {
        const float ms = part_ml[(row0 + s) * 2];
        if (ms != -INFINITY) L += part_ml[(row0 + s) * 2 + 1] * expf(ms - M);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (int s = s_lo; s <= s_hi; ++s) {
            const float ms = part_ml[(row0 + s) * 2];
            if (ms != -INFINITY) o += part_out[(row0 + s) * hd + d] * expf(ms - M);
        }
        out[(size_t)t * out_stride + (size_t)h * hd + d] = __float2bfloat16_rn(o * inv);
    }
}

template <int HS, int NT>
static int launch_decode(const void* q, long q_stride, const void* kc, const void* vc, const int* bt, int max_blocks,
                         const int* seq_of_token, const int* positions, float* part_out, float* part_ml,
                         int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T,
                         cudaStream_t stream) {
    const int G = nq / nkv, NH = NT * 8;
    const size_t loop_bytes = (size_t)AD_WARPS * (16 * NH + NH + 16) * 4;
    const size_t comb_bytes = ((size_t)2 * AD_WARPS * NH + (size_t)AD_WARPS * G * hd) * 4;
    const size_t smem = loop_bytes > comb_bytes ? loop_bytes : comb_bytes;
    auto kern = paged_decode_attention_kernel<HS, NT>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return AIEN_E_STATE;
    }
    dim3 grid(max_splits, nkv, T);
    launch_chain(kern, grid, dim3(AD_WARPS * 32), smem, stream, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc,
                 (const __nv_bfloat16*)vc, bt, max_blocks, seq_of_token, positions,
                 part_out, part_ml, nq, nkv, hd, page_size, window, scale, max_splits);
    return launch_status();
}

}  // namespace aien

using namespace aien;

// Scratch: part_out [T * nq * max_splits * hd] floats, part_ml [T * nq * max_splits * 2] floats.
// max_splits must cover the longest context in the step: ceil((max position + 1) / 256).
AIEN_API int aien_paged_attention_decode(
    const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
    const int* seq_of_token, const int* positions, void* out, long out_stride, float* part_out, float* part_ml,
    int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > 256 || (hd & 15) || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || max_splits <= 0) return AIEN_E_SHAPE;
    const int G = nq / nkv;
    if (G > 16 || T > 65535 || nkv > 65535) return AIEN_E_SHAPE;
    if ((q_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15)) return AIEN_E_ALIGN;
    const int HS = (hd + 31) / 32, NT = (G + 7) / 8;
    int rc = AIEN_E_SHAPE;
#define AD_CASE(hs, nt)                                                                                              \
    if (HS == hs && NT == nt)                                                                                        \
        rc = launch_decode<hs, nt>(q, q_stride, k_cache, v_cache, block_table, max_blocks, seq_of_token, positions,  \
                                   part_out, part_ml, nq, nkv, hd, page_size, window, scale, max_splits, T, stream);
    AD_CASE(1, 1) AD_CASE(2, 1) AD_CASE(3, 1) AD_CASE(4, 1) AD_CASE(5, 1) AD_CASE(6, 1) AD_CASE(7, 1) AD_CASE(8, 1)
    AD_CASE(1, 2) AD_CASE(2, 2) AD_CASE(3, 2) AD_CASE(4, 2) AD_CASE(5, 2) AD_CASE(6, 2) AD_CASE(7, 2) AD_CASE(8, 2)
#undef AD_CASE
    if (rc != 0) return rc;
    dim3 mgrid(nq, T);
    launch_chain(decode_attention_merge_kernel, mgrid, dim3(128), 0, stream, (const float*)part_out, (const float*)part_ml, positions,
                 (__nv_bfloat16*)out, out_stride, nq, hd, window, max_splits);
    return launch_status();
}
