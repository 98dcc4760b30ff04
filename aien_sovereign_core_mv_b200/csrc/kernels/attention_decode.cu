// Decode attention over the paged bfloat16 cache: one query token per request, keys split by
// absolute position into chunks of 128, one CTA per (chunk, kv head, token); the CTA that
// finishes last for a (token, kv head) merges the chunks.
//
// A chunk is the keys [c*128, c*128+128) of the request, so which keys are summed together is
// fixed by their positions and never by the batch or the grid.  A CTA first requests its whole
// chunk of K and of V with cp.async (64 KB in flight per CTA at head size 128, three CTAs per SM),
// then works in three phases.  Scores: each of the eight warps takes 16 keys;
// mma.sync.m16n8k16 with the keys as rows and the (up to 16) query heads that share the kv head as
// columns, fragments from 16-byte reads of the K rows (the contraction index is permuted the same
// way for q and K, see gemv.cu); the scores go to shared memory.  Softmax: one warp per head takes
// maximum, probabilities and denominator over the chunk's keys, float32.  Weighted sum: each warp
// owns 16 output dims and runs V^T . P over all keys of the chunk on the tensor cores (V^T
// fragments by transposing ldmatrix), so nothing is summed across warps.  The CTA's partial result
// (unnormalised sum, max, denominator) goes to scratch, and a ticket counter per (token, kv head)
// tells the last CTA to combine the chunks in chunk order, whichever CTA that is, and to put the
// counter back to zero.
// Formulas: crates/aien-inference-abi/src/backend.rs:311-379 (online softmax over pages, scale
// 1/sqrt(head_dim)).
//
// Needs head_dim % 16 == 0 and <= 256, at most 16 query heads per kv head, bfloat16 q and cache.
#include "common.cuh"
#include "attention_decode_merge.cuh"
#include <math.h>

namespace aien {

constexpr int AD_WARPS = 8;
constexpr int AD_CHUNK = 128;

__device__ __forceinline__ uint4 ad_ldg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }   // q: written by the kernel ahead
__device__ __forceinline__ uint4 ad_lds16(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ void ad_cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ad_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// When `k` is set, the kernel also does the work of the q/k kernel for its token: the per-head
// RMSNorm of q and k, their rotation, and the write of k and v into the token's cache slot (the CTA
// whose chunk holds the token's position does that, and uses the values directly).  The arithmetic
// is that of qk_norm_rope_kv_write_kernel (elementwise.cu), so the cache holds the same bits.
struct FusedQK {
    const __nv_bfloat16* k;          // raw projections of the step's tokens; null: q is ready, cache is written
    long k_stride;
    const __nv_bfloat16* v;
    long v_stride;
    const void* q_norm_w;            // null: no norm
    const void* k_norm_w;
    int wdt;
    float eps;
    const float* cos_t;              // [T, rot/2]; null: no rotation
    const float* sin_t;
    int rot;
    const int* slot_map;             // [T] cache slot of the token
    __nv_bfloat16* k_cache_w;
    __nv_bfloat16* v_cache_w;
};

// One warp: norm (if w) and rotate (if cos_t) the head at src into hb (float32, head_dim values).
__device__ __forceinline__ void ad_norm_rope_head(const __nv_bfloat16* src, float* hb, int hd, const void* w, int wdt, float eps,
                                                  const float* cos_t, const float* sin_t, int rot, int t, int lane) {
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
        const float val = ld_act(src + i);
        hb[i] = val;
        ss += val * val;
    }
    __syncwarp();
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float sc = 1.0f / sqrtf(ss / (float)hd + eps);
        for (int i = lane; i < hd; i += 32) hb[i] = hb[i] * sc * load_dyn(w, wdt, i);
        __syncwarp();
    }
    if (cos_t != nullptr) {
        const int half = rot >> 1;
        for (int i = lane; i < half; i += 32) {
            const float a = hb[i], b = hb[i + half];
            const float cs = cos_t[(size_t)t * half + i], sn = sin_t[(size_t)t * half + i];
            hb[i] = a * cs - b * sn;
            hb[i + half] = a * sn + b * cs;
        }
        __syncwarp();
    }
}

// HS = ceil(head_dim / 32) dim steps of the score product, NT = ceil(G / 8) head tiles
template <int HS, int NT>
__global__ void __launch_bounds__(AD_WARPS * 32)
paged_decode_attention_kernel(const __nv_bfloat16* __restrict__ q, long q_stride,
                              const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                              const int* __restrict__ block_table, int max_blocks,
                              const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                              const int* __restrict__ token_list, float* __restrict__ part_out, float* __restrict__ part_ml, int* __restrict__ counters,
                              __nv_bfloat16* __restrict__ out, long out_stride,
                              int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int misc_bytes,
                              FusedQK fq) {
    constexpr int NH = NT * 8;
    extern __shared__ float smem[];
    __shared__ int s_slot[AD_CHUNK];
    griddep_launch();
    griddep_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    // blockIdx.z counts the tokens this launch serves: all tokens of the step, or those named by
    // token_list (the single-token requests of a mixed step).  Scratch is indexed by blockIdx.z.
    const int split = blockIdx.x, kvh = blockIdx.y, zt = blockIdx.z;
    const int t = token_list ? token_list[zt] : zt;
    const int G = nq / nkv;
    const int pos = positions[t];
    // In a decode-only step token t is request t (seq_of_token may be null): the table row does not
    // hang on another load, so the page lookups go out together with the position load.
    const int* bt = block_table + (size_t)(seq_of_token ? seq_of_token[t] : t) * max_blocks;
    const int chunk_base = split * AD_CHUNK;
    if (tid < AD_CHUNK) {
        // looked up before the position is known: a key beyond the position is masked later, and its
        // page, if the table has one, belongs to this request anyway
        const int key = chunk_base + tid, pi = key / page_size;
        const int pg = pi < max_blocks ? bt[pi] : -1;
        s_slot[tid] = pg < 0 ? -1 : pg * page_size + key % page_size;
    }
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int lo = max(first, chunk_base), hi = min(pos, chunk_base + AD_CHUNK - 1);
    if (lo > hi) return;
    __syncthreads();

    // ---- the whole chunk of K, then of V, is requested at once with cp.async (rows of keys that are
    // masked or absent are zero-filled).  K rows are padded so that the fragment reads below
    // (two rows x four 16-byte pieces per quarter-warp) fall on different banks.
    const int CH = hd / 8;                                   // 16-byte pieces per row
    // Rows of 128-byte multiples are not padded: the pieces of odd rows are stored with bit 2 of
    // their index flipped instead.  Other row sizes are padded to 4 (mod 8) pieces.
    const bool swz = (CH % 8) == 0;
    const int k_stride = swz ? hd * 2 : (CH + ((4 - CH % 8) + 8) % 8) * 16;
    const int v_stride = hd * 2 + 16;                        // an odd number of pieces: ldmatrix rows fall on different banks
    const uint32_t K_u = (uint32_t)__cvta_generic_to_shared(smem) + misc_bytes;
    const uint32_t V_u = K_u + AD_CHUNK * k_stride;
    for (int idx = tid; idx < AD_CHUNK * CH; idx += AD_WARPS * 32) {
        const int r = idx / CH, ch = idx - r * CH;
        const int key = chunk_base + r, sl = s_slot[r];
        if (fq.k != nullptr && key == pos) continue;         // this row is computed here, not read
        const bool valid = key >= lo && key <= hi && sl >= 0;
        const int pc = swz ? (ch ^ ((r & 1) << 2)) : ch;
        ad_cp_async16(K_u + r * k_stride + pc * 16, k_cache + ((size_t)(valid ? sl : 0) * nkv + kvh) * hd + ch * 8, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int idx = tid; idx < AD_CHUNK * CH; idx += AD_WARPS * 32) {
        const int r = idx / CH, ch = idx - r * CH;
        const int key = chunk_base + r, sl = s_slot[r];
        if (fq.k != nullptr && key == pos) continue;
        const bool valid = key >= lo && key <= hi && sl >= 0;
        ad_cp_async16(V_u + r * v_stride + ch * 16, v_cache + ((size_t)(valid ? sl : 0) * nkv + kvh) * hd + ch * 8, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    // shared scratch (floats): scores [AD_CHUNK][NH], then per head max and denominator [2][NH],
    // then the probabilities as bfloat16 [NH][AD_CHUNK]
    float* Sc = smem;
    float* Hm = Sc + AD_CHUNK * NH;
    float* Hl = Hm + NH;
    __nv_bfloat16* Pt = reinterpret_cast<__nv_bfloat16*>(Hl + NH);
    float* Hb = reinterpret_cast<float*>(Pt + NH * AD_CHUNK);          // fused q/k work: [AD_WARPS][256] floats ...
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(Hb + AD_WARPS * 256);   // ... and q as bfloat16 [NH][hd]

    // query fragments: head (nt*8 + g), dims ds*32 + c*8 .. +8
    uint4 qf[NT][HS];
    if (fq.k == nullptr) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int ds = 0; ds < HS; ++ds) {
                const int h = nt * 8 + g, d = ds * 32 + c * 8;
                qf[nt][ds] = (h < G && d < hd) ? ad_ldg16(q + (size_t)t * q_stride + (size_t)(kvh * G + h) * hd + d)
                                               : make_uint4(0u, 0u, 0u, 0u);
            }
    } else {
        // q of this kv head's G query heads, and (in the CTA that owns the token's position) k and v of
        // the token: norm, rotate, round.  One warp per head; the work overlaps the cp.async traffic.
        float* hb = Hb + warp * 256;
        const bool owner = pos >= chunk_base && pos < chunk_base + AD_CHUNK;
        const int n_jobs = G + (owner ? 2 : 0);
        for (int job = warp; job < n_jobs; job += AD_WARPS) {
            if (job < G) {
                ad_norm_rope_head(q + (size_t)t * q_stride + (size_t)(kvh * G + job) * hd, hb, hd, fq.q_norm_w, fq.wdt, fq.eps,
                                  fq.cos_t, fq.sin_t, fq.rot, t, lane);
                for (int i = lane; i < hd; i += 32) Qs[job * hd + i] = __float2bfloat16_rn(hb[i]);
            } else {
                const bool is_k = job == G;
                const int r = pos - chunk_base;
                const long slot = fq.slot_map[t];
                if (is_k) {
                    ad_norm_rope_head(fq.k + (size_t)t * fq.k_stride + (size_t)kvh * hd, hb, hd, fq.k_norm_w, fq.wdt, fq.eps,
                                      fq.cos_t, fq.sin_t, fq.rot, t, lane);
                } else {
                    const __nv_bfloat16* src = fq.v + (size_t)t * fq.v_stride + (size_t)kvh * hd;
                    for (int i = lane; i < hd; i += 32) hb[i] = ld_act(src + i);
                    __syncwarp();
                }
                __nv_bfloat16* cache_row = (is_k ? fq.k_cache_w : fq.v_cache_w) + ((size_t)slot * nkv + kvh) * hd;
                const int swr = (is_k && swz) ? ((r & 1) << 2) : 0;
                for (int i = lane; i < hd; i += 32) {
                    const __nv_bfloat16 val = __float2bfloat16_rn(hb[i]);
                    if (slot >= 0) cache_row[i] = val;
                    const uint32_t dst = is_k ? K_u + r * k_stride + (uint32_t)(((i >> 3) ^ swr) * 16 + (i & 7) * 2)
                                              : V_u + r * v_stride + (uint32_t)i * 2;
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst), "h"(*reinterpret_cast<const unsigned short*>(&val)) : "memory");
                }
            }
            __syncwarp();
        }
        __syncthreads();
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int ds = 0; ds < HS; ++ds) {
                const int h = nt * 8 + g, d = ds * 32 + c * 8;
                qf[nt][ds] = (h < G && d < hd) ? *reinterpret_cast<const uint4*>(Qs + h * hd + d) : make_uint4(0u, 0u, 0u, 0u);
            }
    }

    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();                                         // K of the chunk is in shared memory
    // ---- phase 1: scores of this warp's 16 keys for every head, to shared memory
    {
        const int kj0 = chunk_base + warp * 16 + g, kj1 = kj0 + 8;
        const bool ok0 = kj0 >= lo && kj0 <= hi && s_slot[warp * 16 + g] >= 0;
        const bool ok1 = kj1 >= lo && kj1 <= hi && s_slot[warp * 16 + g + 8] >= 0;
        float S[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
        const uint32_t k0a = K_u + (warp * 16 + g) * k_stride, k1a = k0a + 8 * k_stride;
        const int sw = swz ? ((g & 1) << 2) : 0;                  // rows g and g+8 have the same parity
#pragma unroll
        for (int ds = 0; ds < HS; ++ds) {
            const bool din = ds * 32 + c * 8 < hd;
            const uint32_t piece = (uint32_t)((ds * 4 + c) ^ sw) * 16;
            const uint4 ka = din ? ad_lds16(k0a + piece) : make_uint4(0u, 0u, 0u, 0u);
            const uint4 kb = din ? ad_lds16(k1a + piece) : make_uint4(0u, 0u, 0u, 0u);
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
                const int h = nt * 8 + 2 * c + e;
                Sc[(warp * 16 + g) * NH + h] = ok0 ? S[nt][e] * scale : -INFINITY;
                Sc[(warp * 16 + g + 8) * NH + h] = ok1 ? S[nt][2 + e] * scale : -INFINITY;
            }
    }
    __syncthreads();
    // ---- phase 2: per head, maximum, probabilities and denominator over the chunk (keys in order)
    for (int h = warp; h < NH; h += AD_WARPS) {
        float sv[AD_CHUNK / 32];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < AD_CHUNK / 32; ++i) { sv[i] = Sc[(i * 32 + lane) * NH + h]; mx = fmaxf(mx, sv[i]); }
        mx = warp_max(mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < AD_CHUNK / 32; ++i) {
            const float pv = (mx == -INFINITY || sv[i] == -INFINITY) ? 0.f : expf(sv[i] - mx);
            sum += pv;
            Pt[h * AD_CHUNK + i * 32 + lane] = __float2bfloat16_rn(pv);
        }
        sum = warp_sum(sum);
        if (lane == 0) { Hm[h] = mx; Hl[h] = sum; }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                         // V of the chunk is in shared memory; P is visible
    // ---- phase 3: out^T[dims, heads] = V^T[dims, keys] . P[keys, heads]; a warp owns 16 dims at a time, so
    // no sum over warps is needed.  V^T fragments by transposing ldmatrix reads of the V rows.
    const int s_lo = first / AD_CHUNK, s_hi = pos / AD_CHUNK;
    for (int mt = warp; mt * 16 < hd; mt += AD_WARPS) {
        float oacc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) oacc[nt][0] = oacc[nt][1] = oacc[nt][2] = oacc[nt][3] = 0.f;
        const uint32_t vbase = V_u + ((lane & 7) + ((lane >> 4) << 3)) * v_stride + ((lane >> 3) & 1) * 16 + mt * 32;
#pragma unroll
        for (int ks = 0; ks < AD_CHUNK / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(vbase + ks * 16 * v_stride));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t* prow = reinterpret_cast<const uint32_t*>(Pt + (nt * 8 + g) * AD_CHUNK + ks * 16);
                ad_mma(oacc[nt], a0, a1, a2, a3, prow[c], prow[c + 4]);
            }
        }
        // oacc[nt]: dims 16mt+g (regs 0,1) and 16mt+g+8 (regs 2,3), heads nt*8+2c and +1
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = nt * 8 + 2 * c + e;
                if (h < G) {
                    const size_t row = ((size_t)zt * nq + kvh * G + h) * max_splits + split;
                    part_out[row * hd + mt * 16 + g] = oacc[nt][e];
                    part_out[row * hd + mt * 16 + g + 8] = oacc[nt][2 + e];
                }
            }
    }
    if (tid < G) {
        const size_t row = ((size_t)zt * nq + kvh * G + tid) * max_splits + split;
        part_ml[row * 2] = Hm[tid];
        part_ml[row * 2 + 1] = Hl[tid];
    }

    // ---- the last CTA of this (token, kv head) merges the chunks in chunk order
    __shared__ int is_last;
    __syncthreads();                                         // every thread's partial results are written
    if (threadIdx.x == 0) {
        __threadfence();                                     // ... and ordered before the ticket, device-wide
        const int ticket = atomicAdd(&counters[(size_t)zt * nkv + kvh], 1);
        is_last = ticket == (s_hi - s_lo);
        if (is_last) counters[(size_t)zt * nkv + kvh] = 0;        // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (hd <= 128)
        ad_merge_chunks<NH, 1>(smem, part_out, part_ml, out + (size_t)t * out_stride + (size_t)kvh * G * hd, (size_t)zt * nq + kvh * G,
                               G, hd, max_splits, s_lo, s_hi - s_lo + 1, threadIdx.x, AD_WARPS * 32, [] { __syncthreads(); });
    else
        ad_merge_chunks<NH, 2>(smem, part_out, part_ml, out + (size_t)t * out_stride + (size_t)kvh * G * hd, (size_t)zt * nq + kvh * G,
                               G, hd, max_splits, s_lo, s_hi - s_lo + 1, threadIdx.x, AD_WARPS * 32, [] { __syncthreads(); });
}

template <int HS, int NT>
static int launch_decode(const void* q, long q_stride, const void* kc, const void* vc, const int* bt, int max_blocks,
                         const int* seq_of_token, const int* positions, const int* token_list, float* part_out, float* part_ml, int* counters,
                         void* out, long out_stride,
                         int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T,
                         const FusedQK& fq, cudaStream_t stream) {
    const int NH = NT * 8;
    size_t loop_bytes = ((size_t)AD_CHUNK * NH + 2 * NH) * 4 + (size_t)NH * AD_CHUNK * 2;          // scores, max/denominator, probabilities
    if (fq.k != nullptr) loop_bytes += (size_t)AD_WARPS * 256 * 4 + (size_t)NH * hd * 2 + 16;      // fused q/k scratch, q
    const size_t comb_bytes = 0;
    const size_t merge_bytes = ad_merge_scratch_floats(max_splits, nq / nkv, hd) * 4;
    size_t smem = loop_bytes > comb_bytes ? loop_bytes : comb_bytes;
    if (merge_bytes > smem) smem = merge_bytes;
    const int misc_bytes = (int)((smem + 127) & ~(size_t)127);           // per-warp scratch, combine and merge areas
    const int CH = hd / 8;
    const int k_stride = (CH % 8) == 0 ? hd * 2 : (CH + ((4 - CH % 8) + 8) % 8) * 16;
    const size_t kv_bytes = (size_t)AD_CHUNK * k_stride + (size_t)AD_CHUNK * (hd * 2 + 16);   // K and V of the chunk
    smem = (size_t)misc_bytes + kv_bytes;
    if (smem > 200 * 1024) return AIEN_E_SHAPE;
    auto kern = paged_decode_attention_kernel<HS, NT>;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return AIEN_E_STATE;
        configured = smem;
    }
    dim3 grid(max_splits, nkv, T);
    // A plain launch: measured, this kernel loses when its CTAs become resident early (they wait
    // on the kernel ahead while holding the slots its own tail needs).
    kern<<<grid, AD_WARPS * 32, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc,
                 (const __nv_bfloat16*)vc, bt, max_blocks, seq_of_token, positions, token_list,
                 part_out, part_ml, counters, (__nv_bfloat16*)out, out_stride, nq, nkv, hd, page_size, window, scale, max_splits,
                 misc_bytes, fq);
    return launch_status();
}

}  // namespace aien

using namespace aien;

// T: tokens served (all of the step, or the entries of token_list).
// Scratch: part_out [T * nq * max_splits * hd] floats, part_ml [T * nq * max_splits * 2] floats.
// counters: T * nkv ints that are zero on entry and are left zero.
// max_splits must cover the longest context in the step: ceil((max position + 1) / 128).
static int decode_dispatch(
    const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
    const int* seq_of_token, const int* positions, const int* token_list, void* out, long out_stride, float* part_out,
    float* part_ml, int* counters, int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T,
    const FusedQK& fq, cudaStream_t stream);

AIEN_API int aien_paged_attention_decode(
    const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
    const int* seq_of_token, const int* positions, const int* token_list, void* out, long out_stride, float* part_out,
    float* part_ml, int* counters, int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T, cudaStream_t stream) {
    FusedQK none = {};
    return decode_dispatch(q, q_stride, k_cache, v_cache, block_table, max_blocks, seq_of_token, positions, token_list, out,
                           out_stride, part_out, part_ml, counters, nq, nkv, hd, page_size, window, scale, max_splits, T, none, stream);
}

// The same with the q/k kernel's work folded in: q, k, v are the raw projections of the step's tokens
// (row strides in elements); k and v are written to the token's slot of the caches.
AIEN_API int aien_paged_attention_decode_fused(
    const void* q, long q_stride, const void* k, long k_stride, const void* v, long v_stride,
    const void* q_norm_w, const void* k_norm_w, int w_dt, float eps, const float* cos_t, const float* sin_t, int rot,
    const int* slot_map, void* k_cache, void* v_cache, const int* block_table, int max_blocks,
    const int* positions, void* out, long out_stride, float* part_out, float* part_ml, int* counters,
    int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T, cudaStream_t stream) {
    if (hd > 256 || rot < 0 || rot > hd || (rot & 1) || k == nullptr || v == nullptr || slot_map == nullptr) return AIEN_E_SHAPE;
    FusedQK fq = {(const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, q_norm_w, k_norm_w, w_dt, eps,
                  cos_t, sin_t, rot, slot_map, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache};
    return decode_dispatch(q, q_stride, k_cache, v_cache, block_table, max_blocks, nullptr, positions, nullptr, out, out_stride,
                           part_out, part_ml, counters, nq, nkv, hd, page_size, window, scale, max_splits, T, fq, stream);
}

static int decode_dispatch(
    const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
    const int* seq_of_token, const int* positions, const int* token_list, void* out, long out_stride, float* part_out,
    float* part_ml, int* counters, int nq, int nkv, int hd, int page_size, int window, float scale, int max_splits, int T,
    const FusedQK& fq, cudaStream_t stream) {
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
                                   token_list, part_out, part_ml, counters, out, out_stride, nq, nkv, hd, page_size, window, scale,        \
                                   max_splits, T, fq, stream);
    AD_CASE(1, 1) AD_CASE(2, 1) AD_CASE(3, 1) AD_CASE(4, 1) AD_CASE(5, 1) AD_CASE(6, 1) AD_CASE(7, 1) AD_CASE(8, 1)
    AD_CASE(1, 2) AD_CASE(2, 2) AD_CASE(3, 2) AD_CASE(4, 2) AD_CASE(5, 2) AD_CASE(6, 2) AD_CASE(7, 2) AD_CASE(8, 2)
#undef AD_CASE
    return rc;
}
