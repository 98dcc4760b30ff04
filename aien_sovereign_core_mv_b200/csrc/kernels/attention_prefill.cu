// Prefill attention over the paged bfloat16 cache: portions of prompts (any length, any offset
// into their request) beside single tokens, causal, grouped-query, optional window.
//
// One CTA of eight warps handles 128 consecutive query tokens of one request for one query head;
// the host lists these tiles (request, offset into its portion).  Keys are visited in blocks of
// 64 aligned to absolute positions, read through the block table into shared memory with
// cp.async (rows of masked or absent keys are zero-filled) into two buffers, so that the next
// block's K and V arrive under the current block's math.  A warp whose 16 rows lie beyond the
// portion only helps loading.  Scores and the weighted sum run on
// mma.sync.m16n8k16 (bfloat16 in, float32 accumulate) with ldmatrix-fed fragments; softmax is
// online, float32, per query row, with the per-row causal and window limits applied to the
// scores.  Formulas: crates/aien-inference-abi/src/backend.rs:280-306 (row i of a portion sees
// offset + i + 1 keys), scale 1/sqrt(head_dim).
//
// Head sizes 16..128 in steps of 16 (larger ones take the generic kernel).
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int AP_BM = 128, AP_BN = 64, AP_THREADS = 256;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ap_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

template <int HD>
__global__ void __launch_bounds__(AP_THREADS, (HD <= 128 ? 2 : 1))
paged_prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, long q_stride,
                               const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                               const int* __restrict__ block_table, int max_blocks,
                               const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                               const int* __restrict__ tile_seq, const int* __restrict__ tile_q0,
                               __nv_bfloat16* __restrict__ out, long out_stride,
                               int nq, int nkv, int page_size, int window, float scale_log2e) {
    constexpr int STR = HD + 8;                   // row stride in elements: an odd number of 16-byte chunks
    constexpr int KS = HD / 16;                   // k16 steps of the score product
    constexpr int DT = HD / 8;                    // n8 tiles of the output
    constexpr int CH = HD / 8;                    // 16-byte chunks per row
    extern __shared__ __align__(16) uint8_t ap_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(ap_smem);
    __nv_bfloat16* KVs = Qs + AP_BM * STR;            // [2 buffers][K | V][AP_BN][STR]
    const uint32_t Qs_u = (uint32_t)__cvta_generic_to_shared(Qs), KV_u = (uint32_t)__cvta_generic_to_shared(KVs);
    constexpr uint32_t BUF_BYTES = 2 * AP_BN * STR * 2, V_OFF = AP_BN * STR * 2;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int tile = blockIdx.x, h = blockIdx.y;
    const int s = tile_seq[tile], q0 = tile_q0[tile];
    const int qs = q_start[s], q_len = q_start[s + 1] - qs;
    const int rows = min(AP_BM, q_len - q0);
    const int pos0 = ctx_len[s] - q_len + q0;                      // position of the tile's first query
    const int pos_last = pos0 + rows - 1;
    const int first = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int kvh = h / (nq / nkv);
    const int* bt = block_table + (size_t)s * max_blocks;

    for (int idx = tid; idx < AP_BM * CH; idx += AP_THREADS) {
        const int r = idx / CH, ch = idx - r * CH;
        const bool valid = r < rows;
        const __nv_bfloat16* src = q + (size_t)(qs + q0 + (valid ? r : 0)) * q_stride + (size_t)h * HD + ch * 8;
        cp_async16(Qs_u + (uint32_t)(r * STR + ch * 8) * 2, src, valid);
    }
    cp_async_commit();

    auto load_kv = [&](const __nv_bfloat16* cache, uint32_t dst_u, int kb) {
        for (int idx = tid; idx < AP_BN * CH; idx += AP_THREADS) {
            const int r = idx / CH, ch = idx - r * CH;
            const int key = kb * AP_BN + r;
            bool valid = key >= first && key <= pos_last;
            long slot = 0;
            if (valid) {
                const int page = bt[key / page_size];
                valid = page >= 0;
                slot = (long)page * page_size + key % page_size;
            }
            const __nv_bfloat16* src = cache + ((size_t)(valid ? slot : 0) * nkv + kvh) * HD + ch * 8;
            cp_async16(dst_u + (uint32_t)(r * STR + ch * 8) * 2, src, valid);
        }
    };

    const int kb_begin = first / AP_BN, kb_end = pos_last / AP_BN;
    auto load_block = [&](int kb) {                 // K and V of one block: one commit group
        const uint32_t buf = KV_u + (uint32_t)((kb - kb_begin) & 1) * BUF_BYTES;
        load_kv(k_cache, buf, kb);
        load_kv(v_cache, buf + V_OFF, kb);
        cp_async_commit();
    };
    load_block(kb_begin);

    // query fragments of this warp's 16 rows
    cp_async_wait<1>();
    __syncthreads();
    const bool active = warp * 16 < rows;
    // Q stays in shared memory; its fragments are re-read per k-step (one ldmatrix against the
    // four that fetch K), which keeps the kernel at two CTAs per SM.
    const uint32_t q_frag_u = Qs_u + (uint32_t)((warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * STR + (lane >> 4) * 8) * 2;

    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int qpos0 = pos0 + warp * 16 + g, qpos1 = qpos0 + 8;       // positions of this thread's two rows
    const int wlo0 = window > 0 ? qpos0 - window + 1 : 0, wlo1 = window > 0 ? qpos1 - window + 1 : 0;

    for (int kb = kb_begin; kb <= kb_end; ++kb) {
        const bool more = kb < kb_end;
        if (more) load_block(kb + 1);                // into the other buffer: free since the sync that ended block kb-1
        if (more) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();                             // K(kb), V(kb) have landed for every thread
        const uint32_t Ks_u = KV_u + (uint32_t)((kb - kb_begin) & 1) * BUF_BYTES, Vs_u = Ks_u + V_OFF;
        if (active && kb * AP_BN <= pos0 + warp * 16 + 15) {     // the block is not wholly in this warp's future
        float sc[AP_BN / 8][4];
#pragma unroll
        for (int j = 0; j < AP_BN / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            uint32_t q0r, q1r, q2r, q3r;
            ldmatrix_x4(q_frag_u + kk * 32, q0r, q1r, q2r, q3r);
#pragma unroll
            for (int j = 0; j < AP_BN / 8; j += 2) {
                const int mi = lane >> 3;
                const int row = (j + (mi >> 1)) * 8 + (lane & 7), col = kk * 16 + (mi & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(Ks_u + (uint32_t)(row * STR + col) * 2, b0, b1, b2, b3);
                ap_mma(sc[j], q0r, q1r, q2r, q3r, b0, b1);
                ap_mma(sc[j + 1], q0r, q1r, q2r, q3r, b2, b3);
            }
        }

        // ---- online softmax (scores in log2 units)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < AP_BN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kb * AP_BN + j * 8 + 2 * c + e;
                const bool ok0 = key <= qpos0 && key >= wlo0, ok1 = key <= qpos1 && key >= wlo1;
                sc[j][e] = ok0 ? sc[j][e] * scale_log2e : -INFINITY;
                sc[j][2 + e] = ok1 ? sc[j][2 + e] * scale_log2e : -INFINITY;
                mx0 = fmaxf(mx0, sc[j][e]);
                mx1 = fmaxf(mx1, sc[j][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float corr0 = (m_run[0] == -INFINITY) ? 0.f : exp2f(m_run[0] - mn0);
        const float corr1 = (m_run[1] == -INFINITY) ? 0.f : exp2f(m_run[1] - mn1);
        const float base0 = (mn0 == -INFINITY) ? 0.f : mn0, base1 = (mn1 == -INFINITY) ? 0.f : mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < AP_BN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                sc[j][e] = exp2f(sc[j][e] - base0);            // exp2(-inf) = 0 for masked keys
                sc[j][2 + e] = exp2f(sc[j][2 + e] - base1);
                sum0 += sc[j][e];
                sum1 += sc[j][2 + e];
            }
        }
        l_run[0] = l_run[0] * corr0 + sum0;
        l_run[1] = l_run[1] * corr1 + sum1;
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int d = 0; d < DT; ++d) { o[d][0] *= corr0; o[d][1] *= corr0; o[d][2] *= corr1; o[d][3] *= corr1; }

        // ---- O += P . V
#pragma unroll
        for (int ks = 0; ks < AP_BN / 16; ++ks) {
            const uint32_t a0 = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]), a1 = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
            const uint32_t a2 = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]), a3 = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
            for (int d = 0; d < DT; d += 2) {
                const int row = ks * 16 + (lane & 15), col = (d + (lane >> 4)) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(Vs_u + (uint32_t)(row * STR + col) * 2, b0, b1, b2, b3);
                ap_mma(o[d], a0, a1, a2, a3, b0, b1);
                ap_mma(o[d + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        }
        __syncthreads();                             // every warp is done with this block's buffer
    }

    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1); l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1); l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    const int r0 = warp * 16 + g, r1 = r0 + 8;
#pragma unroll
    for (int d = 0; d < DT; ++d) {
        const int col = d * 8 + 2 * c;
        if (r0 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(qs + q0 + r0) * out_stride + (size_t)h * HD + col) = pack_bf16(o[d][0] * inv0, o[d][1] * inv0);
        if (r1 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(qs + q0 + r1) * out_stride + (size_t)h * HD + col) = pack_bf16(o[d][2] * inv1, o[d][3] * inv1);
    }
}

template <int HD>
static int launch_prefill(const void* q, long q_stride, const void* kc, const void* vc, const int* bt, int max_blocks,
                          const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_q0, int num_tiles,
                          void* out, long out_stride, int nq, int nkv, int page_size, int window, float scale,
                          cudaStream_t stream) {
    constexpr int STR = HD + 8;
    const int smem = (AP_BM + 4 * AP_BN) * STR * 2;
    auto kern = paged_prefill_attention_kernel<HD>;
    static bool configured = false;
    if (smem > 48 * 1024 && !configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return AIEN_E_STATE;
        configured = true;
    }
    dim3 grid(num_tiles, nq);
    kern<<<grid, AP_THREADS, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                              bt, max_blocks, q_start, ctx_len, tile_seq, tile_q0, (__nv_bfloat16*)out, out_stride,
                                              nq, nkv, page_size, window, scale * 1.4426950408889634f);
    return launch_status();
}

}  // namespace aien

using namespace aien;

// tile_seq/tile_q0 [num_tiles]: request index in the step and offset of the tile's first query in
// that request's portion (multiples of 128).
AIEN_API int aien_paged_attention_prefill(
    const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
    const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_q0, int num_tiles,
    void* out, long out_stride, int nq, int nkv, int hd, int page_size, int window, float scale, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    if (hd <= 0 || hd > 128 || (hd & 15) || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || nq > 65535) return AIEN_E_SHAPE;
    if ((q_stride & 7) || (out_stride & 1) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) ||
        ((uintptr_t)out & 3))
        return AIEN_E_ALIGN;
#define AP_CASE(HDV)                                                                                                   \
    if (hd == HDV)                                                                                                     \
        return launch_prefill<HDV>(q, q_stride, k_cache, v_cache, block_table, max_blocks, q_start, ctx_len, tile_seq,  \
                                   tile_q0, num_tiles, out, out_stride, nq, nkv, page_size, window, scale, stream);
    AP_CASE(16) AP_CASE(32) AP_CASE(48) AP_CASE(64) AP_CASE(80) AP_CASE(96) AP_CASE(112) AP_CASE(128)
#undef AP_CASE
    return AIEN_E_SHAPE;
}
