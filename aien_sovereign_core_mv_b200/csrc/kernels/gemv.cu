// Decode-time matrix product: out[M,N] = a[M,K] . W[N,K]^T for a handful of rows (M <= 16),
// bfloat16 operands, float32 accumulation.  The work is reading W once at memory speed.
//
// One CTA owns 16 rows of W; its warps split K and are summed in warp order at the end, so a
// token's result does not depend on M or on the grid.  Inside a warp the 16 x 32 slab of W and
// the 8 x 32 slab of a are fed to mma.sync.m16n8k16 straight from 16-byte global loads: the
// contraction index may be permuted freely as long as both operands use the same permutation,
// so thread (g, c) loads the 8 consecutive values [c*8, c*8+8) of row g (and g+8) and of token
// g, and those registers already are the fragments of two k16 steps.  No shared-memory staging,
// no transposes.  W streams through with no L1 allocation; a stays cache-resident.
//
// Variants: plain store; `gate|up` rows interleaved in groups of 8 with silu(gate)*up applied
// in the epilogue (crates/aien-inference-abi/src/backend.rs:572-579 for the formula).
//
// Needs K % 8 == 0, 16-byte aligned row starts of a and W; any N, any M in 1..16.
#include "common.cuh"

namespace aien {

constexpr int GV_UNROLL = 2;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
// activations: written by the kernel ahead, so read with a load that stays behind griddep_wait()
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    return __ldcg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: token tiles of 8 (1 or 2).  EPI: 0 = store, 1 = silu(gate)*up over interleaved rows
// (rows [0,8) of each 16-row tile are gate, rows [8,16) the matching up rows; out has N/2 columns).
// blockIdx.y = split of K across CTAs: the CTA writes its partial product to out + y * part_stride
// (float32 [splits][M][ldc]); the consumer adds the parts in order.
template <int MT, int EPI, typename TC, int GV_WARPS>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_mma_kernel(const __nv_bfloat16* __restrict__ a, long lda, const __nv_bfloat16* __restrict__ W, long ldw,
                TC* __restrict__ out, long ldc, size_t part_stride, int M, int N, int K) {
    __shared__ float red[GV_WARPS][MT][4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int steps = (K + 31) >> 5;
    const int units = gridDim.y * GV_WARPS, unit = blockIdx.y * GV_WARPS + warp;
    const int s_begin = (int)((long)steps * unit / units), s_end = (int)((long)steps * (unit + 1) / units);
    out += (size_t)blockIdx.y * part_stride;

    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool v0 = r0 < N, v1 = r1 < N;
    const __nv_bfloat16* w0 = W + (size_t)(v0 ? r0 : 0) * ldw + c * 8;
    const __nv_bfloat16* w1 = W + (size_t)(v1 ? r1 : 0) * ldw + c * 8;
    const __nv_bfloat16* xa[MT];
    bool xv[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int tok = mt * 8 + g;
        xv[mt] = tok < M;
        xa[mt] = a + (size_t)(xv[mt] ? tok : 0) * lda + c * 8;
    }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    // The first slabs of W are requested before waiting for the kernel ahead of this one: weights
    // do not depend on it, the activations do.  Inside the loop the next slabs of W are requested
    // before the current ones are used, so two groups of loads are in flight per warp.
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 wa[GV_UNROLL], wb[GV_UNROLL];
    auto load_w = [&](int s) {
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
            const int k = (s + u) * 32;
            const bool in = (s + u) < s_end && (k + c * 8) < K;      // K % 8 == 0: a chunk is whole or absent
            wa[u] = (in && v0) ? ldg_stream(w0 + k) : zero;
            wb[u] = (in && v1) ? ldg_stream(w1 + k) : zero;
        }
    };
    griddep_launch();
    load_w(s_begin);
    griddep_wait();
    for (int s = s_begin; s < s_end; s += GV_UNROLL) {
        uint4 xb[GV_UNROLL][MT], ca[GV_UNROLL], cb[GV_UNROLL];
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
            const int k = (s + u) * 32;
            const bool in = (s + u) < s_end && (k + c * 8) < K;
            ca[u] = wa[u];
            cb[u] = wb[u];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) xb[u][mt] = (in && xv[mt]) ? ldg_cached(xa[mt] + k) : zero;
        }
        if (s + GV_UNROLL < s_end) load_w(s + GV_UNROLL);
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16_16816(acc[mt], ca[u].x, cb[u].x, ca[u].y, cb[u].y, xb[u][mt].x, xb[u][mt].y);
                mma_bf16_16816(acc[mt], ca[u].z, cb[u].z, ca[u].w, cb[u].w, xb[u][mt].z, xb[u][mt].w);
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][mt][i][lane] = acc[mt][i];
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        float sum[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < GV_WARPS; ++w) t += red[w][mt][i][lane];
            sum[i] = t;
        }
        // sum[0], sum[1]: row g, tokens 2c, 2c+1;  sum[2], sum[3]: row g+8, same tokens
        const int t0 = mt * 8 + 2 * c;
        if (EPI == 0) {
            if (v0) {
                if (t0 < M) out[(size_t)t0 * ldc + r0] = from_f<TC>(sum[0]);
                if (t0 + 1 < M) out[(size_t)(t0 + 1) * ldc + r0] = from_f<TC>(sum[1]);
            }
            if (v1) {
                if (t0 < M) out[(size_t)t0 * ldc + r1] = from_f<TC>(sum[2]);
                if (t0 + 1 < M) out[(size_t)(t0 + 1) * ldc + r1] = from_f<TC>(sum[3]);
            }
        } else {
            const int col = blockIdx.x * 8 + g;                 // output column of this gate/up pair
            if (v1) {
                const float y0 = sum[0] / (1.0f + expf(-sum[0])) * sum[2];
                const float y1 = sum[1] / (1.0f + expf(-sum[1])) * sum[3];
                if (t0 < M) out[(size_t)t0 * ldc + col] = from_f<TC>(y0);
                if (t0 + 1 < M) out[(size_t)(t0 + 1) * ldc + col] = from_f<TC>(y1);
            }
        }
    }
}

template <int MT, int EPI>
static int launch_gemv(const void* a, long lda, const void* W, long ldw, void* out, int c_dt, long ldc,
                       int splits, size_t part_stride, int M, int N, int K, cudaStream_t stream) {
    dim3 grid((N + 15) / 16, splits);
    if (splits > 1) {
        if (c_dt != AIEN_DT_F32) return AIEN_E_DTYPE;
        launch_chain(gemv_mma_kernel<MT, EPI, float, 4>, grid, dim3(4 * 32), 0, stream,
                     (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)W, ldw, (float*)out, ldc, part_stride, M, N, K);
    } else if (c_dt == AIEN_DT_BF16)
        launch_chain(gemv_mma_kernel<MT, EPI, __nv_bfloat16, 8>, grid, dim3(8 * 32), 0, stream,
                     (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)W, ldw, (__nv_bfloat16*)out, ldc, (size_t)0, M, N, K);
    else if (c_dt == AIEN_DT_F32)
        launch_chain(gemv_mma_kernel<MT, EPI, float, 8>, grid, dim3(8 * 32), 0, stream,
                     (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)W, ldw, (float*)out, ldc, (size_t)0, M, N, K);
    else
        return AIEN_E_DTYPE;
    return launch_status();
}

}  // namespace aien

using namespace aien;

// epilogue: 0 plain, 1 silu(gate)*up over rows interleaved in groups of 8 (N counts both).
// splits > 1: K is cut into `splits` ranges, out is float32 [splits][M][ldc] partial products
// (part_stride elements apart) for the consumer to add; only with epilogue 0.
AIEN_API int aien_gemv_bf16(const void* a, long lda, const void* W, long ldw, void* out, int c_dt, long ldc,
                            int M, int N, int K, int epilogue, int splits, size_t part_stride, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || (K & 7) || splits < 1 || splits > 64) return AIEN_E_SHAPE;
    if (splits > 1 && epilogue != 0) return AIEN_E_SHAPE;
    if ((lda & 7) || (ldw & 7) || ((uintptr_t)a & 15) || ((uintptr_t)W & 15)) return AIEN_E_ALIGN;
    if (epilogue == 1 && (N & 15)) return AIEN_E_SHAPE;
    if (epilogue == 0) {
        return M <= 8 ? launch_gemv<1, 0>(a, lda, W, ldw, out, c_dt, ldc, splits, part_stride, M, N, K, stream)
                      : launch_gemv<2, 0>(a, lda, W, ldw, out, c_dt, ldc, splits, part_stride, M, N, K, stream);
    }
    if (epilogue == 1) {
        return M <= 8 ? launch_gemv<1, 1>(a, lda, W, ldw, out, c_dt, ldc, 1, 0, M, N, K, stream)
                      : launch_gemv<2, 1>(a, lda, W, ldw, out, c_dt, ldc, 1, 0, M, N, K, stream);
    }
    return AIEN_E_SHAPE;
}
