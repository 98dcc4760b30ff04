// Decode-time matrix product, streamed: out[M,N] = a[M,K] . W[N,K]^T for M <= 16, bfloat16.
//
// A persistent kernel, one CTA per SM.  The work is cut into units of 16 rows of W by one range of
// K (the number of ranges depends on (N, K) only); CTA b takes units b, b + grid, b + 2 grid, ...
// One producer lane streams each unit through a ring of shared-memory stages with TMA
// (one 3-D copy of 16 rows x 512 values of W and one of the matching 8 or 16 rows of a per stage,
// laid out as eight 128-byte-swizzled boxes of 64 values, each CTA its own), so up to ~190 KB per SM are in flight without holding a register.  Eight
// consumer warps each take one box of a stage, read the operand fragments from shared memory
// (conflict-free thanks to the swizzle) and issue mma.sync.m16n8k16 with float32 accumulators;
// at the end of a unit the warps are summed in warp order and the result is written as a
// float32 partial product (the consumer adds the ranges in order), as the final value, or as
// silu(gate)*up when W holds gate|up rows interleaved in runs of 8.  The producer does not stop
// at unit boundaries, so the memory stream never drains.
//
// Two optional fusions with the RMSNorm that sits between two products of a decode step
// (crates/aien-inference-abi/src/transformer_backend.rs: x += delta; h = x * rsqrt(mean(x^2) + eps) * w):
//   * epilogue 2, the product that ends a residual branch: the result is added to the float32
//     residual in place, the sum times the next norm's weight is written as bfloat16 (the next
//     product's operand), and every CTA leaves the sum of squares of the residual values it
//     produced, per token, in ssq_out[cta][16];
//   * scaled input, the product that follows: the operand rows are those unnormalised values, so
//     the result row t is multiplied by 1 / sqrt(sum_cta ssq_in[cta][t] / K + eps); the partial
//     sums are added in CTA order.
// Together they do what the norm kernel between the two products did, without the launch.
//
// Rows beyond N or M are zero-filled by TMA.  Needs K % 64 == 0 and 16-byte aligned bases and row
// strides (other sizes take the direct kernel).  Waits are bounded and report through aien_gemv_stream_error().
#include "tma.cuh"

namespace aien {

constexpr int GS_CONSUMERS = 8;                       // consumer warps = boxes per stage
constexpr int GS_BOX_COLS = 64;                       // 128 bytes
constexpr int GS_STAGE_COLS = GS_CONSUMERS * GS_BOX_COLS;   // 512 values of K per stage
constexpr int GS_W_BOX = 16 * 128;                    // bytes
constexpr int GS_THREADS = (GS_CONSUMERS + 1) * 32;

__device__ __forceinline__ void gs_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}

struct GsFuse {
    const float* ssq_in;       // scaled input: [ssq_parts][16] partial sums of squares per token; null: off
    int ssq_parts;
    float eps;
    float* resid;              // epilogue 2: float32 residual [M, ld_res], updated in place
    long ld_res;
    const void* norm_w;        // the next norm's weight [N]
    int w_dt;
    __nv_bfloat16* xw;         // bfloat16(residual * norm_w) [M, ld_xw]
    long ld_xw;
    float* ssq_out;            // [gridDim.x][16]
};

// MT token tiles of 8; EPI 0 store / 1 swiglu / 2 residual; STAGES ring depth
template <int MT, int EPI, typename TC, int STAGES>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemv_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   TC* __restrict__ out, long ldc, size_t part_stride, int M, int N, int K, int splits, int k_per_split, GsFuse fz) {
    constexpr int X_BOX = MT * 8 * 128;                               // bytes of one box of a
    constexpr int STAGE_BYTES = GS_CONSUMERS * (GS_W_BOX + X_BOX);
    extern __shared__ uint8_t gs_smem_raw[];
    __shared__ float red[2][GS_CONSUMERS][MT][4][32];
    __shared__ float ssq_red[16][16];
    const uint32_t base = (smem_u32(gs_smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, GS_CONSUMERS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    griddep_launch();
    __syncthreads();

    const int tiles = (N + 15) / 16;
    const int units = tiles * splits;

    if (warp == GS_CONSUMERS) {
        // ---------------- producer.  One copy per operand and stage: 16 rows x 512 values of W, 8 or
        // 16 rows x 512 values of a (chunks of 64 values beyond K are zero-filled).  The first ring
        // of W is requested before waiting for the kernel ahead of this one: weights do not depend
        // on it; a does, and is requested after the wait.
        if (lane == 0) {
            uint32_t it = 0;
            bool waited = false;
            uint32_t pending_x[STAGES];
            int pending_k[STAGES], n_pending = 0;
            for (int u = blockIdx.x; u < units; u += gridDim.x) {
                const int tile = u / splits, sp = u - tile * splits;
                const int k_begin = sp * k_per_split, k_end = min(K, k_begin + k_per_split);
                for (int k0 = k_begin; k0 < k_end; k0 += GS_STAGE_COLS, ++it) {
                    const int s = it % STAGES;
                    if (it >= (uint32_t)STAGES) {
                        if (!waited) {
                            griddep_wait();
                            for (int i = 0; i < n_pending; ++i)
                                tma_load_3d(pending_x[i] + GS_CONSUMERS * GS_W_BOX, &map_a, full0 + 8 * i, 0, 0, pending_k[i]);
                            waited = true;
                        }
                        mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1, 1);
                    }
                    const uint32_t stage = base + s * STAGE_BYTES;
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_3d(stage, &map_w, full0 + 8 * s, 0, tile * 16, k0 / GS_BOX_COLS);
                    if (waited) {
                        tma_load_3d(stage + GS_CONSUMERS * GS_W_BOX, &map_a, full0 + 8 * s, 0, 0, k0 / GS_BOX_COLS);
                    } else {
                        pending_x[n_pending] = stage;
                        pending_k[n_pending] = k0 / GS_BOX_COLS;
                        ++n_pending;
                    }
                }
            }
            if (!waited) {
                griddep_wait();
                for (int i = 0; i < n_pending; ++i)
                    tma_load_3d(pending_x[i] + GS_CONSUMERS * GS_W_BOX, &map_a, full0 + 8 * i, 0, 0, pending_k[i]);
            }
        }
        return;
    }
    griddep_wait();                                   // the consumers write out, which the kernel ahead may still read

    // ---------------- consumers
    const int g = lane >> 2, c = lane & 3;
    // scaled input: every consumer thread sums a share of the partial sums of squares now (the loads
    // fly while the ring fills); warp 0, which finishes every unit, combines the shares in order at
    // the end of its first unit and keeps the factors of its tokens in registers
    float rs[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) rs[mt][0] = rs[mt][1] = 1.0f;
    if (fz.ssq_in != nullptr) {
        const int t = threadIdx.x & 15, share = threadIdx.x >> 4;          // 16 shares of the parts
        float sq = 0.f;
        for (int p = share; p < fz.ssq_parts; p += 16) sq += __ldcg(fz.ssq_in + (size_t)p * 16 + t);
        ssq_red[share][t] = sq;
    }
    bool have_rs = fz.ssq_in == nullptr;
    float ss[MT][2];                                   // epilogue 2: sums of squares of this CTA's residual values
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) ss[mt][0] = ss[mt][1] = 0.f;
    uint32_t it = 0;
    int parity = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x, parity ^= 1) {
        const int tile = u / splits, sp = u - tile * splits;
        const int k_begin = sp * k_per_split, k_end = min(K, k_begin + k_per_split);
        float xr[MT][4];                                // epilogue 2: the residual values, fetched under the stream
        if (EPI == 2 && warp == 0) {
            const int r0 = tile * 16 + g, r1 = r0 + 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int t0 = mt * 8 + 2 * c;
                xr[mt][0] = (t0 < M && r0 < N) ? fz.resid[(size_t)t0 * fz.ld_res + r0] : 0.f;
                xr[mt][1] = (t0 + 1 < M && r0 < N) ? fz.resid[(size_t)(t0 + 1) * fz.ld_res + r0] : 0.f;
                xr[mt][2] = (t0 < M && r1 < N) ? fz.resid[(size_t)t0 * fz.ld_res + r1] : 0.f;
                xr[mt][3] = (t0 + 1 < M && r1 < N) ? fz.resid[(size_t)(t0 + 1) * fz.ld_res + r1] : 0.f;
            }
        }
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
        for (int k0 = k_begin; k0 < k_end; k0 += GS_STAGE_COLS, ++it) {
            const int s = it % STAGES;
            mbar_wait(full0 + 8 * s, (it / STAGES) & 1, 2);
            const uint32_t wbox = base + s * STAGE_BYTES + warp * GS_W_BOX;
            const uint32_t xbox = base + s * STAGE_BYTES + GS_CONSUMERS * GS_W_BOX + warp * X_BOX;
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {                           // two k32 steps per 64-value box
                const uint32_t chunk = (uint32_t)(((kk * 4 + c) ^ g) & 7) * 16;   // 128-byte swizzle: chunk ^ (row & 7)
                const uint4 wa = lds128(wbox + g * 128 + chunk);
                const uint4 wb = lds128(wbox + (g + 8) * 128 + chunk);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint4 xb = lds128(xbox + (mt * 8 + g) * 128 + chunk);
                    gs_mma(acc[mt], wa.x, wb.x, wa.y, wb.y, xb.x, xb.y);
                    gs_mma(acc[mt], wa.z, wb.z, wa.w, wb.w, xb.z, xb.w);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
        // ---- sum the warps in warp order; warp 0 finishes the unit while the others go on
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[parity][warp][mt][i][lane] = acc[mt][i];
        asm volatile("bar.sync 1, %0;" ::"n"(GS_CONSUMERS * 32) : "memory");
        if (warp == 0) {
            if (!have_rs) {
                float sq = 0.f;
#pragma unroll
                for (int share = 0; share < 16; ++share) sq += ssq_red[share][lane & 15];
                const float r = 1.0f / sqrtf(sq / (float)K + fz.eps);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    rs[mt][0] = __shfl_sync(0xffffffffu, r, mt * 8 + 2 * c);
                    rs[mt][1] = __shfl_sync(0xffffffffu, r, mt * 8 + 2 * c + 1);
                }
                have_rs = true;
            }
            const int r0 = tile * 16 + g, r1 = r0 + 8;
            TC* o = out + (size_t)sp * part_stride;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                float sum[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float t = 0.f;
#pragma unroll
                    for (int w = 0; w < GS_CONSUMERS; ++w) t += red[parity][w][mt][i][lane];
                    sum[i] = t * rs[mt][i & 1];
                }
                const int t0 = mt * 8 + 2 * c;
                if (EPI == 2) {
                    const float w0 = r0 < N ? load_dyn(fz.norm_w, fz.w_dt, r0) : 0.f, w1 = r1 < N ? load_dyn(fz.norm_w, fz.w_dt, r1) : 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int t = t0 + (i & 1), r = (i < 2) ? r0 : r1;
                        if (t < M && r < N) {
                            const float xn = xr[mt][i] + sum[i];
                            fz.resid[(size_t)t * fz.ld_res + r] = xn;
                            fz.xw[(size_t)t * fz.ld_xw + r] = __float2bfloat16_rn(xn * ((i < 2) ? w0 : w1));
                            ss[mt][i & 1] += xn * xn;
                        }
                    }
                } else if (EPI == 0) {
                    if (r0 < N) {
                        if (t0 < M) o[(size_t)t0 * ldc + r0] = from_f<TC>(sum[0]);
                        if (t0 + 1 < M) o[(size_t)(t0 + 1) * ldc + r0] = from_f<TC>(sum[1]);
                    }
                    if (r1 < N) {
                        if (t0 < M) o[(size_t)t0 * ldc + r1] = from_f<TC>(sum[2]);
                        if (t0 + 1 < M) o[(size_t)(t0 + 1) * ldc + r1] = from_f<TC>(sum[3]);
                    }
                } else if (r1 < N) {
                    const int col = tile * 8 + g;
                    const float y0 = sum[0] / (1.0f + expf(-sum[0])) * sum[2];
                    const float y1 = sum[1] / (1.0f + expf(-sum[1])) * sum[3];
                    if (t0 < M) o[(size_t)t0 * ldc + col] = from_f<TC>(y0);
                    if (t0 + 1 < M) o[(size_t)(t0 + 1) * ldc + col] = from_f<TC>(y1);
                }
            }
        }
    }
    if (EPI == 2 && warp == 0) {
        // rows g of the tile are spread over the lanes with equal c: sum them in a fixed order
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = ss[mt][e];
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (g == 0) fz.ssq_out[(size_t)blockIdx.x * 16 + mt * 8 + 2 * c + e] = v;
            }
        if (MT == 1 && lane < 8) fz.ssq_out[(size_t)blockIdx.x * 16 + 8 + lane] = 0.f;
    }
}

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int MT, int EPI, typename TC>
static int launch_stream(const CUtensorMap& mw, const CUtensorMap& ma, void* out, long ldc, size_t part_stride,
                         int M, int N, int K, int splits, const GsFuse& fz, cudaStream_t stream) {
    constexpr int X_BOX = MT * 8 * 128;
    constexpr int STAGE_BYTES = GS_CONSUMERS * (GS_W_BOX + X_BOX);
    constexpr int STAGES = (200 * 1024) / STAGE_BYTES;                // 8 stages of 24 KB, or 6 of 32 KB
    constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 16 * STAGES + 64;
    auto kern = gemv_stream_kernel<MT, EPI, TC, STAGES>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return AIEN_E_STATE;
        configured = true;
    }
    int k_per_split = (K + splits - 1) / splits;
    k_per_split = ((k_per_split + GS_STAGE_COLS - 1) / GS_STAGE_COLS) * GS_STAGE_COLS;
    const int units = ((N + 15) / 16) * splits;
    const int grid = units < sm_count() ? units : sm_count();
    launch_chain(kern, dim3(grid), dim3(GS_THREADS), (size_t)SMEM, stream, mw, ma, (TC*)out, ldc, part_stride, M, N, K, splits, k_per_split, fz);
    return launch_status();
}

}  // namespace aien

using namespace aien;

static int gemv_stream_dispatch(const void* a, long lda, const void* W, long ldw, void* out, int c_dt, long ldc,
                                int M, int N, int K, int epilogue, int splits, size_t part_stride, const GsFuse& fz, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || (K & 63) || splits < 1 || splits > 64) return AIEN_E_SHAPE;
    if (splits > 1 && (epilogue != 0 || c_dt != AIEN_DT_F32)) return AIEN_E_SHAPE;
    if ((lda & 7) || (ldw & 7) || ((uintptr_t)a & 15) || ((uintptr_t)W & 15)) return AIEN_E_ALIGN;
    if (epilogue == 1 && (N & 15)) return AIEN_E_SHAPE;
    if (epilogue == 2 && (splits != 1 || !fz.resid || !fz.norm_w || !fz.xw || !fz.ssq_out || fz.ssq_in)) return AIEN_E_SHAPE;
    if (fz.ssq_in && (splits != 1 || fz.ssq_parts <= 0)) return AIEN_E_SHAPE;
    CUtensorMap mw, ma;
    const uint32_t xrows = M <= 8 ? 8 : 16;
    if (!make_map_chunked(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 16, GS_CONSUMERS) ||
        !make_map_chunked(&ma, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, xrows, GS_CONSUMERS))
        return AIEN_E_STATE;
#define GS_CASE(mt, epi, T) return launch_stream<mt, epi, T>(mw, ma, out, ldc, part_stride, M, N, K, splits, fz, stream)
    if (epilogue == 0) {
        if (c_dt == AIEN_DT_BF16) { if (M <= 8) GS_CASE(1, 0, __nv_bfloat16); else GS_CASE(2, 0, __nv_bfloat16); }
        if (c_dt == AIEN_DT_F32) { if (M <= 8) GS_CASE(1, 0, float); else GS_CASE(2, 0, float); }
        return AIEN_E_DTYPE;
    }
    if (epilogue == 1) {
        if (c_dt == AIEN_DT_BF16) { if (M <= 8) GS_CASE(1, 1, __nv_bfloat16); else GS_CASE(2, 1, __nv_bfloat16); }
        if (c_dt == AIEN_DT_F32) { if (M <= 8) GS_CASE(1, 1, float); else GS_CASE(2, 1, float); }
        return AIEN_E_DTYPE;
    }
    if (epilogue == 2) { if (M <= 8) GS_CASE(1, 2, float); else GS_CASE(2, 2, float); }
#undef GS_CASE
    return AIEN_E_SHAPE;
}

// Same contract as aien_gemv_bf16.  With splits > 1 out is float32 [splits][M][ldc].  A range of K
// is a multiple of 512 values, so `splits` ranges may cover K with fewer ranges in use; the unused
// partial products are written as zeros.
AIEN_API int aien_gemv_stream_bf16(const void* a, long lda, const void* W, long ldw, void* out, int c_dt, long ldc,
                                   int M, int N, int K, int epilogue, int splits, size_t part_stride, cudaStream_t stream) {
    if (epilogue != 0 && epilogue != 1) return AIEN_E_SHAPE;
    GsFuse none = {};
    return gemv_stream_dispatch(a, lda, W, ldw, out, c_dt, ldc, M, N, K, epilogue, splits, part_stride, none, stream);
}

// The CTAs a product over N rows of W is run by: the number of partial sums of squares that
// aien_gemv_stream_residual leaves.
AIEN_API int aien_gemv_stream_grid(int N) {
    const int units = (N + 15) / 16;
    return units < sm_count() ? units : sm_count();
}

// The product that follows a fused norm: the rows of a are unnormalised, and row t of the result is
// multiplied by 1 / sqrt(sum_p ssq[p][t] / K + eps) before it is stored (epilogue 0) or goes through
// silu(gate)*up (epilogue 1).
AIEN_API int aien_gemv_stream_scaled(const void* a, long lda, const void* W, long ldw, void* out, int c_dt, long ldc,
                                     int M, int N, int K, int epilogue, const float* ssq, int ssq_parts, float eps, cudaStream_t stream) {
    if ((epilogue != 0 && epilogue != 1) || ssq == nullptr) return AIEN_E_SHAPE;
    GsFuse fz = {};
    fz.ssq_in = ssq; fz.ssq_parts = ssq_parts; fz.eps = eps;
    return gemv_stream_dispatch(a, lda, W, ldw, out, c_dt, ldc, M, N, K, epilogue, 1, 0, fz, stream);
}

// The product that ends a residual branch: resid[M, ld_res] += a . W^T in place (float32),
// xw[M, ld_xw] = bfloat16(resid * norm_w), ssq_out[aien_gemv_stream_grid(N)][16] = per-CTA sums of
// squares of the new residual values per token.
AIEN_API int aien_gemv_stream_residual(const void* a, long lda, const void* W, long ldw, float* resid, long ld_res,
                                       const void* norm_w, int w_dt, void* xw, long ld_xw, float* ssq_out,
                                       int M, int N, int K, cudaStream_t stream) {
    if (w_dt != AIEN_DT_BF16 && w_dt != AIEN_DT_F32) return AIEN_E_DTYPE;
    GsFuse fz = {};
    fz.resid = resid; fz.ld_res = ld_res; fz.norm_w = norm_w; fz.w_dt = w_dt; fz.xw = (__nv_bfloat16*)xw; fz.ld_xw = ld_xw; fz.ssq_out = ssq_out;
    return gemv_stream_dispatch(a, lda, W, ldw, resid, AIEN_DT_F32, ld_res, M, N, K, 2, 1, 0, fz, stream);
}

AIEN_API int aien_gemv_stream_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_wait_error, &zero, sizeof(int));
    return v;
}

AIEN_DEFINE_WAIT_ERROR_ADDRESS(aien_gemv_stream_error_address)
