// C[M,N] = A[M,K] . W[N,K]^T with float32 accumulation on the CUDA cores.
//
// This is the engine's true-32-bit matrix product (no tensor-core mode of any kind) and the
// plain product every faster kernel is checked against.  Each output element is one chain of
// fused multiply-adds over k = 0..K-1 in order, so a row's result depends on that row and W
// only: not on M, not on where the row sits in the batch.  Any M, N, K, any leading
// dimensions.  W is the checkpoint's own [out, in] row-major layout (the reference's
// matmul_vec convention, crates/aien-inference-abi/src/tensor.rs:22-61).
#include "common.cuh"

namespace aien {

constexpr int GS_BM = 64, GS_BN = 64, GS_BK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(const TA* __restrict__ A, long lda, const TW* __restrict__ W, long ldw,
                   TC* __restrict__ C, long ldc, int M, int N, int K) {
    __shared__ float As[GS_BK][GS_BM + 4];
    __shared__ float Ws[GS_BK][GS_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, c = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? to_f(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_f<TC>(acc[i][j]);
        }
    }
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_gemm_simple(const void* A, int a_dt, long lda, const void* W, int w_dt, long ldw,
                              void* C, int c_dt, long ldc, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return AIEN_E_SHAPE;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    if (grid.y > 65535) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(a_dt, TA, AIEN_DISPATCH_DTYPE(w_dt, TW, AIEN_DISPATCH_DTYPE(c_dt, TC,
        (gemm_simple_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>(
            (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K)))));
    return launch_status();
}
