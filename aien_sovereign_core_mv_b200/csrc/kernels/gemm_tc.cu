// C[M,N] = A[M,K] . W[N,K]^T on the fifth-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands brought into shared memory by TMA.
//
// Three forms (tc_plan, tc_m256_cols and tc_p_cols choose): one CTA per 128 x 128 tile, described here, for
// products with few tiles and for split-K; a persistent form with 128 x 256 (or 192) tiles and two
// accumulators, and one with tiles of 256 rows, both described further down, for the large products
// of a prefill.  The first form, six warps, three roles:
//   warp 0      producer: one lane issues the TMA loads of the A and W k-blocks (128 rows x 64
//               bfloat16 = one 128-byte swizzled row each) into a 3-stage ring;
//   warp 1      allocates tensor memory, then one lane issues tcgen05.mma (M 128, N 128, K 16,
//               four per k-block) and commits each stage back to the producer;
//   warps 2-5   epilogue: each owns one 32-lane quarter of tensor memory, reads the float32
//               accumulator with tcgen05.ld and stores its rows (bfloat16 or float32), or applies
//               silu(gate)*up first when W holds gate and up rows interleaved in groups of 8.
// Two CTAs fit on an SM (96 KB of stages, 128 tensor-memory columns each), so one tile's epilogue
// runs under the other's main loop.  The grid is M-tiles fastest: the CTAs that share a tile of W
// run together and W is read from HBM once.
//
// Rows of A beyond M, rows of W beyond N and columns beyond K are zero-filled by TMA; stores are
// masked.  Needs K % 8 == 0 and 16-byte aligned bases and row strides (the TMA rules).
// Every wait is bounded: after the limit the kernel records an error code and goes on without
// hanging; the host reads the code with aien_gemm_tc_error().
#include "tma.cuh"
#include "umma.cuh"
#include <cstdlib>
#include <cstring>

namespace aien {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;
// AR rows of A are brought in per k-block (128, or 64 / 32 when M is that small: the MMA still reads
// 128 rows, the rest being whatever follows in shared memory; a row of the result depends on its
// own row of A only, and rows beyond M are never stored).  The shared memory this saves holds more
// stages of W, which is what a product with few rows waits for.
// BN rows of W per tile: 128, or 96 where that spreads a product without split-K more evenly over
// the SMs (tc_tile_cols).  Two CTAs share an SM in every case.
template <int AR, int BN> struct TcT {
    static constexpr int STAGE_A = AR * TC_BK * 2, STAGE_B = BN * TC_BK * 2;
    static constexpr int STAGES = (100 * 1024) / (STAGE_A + STAGE_B);        // BN 128: 3 / 4 / 5 for AR 128 / 64 / 32
    static constexpr int SMEM = STAGES * (STAGE_A + STAGE_B) + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int TMEM_COLS = BN <= 64 ? 64 : 128;
};

// Stores 32 consecutive accumulator columns of one row: r holds columns n0+c0 .. +31 of row `row`.
// EPI 0: as they are; EPI 1: silu(gate)*up over columns interleaved in runs of 8 (out has N/2 columns).
template <int EPI, typename TC>
__device__ __forceinline__ void tc_store_chunk(const uint32_t r[32], TC* __restrict__ out, long ldc, int row, int n0, int c0, int N) {

                if (EPI == 0) {
                    TC* dst = out + (size_t)row * ldc + n0 + c0;
                    const int valid = N - (n0 + c0);
                    if (valid >= 32 && (((uintptr_t)dst & 15) == 0)) {
                        if (sizeof(TC) == 2) {
                            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 o;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                                o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                                o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                                d4[v] = o;
                            }
                        } else {
                            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                            for (int v = 0; v < 8; ++v) d4[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < valid) dst[j] = from_f<TC>(__uint_as_float(r[j]));
                    }
                } else {
                    // columns c0..c0+31 hold two runs of (8 gate, 8 up): 16 outputs
                    const int oc0 = (n0 + c0) / 2;
                    TC* dst = out + (size_t)row * ldc + oc0;
                    const int valid = N / 2 - oc0;
                    float y[16];
#pragma unroll
                    for (int run = 0; run < 2; ++run)
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float g = __uint_as_float(r[run * 16 + j]), u = __uint_as_float(r[run * 16 + 8 + j]);
                            y[run * 8 + j] = __fdividef(g, 1.0f + __expf(-g)) * u;
                        }
                    if (valid >= 16 && sizeof(TC) == 2 && (((uintptr_t)dst & 15) == 0)) {
                        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                        for (int v = 0; v < 2; ++v) {
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(y[8 * v + 0], y[8 * v + 1]), p1 = __floats2bfloat162_rn(y[8 * v + 2], y[8 * v + 3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(y[8 * v + 4], y[8 * v + 5]), p3 = __floats2bfloat162_rn(y[8 * v + 6], y[8 * v + 7]);
                            uint4 o;
                            o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                            o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                            d4[v] = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < valid) dst[j] = from_f<TC>(y[j]);
                    }
                }
            }

// EPI 0: store; EPI 1: silu(gate)*up over columns interleaved in runs of 8 (out has N/2 columns)
template <int EPI, typename TC, int AR, int BN>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               TC* __restrict__ out, long ldc, size_t part_stride, int kb_per_split, int M, int N, int K) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    constexpr int TC_STAGES = TcT<AR, BN>::STAGES, TC_STAGE_A = TcT<AR, BN>::STAGE_A, TC_STAGE_B = TcT<AR, BN>::STAGE_B;
    constexpr int TC_BN = BN;
    const uint32_t sA = base, sB = base + TC_STAGES * TC_STAGE_A;
    const uint32_t bars = sB + TC_STAGES * TC_STAGE_B;     // full[], empty[], tmem_full, then the tmem slot
    const uint32_t full0 = bars, empty0 = bars + 8 * TC_STAGES, tmem_full = bars + 16 * TC_STAGES;
    const uint32_t tmem_slot = tmem_full + 8;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + (tmem_slot - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * TC_BN;
    // blockIdx.z: a range of k-blocks (split-K for small M); the partial product goes to
    // out + z * part_stride and the consumer adds the ranges in order
    const int kb_first = blockIdx.z * kb_per_split;
    const int num_kb = min((K + TC_BK - 1) / TC_BK - kb_first, kb_per_split);
    out += (size_t)blockIdx.z * part_stride;

    griddep_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TcT<AR, BN>::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            // The first ring of W is requested before waiting for the kernel ahead in the stream:
            // weights do not depend on it; A does, and nothing is written before A has arrived.
            const int ahead = min(num_kb, TC_STAGES);
            for (int kb = 0; kb < ahead; ++kb) {
                mbar_expect_tx(full0 + 8 * kb, TC_STAGE_A + TC_STAGE_B);
                tma_load_2d(sB + kb * TC_STAGE_B, &map_w, full0 + 8 * kb, (kb_first + kb) * TC_BK, n0);
            }
            griddep_wait();
            for (int kb = 0; kb < ahead; ++kb)
                tma_load_2d(sA + kb * TC_STAGE_A, &map_a, full0 + 8 * kb, (kb_first + kb) * TC_BK, m0);
            for (int kb = ahead; kb < num_kb; ++kb) {
                const int s = kb % TC_STAGES;
                const uint32_t round = kb / TC_STAGES;
                mbar_wait(empty0 + 8 * s, (round - 1) & 1, 1);
                mbar_expect_tx(full0 + 8 * s, TC_STAGE_A + TC_STAGE_B);
                tma_load_2d(sA + s * TC_STAGE_A, &map_a, full0 + 8 * s, (kb_first + kb) * TC_BK, m0);
                tma_load_2d(sB + s * TC_STAGE_B, &map_w, full0 + 8 * s, (kb_first + kb) * TC_BK, n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, N at bit 17 (>>3), M at bit 24 (>>4)
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % TC_STAGES;
                mbar_wait(full0 + 8 * s, (kb / TC_STAGES) & 1, 2);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = make_desc_sw128(sA + s * TC_STAGE_A), db = make_desc_sw128(sB + s * TC_STAGE_B);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)     // 16 bfloat16 = 32 bytes = 2 descriptor units along K
                    umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);             // the stage may be refilled once these MMAs have read it
            }
            umma_commit(tmem_full);
        }
    } else {
        const int quarter = warp & 3;                    // tensor-memory lanes 32*quarter .. +31
        mbar_wait(tmem_full, 0, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < TC_BN && m0 + quarter * 32 < M; c0 += 32) {      // a quarter beyond M has nothing to store
            uint32_t r[32];
            tmem_ld32(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < M) tc_store_chunk<EPI, TC>(r, out, ldc, row, n0, c0, N);

        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)TcT<AR, BN>::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The persistent form, for products whose tile grid fills the GPU: one CTA per SM walks over
// tiles of 128 x BN (BN 256), M-tiles fastest.  Tensor memory holds two
// accumulators, so the four epilogue warps drain tile i while the MMA lane already works on
// tile i+1, and the producer runs ahead across tile borders.  With BN 256 one k-block reads
// 16 KB of A and 32 KB of W from shared memory for 512 tensor-core cycles, which leaves the
// shared-memory bandwidth headroom that 128 x 128 tiles (32 KB for 256 cycles) do not have.
// With `splits` > 1 (float32 output only) every tile is made `splits` times, each over one range of
// k-blocks, into out + range * part_stride: the caller's consumer adds the ranges in order.  A
// narrow product with long K (40 tiles of 128 x 256) fills the GPU that way; units are ordered
// range-major, so the CTAs that run together share the tiles of A and W they load through L2.
// (Dealing the k-blocks of the last wave out in equal runs, the tiles cut between CTAs put together
// in the kernel through scratch, was measured and not kept: CTAs that are out of step in K re-read
// W from HBM, and the addition at the end cost more than the wave it saved.)
template <int BN> struct TcP {
    static constexpr int STAGE_A = TC_BM * TC_BK * 2, STAGE_B = BN * TC_BK * 2;
    static constexpr int STAGES = (192 * 1024) / (STAGE_A + STAGE_B);          // 4 of 48 KB
    static constexpr int SMEM = STAGES * (STAGE_A + STAGE_B) + 1024 + 256;
    static constexpr int TMEM_COLS = 2 * BN <= 256 ? 256 : 512;                // two accumulators of BN columns; a power of two
};

template <int BN, int EPI, typename TC>
__global__ void __launch_bounds__(192, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                          TC* __restrict__ out, long ldc, int M, int N, int K, int splits, int kb_per_split, size_t part_stride) {
    using P = TcP<BN>;
    constexpr int STAGES = P::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = base, sB = base + STAGES * P::STAGE_A;
    const uint32_t bars = sB + STAGES * P::STAGE_B;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, tfull0 = bars + 16 * STAGES, tempty0 = tfull0 + 16;
    const uint32_t tmem_slot = tempty0 + 16;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + (tmem_slot - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    const int total = tiles * splits;                   // units: (range of K, tile), tiles fastest
    const int all_kb = (K + TC_BK - 1) / TC_BK;
    // k-blocks [kb_lo(u), kb_hi(u)) of unit u
    auto kb_lo = [&](int u) { return (u / tiles) * kb_per_split; };
    auto kb_hi = [&](int u) { return min(all_kb, (u / tiles + 1) * kb_per_split); };

    griddep_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)P::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            // the first ring of W (of this CTA's first tile) goes out before the wait for the kernel
            // ahead in the stream: A is its result, W is not
            const int u0 = blockIdx.x;
            const uint32_t ahead = u0 < total ? (uint32_t)min(kb_hi(u0) - kb_lo(u0), STAGES) : 0u;
            for (uint32_t i = 0; i < ahead; ++i) {
                mbar_expect_tx(full0 + 8 * i, P::STAGE_A + P::STAGE_B);
                tma_load_2d(sB + i * P::STAGE_B, &map_w, full0 + 8 * i, (kb_lo(u0) + (int)i) * TC_BK, ((u0 % tiles) / m_tiles) * BN);
            }
            griddep_wait();
            uint32_t it = 0;
            for (int u = blockIdx.x; u < total; u += gridDim.x) {
                const int tile = u % tiles;
                const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
                for (int kb = kb_lo(u), kbe = kb_hi(u); kb < kbe; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it < ahead) {                                  // W is on its way already
                        tma_load_2d(sA + s * P::STAGE_A, &map_a, full0 + 8 * s, kb * TC_BK, m0);
                        continue;
                    }
                    if (it >= (uint32_t)STAGES) mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1, 1);
                    mbar_expect_tx(full0 + 8 * s, P::STAGE_A + P::STAGE_B);
                    tma_load_2d(sA + s * P::STAGE_A, &map_a, full0 + 8 * s, kb * TC_BK, m0);
                    tma_load_2d(sB + s * P::STAGE_B, &map_w, full0 + 8 * s, kb * TC_BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(TC_BM, BN, false);
            uint32_t it = 0;
            int i = 0;
            for (int u = blockIdx.x; u < total; u += gridDim.x, ++i) {
                const int acc = i & 1;
                if (i >= 2) mbar_wait(tempty0 + 8 * acc, ((i >> 1) - 1) & 1, 4);      // the epilogue has drained this accumulator
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int kb_first = kb_lo(u);
                for (int kb = kb_first, kbe = kb_hi(u); kb < kbe; ++kb, ++it) {
                    const int s = it % STAGES;
                    mbar_wait(full0 + 8 * s, (it / STAGES) & 1, 2);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = make_desc_sw128(sA + s * P::STAGE_A), db = make_desc_sw128(sB + s * P::STAGE_B);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16(tmem_acc + acc * (P::TMEM_COLS / 2), da + 2 * k, db + 2 * k, idesc, (kb > kb_first || k > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);
                }
                umma_commit(tfull0 + 8 * acc);
            }
        }
    } else {
        const int quarter = warp & 3;
        int i = 0;
        for (int u = blockIdx.x; u < total; u += gridDim.x, ++i) {
            const int acc = i & 1;
            const int tile = u % tiles;
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
            TC* out_u = out + (size_t)(u / tiles) * part_stride;
            mbar_wait(tfull0 + 8 * acc, (i >> 1) & 1, 3);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * (P::TMEM_COLS / 2) + c0), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < M && n0 + c0 < N) tc_store_chunk<EPI, TC>(r, out_u, ldc, row, n0, c0, N);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)P::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The persistent form with tiles of 256 x 256: two accumulators of 128 rows side by side in tensor
// memory (all 512 columns), eight products per k-block (the two row halves of A against the same 256
// rows of W).  What bounds the 128 x 256 tile is shared memory, not the tensor core: per k-block TMA
// writes 48 KB and the four products read 48 KB, 768 cycles at 128 bytes a cycle for 512 cycles of
// products (measured: 756).  A 256 x 256 tile writes 64 KB and reads 96 KB for 1,024 cycles of
// products.  The price: no second pair of accumulators, so a tile's epilogue (eight warps) does not
// run under the next tile's main loop (the producer does fill the ring meanwhile), and half as many
// tiles to deal out; tc_plan chooses by the number of waves either way.  No ranges of K.
template <int BNV> struct TcM {
    static constexpr int BM = 256, BN = BNV;                                       // BN 256, or 240 / 224 where that makes fewer waves
    static constexpr int STAGE_A = BM * TC_BK * 2, STAGE_B = 256 * TC_BK * 2;      // 32 KB each (a narrower W tile leaves the rest unused)
    static constexpr int STAGES = 3;
    static constexpr int SMEM = STAGES * (STAGE_A + STAGE_B) + 1024 + 256;
    static constexpr int THREADS = 320;                                            // producer, MMA, eight epilogue warps
};

template <int BNV, int EPI, typename TC>
__global__ void __launch_bounds__(TcM<BNV>::THREADS, 1)
gemm_tc_persistent_m256_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                               TC* __restrict__ out, long ldc, int M, int N, int K) {
    using P = TcM<BNV>;
    constexpr int W_BYTES = P::BN * TC_BK * 2;           // what one copy of W brings
    constexpr int STAGES = P::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = base, sB = base + STAGES * P::STAGE_A;
    const uint32_t bars = sB + STAGES * P::STAGE_B;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, tfull = bars + 16 * STAGES, tempty = tfull + 8;
    const uint32_t tmem_slot = tempty + 8;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + (tmem_slot - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + P::BM - 1) / P::BM, n_tiles = (N + P::BN - 1) / P::BN;
    const int tiles = m_tiles * n_tiles;                 // M-tiles fastest: the CTAs that run together share W
    const int num_kb = (K + TC_BK - 1) / TC_BK;

    griddep_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tfull, 1);
        mbar_init(tempty, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            // the first ring of W goes out before the wait for the kernel ahead in the stream: A is its result, W is not
            const int t0 = blockIdx.x;
            const uint32_t ahead = t0 < tiles ? (uint32_t)min(num_kb, STAGES) : 0u;
            for (uint32_t i = 0; i < ahead; ++i) {
                mbar_expect_tx(full0 + 8 * i, P::STAGE_A + W_BYTES);
                tma_load_2d(sB + i * P::STAGE_B, &map_w, full0 + 8 * i, (int)i * TC_BK, (t0 / m_tiles) * P::BN);
            }
            griddep_wait();
            uint32_t it = 0;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
                const int m0 = (t % m_tiles) * P::BM, n0 = (t / m_tiles) * P::BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it < ahead) {                                  // W is on its way already
                        tma_load_2d(sA + s * P::STAGE_A, &map_a, full0 + 8 * s, kb * TC_BK, m0);
                        continue;
                    }
                    if (it >= (uint32_t)STAGES) mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1, 1);
                    mbar_expect_tx(full0 + 8 * s, P::STAGE_A + W_BYTES);
                    tma_load_2d(sA + s * P::STAGE_A, &map_a, full0 + 8 * s, kb * TC_BK, m0);
                    tma_load_2d(sB + s * P::STAGE_B, &map_w, full0 + 8 * s, kb * TC_BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        // the whole warp walks the schedule; one lane issues
        const bool issuer = lane == 0;
        const uint32_t idesc = umma_idesc_bf16(TC_BM, P::BN, false);
        const uint64_t da0 = make_desc_sw128(sA), db0 = make_desc_sw128(sB);
        uint32_t it = 0;
        int i = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++i) {
            if (i >= 1) {                                              // the epilogue has drained the accumulators
                mbar_wait(tempty, (i - 1) & 1, 4);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                mbar_wait(full0 + 8 * s, (it / STAGES) & 1, 2);        // what TMA wrote is visible once the barrier has completed
                const uint64_t da = da0 + (uint64_t)((s * P::STAGE_A) >> 4), db = db0 + (uint64_t)((s * P::STAGE_B) >> 4);
                if (issuer) {
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
                        umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, accum);                                        // rows 0..127
                        umma_bf16(tmem_acc + P::BN, da + (uint64_t)((TC_BM * 128) >> 4) + 2 * k, db + 2 * k, idesc, accum);   // rows 128..255
                    }
                    umma_commit(empty0 + 8 * s);
                }
            }
            if (issuer) umma_commit(tfull);
        }
    } else {
        const int e = warp - 2, half = e >> 2, quarter = warp & 3;     // a warp reads the lanes 32 (warp % 4) .. of tensor memory
        int i = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++i) {
            const int m0 = (t % m_tiles) * P::BM + half * TC_BM, n0 = (t / m_tiles) * P::BN;
            mbar_wait(tfull, i & 1, 3);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const int n_end = min(N, n0 + P::BN);                      // a tile of 240 or 224 columns ends inside its last chunk of 32
#pragma unroll 1
            for (int c0 = 0; c0 < P::BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * P::BN + c0), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < M && n0 + c0 < n_end) tc_store_chunk<EPI, TC>(r, out, ldc, row, n0, c0, n_end);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512u) : "memory");
    }
}

static int tc_num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int EPI, typename TC>
static int launch_tc_persistent(const void* A, long lda, const void* W, long ldw, void* out, long ldc, int M, int N, int K,
                                int splits, size_t part_stride, cudaStream_t stream) {
    CUtensorMap ma, mw;
    if (!make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BK, TC_BM) || !make_map(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, TC_BK, BN))
        return AIEN_E_STATE;
    auto kern = gemm_tc_persistent_kernel<BN, EPI, TC>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcP<BN>::SMEM) != cudaSuccess) return AIEN_E_STATE;
        configured = true;
    }
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    const int ranges = (total_kb + kb_per_split - 1) / kb_per_split;          // what aien_gemm_tc_ranges says
    const long total = (long)((M + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN) * ranges;
    const unsigned grid = (unsigned)(total < tc_num_sms() ? total : tc_num_sms());
    launch_chain(kern, dim3(grid), dim3(192), (size_t)TcP<BN>::SMEM, stream, ma, mw, (TC*)out, ldc, M, N, K, ranges, kb_per_split, part_stride);
    return launch_status();
}

template <int BNV, int EPI, typename TC>
static int launch_tc_persistent_m256_bn(const void* A, long lda, const void* W, long ldw, void* out, long ldc, int M, int N, int K,
                                        cudaStream_t stream) {
    using P = TcM<BNV>;
    CUtensorMap ma, mw;
    if (!make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BK, P::BM) || !make_map(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, TC_BK, P::BN))
        return AIEN_E_STATE;
    auto kern = gemm_tc_persistent_m256_kernel<BNV, EPI, TC>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P::SMEM) != cudaSuccess) return AIEN_E_STATE;
        configured = true;
    }
    const long total = (long)((M + P::BM - 1) / P::BM) * ((N + P::BN - 1) / P::BN);
    const unsigned grid = (unsigned)(total < tc_num_sms() ? total : tc_num_sms());
    launch_chain(kern, dim3(grid), dim3(P::THREADS), (size_t)P::SMEM, stream, ma, mw, (TC*)out, ldc, M, N, K);
    return launch_status();
}

template <int EPI, typename TC>
static int launch_tc_persistent_m256(int bn, const void* A, long lda, const void* W, long ldw, void* out, long ldc, int M, int N, int K,
                                     cudaStream_t stream) {
    if (sizeof(TC) == 2) {                       // the narrower tiles for bfloat16 results only (fewer kernels to compile)
        if (bn == 240) return launch_tc_persistent_m256_bn<240, EPI, __nv_bfloat16>(A, lda, W, ldw, out, ldc, M, N, K, stream);
        if (bn == 224) return launch_tc_persistent_m256_bn<224, EPI, __nv_bfloat16>(A, lda, W, ldw, out, ldc, M, N, K, stream);
    }
    return launch_tc_persistent_m256_bn<256, EPI, TC>(A, lda, W, ldw, out, ldc, M, N, K, stream);
}

// Which kernel a product takes: 0 the one-tile-per-CTA kernel, 256 the persistent kernel with
// 128 x 256 tiles.  The persistent one once its units (tiles x ranges of K) give every SM one, and
// for any product of more than 64 rows of A by at least 256 of W with three fifths of that: its
// 128 x 256 tile runs at more than twice the rate of the 128 x 128 one, which makes up for idle
// SMs (512 x 6,144 x 2,560: 96 units, 19 us against 22).  (Persistent with 128 x 128 tiles was
// measured 25-35 % slower than either: one CTA per SM at the shared-memory bandwidth limit.)
// AIEN_B200_GEMM_TC=tile | p256 pins the choice.
static int tc_plan(int M, int N, int ranges) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("AIEN_B200_GEMM_TC");
        forced = e == nullptr ? 1 : (!strcmp(e, "tile") ? 0 : ((!strcmp(e, "p256") || !strcmp(e, "m256") || !strcmp(e, "p192")) ? 256 : 1));
    }
    if (forced != 1) return forced;
    const long units = (long)((M + TC_BM - 1) / TC_BM) * ((N + 255) / 256) * ranges;
    if (units >= tc_num_sms()) return 256;
    return (M > 64 && N >= 256 && 5 * units >= 3 * tc_num_sms()) ? 256 : 0;
}

// Whether a product that runs on the persistent kernel takes tiles of 256 rows instead of 128 x 256, and how
// wide (256, 240 or 224 columns; 0: no): by the time either way, in cycles: waves of tiles x (k-blocks x
// the cycles shared memory needs for one + what of a tile's epilogue stays visible).  Per k-block the
// 128 x 256 tile moves 96 KB through shared memory, 768 cycles at 128 bytes a cycle (756 measured); the
// 256 x BN tile (64 + 3 BN / 8) KB, 5 % more measured.  AIEN_B200_GEMM_TC=m256 | p256 pins it (m256: 256 wide).
static int tc_m256_cols(int M, int N, int K, int ranges) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("AIEN_B200_GEMM_TC");
        forced = e == nullptr ? 0 : (!strcmp(e, "m256") ? 1 : ((!strcmp(e, "p256") || !strcmp(e, "p192")) ? 2 : 0));
    }
    if (ranges != 1 || forced == 2) return 0;
    if (forced == 1) return 256;
    if (M <= TC_BM) return 0;
    const long sms = tc_num_sms(), kb = (K + TC_BK - 1) / TC_BK;
    const long t256 = (long)((M + 127) / 128) * ((N + 255) / 256);
    long best = ((t256 + sms - 1) / sms) * (kb * 768 + 700) * 97 / 100;
    int cols = 0;
    for (int bn = 256; bn >= 224; bn -= 16) {
        const long t = (long)((M + 255) / 256) * ((N + bn - 1) / bn), w = (t + sms - 1) / sms;
        // narrower tiles pay where they shorten several waves; in a single wave more, smaller CTAs measured no faster
        // (2,048 x 4,096 x 4,096: 144 tiles of 240 columns 51.9 us, 128 of 256 49.8 us)
        if (bn < 256 && w == 1) continue;
        const long c = w * (kb * (512 + 3 * bn) * 105 / 100 + 4500);
        if (c < best) { best = c; cols = bn; }
    }
    return cols;
}

// How wide the tiles of the persistent kernel with 128 rows are: 256 columns, or 192 where the units of 256 leave
// a quarter of the SMs or more idle and those of 192 fill nine tenths of them in one wave (536 rows x 2,560 x 9,728
// in two ranges: 100 units or 140 on 148 SMs, 39.2 -> 36.2 us; x 4,096: 23.5 -> 21.7 us).  Elsewhere the narrower
// tile measured no faster or slower (80 -> 110 units: 26.8 -> 29.5 us; two waves either way: 36.2 -> 37.1 us): per
// flop it moves a ninth more through shared memory.  AIEN_B200_GEMM_TC=p256 | m256 pins 256, p192 pins 192.
static int tc_p_cols(int M, int N, int ranges) {
    if (const char* e = getenv("AIEN_B200_GEMM_TC")) {
        if (!strcmp(e, "p256") || !strcmp(e, "m256")) return 256;
        if (!strcmp(e, "p192")) return 192;
    }
    const long sms = tc_num_sms(), mt = (M + TC_BM - 1) / TC_BM;
    const long u256 = mt * ((N + 255) / 256) * ranges, u192 = mt * ((N + 191) / 192) * ranges;
    return (u256 * 4 <= sms * 3 && u192 <= sms && u192 * 10 >= sms * 9) ? 192 : 256;
}

static int tc_a_rows(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

// Rows of W per tile.  The CTAs of a launch all run at once (two per SM), and the launch ends when
// the SM with the most rows of W has streamed them: ceil(tiles / SMs) * rows.  96 instead of 128
// where that is less (24,576 rows over 148 SMs: 256 tiles, two each = 192 rows, against 192 tiles,
// some SMs two = 256 rows).  Only without split-K and with 64 rows of A at most.
static int tc_tile_cols(int M, int N, int splits) {
    if (splits != 1 || M > 64) return 128;
    const long sms = tc_num_sms();
    const long t128 = (N + 127) / 128, t96 = (N + 95) / 96;
    if (t96 > 2 * sms) return 128;
    return ((t96 + sms - 1) / sms) * 96 < ((t128 + sms - 1) / sms) * 128 ? 96 : 128;
}

template <int EPI, typename TC, int AR, int BN>
static int launch_tc_rows(const CUtensorMap& ma, const CUtensorMap& mw, void* out, long ldc, int splits, size_t part_stride,
                          int M, int N, int K, cudaStream_t stream) {
    auto kern = gemm_tc_kernel<EPI, TC, AR, BN>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcT<AR, BN>::SMEM) != cudaSuccess) return AIEN_E_STATE;
        configured = true;
    }
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    dim3 grid((M + TC_BM - 1) / TC_BM, (N + BN - 1) / BN, (total_kb + kb_per_split - 1) / kb_per_split);
    launch_chain(kern, grid, dim3(192), (size_t)TcT<AR, BN>::SMEM, stream, ma, mw, (TC*)out, ldc, part_stride, kb_per_split, M, N, K);
    return launch_status();
}

// The tensor maps are made here: their boxes follow the tile (tc_a_rows(M) rows of A, 128 or 96 of W).
template <int EPI, typename TC>
static int launch_tc(const void* A, long lda, const void* W, long ldw, void* out, long ldc, int splits, size_t part_stride,
                     int M, int N, int K, cudaStream_t stream) {
    const int ar = tc_a_rows(M), bn = tc_tile_cols(M, N, splits);
    CUtensorMap ma, mw;
    if (!make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BK, (uint32_t)ar) ||
        !make_map(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, TC_BK, (uint32_t)bn))
        return AIEN_E_STATE;
    if (bn == 96) {
        if (ar == 32) return launch_tc_rows<EPI, TC, 32, 96>(ma, mw, out, ldc, splits, part_stride, M, N, K, stream);
        return launch_tc_rows<EPI, TC, 64, 96>(ma, mw, out, ldc, splits, part_stride, M, N, K, stream);
    }
    if (ar == 32) return launch_tc_rows<EPI, TC, 32, 128>(ma, mw, out, ldc, splits, part_stride, M, N, K, stream);
    if (ar == 64) return launch_tc_rows<EPI, TC, 64, 128>(ma, mw, out, ldc, splits, part_stride, M, N, K, stream);
    return launch_tc_rows<EPI, TC, 128, 128>(ma, mw, out, ldc, splits, part_stride, M, N, K, stream);
}

}  // namespace aien

using namespace aien;

// epilogue 0: out[M,N]; 1: out[M,N/2] = silu(gate)*up with gate/up rows of W interleaved in runs of 8.
// splits > 1 (epilogue 0, float32 out): K is cut into ranges of whole 64-value blocks and out is
// [ranges][M][ldc] partial products, part_stride elements apart; aien_gemm_tc_ranges says how many
// ranges a given (K, splits) really makes.
AIEN_API int aien_gemm_tc_ranges(int K, int splits) {
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    if (splits < 1) splits = 1;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    return (total_kb + kb_per_split - 1) / kb_per_split;
}

// Whether aien_gemm_tc runs this product on the persistent kernel with tiles of 256 x 256 (1) or not (0).
AIEN_API int aien_gemm_tc_m256_supports(int M, int N, int K, int splits) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int ranges = aien_gemm_tc_ranges(K, splits);
    return (tc_plan(M, N, ranges) == 256 && tc_m256_cols(M, N, K, ranges) > 0) ? 1 : 0;
}

AIEN_API int aien_gemm_tc(const void* A, long lda, const void* W, long ldw, void* out, int c_dt, long ldc,
                          int M, int N, int K, int epilogue, int splits, size_t part_stride, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || splits < 1 || splits > 64) return AIEN_E_SHAPE;
    if (splits > 1 && (epilogue != 0 || c_dt != AIEN_DT_F32)) return AIEN_E_SHAPE;
    if ((lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return AIEN_E_ALIGN;
    if (epilogue == 1 && (N & 15)) return AIEN_E_SHAPE;
    if ((M + TC_BM - 1) / TC_BM > 2147483647 / 1 || (N + 95) / 96 > 65535) return AIEN_E_SHAPE;
    if (epilogue == 0 || epilogue == 1) {
        const int plan = tc_plan(M, N, aien_gemm_tc_ranges(K, splits));
#define TCP_CASE(BNV, EPIV, T) return launch_tc_persistent<BNV, EPIV, T>(A, lda, W, ldw, out, ldc, M, N, K, splits, part_stride, stream)
        const int wide = plan == 256 ? tc_m256_cols(M, N, K, aien_gemm_tc_ranges(K, splits)) : 0;
        if (wide > 0) {
            if (epilogue == 0 && c_dt == AIEN_DT_BF16) return launch_tc_persistent_m256<0, __nv_bfloat16>(wide, A, lda, W, ldw, out, ldc, M, N, K, stream);
            if (epilogue == 0 && c_dt == AIEN_DT_F32) return launch_tc_persistent_m256<0, float>(wide, A, lda, W, ldw, out, ldc, M, N, K, stream);
            if (epilogue == 1 && c_dt == AIEN_DT_BF16) return launch_tc_persistent_m256<1, __nv_bfloat16>(wide, A, lda, W, ldw, out, ldc, M, N, K, stream);
            if (epilogue == 1 && c_dt == AIEN_DT_F32) return launch_tc_persistent_m256<1, float>(wide, A, lda, W, ldw, out, ldc, M, N, K, stream);
        }
        if (plan == 256 && epilogue == 0 && tc_p_cols(M, N, aien_gemm_tc_ranges(K, splits)) == 192) {
            if (c_dt == AIEN_DT_BF16) TCP_CASE(192, 0, __nv_bfloat16);
            if (c_dt == AIEN_DT_F32) TCP_CASE(192, 0, float);
        }
        if (plan == 256) {
            if (epilogue == 0 && c_dt == AIEN_DT_BF16) TCP_CASE(256, 0, __nv_bfloat16);
            if (epilogue == 0 && c_dt == AIEN_DT_F32) TCP_CASE(256, 0, float);
            if (epilogue == 1 && c_dt == AIEN_DT_BF16) TCP_CASE(256, 1, __nv_bfloat16);
            if (epilogue == 1 && c_dt == AIEN_DT_F32) TCP_CASE(256, 1, float);
        }
#undef TCP_CASE
    }
    if (epilogue == 0) {
        if (c_dt == AIEN_DT_BF16) return launch_tc<0, __nv_bfloat16>(A, lda, W, ldw, out, ldc, 1, 0, M, N, K, stream);
        if (c_dt == AIEN_DT_F32) return launch_tc<0, float>(A, lda, W, ldw, out, ldc, splits, part_stride, M, N, K, stream);
        return AIEN_E_DTYPE;
    }
    if (epilogue == 1) {
        if (c_dt == AIEN_DT_BF16) return launch_tc<1, __nv_bfloat16>(A, lda, W, ldw, out, ldc, 1, 0, M, N, K, stream);
        if (c_dt == AIEN_DT_F32) return launch_tc<1, float>(A, lda, W, ldw, out, ldc, 1, 0, M, N, K, stream);
        return AIEN_E_DTYPE;
    }
    return AIEN_E_SHAPE;
}

// Reads and clears the error code a bounded wait may have left (0: none; 1 producer, 2 MMA, 3 epilogue).
AIEN_API int aien_gemm_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_wait_error, &zero, sizeof(int));
    return v;
}

AIEN_DEFINE_WAIT_ERROR_ADDRESS(aien_gemm_tc_error_address)
