// TMA and mbarrier helpers shared by the kernels that stream operands through shared memory.
// Every CTA fetches its own tiles; no load here is shared out over a cluster.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

namespace aien {

constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

// One error word per translation unit: a bounded wait that runs out stores its code here.
static __device__ int g_wait_error = 0;

// Gives the translation unit an exported function that tells the device address of its error word,
// so that one small kernel (wait_errors.cu) can read the words of all of them inside the stream.
#define AIEN_DEFINE_WAIT_ERROR_ADDRESS(name)                                                        \
    AIEN_API int name(void** out) {                                                                 \
        return cudaGetSymbolAddress(out, aien::g_wait_error) == cudaSuccess ? 0 : AIEN_E_STATE;     \
    }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after TC_SPIN_LIMIT polls, records `code`, and lets the caller go on.
// Once a wait has given up, the others give up after 2^20 polls (far longer than any wait of a
// working pipeline), so a broken pipeline drains sixteen times faster than one limit per wait.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int code) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 0xFFFFFu) == 0xFFFFFu && *reinterpret_cast<volatile int*>(&g_wait_error) != 0) return;
    }
    atomicCAS(&g_wait_error, 0, code);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}

// ---------------------------------------------------------------- host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// A 2-D bfloat16 row-major matrix [rows, cols] with leading dimension ld, boxes of box_rows x
// box_cols (box_cols * 2 bytes = 128: one swizzled row), 128-byte swizzle, zero fill out of range.
inline bool make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols, uint32_t box_rows) {
    static std::map<std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(ptr, rows, cols, ld, box_cols, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) { *map = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = *map;
    return true;
}

// The same matrix seen as [cols/64][rows][64]: one copy brings box_rows rows x (64 * box_chunks)
// columns, laid out chunk-major in shared memory (chunk j, row r at (j * box_rows + r) * 128 bytes,
// 128-byte swizzle by r).  Needs cols % 64 == 0.
inline bool make_map_chunked(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                             uint32_t box_rows, uint32_t box_chunks) {
    static std::map<std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(ptr, rows, cols, ld, box_rows, box_chunks);
    auto it = cache.find(key);
    if (it != cache.end()) { *map = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn || cols % 64 != 0) return false;
    cuuint64_t dims[3] = {64, rows, cols / 64};
    cuuint64_t strides[2] = {ld * 2, 128};
    cuuint32_t box[3] = {64, box_rows, box_chunks};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = *map;
    return true;
}

}  // namespace aien
