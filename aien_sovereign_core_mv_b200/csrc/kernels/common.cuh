// Shared helpers for the engine's CUDA kernels (sm_100a).
//
// Conventions used by every launcher in this directory:
//   * exported with C linkage, named aien_<op>; returns 0 on success, a cudaError_t value if
//     the launch failed, or a negative AIEN_E_* code when an argument is refused;
//   * takes raw device pointers, sizes, a dtype code per tensor family and a cudaStream_t;
//   * never allocates; scratch comes from the caller.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define AIEN_DT_F32 0
#define AIEN_DT_BF16 1

#define AIEN_E_DTYPE (-2)      // unsupported dtype combination
#define AIEN_E_SHAPE (-3)      // a size the kernel refuses
#define AIEN_E_ALIGN (-4)      // pointer or stride not aligned as required
#define AIEN_E_STATE (-5)      // library state (tensor map encode, attribute set) failed

#define AIEN_API extern "C" __attribute__((visibility("default")))

namespace aien {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Reads element i of a vector whose dtype is only known at run time (norm weights may be
// stored in 32 bits beside a bfloat16 model).
__device__ __forceinline__ float load_dyn(const void* p, int dt, size_t i) {
    return dt == AIEN_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                             : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed combination order (warp tree, then warps in index order), so the
// result for a row does not depend on what else is in the grid.  `red` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += red[w];
    return total;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = red[0];
    for (int w = 1; w < nwarps; ++w) total = fmaxf(total, red[w]);
    return total;
}

// ---- programmatic dependent launch
// The decode step is a chain of short kernels.  Launched with the programmatic-serialization
// attribute, a kernel may become resident while its predecessor is still running; it must not
// read what the predecessor writes, nor write anything, before griddep_wait() returns (which is
// when the predecessor has completed and its writes are visible).  Weights are never written
// during a step, so a kernel may prefetch them first.  griddep_launch() lets the successor start
// its own prologue.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// What an earlier kernel of the step wrote must be read with these in a kernel launched with
// launch_chain: a pointer that the compiler can prove read-only (const, no aliasing store) gets
// ld.global.nc loads, which the assembler may move above griddepcontrol.wait, where the producer
// may still be running (seen: the q/k kernel read stale projections).  ld.global.cg is never moved.
__device__ __forceinline__ float ld_act(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_act(const __nv_bfloat16* p) {
    const unsigned short b = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return __bfloat162float(__ushort_as_bfloat16(b));
}
__device__ __forceinline__ float4 ld_act4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ld_act4(const __nv_bfloat16* p) {
    const uint2 r = __ldcg(reinterpret_cast<const uint2*>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("AIEN_B200_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Launch `kernel` so that it may overlap the tail of the kernel before it on the stream.  Only for
// kernels that call griddep_wait() before touching anything but weights.
template <typename... KArgs, typename... Args>
inline void launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace aien

// Dispatch on one dtype code; T is bound inside BODY.
#define AIEN_DISPATCH_DTYPE(code, T, BODY)                     \
    do {                                                       \
        if ((code) == AIEN_DT_F32) { using T = float; BODY; }  \
        else if ((code) == AIEN_DT_BF16) { using T = __nv_bfloat16; BODY; } \
        else return AIEN_E_DTYPE;                              \
    } while (0)
