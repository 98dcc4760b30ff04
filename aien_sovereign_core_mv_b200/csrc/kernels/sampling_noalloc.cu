// aien_sample_rows_static: the sampling kernel of sampling.cu run on scratch that the library
// owns, for callers that cannot allocate (see sampling_noalloc.h for who they are and why).
#include "common.cuh"
#include "sampling_noalloc.h"
#include <atomic>

namespace aien {

// Defined in sampling.cu; launched from here through its host-side stub.
__global__ void sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                                   const float* __restrict__ top_p, const int* __restrict__ top_k,
                                   const unsigned long long* __restrict__ seeds, const long long* __restrict__ request_ids,
                                   const int* __restrict__ positions, float* __restrict__ probs_scratch,
                                   int* __restrict__ out_ids, float* __restrict__ out_logprob);

// The scratch itself.  In host code this name is only a handle for the runtime, not an address a
// kernel could use: the device address is asked for once per device below.
static __device__ __align__(256) float g_static_probs[AIEN_SAMPLE_STATIC_MAX_ELEMS];

constexpr int kMaxDevices = 64;
static std::atomic<float*> g_scratch_addr[kMaxDevices] = {};     // every thread that asks gets the same answer

}  // namespace aien

using namespace aien;

AIEN_API int aien_sample_rows_static(const float* logits, int R, int V, const float* temperature, const float* top_p,
                                     const int* top_k, const unsigned long long* seeds, const long long* request_ids,
                                     const int* positions, int* out_ids, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || (long long)R * (long long)V > (long long)AIEN_SAMPLE_STATIC_MAX_ELEMS) return AIEN_E_SHAPE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return AIEN_E_STATE;
    float* scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {                                // set-up, once per device, with that device current
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_probs);
        if (e != cudaSuccess) return static_cast<int>(e);
        scratch = static_cast<float*>(p);
        g_scratch_addr[dev].store(scratch, std::memory_order_release);
    }
    sample_rows_kernel<<<R, 1024, 0, stream>>>(logits, V, temperature, top_p, top_k, seeds, request_ids, positions,
                                               scratch, out_ids, nullptr);
    return launch_status();
}
