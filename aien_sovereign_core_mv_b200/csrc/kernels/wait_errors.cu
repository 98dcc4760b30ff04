// The error words of the kernels with bounded waits, read inside the stream.
//
// Every kernel that waits on an mbarrier gives up after a fixed number of polls and stores a code
// in the error word of its translation unit (tma.cuh).  The host functions aien_*_error() read one
// word each with a synchronous copy; a step cannot afford four of those.  This kernel copies the
// four words into a caller's buffer, in the stream, behind the step's own launches: the engine
// puts that buffer beside the sampled token ids, so the one device-to-host copy a step makes
// anyway also tells whether every wait of the step was met.
#include "common.cuh"

extern "C" {
int aien_gemm_tc_error_address(void** out);
int aien_gemv_stream_error_address(void** out);
int aien_attention_prefill_tc_error_address(void** out);
int aien_attention_decode_stream_error_address(void** out);
}

namespace aien {

struct WaitWords {
    const int* w[4];
};

__global__ void collect_wait_errors_kernel(WaitWords words, int* __restrict__ out) {
    const int i = threadIdx.x;
    if (i < 4) out[i] = *reinterpret_cast<const volatile int*>(words.w[i]);
}

constexpr int kMaxDevices = 64;
static WaitWords g_words[kMaxDevices] = {};
static bool g_words_known[kMaxDevices] = {};

}  // namespace aien

using namespace aien;

// out: 4 x int32 on the device, in the order gemm_tc, gemv_stream, attention_prefill_tc,
// attention_decode_stream (0: every wait was met).  The words are left as they are: the
// aien_*_error() functions clear them.  The first call on a device looks the addresses up.
AIEN_API int aien_collect_wait_errors(int* out, cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return AIEN_E_STATE;
    if (!g_words_known[dev]) {
        void* p[4] = {nullptr, nullptr, nullptr, nullptr};
        if (aien_gemm_tc_error_address(&p[0]) || aien_gemv_stream_error_address(&p[1]) ||
            aien_attention_prefill_tc_error_address(&p[2]) || aien_attention_decode_stream_error_address(&p[3]))
            return AIEN_E_STATE;
        for (int i = 0; i < 4; ++i) g_words[dev].w[i] = static_cast<const int*>(p[i]);
        g_words_known[dev] = true;
    }
    collect_wait_errors_kernel<<<1, 32, 0, stream>>>(g_words[dev], out);
    return launch_status();
}
