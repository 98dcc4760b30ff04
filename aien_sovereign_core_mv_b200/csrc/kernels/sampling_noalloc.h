// Token sampling for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library.
// Some hosts of an inference library cannot call cudaMalloc at the time they sample: code running
// under a memory budget that was handed out at start-up and is now closed, plugins that are
// forbidden to touch the allocator of the process they live in, and real-time loops where an
// allocation (and the implicit synchronisation it may bring) is not acceptable.  The regular entry
// point, aien_sample_rows, wants a scratch buffer of R * V floats from its caller; this one keeps
// that scratch inside the library instead, in a fixed array that lives in device memory for as
// long as the library is loaded.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Most float32 values the built-in scratch holds: rows * vocabulary of one call must not exceed it
// (4 MB per GPU that loads the library, held until the process exits).
#define AIEN_SAMPLE_STATIC_MAX_ELEMS (1 << 20)

// Same rules and same results as aien_sample_rows (greedy at temperature <= 0.001, top-k, top-p,
// one Philox draw per row), but without a scratch argument.
//   logits [R, V] float32; temperature, top_p [R] float32; top_k, positions [R] int32;
//   seeds [R] uint64; request_ids [R] int64; out_ids [R] int32; all device pointers.
// Returns 0, a cudaError_t value, -3 when R * V exceeds AIEN_SAMPLE_STATIC_MAX_ELEMS, or -5 when the
// current device's index is 64 or more (the table of per-device addresses ends there); nothing is
// launched in either case.  It calls no allocating routine.
//
// The first call on each device looks up the device address of the scratch array (one
// cudaGetSymbolAddress with that device current) and remembers it; make that first call outside
// any stream capture.  All calls on a device share the one array: it keeps whatever the last
// call left there, which is harmless because every row that samples writes its V slots before it
// reads them, but two calls that overlap on the GPU (different streams, no ordering between
// them) would overwrite each other's probabilities and must be serialised by the caller.
int aien_sample_rows_static(const float* logits, int R, int V, const float* temperature, const float* top_p,
                            const int* top_k, const unsigned long long* seeds, const long long* request_ids,
                            const int* positions, int* out_ids, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
