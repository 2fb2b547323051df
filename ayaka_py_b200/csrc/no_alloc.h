// An entry point for callers that must not allocate.
//
// This declaration has no counterpart in the reference project; it exists for
// programs that embed this library where memory allocation is off the table at
// call time: a host that has given the whole device to a memory pool of its own
// (so that cudaMalloc from a library would fail or fragment it), or a serving
// thread with a latency budget that cannot absorb the device-wide
// synchronisation that cudaMalloc and cudaFree imply.  Such callers still pass
// their own inputs and outputs; what they cannot provide is the scratch memory
// that the split-K form of the tensor-core product needs.
//
// ayk_gemm_tc_no_alloc computes the same product as ayk_gemm_tc,
//
//   C[M, N] = act(X[M, K] * W[N, K]^T + bias[N]) (+ residual[M, N]),
//
// with X and W bfloat16, but keeps the split-K partial sums and the tile
// counters in arrays that are part of the library image (static __device__
// storage), so the call allocates nothing: no cudaMalloc, no cudaFree, no
// pinned host memory, no allocator of a framework.
//
// Limits and rules:
//   * splits * M * N must not exceed AYK_NO_ALLOC_MAX_PARTIALS floats (4 MiB of
//     scratch) and the number of 128-wide output tiles must not exceed
//     AYK_NO_ALLOC_MAX_TILES; larger problems are refused with an error text.
//     Every GPU whose context loads the library holds these arrays (about
//     4 MiB) until the process exits.
//   * The first call on a device looks up the arrays' device addresses (and the
//     driver's tensor-map encoder) and sets the kernel's shared-memory
//     attribute on that device; it does so under the library's mutex, so first
//     calls from several threads, or on several devices, are safe.  Make that
//     first call outside any stream capture.
//   * With splits <= 0 the library chooses a split count that fits the built-in
//     scratch (down to no split at all); only a count that the caller asks for
//     can be refused as too large.
//   * All calls share the one scratch region, which keeps whatever the last
//     call left in it; the entry point clears the counters itself before each
//     launch.  Two calls that overlap on the GPU (different streams, or one
//     stream and a graph replay) would race on the scratch: serialise them.
//   * A bounded wait inside the kernel that runs out is reported by
//     ayk_gemm_tc_no_alloc_error() (which synchronises the device to read the
//     word); 0 means no wait ran out since the library was loaded.
#pragma once

#include <cuda_runtime.h>

#define AYK_NO_ALLOC_MAX_PARTIALS (1 << 20)
#define AYK_NO_ALLOC_MAX_TILES 1024

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or a negative code with a text in ayk_last_error().
// dtype tags: 0 = float32, 1 = bfloat16 (out_dtype); act: 0 none, 1 gelu (erf),
// 2 gelu (tanh), 3 quick_gelu.  splits <= 0 lets the library choose.
int ayk_gemm_tc_no_alloc(void* C, const void* X, const void* W, const float* bias, const float* residual,
                         int M, int N, int K, int act, int out_dtype, int splits, cudaStream_t stream);

int ayk_gemm_tc_no_alloc_error(void);

#ifdef __cplusplus
}
#endif
