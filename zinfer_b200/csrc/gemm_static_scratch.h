// A matrix product for callers that cannot allocate GPU memory.
//
// This entry point has no counterpart in NeoZedAtlas/Zinfer (which runs on the CPU
// and has no device memory to manage); it exists for users of this library.
//
// Who needs it: code that runs where cudaMalloc is not an option.  Examples are a
// plug-in called from inside a host application's CUDA-graph capture or from a
// real-time loop that forbids allocation, a process whose memory pool is owned and
// fully handed out by another runtime, and C callers that link this library
// without torch, which is what normally provides the split-K workspace.
// zi_gemm_tcgen05() asks its caller for that workspace; this variant brings its own.
//
//   out[M, N] = x[M, K] * w[N, K]^T   (bfloat16 operands, 32-bit accumulation)
//
// The caller passes inputs and outputs only.  When the product is split along K,
// the partial sums go to a 8 MiB array that is part of the library's device image:
// every GPU that loads the library keeps those 8 MiB until the process exits.
// Products that would need more (splits * M * N * 4 bytes; the capacity is
// zi_gemm_static_scratch_capacity_bytes()) are refused with a message in
// zi_last_error(), and nothing is launched.
//
// Rules for callers:
//  * The first call on a device looks up the device address of the built-in array
//    (cudaGetSymbolAddress, with that device current) and sets a kernel attribute.
//    Make that first call before you begin any stream capture.
//  * All calls on one device share the one array, and it keeps what the last call
//    left in it.  Nothing in it has to be zero at the start (every partial sum that
//    is read is written first).  Two calls
//    whose kernels may overlap on the GPU (different streams without an ordering
//    between them) race on the array: order them yourself.
//  * The function calls no cudaMalloc, cudaFree or any allocating library routine.
//  * How a failure shows.  Every wait inside the kernel is bounded; if one ever ran
//    out (never seen in practice) the kernel stores a non-zero code in a status word
//    and returns, and its output is not to be trusted.  The word is only ever written
//    with non-zero codes and never cleared by a call, so a failure of an earlier call
//    stays visible until you read it.  `wait_status` is a device int of yours (zero it
//    once, read it when you synchronise anyway), or NULL to use a word inside the
//    library, which zi_gemm_static_scratch_status() reads and clears (it waits for the
//    device and allocates nothing).
//
// Returns 0, a cudaError_t (> 0) of the launch, or -1 with zi_last_error() set.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long zi_gemm_static_scratch_capacity_bytes();

// The library's own status word on the current device: 0, or the code of a wait that ran out
// since the last read (then cleared); negative if the word cannot be read.
int zi_gemm_static_scratch_status();

int zi_gemm_tcgen05_static_scratch(void* out, int out_dtype /* 0 = float32, 1 = bfloat16 */, const void* x,
                                   const void* w, int M, int N, int K, int ldx, int ldw, int ldo, int sm_count,
                                   int* wait_status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
