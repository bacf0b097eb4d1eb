// Allocation-free entry point of the split-K tensor-core GEMM.
//
// This function has no counterpart in the reference implementation; it exists for callers of this
// library that are not allowed to allocate device memory:
//   * a serving process that hands the whole device to its KV-cache pool at start-up, after which
//     any further cudaMalloc fails or eats into memory the scheduler has already promised away;
//   * a decode thread with a latency bound, where cudaMalloc / cudaFree would synchronise the
//     whole device and stall every stream in the process;
//   * plugin code running under a host framework that owns all allocation and forbids the CUDA
//     allocator inside its callbacks.
//
// The split-K partial sums and the per-tile arrival counters, which sfb_umma_dense takes from the
// caller, live here in arrays that are part of the library image:
//     SFB_NOALLOC_MAX_FLOATS  floats of partial sums  (8 MiB)
//     SFB_NOALLOC_MAX_TILES   32-bit counters         (16 KiB)
// Every GPU that loads the library holds these arrays until the process exits.
//
// Rules for the caller:
//   * Inputs and outputs are still the caller's: tensor maps (sfb_tmap_encode), scale atoms, output.
//   * tiles * splits * 128 * NP must not exceed SFB_NOALLOC_MAX_FLOATS and tiles (= groups * N/128)
//     must not exceed SFB_NOALLOC_MAX_TILES; otherwise the call launches nothing, returns
//     SFB_NOALLOC_TOO_LARGE and sfb_noalloc_last_error() says which limit was hit.
//   * The first call on each device looks up the device addresses of the arrays (with that device
//     current).  Make that first call before any stream capture begins on that device.
//   * All calls share the arrays and find in them whatever the previous call left; the counters
//     are cleared on the stream before each launch.  Two calls that overlap on the GPU (different
//     streams, or the same stream with programmatic overlap) race on the arrays: serialise them.
//   * With splits == 1 nothing is accumulated across CTAs, so the arrays are not touched and the
//     size limits above do not apply.
//   * The address lookup of the first call is not locked.  Two host threads that make their first
//     call on the same device at the same time both run the lookup and store the same two
//     addresses; that is harmless, but a caller that wants no such overlap makes one call per
//     device from one thread during start-up.
//   * A peer push armed with sfb_umma_set_push (or a gather armed with sfb_umma_set_gather) for
//     some other call is discarded here, not inherited: this entry point writes only out_b / out_f.
//   * The function calls no cudaMalloc, cudaFree or allocating library routine.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define SFB_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)
#define SFB_NOALLOC_MAX_TILES 4096
#define SFB_NOALLOC_TOO_LARGE (-2)
#define SFB_NOALLOC_SETUP_FAILED (-3)

#ifdef __cplusplus
extern "C" {
#endif

// Same contract and argument meaning as sfb_umma_dense (k_umma.cu) without the scratch and ticket
// pointers.  Returns 0, a cudaError_t from the launch, or one of the negative codes above.
int sfb_umma_dense_noalloc(const void* tmapA, const void* tmapB, const void* sfa, int katoms_a, const void* sfb,
                           int katoms_b, int n, int NP, int N, int K, int groups, int a_fp4, int splits,
                           void* out_b, float* out_f, int64_t out_stride, void* status, cudaStream_t stream);

// Text of the last error this thread got from sfb_umma_dense_noalloc ("" when none).
const char* sfb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
