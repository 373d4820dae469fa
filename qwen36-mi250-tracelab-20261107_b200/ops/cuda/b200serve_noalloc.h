// Allocation-free entry point of the kernel library. It has no counterpart in the reference
// engine; it exists for hosts that embed these kernels where device memory cannot be requested.
//
// Who needs it: code that runs inside a fixed memory plan and therefore must not call cudaMalloc
// (or anything that does so behind its back, a framework's caching allocator included) - for
// example a serving process whose whole device memory was carved up at start-up, a plugin called
// from another runtime that owns the allocator, or a latency-critical loop in which an allocation
// could synchronise the device. The regular greedy-head entry point (b200_gemm_dense with the
// argmax epilogue) asks its caller for a workspace of per-vocabulary-tile partial results; such
// callers have nowhere to take it from.
//
// b200_lm_head_argmax_noalloc computes, for each of T activation rows X[t, :K] (bf16), the index
// of the largest logit X[t] . W[v] over the V rows of W (bf16, [V, K]); ties go to the lower
// index. Inputs and outputs are the caller's; the partial results live in an array that is part
// of the library image:
//
//   * Limits: T <= B200_NOALLOC_MAX_ROWS rows and V <= 128 * B200_NOALLOC_MAX_TILES vocabulary
//     entries per call. Larger sizes are refused with B200_NOALLOC_TOO_LARGE and a message on
//     stderr; nothing is launched.
//   * Cost: the array takes (MAX_ROWS * MAX_TILES * 8) bytes = 4 MiB of device memory on every GPU
//     that loads the library, from load until the process exits, whether or not this function
//     is ever called.
//   * The first call on each device looks up the array's device address (one runtime query, no
//     launch) and caches it per device ordinal. Make that first call before any CUDA stream capture
//     begins. Two host threads that make their first call on the same device at the same moment
//     both store the same address; no lock is taken.
//   * All calls on a device share the one array. It keeps whatever the previous call left; a call
//     whose kernels ran to completion overwrites every element it later reads, so nothing has to
//     be cleared. If an internal bounded wait gives up (*err != 0 afterwards) the partial results
//     are not written and out_idx / out_val come from the previous call's leftovers: read *err
//     before trusting the outputs. Two calls that can overlap on the GPU (different streams, or
//     concurrent host threads) would overwrite each other's partial results: serialise them.
//   * The function calls no cudaMalloc, cudaFree or allocating library routine.
//
// out_idx: int64 [T]; out_val: float [T] with the winning logit, or NULL; ldx / ldw: row strides of
// X and W in elements; err: device int the kernels set when an internal bounded wait gives up
// (may be shared with the other entry points); returns 0 on success.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define B200_NOALLOC_MAX_ROWS 256
#define B200_NOALLOC_MAX_TILES 2048

#define B200_NOALLOC_TOO_LARGE (-20)
#define B200_NOALLOC_BAD_DEVICE (-21)
#define B200_NOALLOC_NO_SYMBOL (-22)

#ifdef __cplusplus
extern "C" {
#endif

int b200_lm_head_argmax_noalloc(const void* X, const void* W, int64_t* out_idx, float* out_val, int T, int V, int K,
                                int ldx, int ldw, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
