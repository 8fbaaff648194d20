// Norm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference library.  It exists for
// code that runs where cudaMalloc is off limits: inside a region whose memory
// plan is frozen (a captured or replayed step, a fixed arena handed out by a
// serving runtime), from a plain C host without a tensor library, or from a
// component that is forbidden to grow the process' device footprint.  The
// regular norm backward needs a scratch buffer for its two-stage reduction of
// the weight gradient; here that scratch is a fixed array that lives inside the
// library image on every GPU that loads it (TEB200_NOALLOC_SCRATCH_FLOATS * 4 bytes,
// held until the process exits).
//
// Rules of use:
//   * The first call on a device looks up the device address of the scratch
//     array; make that first call outside any stream capture.
//   * Problem sizes whose scratch need, teb200_norm_bwd_noalloc_scratch_floats(R, C),
//     exceeds TEB200_NOALLOC_SCRATCH_FLOATS are rejected with cudaErrorInvalidValue and a
//     message on stderr; nothing is launched.
//   * All calls share the one array.  Two calls that may run at the same time on
//     one GPU (different streams) race on it; serialize them.  Nothing in the
//     array has to be zero on entry: each call overwrites every word it later
//     reads, so leftovers of the previous call are harmless.
//   * The function calls no cudaMalloc / cudaFree and no allocating library
//     routine.  Inputs and outputs are the caller's.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// 4 Mi floats = 16 MiB per GPU.
#define TEB200_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

// Scratch floats the backward of an [R, C] problem needs.
long long teb200_norm_bwd_noalloc_scratch_floats(int R, int C);

// dx = d(norm)/dx, dgamma (and dbeta for LayerNorm) from dy, x and the saved statistics.
//   layernorm: 0 RMSNorm (mu, dbeta ignored), 1 LayerNorm
//   x_dtype / w_dtype: 0 fp32, 1 fp16, 2 bf16 (activations / gamma)
//   add: optional tensor added to dx, or NULL
// Returns a cudaError_t value (0 on success).
int teb200_norm_bwd_noalloc(int layernorm, int R, int C, int x_dtype, int w_dtype, int zero_centered_gamma,
                            const void* dy, const void* x, const float* mu, const float* rsigma, const void* gamma,
                            const void* add, void* dx, void* dgamma, void* dbeta, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
