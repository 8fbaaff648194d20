// LayerNorm / RMSNorm launchers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace teb200 {

struct NormArgs {
  int layernorm = 0;  // 0 = RMSNorm, 1 = LayerNorm
  int R = 0, C = 0;
  int x_dtype = 2, w_dtype = 2;  // DType of activations / of gamma, beta
  float eps = 1e-5f;
  int zero_centered = 0;
  const void* x = nullptr;
  const void* gamma = nullptr;
  const void* beta = nullptr;
  void* y = nullptr;    // optional: null computes the statistics only
  float* mu = nullptr;  // [R] LayerNorm only
  float* rs = nullptr;  // [R]
  // backward
  const void* dy = nullptr;
  const void* add = nullptr;  // optional tensor added to dx (residual gradient)
  void* dx = nullptr;
  void* dgamma = nullptr;
  void* dbeta = nullptr;
  // scratch of norm_bwd_parts(R) * 2 * C floats for the two-stage parameter-gradient reduction
  float* workspace = nullptr;
};

int norm_bwd_parts(int R);
cudaError_t norm_fwd(const NormArgs& a, cudaStream_t s);
cudaError_t norm_bwd(const NormArgs& a, cudaStream_t s);

}  // namespace teb200
