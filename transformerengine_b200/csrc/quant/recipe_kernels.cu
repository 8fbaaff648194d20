// Delayed-scaling bookkeeping in one launch: amax = max (or most recent) over the history,
// new scale = (fp8_max / amax) / 2^margin with the guards of the reference, history rolled by one
// and slot 0 cleared.  (Reference behaviour: common/recipe/delayed_scaling.cu.)
#include <cuda_runtime.h>
#include <stdint.h>

#include "teb200/api.h"
#include "teb200/quant.h"

namespace teb200 {
namespace {

// history [H, n] row-major; one thread per quantizer column
__global__ void delayed_scaling_update_kernel(float* history, float* scale, int H, int n, float fp8_max, float inv_pow2_margin,
                                              int most_recent) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  float amax = history[j];
  if (!most_recent)
    for (int h = 1; h < H; ++h) amax = fmaxf(amax, history[static_cast<size_t>(h) * n + j]);
  if (amax > 0.f && isfinite(amax)) {
    float sf = __fdiv_rn(fp8_max, amax) * inv_pow2_margin;
    if (isinf(sf)) sf = 3.402823466e+38f;
    scale[j] = sf;
  }
  // roll: row h takes row h+1, the last row takes the old row 0, then slot 0 is cleared
  float carry = history[j];
  for (int h = 0; h + 1 < H; ++h) history[static_cast<size_t>(h) * n + j] = history[static_cast<size_t>(h + 1) * n + j];
  if (H > 1) history[static_cast<size_t>(H - 1) * n + j] = carry;
  history[j] = 0.f;
}

}  // namespace

cudaError_t delayed_scaling_update(float* history, float* scale, int H, int n, float fp8_max, int margin, int most_recent,
                                   cudaStream_t s) {
  if (n == 0 || H == 0) return cudaSuccess;
  float inv = 1.f;
  for (int i = 0; i < (margin > 0 ? margin : -margin); ++i) inv *= margin > 0 ? 0.5f : 2.f;
  delayed_scaling_update_kernel<<<(n + 127) / 128, 128, 0, s>>>(history, scale, H, n, fp8_max, inv, most_recent);
  return cudaGetLastError();
}

}  // namespace teb200
