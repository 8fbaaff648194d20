// Sum of the same region of up to 8 ranks' symmetric buffers into a local tensor (16-bit in,
// fp32 accumulate), read with 16-byte peer loads.  Used to return dK/dV partial results to the
// rank that owns the keys in context-parallel attention.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "teb200/api.h"
#include "teb200/comm.h"
#include "teb200/ptx.cuh"

namespace teb200 {
namespace {

template <bool BF>
__global__ void peer_sum_kernel(PeerSumArgs a) {
  const long long n = a.vecs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < a.n; ++r) {
      const uint4 v = reinterpret_cast<const uint4*>(a.src[r])[i];
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (BF) {
          acc[2 * k] += __uint_as_float(w[k] << 16);
          acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
        } else {
          const __half2 h = *reinterpret_cast<const __half2*>(&w[k]);
          acc[2 * k] += __low2float(h);
          acc[2 * k + 1] += __high2float(h);
        }
      }
    }
    uint4 o;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) o32[k] = BF ? pack_bf16x2(acc[2 * k], acc[2 * k + 1]) : pack_f16x2(acc[2 * k], acc[2 * k + 1]);
    reinterpret_cast<uint4*>(a.out)[i] = o;
  }
}

}  // namespace

cudaError_t peer_sum(const PeerSumArgs& a, cudaStream_t s) {
  if (a.n < 1 || a.n > kCommMaxRanks) return cudaErrorInvalidValue;
  if (a.vecs == 0) return cudaSuccess;
  const int grid = static_cast<int>(a.vecs / 256 + 1 < 148 * 8 ? a.vecs / 256 + 1 : 148 * 8);
  if (a.is_bf16) peer_sum_kernel<true><<<grid, 256, 0, s>>>(a);
  else peer_sum_kernel<false><<<grid, 256, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace teb200
