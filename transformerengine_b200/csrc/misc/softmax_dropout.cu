// Scaled masked softmax (forward / backward) and dropout with a packed keep-mask, for the
// unfused attention path.  One warp per row, fp32 math, 16-bit or fp32 storage.
// (Reference behaviour: common/fused_softmax/scaled_masked_softmax.cu,
//  scaled_upper_triang_masked_softmax.cu, common/dropout/dropout.cu.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "teb200/api.h"
#include "teb200/misc.h"

namespace teb200 {
namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, size_t i) { return static_cast<float>(p[i]); }

__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// rows = b*h*sq; mask [b, 1, sq, sk] bytes (non-zero = masked out); causal aligned bottom-right
template <typename T>
__global__ void softmax_fwd_kernel(SoftmaxArgs a) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const T* x = static_cast<const T*>(a.x) + row * a.cols;
  T* y = static_cast<T*>(a.y) + row * a.cols;
  const int qi = static_cast<int>(row % a.sq);
  const long long bi = row / (static_cast<long long>(a.sq) * a.heads);
  const uint8_t* m = a.mask ? a.mask + (bi * a.sq + qi) * a.cols : nullptr;
  const int lim = a.causal ? qi + (a.cols - a.sq) : a.cols - 1;  // last visible column
  float mx = -3.0e38f;
  for (int c = lane; c < a.cols; c += 32) {
    const bool vis = c <= lim && !(m && m[c]);
    if (vis) mx = fmaxf(mx, ldf(x, c) * a.scale);
  }
  mx = wmax(mx);
  float sum = 0.f;
  for (int c = lane; c < a.cols; c += 32) {
    const bool vis = c <= lim && !(m && m[c]);
    if (vis) sum += __expf(ldf(x, c) * a.scale - mx);
  }
  sum = wsum(sum);
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  for (int c = lane; c < a.cols; c += 32) {
    const bool vis = c <= lim && !(m && m[c]);
    y[c] = static_cast<T>(vis ? __expf(ldf(x, c) * a.scale - mx) * inv : 0.f);
  }
}

// dx = scale * p * (dy - sum(dy * p))
template <typename T>
__global__ void softmax_bwd_kernel(SoftmaxArgs a) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const T* p = static_cast<const T*>(a.x) + row * a.cols;
  const T* dy = static_cast<const T*>(a.dy) + row * a.cols;
  T* dx = static_cast<T*>(a.y) + row * a.cols;
  float dot = 0.f;
  for (int c = lane; c < a.cols; c += 32) dot += ldf(p, c) * ldf(dy, c);
  dot = wsum(dot);
  for (int c = lane; c < a.cols; c += 32) dx[c] = static_cast<T>(a.scale * ldf(p, c) * (ldf(dy, c) - dot));
}

__device__ __forceinline__ uint32_t mix(uint64_t k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdULL; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ULL; k ^= k >> 33;
  return static_cast<uint32_t>(k);
}

// one thread per 8 elements; keep bits packed one byte per group
template <typename T>
__global__ void dropout_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ bits, int64_t n,
                                   float p, uint64_t seed, uint64_t offset) {
  const int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t i0 = g * 8;
  if (i0 >= n) return;
  const float inv = 1.f / (1.f - p);
  const uint32_t thr = static_cast<uint32_t>(p * 16777216.f);
  uint8_t b = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int64_t i = i0 + k;
    if (i >= n) break;
    const uint32_t r = mix(static_cast<uint64_t>(i) * 0x9E3779B97F4A7C15ULL + seed * 0xD1B54A32D192ED03ULL + offset) >> 8;
    const bool keep = r >= thr;
    b |= static_cast<uint8_t>(keep) << k;
    y[i] = static_cast<T>(keep ? static_cast<float>(x[i]) * inv : 0.f);
  }
  bits[g] = b;
}

template <typename T>
__global__ void dropout_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ bits, T* __restrict__ dx,
                                   int64_t n, float p) {
  const int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t i0 = g * 8;
  if (i0 >= n) return;
  const float inv = 1.f / (1.f - p);
  const uint8_t b = bits[g];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int64_t i = i0 + k;
    if (i >= n) break;
    dx[i] = static_cast<T>(((b >> k) & 1) ? static_cast<float>(dy[i]) * inv : 0.f);
  }
}

}  // namespace

#define TEB_DISPATCH(dtype, CALL)                     \
  switch (dtype) {                                    \
    case kFloat32: { using T = float; CALL; break; }  \
    case kFloat16: { using T = __half; CALL; break; } \
    default: { using T = __nv_bfloat16; CALL; }       \
  }

cudaError_t softmax_fwd(const SoftmaxArgs& a, cudaStream_t s) {
  if (a.rows == 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>((a.rows + 7) / 8);
  TEB_DISPATCH(a.dtype, (softmax_fwd_kernel<T><<<grid, 256, 0, s>>>(a)));
  return cudaGetLastError();
}
cudaError_t softmax_bwd(const SoftmaxArgs& a, cudaStream_t s) {
  if (a.rows == 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>((a.rows + 7) / 8);
  TEB_DISPATCH(a.dtype, (softmax_bwd_kernel<T><<<grid, 256, 0, s>>>(a)));
  return cudaGetLastError();
}
cudaError_t dropout_fwd(const void* x, void* y, uint8_t* mask_bits, int64_t n, int dtype, float p, uint64_t seed,
                        uint64_t offset, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>(((n + 7) / 8 + 255) / 256);
  TEB_DISPATCH(dtype, (dropout_fwd_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(y), mask_bits, n,
                                                                   p, seed, offset)));
  return cudaGetLastError();
}
cudaError_t dropout_bwd(const void* dy, const uint8_t* mask_bits, void* dx, int64_t n, int dtype, float p, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>(((n + 7) / 8 + 255) / 256);
  TEB_DISPATCH(dtype, (dropout_bwd_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(dy), mask_bits, static_cast<T*>(dx), n, p)));
  return cudaGetLastError();
}

}  // namespace teb200
