// Rotary position embedding, forward and backward, strided SBHD / BSHD input so it
// can run in place on the Q and K slices of a fused QKV projection output.
// out = x*cos + rot(x)*sin over the first d_rot dims, the rest is copied
// (reference: common/fused_rope/fused_rope.cu:39-92; context-parallel position
// remap for the dual-chunk split at :181-191).
#include <teb200/api.h>
#include <teb200/misc.h>
#include <teb200/ptx.cuh>

namespace teb200 {
namespace {

template <typename T>
__global__ void rope_kernel(const RopeArgs a) {
  extern __shared__ float cs[];  // cos[d_rot], sin[d_rot]
  const int si = blockIdx.x, bi = blockIdx.y;
  int pos = si;
  if (a.cp_size > 1) {
    const int half = a.s / 2;
    pos = si < half ? si + a.cp_rank * half : si + a.s * a.cp_size - (a.cp_rank + 1) * half - half;
  }
  pos += a.pos_offset + (a.start_positions ? a.start_positions[bi] : 0);
  for (int j = threadIdx.x; j < a.d_rot; j += blockDim.x) {
    float sn, c;
    sincosf(a.freqs[static_cast<size_t>(pos) * a.d_rot + j], &sn, &c);
    cs[j] = c;
    cs[a.d_rot + j] = sn;
  }
  __syncthreads();
  const T* x = static_cast<const T*>(a.x) + si * a.stride_s + bi * a.stride_b;
  T* out = static_cast<T*>(a.out) + si * a.stride_s + bi * a.stride_b;
  const int half = a.d_rot / 2;
  for (int idx = threadIdx.x; idx < a.h * a.d; idx += blockDim.x) {
    const int hi = idx / a.d, j = idx % a.d;
    const T* xh = x + hi * a.stride_h;
    float v = static_cast<float>(xh[j]);
    if (j < a.d_rot) {
      int jp;
      float sign;
      if (a.interleaved) {
        jp = (j & 1) ? j - 1 : j + 1;
        sign = (j & 1) ? 1.f : -1.f;
      } else {
        jp = j < half ? j + half : j - half;
        sign = j < half ? -1.f : 1.f;
      }
      const float other = static_cast<float>(xh[jp]);
      if (!a.backward) v = v * cs[j] + sign * other * cs[a.d_rot + j];
      else v = v * cs[j] - sign * other * cs[a.d_rot + jp];
    }
    // in-place: every thread reads both operands before any thread of this (s,b) writes
    reinterpret_cast<float*>(cs)[2 * a.d_rot + idx] = v;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < a.h * a.d; idx += blockDim.x) {
    const int hi = idx / a.d, j = idx % a.d;
    out[hi * a.stride_h + j] = static_cast<T>(cs[2 * a.d_rot + idx]);
  }
}

}  // namespace

cudaError_t rope_apply(const RopeArgs& a, cudaStream_t s) {
  if (a.s <= 0 || a.b <= 0) return cudaSuccess;
  const size_t smem = (2 * static_cast<size_t>(a.d_rot) + static_cast<size_t>(a.h) * a.d) * sizeof(float);
  dim3 grid(a.s, a.b);
  cudaError_t e = cudaSuccess;
#define TEB_ROPE(T)                                                                                       \
  do {                                                                                                    \
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(rope_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
    if (e != cudaSuccess) return e;                                                                       \
    rope_kernel<T><<<grid, 256, smem, s>>>(a);                                                            \
  } while (0)
  if (a.dtype == kBFloat16) TEB_ROPE(__nv_bfloat16);
  else if (a.dtype == kFloat16) TEB_ROPE(__half);
  else if (a.dtype == kFloat32) TEB_ROPE(float);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace teb200
