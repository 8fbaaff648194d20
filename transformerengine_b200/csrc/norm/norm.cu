// LayerNorm / RMSNorm forward statistics (+ optional high-precision output) and
// backward.  The quantized forward output is produced by the tile quantizer's
// norm prologue from the statistics computed here, so the normalised
// activations never make a round trip through HBM in 16-bit form.
// Reference kernels: common/normalization/layernorm/ln_fwd_kernels.cuh:26,
// ln_bwd_kernels.cuh:22-329, rmsnorm/rmsnorm_fwd_kernels.cuh:25,
// rmsnorm_bwd_kernels.cuh:53-327 (formulas in :96-120).
#include <teb200/api.h>
#include <teb200/norm.h>
#include <teb200/ptx.cuh>

namespace teb200 {
namespace {

constexpr int NT = 256;

template <typename T>
__device__ __forceinline__ float to_f(T v) { return static_cast<float>(v); }

template <typename T>
struct Vec8 {
  T v[8];
};
template <>
struct __align__(16) Vec8<__nv_bfloat16> { __nv_bfloat16 v[8]; };
template <>
struct __align__(16) Vec8<__half> { __half v[8]; };
template <>
struct __align__(32) Vec8<float> { float v[8]; };

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) s += red[i];
  return s;
}

// One CTA per row.  C must be a multiple of 8.
template <typename T, typename W, bool LN>
__global__ void __launch_bounds__(NT) norm_fwd_kernel(const T* __restrict__ x, const W* __restrict__ gamma,
                                                      const W* __restrict__ beta, T* __restrict__ y,
                                                      float* __restrict__ mu_out, float* __restrict__ rs_out, int R,
                                                      int C, float eps, int zero_centered) {
  __shared__ float red[NT / 32];
  const int row = blockIdx.x;
  const T* xr = x + static_cast<size_t>(row) * C;
  float mu = 0.f;
  if (LN) {
    float s = 0.f;
    for (int c = threadIdx.x * 8; c < C; c += NT * 8) {
      const Vec8<T> v = *reinterpret_cast<const Vec8<T>*>(xr + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += to_f(v.v[i]);
    }
    mu = block_sum(s, red) / C;
  }
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < C; c += NT * 8) {
    const Vec8<T> v = *reinterpret_cast<const Vec8<T>*>(xr + c);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float d = to_f(v.v[i]) - mu;
      ss += d * d;
    }
  }
  const float var = block_sum(ss, red) / C;
  const float rs = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (LN && mu_out) mu_out[row] = mu;
    rs_out[row] = rs;
  }
  if (y == nullptr) return;
  const float zc = zero_centered ? 1.f : 0.f;
  T* yr = y + static_cast<size_t>(row) * C;
  for (int c = threadIdx.x * 8; c < C; c += NT * 8) {
    const Vec8<T> v = *reinterpret_cast<const Vec8<T>*>(xr + c);
    const Vec8<W> g = *reinterpret_cast<const Vec8<W>*>(gamma + c);
    Vec8<T> o;
    if (LN && beta != nullptr) {
      const Vec8<W> b = *reinterpret_cast<const Vec8<W>*>(beta + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) o.v[i] = static_cast<T>((to_f(v.v[i]) - mu) * rs * (to_f(g.v[i]) + zc) + to_f(b.v[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) o.v[i] = static_cast<T>((to_f(v.v[i]) - mu) * rs * (to_f(g.v[i]) + zc));
    }
    *reinterpret_cast<Vec8<T>*>(yr + c) = o;
  }
}

// Persistent CTAs walk rows; each thread owns fixed columns so the per-CTA
// dgamma/dbeta partial sums live in shared memory without atomics.  Partials go
// to `ws` [gridDim.x, 2, C]; a second kernel reduces them in a fixed order.
template <typename T, typename W, bool LN>
__global__ void __launch_bounds__(NT) norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                      const float* __restrict__ mu_in,
                                                      const float* __restrict__ rs_in, const W* __restrict__ gamma,
                                                      const T* __restrict__ add, T* __restrict__ dx,
                                                      float* __restrict__ ws, int R, int C, int zero_centered) {
  extern __shared__ float sm[];
  float* dg = sm;          // [C]
  float* db = sm + C;      // [C] (LN only)
  __shared__ float red[NT / 32];
  for (int c = threadIdx.x; c < C; c += NT) {
    dg[c] = 0.f;
    if (LN) db[c] = 0.f;
  }
  const float zc = zero_centered ? 1.f : 0.f;
  for (int row = blockIdx.x; row < R; row += gridDim.x) {
    const T* xr = x + static_cast<size_t>(row) * C;
    const T* dr = dy + static_cast<size_t>(row) * C;
    const float mu = LN ? mu_in[row] : 0.f;
    const float rs = rs_in[row];
    float s1 = 0.f, s2 = 0.f;  // sum(dy*g*xhat), sum(dy*g)
    for (int c = threadIdx.x * 8; c < C; c += NT * 8) {
      const Vec8<T> xv = *reinterpret_cast<const Vec8<T>*>(xr + c);
      const Vec8<T> dv = *reinterpret_cast<const Vec8<T>*>(dr + c);
      const Vec8<W> g = *reinterpret_cast<const Vec8<W>*>(gamma + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (to_f(xv.v[i]) - mu) * rs;
        const float dg_ = to_f(dv.v[i]) * (to_f(g.v[i]) + zc);
        s1 += dg_ * xh;
        s2 += dg_;
      }
    }
    s1 = block_sum(s1, red) / C;
    if (LN) s2 = block_sum(s2, red) / C;
    T* dxr = dx + static_cast<size_t>(row) * C;
    for (int c = threadIdx.x * 8; c < C; c += NT * 8) {
      const Vec8<T> xv = *reinterpret_cast<const Vec8<T>*>(xr + c);
      const Vec8<T> dv = *reinterpret_cast<const Vec8<T>*>(dr + c);
      const Vec8<W> g = *reinterpret_cast<const Vec8<W>*>(gamma + c);
      Vec8<T> av;
      if (add != nullptr) av = *reinterpret_cast<const Vec8<T>*>(add + static_cast<size_t>(row) * C + c);
      Vec8<T> o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (to_f(xv.v[i]) - mu) * rs;
        const float d = to_f(dv.v[i]);
        const float dg_ = d * (to_f(g.v[i]) + zc);
        float r = rs * (dg_ - xh * s1 - (LN ? s2 : 0.f));
        if (add != nullptr) r += to_f(av.v[i]);
        o.v[i] = static_cast<T>(r);
        dg[c + i] += d * xh;
        if (LN) db[c + i] += d;
      }
      *reinterpret_cast<Vec8<T>*>(dxr + c) = o;
    }
  }
  __syncthreads();
  float* wrow = ws + static_cast<size_t>(blockIdx.x) * 2 * C;
  for (int c = threadIdx.x; c < C; c += NT) {
    wrow[c] = dg[c];
    wrow[C + c] = LN ? db[c] : 0.f;
  }
}

// Column sums of the per-part partial dgamma / dbeta.  One block owns 32 columns; its 16 thread rows walk the
// parts interleaved (128-byte coalesced loads), then combine through shared memory.
constexpr int FIN_COLS = 32, FIN_ROWS = 16;

template <typename W>
__global__ void __launch_bounds__(FIN_COLS * FIN_ROWS)
norm_bwd_finalize_kernel(const float* __restrict__ ws, int parts, int C, W* __restrict__ dgamma,
                         W* __restrict__ dbeta) {
  __shared__ float sg[FIN_ROWS][FIN_COLS + 1], sb[FIN_ROWS][FIN_COLS + 1];
  const int tx = threadIdx.x % FIN_COLS, ty = threadIdx.x / FIN_COLS;
  const int c = blockIdx.x * FIN_COLS + tx;
  float g = 0.f, b = 0.f;
  if (c < C) {
    for (int p = ty; p < parts; p += FIN_ROWS) {
      g += ws[static_cast<size_t>(p) * 2 * C + c];
      if (dbeta != nullptr) b += ws[static_cast<size_t>(p) * 2 * C + C + c];
    }
  }
  sg[ty][tx] = g;
  sb[ty][tx] = b;
  __syncthreads();
  if (ty == 0 && c < C) {
#pragma unroll
    for (int r = 1; r < FIN_ROWS; ++r) {
      g += sg[r][tx];
      b += sb[r][tx];
    }
    dgamma[c] = static_cast<W>(g);
    if (dbeta != nullptr) dbeta[c] = static_cast<W>(b);
  }
}

template <typename T, typename W>
cudaError_t fwd_t(const NormArgs& a, cudaStream_t s) {
  if (a.layernorm)
    norm_fwd_kernel<T, W, true><<<a.R, NT, 0, s>>>(static_cast<const T*>(a.x), static_cast<const W*>(a.gamma),
                                                    static_cast<const W*>(a.beta), static_cast<T*>(a.y), a.mu, a.rs,
                                                    a.R, a.C, a.eps, a.zero_centered);
  else
    norm_fwd_kernel<T, W, false><<<a.R, NT, 0, s>>>(static_cast<const T*>(a.x), static_cast<const W*>(a.gamma),
                                                     nullptr, static_cast<T*>(a.y), nullptr, a.rs, a.R, a.C, a.eps,
                                                     a.zero_centered);
  return cudaGetLastError();
}

template <typename T, typename W>
cudaError_t bwd_t(const NormArgs& a, cudaStream_t s) {
  const int parts = norm_bwd_parts(a.R);
  const size_t smem = static_cast<size_t>(a.C) * 2 * sizeof(float);
  cudaError_t e = cudaSuccess;
  if (a.layernorm) {
    if (smem > 48 * 1024)
      e = cudaFuncSetAttribute(norm_bwd_kernel<T, W, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    norm_bwd_kernel<T, W, true><<<parts, NT, smem, s>>>(
        static_cast<const T*>(a.dy), static_cast<const T*>(a.x), a.mu, a.rs, static_cast<const W*>(a.gamma),
        static_cast<const T*>(a.add), static_cast<T*>(a.dx), a.workspace, a.R, a.C, a.zero_centered);
  } else {
    if (smem > 48 * 1024)
      e = cudaFuncSetAttribute(norm_bwd_kernel<T, W, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    norm_bwd_kernel<T, W, false><<<parts, NT, smem, s>>>(
        static_cast<const T*>(a.dy), static_cast<const T*>(a.x), nullptr, a.rs, static_cast<const W*>(a.gamma),
        static_cast<const T*>(a.add), static_cast<T*>(a.dx), a.workspace, a.R, a.C, a.zero_centered);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  norm_bwd_finalize_kernel<W><<<(a.C + FIN_COLS - 1) / FIN_COLS, FIN_COLS * FIN_ROWS, 0, s>>>(a.workspace, parts, a.C, static_cast<W*>(a.dgamma),
                                                                a.layernorm ? static_cast<W*>(a.dbeta) : nullptr);
  return cudaGetLastError();
}

#define DISPATCH_TW(FN)                                                                  \
  if (a.x_dtype == kBFloat16 && a.w_dtype == kBFloat16) return FN<__nv_bfloat16, __nv_bfloat16>(a, s); \
  if (a.x_dtype == kBFloat16 && a.w_dtype == kFloat32) return FN<__nv_bfloat16, float>(a, s);          \
  if (a.x_dtype == kFloat16 && a.w_dtype == kFloat16) return FN<__half, __half>(a, s);                 \
  if (a.x_dtype == kFloat16 && a.w_dtype == kFloat32) return FN<__half, float>(a, s);                  \
  if (a.x_dtype == kFloat32 && a.w_dtype == kFloat32) return FN<float, float>(a, s);                   \
  return cudaErrorInvalidValue;

}  // namespace

int norm_bwd_parts(int R) {
  const int cap = 148 * 2;
  return R < cap ? (R > 0 ? R : 1) : cap;
}

cudaError_t norm_fwd(const NormArgs& a, cudaStream_t s) {
  if (a.R <= 0) return cudaSuccess;
  if (a.C % 8 != 0) return cudaErrorInvalidValue;
  DISPATCH_TW(fwd_t)
}

cudaError_t norm_bwd(const NormArgs& a, cudaStream_t s) {
  if (a.R <= 0) return cudaSuccess;
  if (a.C % 8 != 0 || a.workspace == nullptr) return cudaErrorInvalidValue;
  DISPATCH_TW(bwd_t)
}

}  // namespace teb200
