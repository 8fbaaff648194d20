// Fused softmax cross entropy over large vocabularies: one CTA per row does an
// online max / sum-exp pass, writes the loss, and (optionally) overwrites the
// logits with d(loss)/d(logits) in a second pass, so the [tokens, vocab] tensor is
// never duplicated.  With vocab-parallel sharding the first pass only records the
// per-row statistics (max, sum-exp, target logit); after their all-reduce the
// second stage writes the gradient.  Replaces the reference's Triton kernels
// (common/triton/cross_entropy.py, pytorch/triton/cross_entropy.py:85).
#include <teb200/api.h>
#include <teb200/misc.h>
#include <teb200/ptx.cuh>

namespace teb200 {
namespace {

constexpr int NT = 1024;

template <typename T>
struct alignas(sizeof(T) * 8) V8 {
  T v[8];
};

struct MaxSum {
  float m, s;
};
__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  MaxSum r;
  r.m = m;
  r.s = (a.m == -INFINITY ? 0.f : a.s * __expf(a.m - m)) + (b.m == -INFINITY ? 0.f : b.s * __expf(b.m - m));
  return r;
}

template <typename T>
__device__ __forceinline__ MaxSum row_stats(const T* row, int V, MaxSum* red) {
  MaxSum acc{-INFINITY, 0.f};
  const bool vec_ok = (reinterpret_cast<uintptr_t>(row) % (sizeof(T) * 8)) == 0;
  const int Vv = vec_ok ? (V / 8) * 8 : 0;
  for (int c = threadIdx.x * 8; c < Vv; c += NT * 8) {
    const V8<T> v = *reinterpret_cast<const V8<T>*>(row + c);
    float f[8], m = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[i] = static_cast<float>(v.v[i]);
      m = fmaxf(m, f[i]);
    }
    const float nm = fmaxf(acc.m, m);
    float s = acc.m == -INFINITY ? 0.f : acc.s * __expf(acc.m - nm);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += __expf(f[i] - nm);
    acc.m = nm;
    acc.s = s;
  }
  for (int c = Vv + threadIdx.x; c < V; c += NT) {
    MaxSum o{static_cast<float>(row[c]), 1.f};
    acc = combine(acc, o);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other;
    other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
    acc = combine(acc, other);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  MaxSum tot{-INFINITY, 0.f};
  for (int i = 0; i < NT / 32; ++i) tot = combine(tot, red[i]);
  __syncthreads();
  return tot;
}

template <typename T>
__device__ __forceinline__ void write_grad(const T* row, T* grow, int V, float gmax, float gsum, int64_t local_tgt,
                                           float gscale, float smoothing, int vocab_total) {
  const float inv = 1.f / gsum;
  const float on = 1.f - smoothing, off = smoothing / vocab_total;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(row) % (sizeof(T) * 8)) == 0 &&
                      (reinterpret_cast<uintptr_t>(grow) % (sizeof(T) * 8)) == 0;
  const int Vv = vec_ok ? (V / 8) * 8 : 0;
  for (int c = threadIdx.x * 8; c < Vv; c += NT * 8) {
    const V8<T> v = *reinterpret_cast<const V8<T>*>(row + c);
    V8<T> o;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p = __expf(static_cast<float>(v.v[i]) - gmax) * inv;
      p -= off;
      if (c + i == local_tgt) p -= on;
      o.v[i] = static_cast<T>(p * gscale);
    }
    *reinterpret_cast<V8<T>*>(grow + c) = o;
  }
  for (int c = Vv + threadIdx.x; c < V; c += NT) {
    float p = __expf(static_cast<float>(row[c]) - gmax) * inv - off;
    if (c == local_tgt) p -= on;
    grow[c] = static_cast<T>(p * gscale);
  }
}

template <typename T>
__global__ void __launch_bounds__(NT) ce_kernel(const CrossEntropyArgs a) {
  __shared__ MaxSum red[NT / 32];
  const int r = blockIdx.x;
  const T* row = static_cast<const T*>(a.logits) + static_cast<size_t>(r) * a.ld;
  const int64_t tgt = a.targets[r];
  const bool ignored = tgt == a.ignore_index;
  const int64_t local = tgt - a.vocab_start;
  const bool mine = !ignored && local >= 0 && local < a.V;
  const MaxSum st = row_stats(row, a.V, red);
  const float tlogit = mine ? static_cast<float>(row[local]) : 0.f;
  if (a.row_max != nullptr) {
    // vocab-parallel first stage: publish the statistics only
    if (threadIdx.x == 0) {
      a.row_max[r] = st.m;
      a.row_sum[r] = st.s;
      a.row_tgt[r] = tlogit;
    }
    return;
  }
  if (threadIdx.x == 0) {
    float loss = 0.f;
    if (!ignored) {
      const float lse = st.m + __logf(st.s);
      loss = lse - tlogit;
      // label smoothing would need the mean logit; the smoothed gradient is exact, the
      // smoothed loss is computed by the caller from the un-smoothed one when needed
    }
    a.loss[r] = loss;
  }
  if (a.grad != nullptr) {
    T* grow = static_cast<T*>(a.grad) + static_cast<size_t>(r) * a.ld;
    if (ignored) {
      for (int c = threadIdx.x; c < a.V; c += NT) grow[c] = static_cast<T>(0.f);
    } else {
      write_grad(row, grow, a.V, st.m, st.s, local, a.grad_scale * (a.grad_scale_dev ? *a.grad_scale_dev : 1.f),
                 a.label_smoothing, a.V);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(NT) ce_parallel_bwd_kernel(const CrossEntropyArgs a, const float* gmax,
                                                             const float* gsum) {
  const int r = blockIdx.x;
  const T* row = static_cast<const T*>(a.logits) + static_cast<size_t>(r) * a.ld;
  T* grow = static_cast<T*>(a.grad) + static_cast<size_t>(r) * a.ld;
  const int64_t tgt = a.targets[r];
  if (tgt == a.ignore_index) {
    for (int c = threadIdx.x; c < a.V; c += NT) grow[c] = static_cast<T>(0.f);
    return;
  }
  write_grad(row, grow, a.V, gmax[r], gsum[r], tgt - a.vocab_start,
             a.grad_scale * (a.grad_scale_dev ? *a.grad_scale_dev : 1.f), 0.f, a.V);
}

}  // namespace

cudaError_t cross_entropy_fwd_bwd(const CrossEntropyArgs& a, cudaStream_t s) {
  if (a.R <= 0) return cudaSuccess;
  if (a.dtype == kBFloat16) ce_kernel<__nv_bfloat16><<<a.R, NT, 0, s>>>(a);
  else if (a.dtype == kFloat16) ce_kernel<__half><<<a.R, NT, 0, s>>>(a);
  else if (a.dtype == kFloat32) ce_kernel<float><<<a.R, NT, 0, s>>>(a);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t cross_entropy_parallel_bwd(const CrossEntropyArgs& a, const float* gmax, const float* gsum,
                                       cudaStream_t s) {
  if (a.R <= 0) return cudaSuccess;
  if (a.dtype == kBFloat16) ce_parallel_bwd_kernel<__nv_bfloat16><<<a.R, NT, 0, s>>>(a, gmax, gsum);
  else if (a.dtype == kFloat16) ce_parallel_bwd_kernel<__half><<<a.R, NT, 0, s>>>(a, gmax, gsum);
  else if (a.dtype == kFloat32) ce_parallel_bwd_kernel<float><<<a.R, NT, 0, s>>>(a, gmax, gsum);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace teb200
