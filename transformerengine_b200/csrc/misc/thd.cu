// Packed-sequence ("thd") helpers: context-parallel token partitioning and softmax-state merging,
// thd <-> bshd conversion, and the KV-cache step (append the new tokens, gather every live
// sequence's keys / values into one packed tensor).  All are bandwidth-bound row movers: one CTA
// per token row (or a few), 16-byte accesses, the token -> sequence map found by binary search in
// the cumulative lengths.
// (Reference behaviour: common/fused_attn/context_parallel.cu, common/fused_attn/kv_cache.cu.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "teb200/misc.h"

namespace teb200 {
namespace {

// largest i in [0, nb) with cu[i] / div <= t
__device__ __forceinline__ int find_seq(const int* __restrict__ cu, int nb, int t, int div) {
  int lo = 0, hi = nb - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] / div <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ void copy_row(void* dst, const void* src, int row_bytes) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  for (int i = threadIdx.x; i < (row_bytes >> 4); i += blockDim.x) d[i] = s[i];
}

// ---------------------------------------------------------------------------- partition indices
__global__ void thd_partition_kernel(int* __restrict__ out, const int* __restrict__ cu, int nb, int n_local,
                                     int world, int rank) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n_local) return;
  const int i = find_seq(cu, nb, j, world);
  const int p = j - cu[i] / world;
  const int chunk = (cu[i + 1] - cu[i]) / (2 * world);
  out[j] = p < chunk ? cu[i] + rank * chunk + p : cu[i] + (2 * world - 1 - rank) * chunk + (p - chunk);
}

// token of the packed tensor that half-token j (of the chosen half of every sequence) refers to
__device__ __forceinline__ int half_token(const int* __restrict__ cu, int nb, int j, int half_idx) {
  const int i = find_seq(cu, nb, j, 2);
  const int p = j - cu[i] / 2;
  const int hl = (cu[i + 1] - cu[i]) / 2;
  return cu[i] + half_idx * hl + p;
}

// ---------------------------------------------------------------------------- read half tensor
__global__ void thd_read_half_kernel(void* __restrict__ half, const void* __restrict__ full, const int* __restrict__ cu,
                                     int nb, int t_half, int row_bytes, int half_idx) {
  const int j = blockIdx.x;
  const int tok = half_token(cu, nb, j, half_idx);
  const size_t lead = blockIdx.y;  // leading [2] of a stacked K/V tensor
  copy_row(static_cast<uint8_t*>(half) + (lead * t_half + j) * row_bytes,
           static_cast<const uint8_t*>(full) + (lead * 2 * t_half + tok) * row_bytes, row_bytes);
}

// ---------------------------------------------------------------------------- LSE of the second half
// mode 0: lse[h, tok] = logaddexp(lse[h, tok], half[h, j]);  mode 1: half[h, j] = lse[h, tok]
__global__ void thd_lse_half_kernel(float* __restrict__ lse, float* __restrict__ half, const int* __restrict__ cu,
                                    int nb, int heads, int t, int mode) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int t_half = t / 2;
  if (j >= t_half) return;
  const int tok = half_token(cu, nb, j, 1);
  for (int h = blockIdx.y; h < heads; h += gridDim.y) {
    float* a = lse + static_cast<size_t>(h) * t + tok;
    float* b = half + static_cast<size_t>(h) * t_half + j;
    if (mode == 1) {
      *b = *a;
    } else {
      const float x = *a, y = *b;
      const float m = fmaxf(x, y);
      *a = m == -INFINITY ? m : m + log1pf(expf(fminf(x, y) - m));
    }
  }
}

// ---------------------------------------------------------------------------- output correction
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

// out[tok, h, :] += step[j, h, :] * exp(lse_step[h, j] - lse[h, tok]); one CTA per (row j, head h)
template <typename T>
__global__ void thd_out_correction_kernel(T* __restrict__ out, const T* __restrict__ step,
                                          const float* __restrict__ lse, const float* __restrict__ lse_step,
                                          const int* __restrict__ cu, int nb, int heads, int d, int t, int t_step,
                                          int only_second_half) {
  const int j = blockIdx.x, h = blockIdx.y;
  const int tok = only_second_half ? half_token(cu, nb, j, 1) : j;
  const float ls = lse_step[static_cast<size_t>(h) * t_step + j];
  const float w = ls == -INFINITY ? 0.f : __expf(ls - lse[static_cast<size_t>(h) * t + tok]);  // empty partial result
  T* o = out + (static_cast<size_t>(tok) * heads + h) * d;
  const T* s = step + (static_cast<size_t>(j) * heads + h) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = from_f<T>(to_f<T>(o[c]) + to_f<T>(s[c]) * w);
}

// ---------------------------------------------------------------------------- gradient correction
// per half of every sequence: 0 leave, 1 copy, 2 add.  step holds all tokens (t_step == t) or only
// the tokens of the one active half (t_step == t / 2).
template <typename T>
__global__ void thd_grad_correction_kernel(T* __restrict__ grad, const T* __restrict__ step,
                                           const int* __restrict__ cu, int nb, int row, int t, int t_step,
                                           int mode_first, int mode_second) {
  const int tok = blockIdx.x;
  if (tok >= cu[nb]) return;  // padding after the last sequence
  const int i = find_seq(cu, nb, tok, 1);
  const int p = tok - cu[i];
  const int hl = (cu[i + 1] - cu[i]) / 2;
  const int second = p >= hl ? 1 : 0;
  const int mode = second ? mode_second : mode_first;
  if (mode == 0) return;
  const int src = t_step == t ? tok : cu[i] / 2 + (p - second * hl);
  const size_t lead = blockIdx.y;
  T* g = grad + (lead * t + tok) * row;
  const T* s = step + (lead * t_step + src) * row;
  for (int c = threadIdx.x; c < row; c += blockDim.x)
    g[c] = mode == 1 ? s[c] : from_f<T>(to_f<T>(g[c]) + to_f<T>(s[c]));
}

// ---------------------------------------------------------------------------- thd <-> bshd
// to_bshd = 1: padded[i, p] = packed[cu[i] + p];  else packed[cu[i] + p] = padded[i, p]
__global__ void thd_bshd_kernel(void* __restrict__ packed, void* __restrict__ padded, const int* __restrict__ cu, int nb,
                                int s_max, int row_bytes, int to_bshd) {
  const int tok = blockIdx.x;
  if (tok >= cu[nb]) return;
  const int i = find_seq(cu, nb, tok, 1);
  const int p = tok - cu[i];
  if (p >= s_max) return;
  uint8_t* a = static_cast<uint8_t*>(packed) + static_cast<size_t>(tok) * row_bytes;
  uint8_t* b = static_cast<uint8_t*>(padded) + (static_cast<size_t>(i) * s_max + p) * row_bytes;
  if (to_bshd) copy_row(b, a, row_bytes); else copy_row(a, b, row_bytes);
}

// ---------------------------------------------------------------------------- KV cache step
__global__ void kv_cache_step_kernel(KvCacheArgs a) {
  const int tok = blockIdx.x;  // row of the packed outputs
  const int i = find_seq(a.cu_kv, a.nb, tok, 1);
  const int p = tok - a.cu_kv[i];
  const int old = a.cu_kv[i + 1] - a.cu_kv[i] - (a.cu_new[i + 1] - a.cu_new[i]);
  const int pslot = p / a.page_size;
  const int page = pslot < a.width ? a.page_table[i * a.width + pslot] : -1;
  if (page < 0 || page >= a.num_pages || old < 0) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, 31);  // inconsistent page table / lengths
    return;
  }
  const size_t slot = static_cast<size_t>(page) * a.page_size + p % a.page_size;
  for (int which = 0; which < 2; ++which) {
    const int rb = which ? a.row_bytes_v : a.row_bytes_k;
    uint8_t* cache = static_cast<uint8_t*>(which ? a.cache_v : a.cache_k) + slot * rb;
    uint8_t* out = static_cast<uint8_t*>(which ? a.out_v : a.out_k) + static_cast<size_t>(tok) * rb;
    if (p >= old) {
      const uint8_t* src = static_cast<const uint8_t*>(which ? a.new_v : a.new_k) +
                           static_cast<size_t>(a.cu_new[i] + p - old) * rb;
      const uint4* s = reinterpret_cast<const uint4*>(src);
      for (int c = threadIdx.x; c < (rb >> 4); c += blockDim.x) {
        const uint4 v = s[c];
        reinterpret_cast<uint4*>(cache)[c] = v;
        reinterpret_cast<uint4*>(out)[c] = v;
      }
    } else {
      copy_row(out, cache, rb);
    }
  }
}

}  // namespace

cudaError_t thd_partition_indices(int* out, const int* cu, int nb, int total_tokens, int world, int rank,
                                  cudaStream_t s) {
  if (nb < 1 || world < 1 || rank < 0 || rank >= world || total_tokens % (2 * world)) return cudaErrorInvalidValue;
  const int n = total_tokens / world;
  if (n == 0) return cudaSuccess;
  thd_partition_kernel<<<(n + 255) / 256, 256, 0, s>>>(out, cu, nb, n, world, rank);
  return cudaGetLastError();
}

cudaError_t thd_read_half(void* half, const void* full, const int* cu, int nb, int t, int lead, int row_bytes,
                          int half_idx, cudaStream_t s) {
  if (row_bytes % 16 || t % 2 || nb < 1 || half_idx < 0 || half_idx > 1 || lead < 1) return cudaErrorInvalidValue;
  if (t == 0) return cudaSuccess;
  thd_read_half_kernel<<<dim3(t / 2, lead), 128, 0, s>>>(half, full, cu, nb, t / 2, row_bytes, half_idx);
  return cudaGetLastError();
}

cudaError_t thd_lse_half(float* lse, float* half, const int* cu, int nb, int heads, int t, int mode, cudaStream_t s) {
  if (t % 2 || nb < 1 || heads < 1) return cudaErrorInvalidValue;
  if (t == 0) return cudaSuccess;
  thd_lse_half_kernel<<<dim3((t / 2 + 127) / 128, heads < 64 ? heads : 64), 128, 0, s>>>(lse, half, cu, nb, heads, t, mode);
  return cudaGetLastError();
}

cudaError_t thd_out_correction(void* out, const void* step, const float* lse, const float* lse_step, const int* cu,
                               int nb, int heads, int d, int t, int only_second_half, int dtype, cudaStream_t s) {
  if (nb < 1 || t % 2 || heads < 1 || heads > 65535) return cudaErrorInvalidValue;
  const int t_step = only_second_half ? t / 2 : t;
  if (t_step == 0) return cudaSuccess;
  const dim3 grid(t_step, heads);
  if (dtype == 0)
    thd_out_correction_kernel<float><<<grid, 128, 0, s>>>(static_cast<float*>(out), static_cast<const float*>(step), lse,
                                                         lse_step, cu, nb, heads, d, t, t_step, only_second_half);
  else if (dtype == 2)
    thd_out_correction_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(static_cast<__nv_bfloat16*>(out),
                                                                 static_cast<const __nv_bfloat16*>(step), lse, lse_step,
                                                                 cu, nb, heads, d, t, t_step, only_second_half);
  else if (dtype == 1)
    thd_out_correction_kernel<__half><<<grid, 128, 0, s>>>(static_cast<__half*>(out), static_cast<const __half*>(step),
                                                          lse, lse_step, cu, nb, heads, d, t, t_step, only_second_half);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t thd_grad_correction(void* grad, const void* step, const int* cu, int nb, int lead, int row, int t,
                                int t_step, int mode_first, int mode_second, int dtype, cudaStream_t s) {
  if (nb < 1 || t % 2 || (t_step != t && t_step != t / 2) || lead < 1) return cudaErrorInvalidValue;
  if (t_step != t && mode_first != 0 && mode_second != 0) return cudaErrorInvalidValue;
  if (t == 0) return cudaSuccess;
  const dim3 grid(t, lead);
  if (dtype == 0)
    thd_grad_correction_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(grad), static_cast<const float*>(step), cu,
                                                          nb, row, t, t_step, mode_first, mode_second);
  else if (dtype == 2)
    thd_grad_correction_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(grad),
                                                                  static_cast<const __nv_bfloat16*>(step), cu, nb, row,
                                                                  t, t_step, mode_first, mode_second);
  else if (dtype == 1)
    thd_grad_correction_kernel<__half><<<grid, 256, 0, s>>>(static_cast<__half*>(grad), static_cast<const __half*>(step),
                                                           cu, nb, row, t, t_step, mode_first, mode_second);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t thd_bshd_convert(void* packed, void* padded, const int* cu, int nb, int t, int s_max, int row_bytes,
                             int to_bshd, cudaStream_t s) {
  if (row_bytes % 16 || nb < 1 || s_max < 1) return cudaErrorInvalidValue;
  if (t == 0) return cudaSuccess;
  thd_bshd_kernel<<<t, 128, 0, s>>>(packed, padded, cu, nb, s_max, row_bytes, to_bshd);
  return cudaGetLastError();
}

cudaError_t kv_cache_step(const KvCacheArgs& a, cudaStream_t s) {
  if (a.row_bytes_k % 16 || a.row_bytes_v % 16 || a.nb < 1 || a.width < 1 || a.page_size < 1 || a.num_pages < 1)
    return cudaErrorInvalidValue;
  if (a.total == 0) return cudaSuccess;
  kv_cache_step_kernel<<<a.total, 128, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace teb200
