// MoE routing kernels: score function + top-k (+ expert bias, scaling, per-expert token counts,
// full scores for the auxiliary loss) with its backward, and the row gather/scatter that groups
// tokens expert-major and merges expert outputs back with their routing weights.
// (Reference behaviour: common/fused_router/fused_topk_with_score_function.cu,
//  common/fused_router/fused_moe_aux_loss.cu, common/permutation/permutation.cu.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "teb200/api.h"
#include "teb200/misc.h"

namespace teb200 {
namespace {

constexpr int kMaxPerLane = 8;  // experts per lane: E <= 256
constexpr float kNegInf = -3.0e38f;

template <typename T>
__device__ __forceinline__ float ld(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
template <>
__device__ __forceinline__ float ld<__half>(const __half* p, size_t i) { return __half2float(p[i]); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float score_of(float l, int fn) {
  if (fn == 0) return 1.f / (1.f + __expf(-l));
  const float sp = l > 20.f ? l : log1pf(__expf(l));  // softplus
  return sqrtf(sp);
}

// One warp per token.  Lane i owns experts i, i+32, ...
template <typename T>
__global__ void router_fwd_kernel(RouterArgs a) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= a.T) return;
  const T* lg = static_cast<const T*>(a.logits) + static_cast<size_t>(t) * a.E;
  float l[kMaxPerLane], s[kMaxPerLane], sel[kMaxPerLane];
  bool taken[kMaxPerLane];
  float mx = kNegInf;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    l[i] = e < a.E ? ld<T>(lg, e) : kNegInf;
    taken[i] = false;
    mx = fmaxf(mx, l[i]);
  }
  mx = warp_max(mx);
  if (a.score_fn == 1) {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      s[i] = lane + 32 * i < a.E ? __expf(l[i] - mx) : 0.f;
      sum += s[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      s[i] *= inv;                                   // full softmax (used by pre-softmax and by the aux loss)
      sel[i] = a.use_pre_softmax ? s[i] : l[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < a.E ? score_of(l[i], a.score_fn) : 0.f;
      sel[i] = s[i] + (a.expert_bias != nullptr && e < a.E ? a.expert_bias[e] : 0.f);
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i)
    if (lane + 32 * i >= a.E) sel[i] = kNegInf;
  // top-k by repeated arg-max (ties: lowest expert index)
  int picked_e[8];
  float picked_raw[8];
  for (int k = 0; k < a.topk; ++k) {
    float best = kNegInf;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (!taken[i] && e < a.E && (sel[i] > best || (sel[i] == best && e < best_e))) { best = sel[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    picked_e[k] = best_e;
    // raw value that becomes the probability: softmax -> logit (post) or prob (pre); others -> score without bias
    const int own_lane = best_e & 31, own_i = best_e >> 5;
    float raw = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (i == own_i && lane == own_lane) {
        taken[i] = true;
        raw = (a.score_fn == 1 && !a.use_pre_softmax) ? l[i] : s[i];
      }
    picked_raw[k] = __shfl_sync(0xffffffffu, raw, own_lane);
  }
  // normalise the picked values
  float w[8];
  if (a.score_fn == 1 && !a.use_pre_softmax) {
    float m2 = kNegInf, sum = 0.f;
    for (int k = 0; k < a.topk; ++k) m2 = fmaxf(m2, picked_raw[k]);
    for (int k = 0; k < a.topk; ++k) { w[k] = __expf(picked_raw[k] - m2); sum += w[k]; }
    for (int k = 0; k < a.topk; ++k) w[k] /= sum;
  } else if (a.score_fn != 1 && a.topk > 1) {
    float sum = 0.f;
    for (int k = 0; k < a.topk; ++k) sum += picked_raw[k];
    for (int k = 0; k < a.topk; ++k) w[k] = picked_raw[k] / (sum + 1e-20f);
  } else {
    for (int k = 0; k < a.topk; ++k) w[k] = picked_raw[k];
  }
  for (int k = 0; k < a.topk; ++k) w[k] *= a.scaling_factor;
  // outputs
  float* pr = a.probs + static_cast<size_t>(t) * a.E;
  uint8_t* rm = a.routing_map + static_cast<size_t>(t) * a.E;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    if (e < a.E) {
      float pv = 0.f;
      for (int k = 0; k < a.topk; ++k)
        if (picked_e[k] == e) pv = w[k];
      pr[e] = pv;
      rm[e] = taken[i] ? 1 : 0;
      if (a.scores != nullptr) {
        float sc = s[i];
        a.scores[static_cast<size_t>(t) * a.E + e] = sc;
      }
      if (taken[i] && a.tokens_per_expert != nullptr) atomicAdd(a.tokens_per_expert + e, 1);
    }
  }
  if (lane < a.topk) {
    if (a.topk_idx != nullptr) a.topk_idx[static_cast<size_t>(t) * a.topk + lane] = picked_e[lane];
    if (a.topk_w != nullptr) a.topk_w[static_cast<size_t>(t) * a.topk + lane] = w[lane];
  }
}

// Backward through the kept probabilities (selection itself is not differentiated).
template <typename T>
__global__ void router_bwd_kernel(RouterArgs a, const float* __restrict__ gprobs, T* __restrict__ glogits) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= a.T) return;
  const T* lg = static_cast<const T*>(a.logits) + static_cast<size_t>(t) * a.E;
  const uint8_t* rm = a.routing_map + static_cast<size_t>(t) * a.E;
  const float* gp = gprobs + static_cast<size_t>(t) * a.E;
  float l[kMaxPerLane], g[kMaxPerLane];
  bool on[kMaxPerLane];
  float mx = kNegInf, mx_sel = kNegInf;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    const bool in = e < a.E;
    l[i] = in ? ld<T>(lg, e) : kNegInf;
    on[i] = in && rm[e] != 0;
    g[i] = on[i] ? gp[e] * a.scaling_factor : 0.f;
    mx = fmaxf(mx, l[i]);
    if (on[i]) mx_sel = fmaxf(mx_sel, l[i]);
  }
  mx = warp_max(mx);
  mx_sel = warp_max(mx_sel);
  float out[kMaxPerLane];
  if (a.score_fn == 1) {
    // softmax over all experts (pre) or over the selected ones (post): dl = p * (g - sum g p)
    const bool pre = a.use_pre_softmax != 0;
    float p[kMaxPerLane], sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const bool part = pre ? (lane + 32 * i < a.E) : on[i];
      p[i] = part ? __expf(l[i] - (pre ? mx : mx_sel)) : 0.f;
      sum += p[i];
    }
    sum = warp_sum(sum);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) { p[i] /= sum; dot += g[i] * p[i]; }
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) out[i] = p[i] * (g[i] - dot);
  } else {
    // v_k = s_k / (sum_sel s + eps) (topk > 1) or s_k;  ds/dl: sigmoid s(1-s), sqrt-softplus sigmoid(l)/(2s)
    float s[kMaxPerLane], ssum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      s[i] = on[i] ? score_of(l[i], a.score_fn) : 0.f;
      ssum += s[i];
    }
    ssum = warp_sum(ssum);
    float dot = 0.f;
    const float denom = ssum + 1e-20f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) dot += g[i] * s[i];
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      float ds = g[i];
      if (a.topk > 1) ds = on[i] ? (g[i] - dot / denom) / denom : 0.f;
      float dsdl = 0.f;
      if (on[i]) {
        const float sg = 1.f / (1.f + __expf(-l[i]));
        dsdl = a.score_fn == 0 ? sg * (1.f - sg) : sg / (2.f * fmaxf(s[i], 1e-20f));
      }
      out[i] = ds * dsdl;
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    if (e < a.E) glogits[static_cast<size_t>(t) * a.E + e] = static_cast<T>(out[i]);
  }
}

// ------------------------------------------------------------------------------ row movement
// one block per (token, slot); 16-byte vectors
__global__ void permute_rows_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                    const int32_t* __restrict__ dest_row, const float* __restrict__ probs,
                                    float* __restrict__ probs_out, int T, int slots, int vec_per_row) {
  const long long pair = blockIdx.x;
  const int t = static_cast<int>(pair / slots);
  const int d = dest_row[pair];
  if (d < 0) return;
  const uint4* src = in + static_cast<size_t>(t) * vec_per_row;
  uint4* dst = out + static_cast<size_t>(d) * vec_per_row;
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
  if (probs != nullptr && threadIdx.x == 0) probs_out[d] = probs[pair];
}

template <typename T>
__global__ void unpermute_rows_kernel(const T* __restrict__ in, T* __restrict__ out,
                                      const int32_t* __restrict__ dest_row, const float* __restrict__ w, int T_, int slots,
                                      int H) {
  const int t = blockIdx.x;
  for (int h = threadIdx.x * 2; h < H; h += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int k = 0; k < slots; ++k) {
      const int d = dest_row[static_cast<size_t>(t) * slots + k];
      if (d < 0) continue;
      const float wk = w != nullptr ? w[static_cast<size_t>(t) * slots + k] : 1.f;
      a0 += wk * static_cast<float>(in[static_cast<size_t>(d) * H + h]);
      a1 += wk * static_cast<float>(in[static_cast<size_t>(d) * H + h + 1]);
    }
    out[static_cast<size_t>(t) * H + h] = static_cast<T>(a0);
    out[static_cast<size_t>(t) * H + h + 1] = static_cast<T>(a1);
  }
}

// 16-bit rows with 16-byte vectors: one thread sums 8 adjacent elements over the slots
template <bool BF>
__global__ void unpermute_rows_vec_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                          const int32_t* __restrict__ dest_row, const float* __restrict__ w, int slots,
                                          int vec_per_row) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < slots; ++k) {
      const int d = dest_row[static_cast<size_t>(t) * slots + k];
      if (d < 0) continue;
      const float wk = w != nullptr ? w[static_cast<size_t>(t) * slots + k] : 1.f;
      const uint4 v = in[static_cast<size_t>(d) * vec_per_row + i];
      const uint32_t* w32 = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float lo, hi;
        if (BF) {
          lo = __uint_as_float(w32[j] << 16);
          hi = __uint_as_float(w32[j] & 0xffff0000u);
        } else {
          const __half2 h = *reinterpret_cast<const __half2*>(&w32[j]);
          lo = __low2float(h);
          hi = __high2float(h);
        }
        acc[2 * j] += wk * lo;
        acc[2 * j + 1] += wk * hi;
      }
    }
    uint4 o;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (BF) {
        const __nv_bfloat162 b2 = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        o32[j] = *reinterpret_cast<const uint32_t*>(&b2);
      } else {
        const __half2 h2 = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        o32[j] = *reinterpret_cast<const uint32_t*>(&h2);
      }
    }
    out[static_cast<size_t>(t) * vec_per_row + i] = o;
  }
}

// dest rows of an index routing [T, topk]: stable expert-major order with per-expert padding.
// Single block: counts, exclusive scan, then a serial-in-token assignment per expert lane.
__global__ void build_dest_rows_kernel(const int32_t* __restrict__ topk_idx, int T, int topk, int E, int align,
                                       int32_t* counts, int32_t* offsets, int32_t* dest_row) {
  extern __shared__ int32_t sh[];  // [E] counts, [E+1] offsets
  int32_t* c = sh;
  int32_t* off = sh + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) c[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < T * topk; i += blockDim.x) atomicAdd(&c[topk_idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = acc;
      acc += (c[e] + align - 1) / align * align;
    }
    off[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = off[e];
    if (e < E) counts[e] = c[e];
  }
  // expert e's rows in token order: one thread per expert walks the routing
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int pos = off[e];
    for (int i = 0; i < T * topk; ++i)
      if (topk_idx[i] == e) dest_row[i] = pos++;
  }
}

}  // namespace

cudaError_t router_topk_fwd(const RouterArgs& a, cudaStream_t s) {
  if (a.E > 32 * kMaxPerLane || a.topk > 8 || a.topk < 1 || a.num_groups > 1) return cudaErrorInvalidValue;
  if (a.T == 0) return cudaSuccess;
  if (a.tokens_per_expert != nullptr) {
    cudaError_t e = cudaMemsetAsync(a.tokens_per_expert, 0, sizeof(int32_t) * a.E, s);
    if (e != cudaSuccess) return e;
  }
  const int warps = 8;
  const int grid = (a.T + warps - 1) / warps;
  switch (a.dtype) {
    case kFloat32: router_fwd_kernel<float><<<grid, warps * 32, 0, s>>>(a); break;
    case kFloat16: router_fwd_kernel<__half><<<grid, warps * 32, 0, s>>>(a); break;
    default: router_fwd_kernel<__nv_bfloat16><<<grid, warps * 32, 0, s>>>(a);
  }
  return cudaGetLastError();
}

cudaError_t router_topk_bwd(const RouterArgs& a, const float* grad_probs, void* grad_logits, cudaStream_t s) {
  if (a.E > 32 * kMaxPerLane) return cudaErrorInvalidValue;
  if (a.T == 0) return cudaSuccess;
  const int warps = 8;
  const int grid = (a.T + warps - 1) / warps;
  switch (a.dtype) {
    case kFloat32: router_bwd_kernel<float><<<grid, warps * 32, 0, s>>>(a, grad_probs, static_cast<float*>(grad_logits)); break;
    case kFloat16: router_bwd_kernel<__half><<<grid, warps * 32, 0, s>>>(a, grad_probs, static_cast<__half*>(grad_logits)); break;
    default:
      router_bwd_kernel<__nv_bfloat16><<<grid, warps * 32, 0, s>>>(a, grad_probs, static_cast<__nv_bfloat16*>(grad_logits));
  }
  return cudaGetLastError();
}

cudaError_t permute_rows(const void* in, void* out, const int32_t* dest_row, const float* probs, float* probs_out, int T,
                         int topk, int H, int dtype, cudaStream_t s) {
  const size_t row_bytes = static_cast<size_t>(H) * dtype_size(dtype);
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return cudaErrorInvalidValue;
  if (T == 0 || topk == 0) return cudaSuccess;
  permute_rows_kernel<<<static_cast<unsigned>(static_cast<long long>(T) * topk), 128, 0, s>>>(
      static_cast<const uint4*>(in), static_cast<uint4*>(out), dest_row, probs, probs_out, T, topk,
      static_cast<int>(row_bytes / 16));
  return cudaGetLastError();
}

cudaError_t unpermute_rows(const void* in, void* out, const int32_t* dest_row, const float* w, int T, int topk, int H,
                           int dtype, cudaStream_t s) {
  if (H % 2 != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  if (dtype != kFloat32 && H % 8 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    if (dtype == kBFloat16)
      unpermute_rows_vec_kernel<true><<<T, 256, 0, s>>>(static_cast<const uint4*>(in), static_cast<uint4*>(out), dest_row, w, topk, H / 8);
    else
      unpermute_rows_vec_kernel<false><<<T, 256, 0, s>>>(static_cast<const uint4*>(in), static_cast<uint4*>(out), dest_row, w, topk, H / 8);
    return cudaGetLastError();
  }
  switch (dtype) {
    case kFloat32:
      unpermute_rows_kernel<float><<<T, 256, 0, s>>>(static_cast<const float*>(in), static_cast<float*>(out), dest_row, w, T, topk, H);
      break;
    case kFloat16:
      unpermute_rows_kernel<__half><<<T, 256, 0, s>>>(static_cast<const __half*>(in), static_cast<__half*>(out), dest_row, w, T, topk, H);
      break;
    default:
      unpermute_rows_kernel<__nv_bfloat16><<<T, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in),
                                                              static_cast<__nv_bfloat16*>(out), dest_row, w, T, topk, H);
  }
  return cudaGetLastError();
}

cudaError_t build_dest_rows(const int32_t* topk_idx, int T, int topk, int E, int align, int32_t* counts, int32_t* offsets,
                            int32_t* dest_row, cudaStream_t s) {
  if (E > 4096 || align < 1) return cudaErrorInvalidValue;
  build_dest_rows_kernel<<<1, 256, sizeof(int32_t) * (2 * E + 1), s>>>(topk_idx, T, topk, E, align, counts, offsets, dest_row);
  return cudaGetLastError();
}

}  // namespace teb200
