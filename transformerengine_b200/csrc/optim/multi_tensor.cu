// Multi-tensor optimizer kernels: one launch updates up to kMtMaxTensors tensors of any size.
// The tensors are cut in chunks; a fixed grid strides over the chunks and finds each chunk's
// tensor in a prefix table passed by value in the kernel arguments (no device-side table upload,
// CUDA-graph friendly).
// Math follows the reference Adam functor (common/multi_tensor/adam.cu:124-143):
//   m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g ; denom = sqrt(v/bc2) + eps
//   AdamW: p -= lr*((m/bc1)/denom + wd*p) ; L2 mode adds wd*p to g first.
// The master copy (fp32) is updated and the model-dtype copy is refreshed in the
// same pass, so the step touches every byte once.
#include <teb200/api.h>
#include <teb200/misc.h>
#include <teb200/ptx.cuh>

namespace teb200 {
namespace {

constexpr int NT = 256;

// Chunk c -> tensor index (advancing ti; c only grows inside a block's loop) and the chunk's element range.
__device__ __forceinline__ bool mt_chunk(const MultiTensorTable& t, int c, int nchunks, int64_t chunk, int& ti,
                                         int64_t& start, int64_t& end) {
  if (c >= nchunks) return false;
  while (c >= t.chunk_start[ti + 1]) ++ti;
  start = static_cast<int64_t>(c - t.chunk_start[ti]) * chunk;
  const int64_t n = t.numel[ti];
  end = start + chunk < n ? start + chunk : n;
  return true;
}

template <typename T>
struct alignas(sizeof(T) * 4) V4 {
  T v[4];
};

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int64_t i) { return static_cast<float>(p[i]); }

template <typename G, typename P, typename S>
__global__ void __launch_bounds__(NT) adam_kernel(const __grid_constant__ MultiTensorTable t, const AdamArgs a,
                                                  const int nchunks) {
  if (a.noop != nullptr && *a.noop != 0) return;
  int ti = 0;
  int64_t start, end;
  for (int c = blockIdx.x; mt_chunk(t, c, nchunks, a.chunk, ti, start, end); c += gridDim.x) {
  const G* g = static_cast<const G*>(t.ptr[0][ti]);
  P* p = static_cast<P*>(t.ptr[1][ti]);
  S* m = static_cast<S*>(t.ptr[2][ti]);
  S* v = static_cast<S*>(t.ptr[3][ti]);
  float* master = a.has_master == 1 ? static_cast<float*>(t.ptr[4][ti]) : nullptr;
  int16_t* rem = a.has_master == 2 ? static_cast<int16_t*>(t.ptr[4][ti]) : nullptr;
  const float gs = a.grad_scale * (a.inv_scale_dev ? *a.inv_scale_dev : 1.f);
  const float b1 = a.beta1, b2 = a.beta2;
  float rbc1 = 1.f / a.bias_correction1, rbc2 = 1.f / a.bias_correction2;
  if (a.step_dev != nullptr && a.bias_correction) {
    const float st = static_cast<float>(*a.step_dev);
    rbc1 = 1.f / (1.f - powf(b1, st));
    rbc2 = 1.f / (1.f - powf(b2, st));
  }
  const float lr = a.lr_dev != nullptr ? *a.lr_dev : a.lr;
  // bf16 parameter + 16-bit remainder = the fp32 value, split so that the parameter is the fp32 value rounded
  // half up: a negative remainder means the high half was incremented
  auto join = [](uint16_t hi16, int16_t r) {
    uint32_t hi = hi16;
    if (r < 0) hi -= 1u;
    return __uint_as_float((hi << 16) | static_cast<uint16_t>(r));
  };
  auto split = [](float w, uint16_t& hi16, int16_t& r) {
    const uint32_t u = __float_as_uint(w);
    r = static_cast<int16_t>(u & 0xffffu);
    uint32_t nh = u >> 16;
    if (r < 0) nh += 1u;
    hi16 = static_cast<uint16_t>(nh);
  };
  if (rem != nullptr && sizeof(P) != 2) continue;  // remainders belong to 16-bit parameters (checked by the caller)
  // 4 elements per thread per iteration; tensors are 16-byte aligned and chunks are multiples of 4
  for (int64_t i = start + threadIdx.x * 4; i < end; i += NT * 4) {
    float gv[4], pv[4], mv[4], vv[4];
    const int cnt = end - i < 4 ? static_cast<int>(end - i) : 4;
    if (cnt == 4) {
      const V4<G> g4 = *reinterpret_cast<const V4<G>*>(g + i);
      const V4<S> m4 = *reinterpret_cast<const V4<S>*>(m + i);
      const V4<S> v4 = *reinterpret_cast<const V4<S>*>(v + i);
      if (master) {
        const V4<float> p4 = *reinterpret_cast<const V4<float>*>(master + i);
#pragma unroll
        for (int k = 0; k < 4; ++k) pv[k] = p4.v[k];
      } else if (rem) {
        const V4<uint16_t> h4 = *reinterpret_cast<const V4<uint16_t>*>(reinterpret_cast<const uint16_t*>(p) + i);
        const V4<int16_t> r4 = *reinterpret_cast<const V4<int16_t>*>(rem + i);
#pragma unroll
        for (int k = 0; k < 4; ++k) pv[k] = join(h4.v[k], r4.v[k]);
      } else {
        const V4<P> p4 = *reinterpret_cast<const V4<P>*>(p + i);
#pragma unroll
        for (int k = 0; k < 4; ++k) pv[k] = static_cast<float>(p4.v[k]);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        gv[k] = static_cast<float>(g4.v[k]) * gs;
        mv[k] = static_cast<float>(m4.v[k]);
        vv[k] = static_cast<float>(v4.v[k]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (k < cnt) {
          gv[k] = ldf(g, i + k) * gs;
          pv[k] = master ? master[i + k]
                         : (rem ? join(reinterpret_cast<const uint16_t*>(p)[i + k], rem[i + k]) : ldf(p, i + k));
          mv[k] = ldf(m, i + k);
          vv[k] = ldf(v, i + k);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k < cnt) {
        float gr = gv[k];
        if (!a.adamw) gr += a.weight_decay * pv[k];
        mv[k] = b1 * mv[k] + (1.f - b1) * gr;
        vv[k] = b2 * vv[k] + (1.f - b2) * gr * gr;
        const float denom = sqrtf(vv[k] * rbc2) + a.eps;
        float upd = (mv[k] * rbc1) / denom;
        if (a.adamw) upd += a.weight_decay * pv[k];
        pv[k] -= lr * upd;
      }
    }
    if (cnt == 4) {
      V4<S> m4, v4;
      V4<P> p4;
      V4<float> w4;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        m4.v[k] = static_cast<S>(mv[k]);
        v4.v[k] = static_cast<S>(vv[k]);
        p4.v[k] = static_cast<P>(pv[k]);
        w4.v[k] = pv[k];
      }
      *reinterpret_cast<V4<S>*>(m + i) = m4;
      *reinterpret_cast<V4<S>*>(v + i) = v4;
      if (master) *reinterpret_cast<V4<float>*>(master + i) = w4;
      if (rem) {
        V4<uint16_t> h4;
        V4<int16_t> r4;
#pragma unroll
        for (int k = 0; k < 4; ++k) split(pv[k], h4.v[k], r4.v[k]);
        *reinterpret_cast<V4<int16_t>*>(rem + i) = r4;
        *reinterpret_cast<V4<uint16_t>*>(reinterpret_cast<uint16_t*>(p) + i) = h4;
      } else {
        *reinterpret_cast<V4<P>*>(p + i) = p4;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (k < cnt) {
          m[i + k] = static_cast<S>(mv[k]);
          v[i + k] = static_cast<S>(vv[k]);
          if (master) master[i + k] = pv[k];
          if (rem) {
            uint16_t h;
            int16_t r;
            split(pv[k], h, r);
            rem[i + k] = r;
            reinterpret_cast<uint16_t*>(p)[i + k] = h;
          } else {
            p[i + k] = static_cast<P>(pv[k]);
          }
        }
      }
    }
  }
  }
}

template <typename G, typename P>
__global__ void __launch_bounds__(NT) sgd_kernel(const __grid_constant__ MultiTensorTable t, const SgdArgs a,
                                                 const int nchunks) {
  if (a.noop != nullptr && *a.noop != 0) return;
  int ti = 0;
  int64_t start, end;
  for (int c = blockIdx.x; mt_chunk(t, c, nchunks, a.chunk, ti, start, end); c += gridDim.x) {
  const G* g = static_cast<const G*>(t.ptr[0][ti]);
  P* p = static_cast<P*>(t.ptr[1][ti]);
  float* mom = static_cast<float*>(t.ptr[2][ti]);
  float* master = a.has_master ? static_cast<float*>(t.ptr[3][ti]) : nullptr;
  for (int64_t i = start + threadIdx.x; i < end; i += NT) {
    float gr = ldf(g, i) * a.grad_scale;
    float w = master ? master[i] : ldf(p, i);
    if (a.weight_decay != 0.f && !a.wd_after_momentum) gr += a.weight_decay * w;
    if (a.momentum != 0.f) {
      float b = a.first_run ? gr : mom[i] * a.momentum + (1.f - a.dampening) * gr;
      mom[i] = b;
      gr = a.nesterov ? gr + a.momentum * b : b;
    }
    if (a.weight_decay != 0.f && a.wd_after_momentum) gr += a.weight_decay * w;
    w -= a.lr * gr;
    if (master) master[i] = w;
    p[i] = static_cast<P>(w);
  }
  }
}

template <typename I, typename O>
__global__ void __launch_bounds__(NT) scale_kernel(const __grid_constant__ MultiTensorTable t, float scale, int* noop,
                                                   int64_t chunk, const int nchunks) {
  bool bad = false;
  int ti = 0;
  int64_t start, end;
  for (int c = blockIdx.x; mt_chunk(t, c, nchunks, chunk, ti, start, end); c += gridDim.x) {
    const I* in = static_cast<const I*>(t.ptr[0][ti]);
    O* out = static_cast<O*>(t.ptr[1][ti]);
    for (int64_t i = start + threadIdx.x; i < end; i += NT) {
      const float x = ldf(in, i);
      bad |= !isfinite(x);
      out[i] = static_cast<O>(x * scale);
    }
  }
  if (bad && noop != nullptr) *noop = 1;
}

template <typename T>
__global__ void __launch_bounds__(NT) l2norm_kernel(const __grid_constant__ MultiTensorTable t, float* out,
                                                    float* per_tensor, int tensor_base, int64_t chunk,
                                                    const int nchunks) {
  __shared__ float red[NT / 32];
  int ti = 0;
  int64_t start, end;
  for (int c = blockIdx.x; mt_chunk(t, c, nchunks, chunk, ti, start, end); c += gridDim.x) {
    const T* in = static_cast<const T*>(t.ptr[0][ti]);
    float s = 0.f;
    for (int64_t i = start + threadIdx.x; i < end; i += NT) {
      const float x = ldf(in, i);
      s += x * x;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int i = 0; i < NT / 32; ++i) tot += red[i];
      atomicAdd(out, tot);
      if (per_tensor != nullptr) atomicAdd(per_tensor + tensor_base + ti, tot);
    }
    __syncthreads();
  }
}

}  // namespace

// a few blocks per SM stride over all chunks of the launch
int mt_grid(int nchunks) {
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (sms[dev] == 0) {
    int n = 148;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    sms[dev] = n > 0 ? n : 148;
  }
  const int cap = sms[dev] * 6;
  return nchunks < cap ? nchunks : cap;
}

#define TEB_ADAM(G, P, S) adam_kernel<G, P, S><<<mt_grid(nchunks), NT, 0, s>>>(t, a, nchunks)

cudaError_t multi_tensor_adam(const MultiTensorTable& t, int nchunks, const AdamArgs& a, cudaStream_t s) {
  if (nchunks <= 0) return cudaSuccess;
  using bf = __nv_bfloat16;
  const int g = a.grad_dtype, p = a.param_dtype, st = a.state_dtype;
  if (st == kFloat32) {
    if (g == kBFloat16 && p == kBFloat16) TEB_ADAM(bf, bf, float);
    else if (g == kFloat32 && p == kBFloat16) TEB_ADAM(float, bf, float);
    else if (g == kFloat32 && p == kFloat32) TEB_ADAM(float, float, float);
    else if (g == kBFloat16 && p == kFloat32) TEB_ADAM(bf, float, float);
    else if (g == kFloat16 && p == kFloat16) TEB_ADAM(__half, __half, float);
    else if (g == kFloat32 && p == kFloat16) TEB_ADAM(float, __half, float);
    else return cudaErrorInvalidValue;
  } else if (st == kBFloat16) {
    if (g == kBFloat16 && p == kBFloat16) TEB_ADAM(bf, bf, bf);
    else if (g == kFloat32 && p == kBFloat16) TEB_ADAM(float, bf, bf);
    else if (g == kFloat32 && p == kFloat32) TEB_ADAM(float, float, bf);
    else return cudaErrorInvalidValue;
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t multi_tensor_sgd(const MultiTensorTable& t, int nchunks, const SgdArgs& a, cudaStream_t s) {
  if (nchunks <= 0) return cudaSuccess;
  using bf = __nv_bfloat16;
  if (a.grad_dtype == kFloat32 && a.param_dtype == kFloat32) sgd_kernel<float, float><<<mt_grid(nchunks), NT, 0, s>>>(t, a, nchunks);
  else if (a.grad_dtype == kBFloat16 && a.param_dtype == kBFloat16) sgd_kernel<bf, bf><<<mt_grid(nchunks), NT, 0, s>>>(t, a, nchunks);
  else if (a.grad_dtype == kFloat32 && a.param_dtype == kBFloat16) sgd_kernel<float, bf><<<mt_grid(nchunks), NT, 0, s>>>(t, a, nchunks);
  else if (a.grad_dtype == kFloat16 && a.param_dtype == kFloat16) sgd_kernel<__half, __half><<<mt_grid(nchunks), NT, 0, s>>>(t, a, nchunks);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t multi_tensor_scale(const MultiTensorTable& t, int nchunks, int in_dtype, int out_dtype, float scale,
                               int* noop, int64_t chunk, cudaStream_t s) {
  if (nchunks <= 0) return cudaSuccess;
  using bf = __nv_bfloat16;
#define TEB_SCALE(I, O) scale_kernel<I, O><<<mt_grid(nchunks), NT, 0, s>>>(t, scale, noop, chunk, nchunks)
  if (in_dtype == kFloat32 && out_dtype == kFloat32) TEB_SCALE(float, float);
  else if (in_dtype == kBFloat16 && out_dtype == kBFloat16) TEB_SCALE(bf, bf);
  else if (in_dtype == kBFloat16 && out_dtype == kFloat32) TEB_SCALE(bf, float);
  else if (in_dtype == kFloat32 && out_dtype == kBFloat16) TEB_SCALE(float, bf);
  else if (in_dtype == kFloat16 && out_dtype == kFloat16) TEB_SCALE(__half, __half);
  else if (in_dtype == kFloat16 && out_dtype == kFloat32) TEB_SCALE(__half, float);
  else if (in_dtype == kFloat32 && out_dtype == kFloat16) TEB_SCALE(float, __half);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t multi_tensor_l2norm_sq(const MultiTensorTable& t, int nchunks, int dtype, float* out, float* per_tensor,
                                   int tensor_base, int64_t chunk, cudaStream_t s) {
  if (nchunks <= 0) return cudaSuccess;
  if (dtype == kFloat32) l2norm_kernel<float><<<mt_grid(nchunks), NT, 0, s>>>(t, out, per_tensor, tensor_base, chunk, nchunks);
  else if (dtype == kBFloat16) l2norm_kernel<__nv_bfloat16><<<mt_grid(nchunks), NT, 0, s>>>(t, out, per_tensor, tensor_base, chunk, nchunks);
  else if (dtype == kFloat16) l2norm_kernel<__half><<<mt_grid(nchunks), NT, 0, s>>>(t, out, per_tensor, tensor_base, chunk, nchunks);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace teb200
