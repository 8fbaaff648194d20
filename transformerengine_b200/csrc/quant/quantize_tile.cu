// Tile quantizer with a fused element-wise producer.
//
// One CTA owns a 128x128 tile of the OUTPUT matrix.  In the row pass each thread
// produces 32 consecutive values of one row through the selected prologue
// (identity, norm-apply, activation, gated activation, or their gradients),
// rounds them to bf16 (so that fused and unfused pipelines agree bit for bit),
// quantizes them along the row and parks them in shared memory.  In the column
// pass each thread walks 32 rows of one column and emits the transposed,
// column-scaled copy.  Scales go straight to the 128x4-tile layout that the GEMM's
// tcgen05.cp expects, so no separate swizzle kernel runs.
//
// Covers the reference's MXFP8 cast kernels (common/cast/mxfp8/quantize_mxfp8.cuh:49,
// gated_mxfp8.cuh:57), per-tensor FP8 cast / cast-transpose (common/cast/fp8/
// quantize_fp8.cuh:58-252, common/transpose/cast_transpose.cu:104) and the
// activation kernels of common/activation with quantized output.
#include <cuda_fp8.h>
#include <teb200/api.h>
#include <teb200/ptx.cuh>
#include <teb200/quant.h>

namespace teb200 {
namespace {

constexpr int TR = 128, TC = 128, NT = 256;
constexpr int PITCH = TC + 8;  // bf16 elements

enum Mode : int { kModeMx = 0, kModeTensor = 1, kModeNone = 2 };

__device__ __forceinline__ uint8_t f32_to_e8m0_rp(float v) {
  uint16_t out;
  asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, 0.0, %1;" : "=h"(out) : "f"(v));
  return static_cast<uint8_t>(out & 0xFF);
}
__device__ __forceinline__ float e8m0_rcp(uint8_t e) {
  if (e == 255) return __int_as_float(0x7fffffff);
  if (e == 254) return __int_as_float(0x00400000);
  return __int_as_float((254 - static_cast<int>(e)) << 23);
}
__device__ __forceinline__ float e8m0_val(uint8_t e) {
  if (e == 255) return __int_as_float(0x7fffffff);
  if (e == 0) return __int_as_float(0x00400000);
  return __int_as_float(static_cast<int>(e) << 23);
}
__device__ __forceinline__ uint16_t cvt_fp8x2(float a, float b, int e5m2) {
  return e5m2 ? __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E5M2)
              : __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ size_t swizzled_sf_offset(int i, int j, int k_tiles) {
  return (static_cast<size_t>(i >> 7) * k_tiles + (j >> 2)) * 512 + (i & 31) * 16 + ((i & 127) >> 5) * 4 + (j & 3);
}

__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float act_fwd(float x, int act) {
  switch (act) {
    case kActGelu: return x * (0.5f + 0.5f * tanhf(x * (0.79788456f + 0.03567741f * x * x)));
    case kActSilu: return x * sigmoidf(x);
    case kActRelu: return fmaxf(x, 0.f);
    case kActQGelu: return x * sigmoidf(1.702f * x);
    case kActSRelu: return x > 0.f ? x * x : 0.f;
    default: return x;
  }
}
__device__ __forceinline__ float act_bwd(float x, int act) {
  switch (act) {
    case kActGelu: {
      const float t = tanhf(0.79788456f * x * (1.f + 0.044715f * x * x));
      return 0.5f * x * ((1.f - t * t) * (0.79788456f + 0.1070322243f * x * x)) + 0.5f * (1.f + t);
    }
    case kActSilu: {
      const float s = sigmoidf(x);
      return s * (1.f + x * (1.f - s));
    }
    case kActRelu: return x > 0.f ? 1.f : 0.f;
    case kActQGelu: {
      const float s = sigmoidf(1.702f * x);
      return s + 1.702f * x * s * (1.f - s);
    }
    case kActSRelu: return x > 0.f ? 2.f * x : 0.f;
    default: return 1.f;
  }
}

// load 32 consecutive elements as fp32
__device__ __forceinline__ void load32(const void* base, int dtype, size_t off, float (&v)[32]) {
  if (dtype == kFloat32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 t = p[i];
      v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + off);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 t = p[i];
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (dtype == kBFloat16) {
          v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
          v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        } else {
          const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
          v[8 * i + 2 * j] = __low2float(h);
          v[8 * i + 2 * j + 1] = __high2float(h);
        }
      }
    }
  }
}

__device__ __forceinline__ void produce32(const QuantArgs& a, int gr, int gc, float (&v)[32]) {
  switch (a.prologue) {
    case kProIdentity: load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v); break;
    case kProNorm: {
      load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
      float g[32];
      load32(a.gamma, a.gamma_dtype, gc, g);
      const float mu = a.mu ? a.mu[gr] : 0.f;
      const float rs = a.rs[gr];
      const float zc = a.zero_centered ? 1.f : 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = (v[i] - mu) * rs * (g[i] + zc);
      if (a.beta) {
        load32(a.beta, a.gamma_dtype, gc, g);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += g[i];
      }
      break;
    }
    case kProAct: {
      load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = act_fwd(v[i], a.act);
      break;
    }
    case kProGated: {
      float u[32];
      load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
      load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + a.C + gc, u);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = act_fwd(v[i], a.act) * u[i];
      break;
    }
    case kProDAct: {
      float d[32];
      load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
      load32(a.dy, a.x_dtype, static_cast<size_t>(gr) * a.C + gc, d);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = d[i] * act_bwd(v[i], a.act);
      break;
    }
    case kProDGated: {
      const int n = a.C / 2;
      const int c = gc < n ? gc : gc - n;
      float d[32], x1[32];
      load32(a.dy, a.x_dtype, static_cast<size_t>(gr) * n + c, d);
      load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + c, x1);
      if (gc < n) {
        float x2[32];
        load32(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + n + c, x2);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = d[i] * x2[i] * act_bwd(x1[i], a.act);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = d[i] * act_fwd(x1[i], a.act);
      }
      break;
    }
  }
  if (a.row_scale) {
    const float s = a.row_scale[gr];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= s;
  }
}

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  // values are non-negative: integer compare preserves order
  atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

template <int MODE>
__global__ void __launch_bounds__(NT) quantize_tile_kernel(const QuantArgs a) {
  __shared__ __align__(16) __nv_bfloat16 tile[TR * PITCH];
  __shared__ float red[NT / 32];
  const int tid = threadIdx.x;
  const int r0 = blockIdx.y * TR, c0 = blockIdx.x * TC;
  const bool want_col = a.col_data != nullptr || a.dbias != nullptr;
  const float tscale = (MODE == kModeTensor) ? *a.scale : 1.f;
  const float fmax_rcp = a.fp8_e5m2 ? (1.f / 57344.f) : (1.f / 448.f);
  float local_amax = 0.f;

  // ---------------------------------------------------------------- row pass
#pragma unroll 1
  for (int it = 0; it < (TR * TC / 32) / NT; ++it) {
    const int item = tid + it * NT;
    const int row = item >> 2, blk = item & 3;
    const int gr = r0 + row, gc = c0 + blk * 32;
    __nv_bfloat16* trow = tile + row * PITCH + blk * 32;
    if (gr < a.R && gc < a.C) {
      float v[32];
      produce32(a, gr, gc, v);
      uint32_t packed[16];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        packed[i] = *reinterpret_cast<const uint32_t*>(&h);
        v[2 * i] = __low2float(h);
        v[2 * i + 1] = __high2float(h);
        amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
      }
      if (want_col) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          reinterpret_cast<uint4*>(trow)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      }
      if (a.y != nullptr) {
        const size_t off = static_cast<size_t>(gr) * a.C + gc;
        if (a.y_dtype == kBFloat16) {
          uint4* yp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.y) + off);
#pragma unroll
          for (int i = 0; i < 4; ++i) yp[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        } else if (a.y_dtype == kFloat32) {
          float4* yp = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + off);
#pragma unroll
          for (int i = 0; i < 8; ++i) yp[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
          uint4* yp = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.y) + off);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            yp[i] = make_uint4(pack_f16x2(v[8 * i], v[8 * i + 1]), pack_f16x2(v[8 * i + 2], v[8 * i + 3]),
                               pack_f16x2(v[8 * i + 4], v[8 * i + 5]), pack_f16x2(v[8 * i + 6], v[8 * i + 7]));
          }
        }
      }
      local_amax = fmaxf(local_amax, amax);
      if (MODE != kModeNone && a.row_data != nullptr) {
        float mul;
        if (MODE == kModeMx) {
          const uint8_t e = f32_to_e8m0_rp(amax * fmax_rcp);
          mul = e8m0_rcp(e);
          a.row_scale_out[swizzled_sf_offset(gr, gc >> 5, ((a.C >> 5) + 3) >> 2)] = e;
        } else {
          mul = tscale;
        }
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t lo = cvt_fp8x2(v[4 * i] * mul, v[4 * i + 1] * mul, a.fp8_e5m2);
          const uint32_t hi = cvt_fp8x2(v[4 * i + 2] * mul, v[4 * i + 3] * mul, a.fp8_e5m2);
          q[i] = lo | (hi << 16);
        }
        uint4* qp = reinterpret_cast<uint4*>(a.row_data + static_cast<size_t>(gr) * a.C + gc);
        qp[0] = make_uint4(q[0], q[1], q[2], q[3]);
        qp[1] = make_uint4(q[4], q[5], q[6], q[7]);
      }
    } else if (want_col) {
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(trow)[i] = make_uint4(0, 0, 0, 0);
    }
  }

  if (a.amax != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_amax = fmaxf(local_amax, __shfl_xor_sync(0xffffffffu, local_amax, o));
    if ((tid & 31) == 0) red[tid >> 5] = local_amax;
  }
  __syncthreads();
  if (a.amax != nullptr && tid == 0) {
    float m = 0.f;
    for (int i = 0; i < NT / 32; ++i) m = fmaxf(m, red[i]);
    atomic_max_float(a.amax, m);
  }
  if (MODE == kModeTensor && a.scale_inv != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0)
    *a.scale_inv = 1.f / tscale;
  if (!want_col) return;

  // ---------------------------------------------------------------- column pass
#pragma unroll 1
  for (int it = 0; it < (TR * TC / 32) / NT; ++it) {
    const int item = tid + it * NT;
    const int col = item & (TC - 1), rb = item >> 7;
    const int gc = c0 + col, gr = r0 + rb * 32;
    if (gc >= a.C || gr >= a.R) continue;
    float v[32];
    float amax = 0.f, sum = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      v[i] = __bfloat162float(tile[(rb * 32 + i) * PITCH + col]);
      amax = fmaxf(amax, fabsf(v[i]));
      sum += v[i];
    }
    if (a.dbias != nullptr) atomicAdd(a.dbias + gc, sum);
    if (MODE == kModeNone || a.col_data == nullptr) continue;
    float mul;
    if (MODE == kModeMx) {
      const uint8_t e = f32_to_e8m0_rp(amax * fmax_rcp);
      mul = e8m0_rcp(e);
      a.col_scale_out[swizzled_sf_offset(gc, gr >> 5, ((a.R >> 5) + 3) >> 2)] = e;
    } else {
      mul = tscale;
    }
    uint32_t q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t lo = cvt_fp8x2(v[4 * i] * mul, v[4 * i + 1] * mul, a.fp8_e5m2);
      const uint32_t hi = cvt_fp8x2(v[4 * i + 2] * mul, v[4 * i + 3] * mul, a.fp8_e5m2);
      q[i] = lo | (hi << 16);
    }
    uint4* qp = reinterpret_cast<uint4*>(a.col_data + static_cast<size_t>(gc) * a.R + gr);
    qp[0] = make_uint4(q[0], q[1], q[2], q[3]);
    qp[1] = make_uint4(q[4], q[5], q[6], q[7]);
  }
}

template <int MODE>
cudaError_t launch_tile(const QuantArgs& a, cudaStream_t s) {
  if (a.R <= 0 || a.C <= 0) return cudaSuccess;
  if (a.R % 32 != 0 || a.C % 32 != 0) return cudaErrorInvalidValue;
  dim3 grid((a.C + TC - 1) / TC, (a.R + TR - 1) / TR);
  quantize_tile_kernel<MODE><<<grid, NT, 0, s>>>(a);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ simple element-wise kernels
template <typename OutT>
__global__ void dequant_mx_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf, int R, int C,
                                  int e5m2, OutT* __restrict__ out) {
  const int nblk = C >> 5;
  const size_t total = static_cast<size_t>(R) * nblk;
  const int k_tiles = (nblk + 3) >> 2;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(idx / nblk), b = static_cast<int>(idx % nblk);
    const float s = e8m0_val(sf[swizzled_sf_offset(r, b, k_tiles)]);
    const uint8_t* qp = q + static_cast<size_t>(r) * C + b * 32;
    OutT* op = out + static_cast<size_t>(r) * C + b * 32;
#pragma unroll 8
    for (int i = 0; i < 32; ++i) {
      const __half_raw h = __nv_cvt_fp8_to_halfraw(qp[i], e5m2 ? __NV_E5M2 : __NV_E4M3);
      op[i] = static_cast<OutT>(__half2float(__half(h)) * s);
    }
  }
}

template <typename OutT>
__global__ void dequant_tensor_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale_inv, int64_t n,
                                      int e5m2, OutT* __restrict__ out) {
  const float s = *scale_inv;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(q[i], e5m2 ? __NV_E5M2 : __NV_E4M3);
    out[i] = static_cast<OutT>(__half2float(__half(h)) * s);
  }
}

template <typename T>
__global__ void amax_kernel(const T* __restrict__ x, int64_t n, float* out) {
  float m = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    m = fmaxf(m, fabsf(static_cast<float>(x[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < static_cast<int>(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    atomic_max_float(out, m);
  }
}

__global__ void swizzle_kernel(const uint8_t* __restrict__ in, int rows, int cols, uint8_t* __restrict__ out,
                               int to_swizzled) {
  const int k_tiles = (cols + 3) >> 2;
  const size_t total = static_cast<size_t>(rows) * cols;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx / cols), j = static_cast<int>(idx % cols);
    const size_t so = swizzled_sf_offset(i, j, k_tiles);
    if (to_swizzled) out[so] = in[idx];
    else out[idx] = in[so];
  }
}

inline int grid_for(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  return static_cast<int>(g > 148 * 16 ? 148 * 16 : (g == 0 ? 1 : g));
}

}  // namespace

cudaError_t quantize_mxfp8(const QuantArgs& a, cudaStream_t s) { return launch_tile<kModeMx>(a, s); }
cudaError_t quantize_fp8_tensor(const QuantArgs& a, cudaStream_t s) { return launch_tile<kModeTensor>(a, s); }
cudaError_t apply_prologue(const QuantArgs& a, cudaStream_t s) { return launch_tile<kModeNone>(a, s); }

cudaError_t dequantize_mxfp8(const uint8_t* q, const uint8_t* sf, int R, int C, int e5m2, void* out, int out_dtype,
                             cudaStream_t s) {
  if (R <= 0 || C <= 0) return cudaSuccess;
  const int g = grid_for(static_cast<size_t>(R) * (C / 32), 256);
  if (out_dtype == kFloat32) dequant_mx_kernel<float><<<g, 256, 0, s>>>(q, sf, R, C, e5m2, static_cast<float*>(out));
  else if (out_dtype == kBFloat16)
    dequant_mx_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(q, sf, R, C, e5m2, static_cast<__nv_bfloat16*>(out));
  else dequant_mx_kernel<__half><<<g, 256, 0, s>>>(q, sf, R, C, e5m2, static_cast<__half*>(out));
  return cudaGetLastError();
}

cudaError_t dequantize_fp8_tensor(const uint8_t* q, const float* scale_inv, int64_t n, int e5m2, void* out,
                                  int out_dtype, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int g = grid_for(static_cast<size_t>(n), 256);
  if (out_dtype == kFloat32) dequant_tensor_kernel<float><<<g, 256, 0, s>>>(q, scale_inv, n, e5m2, static_cast<float*>(out));
  else if (out_dtype == kBFloat16)
    dequant_tensor_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(q, scale_inv, n, e5m2, static_cast<__nv_bfloat16*>(out));
  else dequant_tensor_kernel<__half><<<g, 256, 0, s>>>(q, scale_inv, n, e5m2, static_cast<__half*>(out));
  return cudaGetLastError();
}

cudaError_t amax_abs(const void* x, int dtype, int64_t n, float* out, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float), s);
  if (e != cudaSuccess || n <= 0) return e;
  const int g = grid_for(static_cast<size_t>(n), 512);
  if (dtype == kFloat32) amax_kernel<float><<<g, 512, 0, s>>>(static_cast<const float*>(x), n, out);
  else if (dtype == kBFloat16) amax_kernel<__nv_bfloat16><<<g, 512, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, out);
  else amax_kernel<__half><<<g, 512, 0, s>>>(static_cast<const __half*>(x), n, out);
  return cudaGetLastError();
}

cudaError_t swizzle_scales(const uint8_t* compact, int rows, int cols, uint8_t* out, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  swizzle_kernel<<<grid_for(static_cast<size_t>(rows) * cols, 256), 256, 0, s>>>(compact, rows, cols, out, 1);
  return cudaGetLastError();
}
cudaError_t unswizzle_scales(const uint8_t* swz, int rows, int cols, uint8_t* out, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  swizzle_kernel<<<grid_for(static_cast<size_t>(rows) * cols, 256), 256, 0, s>>>(swz, rows, cols, out, 0);
  return cudaGetLastError();
}

}  // namespace teb200
