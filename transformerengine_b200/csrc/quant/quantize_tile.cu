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

__device__ __forceinline__ float sigmoidf(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
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

// load 8 consecutive elements as fp32
__device__ __forceinline__ void load8(const void* base, int dtype, size_t off, float (&v)[8]) {
  if (dtype == kFloat32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    const float4 a = p[0], b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 t = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + off);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (dtype == kBFloat16) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
        v[2 * j] = __low2float(h);
        v[2 * j + 1] = __high2float(h);
      }
    }
  }
}

// Produce 8 consecutive output values of row gr starting at column gc.
// PRO / ACT are compile-time so that the loads of the four chunks of a thread can be hoisted
// ahead of the math; ACT < 0 reads the activation id at run time.
template <int PRO, int ACT>
__device__ __forceinline__ void produce8(const QuantArgs& a, int gr, int gc, float (&v)[8]) {
  const int act = ACT >= 0 ? ACT : a.act;
  switch (PRO) {
    case kProIdentity: load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v); break;
    case kProNorm: {
      load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
      float g[8];
      load8(a.gamma, a.gamma_dtype, gc, g);
      const float mu = a.mu ? a.mu[gr] : 0.f;
      const float rs = a.rs[gr];
      const float zc = a.zero_centered ? 1.f : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (v[i] - mu) * rs * (g[i] + zc);
      if (a.beta) {
        load8(a.beta, a.gamma_dtype, gc, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += g[i];
      }
      break;
    }
    case kProAct: {
      load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = act_fwd(v[i], act);
      break;
    }
    case kProGated: {
      float u[8];
      load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
      load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + a.C + gc, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = act_fwd(v[i], act) * u[i];
      break;
    }
    case kProDAct: {
      float d[8];
      load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + gc, v);
      load8(a.dy, a.x_dtype, static_cast<size_t>(gr) * a.C + gc, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = d[i] * act_bwd(v[i], act);
      break;
    }
    case kProDGated: {
      const int n = a.C / 2;
      const int c = gc < n ? gc : gc - n;
      float d[8], x1[8];
      load8(a.dy, a.x_dtype, static_cast<size_t>(gr) * n + c, d);
      load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + c, x1);
      if (gc < n) {
        float x2[8];
        load8(a.x, a.x_dtype, static_cast<size_t>(gr) * a.ldx + n + c, x2);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d[i] * x2[i] * act_bwd(x1[i], act);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d[i] * act_fwd(x1[i], act);
      }
      break;
    }
  }
  if (a.row_scale) {
    const float s = a.row_scale[gr];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= s;
  }
}

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  // values are non-negative: integer compare preserves order
  atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t habs2_u(uint32_t w) { return w & 0x7FFF7FFFu; }
// element-wise max of two packed non-negative bf16 pairs (bit patterns order like integers)
__device__ __forceinline__ uint32_t hmax2_u(uint32_t a, uint32_t b) {
  return __vmaxu2(a, b);
}

constexpr int QPITCH = TR + 16;  // bytes per column of the transposed fp8 staging tile

template <int PRO, int ACT>
__global__ void __launch_bounds__(NT, 4) quantize_tile_kernel(const QuantArgs a, const int MODE) {
  __shared__ __align__(16) __nv_bfloat16 tile[TR * PITCH];
  // the transposed fp8 staging tile reuses the bf16 tile once every thread holds its column data in registers
  uint8_t* tq = reinterpret_cast<uint8_t*>(tile);
  static_assert(TC * QPITCH <= TR * PITCH * 2, "staging tile must fit in the bf16 tile");
  __shared__ float red[NT / 32];
  const int tid = threadIdx.x;
  const int r0 = blockIdx.y * TR, c0 = blockIdx.x * TC;
  const bool want_col = a.col_data != nullptr || a.dbias != nullptr;
  const float tscale = (MODE == kModeTensor) ? *a.scale : 1.f;
  const float fmax_rcp = a.fp8_e5m2 ? (1.f / 57344.f) : (1.f / 448.f);
  uint32_t local_amax = 0;  // packed bf16 pair, non-negative

  // ---------------------------------------------------------------- row pass
#pragma unroll 1
  for (int it = 0; it < (TR * TC / 32) / NT; ++it) {
    const int item = tid + it * NT;
    const int row = item >> 2, blk = item & 3;
    const int gr = r0 + row, gc = c0 + blk * 32;
    __nv_bfloat16* trow = tile + row * PITCH + blk * 32;
    if (gr < a.R && gc < a.C) {
      uint32_t packed[16];
      uint32_t am2 = 0;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float v[8];
        produce8<PRO, ACT>(a, gr, gc + ch * 8, v);
        if (a.y != nullptr && a.y_dtype != kBFloat16) {
          const size_t off = static_cast<size_t>(gr) * a.C + gc + ch * 8;
          if (a.y_dtype == kFloat32) {
            float4* yp = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + off);
            yp[0] = make_float4(v[0], v[1], v[2], v[3]);
            yp[1] = make_float4(v[4], v[5], v[6], v[7]);
          } else {
            *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.y) + off) =
                make_uint4(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]), pack_f16x2(v[4], v[5]), pack_f16x2(v[6], v[7]));
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t w = pack_bf16x2(v[2 * j], v[2 * j + 1]);
          packed[ch * 4 + j] = w;
          am2 = hmax2_u(am2, habs2_u(w));
        }
      }
      if (want_col) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          reinterpret_cast<uint4*>(trow)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      }
      if (a.y != nullptr && a.y_dtype == kBFloat16) {
        uint4* yp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.y) + static_cast<size_t>(gr) * a.C + gc);
#pragma unroll
        for (int i = 0; i < 4; ++i) yp[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      }
      local_amax = hmax2_u(local_amax, am2);
      if (MODE != kModeNone && a.row_data != nullptr) {
        float mul;
        if (MODE == kModeMx) {
          const float amax = fmaxf(bf_lo(am2), bf_hi(am2));
          const uint8_t e = f32_to_e8m0_rp(amax * fmax_rcp);
          mul = e8m0_rcp(e);
          a.row_scale_out[swizzled_sf_offset(gr, gc >> 5, ((a.C >> 5) + 3) >> 2)] = e;
        } else {
          mul = tscale;
        }
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t lo = cvt_fp8x2(bf_lo(packed[2 * i]) * mul, bf_hi(packed[2 * i]) * mul, a.fp8_e5m2);
          const uint32_t hi = cvt_fp8x2(bf_lo(packed[2 * i + 1]) * mul, bf_hi(packed[2 * i + 1]) * mul, a.fp8_e5m2);
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
    float m = fmaxf(bf_lo(local_amax), bf_hi(local_amax));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) red[tid >> 5] = m;
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
  // one thread = two adjacent columns x 32 rows; results are staged transposed in shared
  // memory so that the global stores are 128 contiguous bytes per output row
  const int cp = tid & 63, rb = tid >> 6;
  const int col = cp * 2;
  const int gcol = c0 + col, grow = r0 + rb * 32;
  const bool active = gcol < a.C && grow < a.R;
  uint32_t w[32];
  uint32_t am2 = 0;
  if (active) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      w[i] = *reinterpret_cast<const uint32_t*>(&tile[(rb * 32 + i) * PITCH + col]);
      am2 = hmax2_u(am2, habs2_u(w[i]));
    }
    if (a.dbias != nullptr) {
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        s0 += bf_lo(w[i]);
        s1 += bf_hi(w[i]);
      }
      atomicAdd(a.dbias + gcol, s0);
      atomicAdd(a.dbias + gcol + 1, s1);
    }
  }
  if (MODE == kModeNone || a.col_data == nullptr) return;
  __syncthreads();  // all column data is in registers: the tile memory becomes the staging buffer
  if (active) {
    float m0, m1;
    if (MODE == kModeMx) {
      const uint8_t e0 = f32_to_e8m0_rp(bf_lo(am2) * fmax_rcp);
      const uint8_t e1 = f32_to_e8m0_rp(bf_hi(am2) * fmax_rcp);
      m0 = e8m0_rcp(e0);
      m1 = e8m0_rcp(e1);
      const int kt = ((a.R >> 5) + 3) >> 2;
      a.col_scale_out[swizzled_sf_offset(gcol, grow >> 5, kt)] = e0;
      a.col_scale_out[swizzled_sf_offset(gcol + 1, grow >> 5, kt)] = e1;
    } else {
      m0 = m1 = tscale;
    }
    uint32_t q0[8], q1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // rows 4i .. 4i+3: each conversion yields (col0 byte, col1 byte)
      const uint32_t a0 = cvt_fp8x2(bf_lo(w[4 * i]) * m0, bf_hi(w[4 * i]) * m1, a.fp8_e5m2);
      const uint32_t a1 = cvt_fp8x2(bf_lo(w[4 * i + 1]) * m0, bf_hi(w[4 * i + 1]) * m1, a.fp8_e5m2);
      const uint32_t a2 = cvt_fp8x2(bf_lo(w[4 * i + 2]) * m0, bf_hi(w[4 * i + 2]) * m1, a.fp8_e5m2);
      const uint32_t a3 = cvt_fp8x2(bf_lo(w[4 * i + 3]) * m0, bf_hi(w[4 * i + 3]) * m1, a.fp8_e5m2);
      const uint32_t t01 = a0 | (a1 << 16), t23 = a2 | (a3 << 16);
      q0[i] = __byte_perm(t01, t23, 0x6420);
      q1[i] = __byte_perm(t01, t23, 0x7531);
    }
    uint4* p0 = reinterpret_cast<uint4*>(tq + col * QPITCH + rb * 32);
    uint4* p1 = reinterpret_cast<uint4*>(tq + (col + 1) * QPITCH + rb * 32);
    p0[0] = make_uint4(q0[0], q0[1], q0[2], q0[3]);
    p0[1] = make_uint4(q0[4], q0[5], q0[6], q0[7]);
    p1[0] = make_uint4(q1[0], q1[1], q1[2], q1[3]);
    p1[1] = make_uint4(q1[4], q1[5], q1[6], q1[7]);
  }
  __syncthreads();
  // 128 output rows (columns of the tile) x 8 chunks of 16 bytes
#pragma unroll
  for (int k = 0; k < (TC * TR / 16) / NT; ++k) {
    const int q = tid + k * NT;
    const int ocol = q >> 3, part = q & 7;
    const int gc = c0 + ocol, gr = r0 + part * 16;
    if (gc < a.C && gr < a.R)
      *reinterpret_cast<uint4*>(a.col_data + static_cast<size_t>(gc) * a.R + gr) =
          *reinterpret_cast<const uint4*>(tq + ocol * QPITCH + part * 16);
  }
}

template <int PRO>
cudaError_t launch_pro(const QuantArgs& a, int mode, dim3 grid, cudaStream_t s) {
  if (PRO == kProIdentity || PRO == kProNorm) {
    quantize_tile_kernel<PRO, -1><<<grid, NT, 0, s>>>(a, mode);
  } else if (a.act == kActSilu) {
    quantize_tile_kernel<PRO, kActSilu><<<grid, NT, 0, s>>>(a, mode);
  } else if (a.act == kActGelu) {
    quantize_tile_kernel<PRO, kActGelu><<<grid, NT, 0, s>>>(a, mode);
  } else {
    quantize_tile_kernel<PRO, -1><<<grid, NT, 0, s>>>(a, mode);
  }
  return cudaGetLastError();
}

cudaError_t launch_tile(const QuantArgs& a, int mode, cudaStream_t s) {
  if (a.R <= 0 || a.C <= 0) return cudaSuccess;
  if (a.R % 32 != 0 || a.C % 32 != 0) return cudaErrorInvalidValue;
  dim3 grid((a.C + TC - 1) / TC, (a.R + TR - 1) / TR);
  switch (a.prologue) {
    case kProIdentity: return launch_pro<kProIdentity>(a, mode, grid, s);
    case kProNorm: return launch_pro<kProNorm>(a, mode, grid, s);
    case kProAct: return launch_pro<kProAct>(a, mode, grid, s);
    case kProGated: return launch_pro<kProGated>(a, mode, grid, s);
    case kProDAct: return launch_pro<kProDAct>(a, mode, grid, s);
    case kProDGated: return launch_pro<kProDGated>(a, mode, grid, s);
    default: return cudaErrorInvalidValue;
  }
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

cudaError_t quantize_mxfp8(const QuantArgs& a, cudaStream_t s) { return launch_tile(a, kModeMx, s); }
cudaError_t quantize_fp8_tensor(const QuantArgs& a, cudaStream_t s) { return launch_tile(a, kModeTensor, s); }
cudaError_t apply_prologue(const QuantArgs& a, cudaStream_t s) { return launch_tile(a, kModeNone, s); }

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
