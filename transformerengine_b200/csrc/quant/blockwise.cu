// FP8 block scaling with 128-wide blocks (1 x 128 for activations / gradients, 128 x 128 for
// weights): one pass over a 128 x 128 tile of the input produces
//   * the row-wise copy  [R, C]  and the column-wise (transposed) copy [C, R] in FP8,
//   * their fp32 decode scales in the compact layout ([rows, ceil(k/128)] or
//     [ceil(rows/128), ceil(k/128)]), the layout checkpoints and the reference use, and
//   * when the scales are powers of two, the same scales as UE8M0 bytes in the 128x4-tile layout that
//     the block-scaled tcgen05 MMA reads (each 128-block scale repeated for its four 32-element
//     sub-blocks), so that the MXFP8 GEMM kernels multiply these tensors exactly, without any
//     conversion pass.
// Reference kernels: common/transpose/quantize_transpose_square_blockwise.cu:66,256 and
// quantize_transpose_vector_blockwise.cu:170; the reference converts to MXFP8 scales before the GEMM
// on this architecture (pytorch/csrc/extensions/gemm.cpp:312-323).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <teb200/api.h>
#include <teb200/quant.h>

namespace teb200 {
namespace {

constexpr int T = 128;        // tile edge = block edge
constexpr int PITCH = T + 1;  // shared-memory row pitch in floats
constexpr int NT = 256;

template <typename X>
__device__ __forceinline__ float ldx(const X* p, long long i) { return static_cast<float>(p[i]); }

// scale = fp8_max / amax, floored to a power of two when pow2 (mantissa cleared), 1 when amax is 0 or not finite;
// with pow2 the exponent is kept inside what a UE8M0 byte can hold for 1 / scale
__device__ __forceinline__ float block_scale(float amax, float fmax, float eps, bool pow2) {
  if (eps > 0.f) amax = fmaxf(amax, eps);
  if (!(amax > 0.f) || !isfinite(amax)) return 1.f;
  float sf = fmax / amax;
  if (isinf(sf)) sf = 3.402823466e38f;
  if (pow2) {
    uint32_t bits = __float_as_uint(sf) & 0x7F800000u;
    uint32_t e = bits >> 23;           // biased exponent of the scale
    if (e > 254u) e = 254u;            // 1/scale = 2^(127 - e): keep it >= 2^-127
    if (e < 1u) e = 1u;
    sf = __uint_as_float(e << 23);
  }
  return sf;
}

__device__ __forceinline__ uint8_t to_fp8(float v, bool e5m2) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3));
}

// UE8M0 byte of the DECODE scale 1 / sf for a power-of-two sf
__device__ __forceinline__ uint32_t ue8m0_of_inverse(float sf) {
  const int e = static_cast<int>((__float_as_uint(sf) >> 23) & 0xFFu);  // sf = 2^(e - 127)
  return static_cast<uint32_t>(254 - e);                                 // 1/sf = 2^(127 - e) -> byte 254 - e
}

// Writes the four identical scale bytes of (operand row i, 128-block kb) into the 128x4-tile layout.
__device__ __forceinline__ void put_mx_scale(uint8_t* mx, int i, int kb, int k_tiles, uint32_t byte) {
  const size_t off = (static_cast<size_t>(i >> 7) * k_tiles + kb) * 512 + (i & 31) * 16 + ((i & 127) >> 5) * 4;
  *reinterpret_cast<uint32_t*>(mx + off) = byte * 0x01010101u;
}

template <typename X>
__global__ void __launch_bounds__(NT) quantize_block128_kernel(const BlockQuantArgs a) {
  extern __shared__ float tile[];  // [T][PITCH]
  __shared__ float red[NT / 32];
  __shared__ float tile_amax;
  const int tr = blockIdx.y, tc = blockIdx.x;
  const int r0 = tr * T, c0 = tc * T;
  const X* x = static_cast<const X*>(a.x);
  for (int i = threadIdx.x; i < T * T; i += NT) {
    const int r = i >> 7, c = i & 127;
    const int gr = r0 + r, gc = c0 + c;
    tile[r * PITCH + c] = (gr < a.R && gc < a.C) ? ldx(x, static_cast<long long>(gr) * a.ld + gc) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool e5 = a.e5m2 != 0;
  const float fmax = e5 ? 57344.f : 448.f;
  const bool pow2 = a.pow2 != 0;
  float sf2d = 1.f;
  if (a.dim == 2) {
    float m = 0.f;
    for (int i = threadIdx.x; i < T * T; i += NT) m = fmaxf(m, fabsf(tile[(i >> 7) * PITCH + (i & 127)]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < NT / 32; ++i) t = fmaxf(t, red[i]);
      tile_amax = t;
    }
    __syncthreads();
    sf2d = block_scale(tile_amax, fmax, a.eps, pow2);
  }
  const int row_kt = (a.C + 127) / 128;  // 128-blocks along the contraction dim of the row-wise operand
  const int col_kt = (a.R + 127) / 128;
  // ---- row-wise copy: lane owns 4 consecutive columns of a row
  if (a.row_data != nullptr) {
    for (int r = warp; r < T; r += NT / 32) {
      const int gr = r0 + r;
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = tile[r * PITCH + lane * 4 + k];
      float sf = sf2d;
      if (a.dim == 1) {
        float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        sf = block_scale(m, fmax, a.eps, pow2);
      }
      if (gr >= a.R) continue;
      const int gc = c0 + lane * 4;
      if (gc + 3 < a.C && (a.C & 3) == 0) {
        const uint32_t pk = to_fp8(v[0] * sf, e5) | (to_fp8(v[1] * sf, e5) << 8) | (to_fp8(v[2] * sf, e5) << 16) |
                            (to_fp8(v[3] * sf, e5) << 24);
        *reinterpret_cast<uint32_t*>(a.row_data + static_cast<size_t>(gr) * a.C + gc) = pk;
      } else {
        for (int k = 0; k < 4; ++k)
          if (gc + k < a.C) a.row_data[static_cast<size_t>(gr) * a.C + gc + k] = to_fp8(v[k] * sf, e5);
      }
      if (lane == 0) {
        if (a.dim == 1) a.row_sinv[static_cast<size_t>(gr) * row_kt + tc] = 1.f / sf;
        else if (r == 0) a.row_sinv[static_cast<size_t>(tr) * row_kt + tc] = 1.f / sf;
        if (a.row_mx != nullptr) put_mx_scale(a.row_mx, gr, tc, row_kt, ue8m0_of_inverse(sf));
      }
    }
  }
  // ---- column-wise copy (transposed output [C, R]): lane owns 4 consecutive ROWS of a column
  if (a.col_data != nullptr) {
    for (int c = warp; c < T; c += NT / 32) {
      const int gc = c0 + c;
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = tile[(lane * 4 + k) * PITCH + c];
      float sf = sf2d;
      if (a.dim == 1) {
        float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        sf = block_scale(m, fmax, a.eps, pow2);
      }
      if (gc >= a.C) continue;
      const int gr = r0 + lane * 4;
      if (gr + 3 < a.R && (a.R & 3) == 0) {
        const uint32_t pk = to_fp8(v[0] * sf, e5) | (to_fp8(v[1] * sf, e5) << 8) | (to_fp8(v[2] * sf, e5) << 16) |
                            (to_fp8(v[3] * sf, e5) << 24);
        *reinterpret_cast<uint32_t*>(a.col_data + static_cast<size_t>(gc) * a.R + gr) = pk;
      } else {
        for (int k = 0; k < 4; ++k)
          if (gr + k < a.R) a.col_data[static_cast<size_t>(gc) * a.R + gr + k] = to_fp8(v[k] * sf, e5);
      }
      if (lane == 0) {
        if (a.dim == 1) a.col_sinv[static_cast<size_t>(gc) * col_kt + tr] = 1.f / sf;
        else if (c == 0) a.col_sinv[static_cast<size_t>(tc) * col_kt + tr] = 1.f / sf;
        if (a.col_mx != nullptr) put_mx_scale(a.col_mx, gc, tr, col_kt, ue8m0_of_inverse(sf));
      }
    }
  }
}

}  // namespace

cudaError_t quantize_block128(const BlockQuantArgs& a, cudaStream_t s) {
  if (a.R <= 0 || a.C <= 0) return cudaSuccess;
  if (a.dim != 1 && a.dim != 2) return cudaErrorInvalidValue;
  if ((a.row_mx != nullptr || a.col_mx != nullptr) && !a.pow2) return cudaErrorInvalidValue;
  const dim3 grid((a.C + T - 1) / T, (a.R + T - 1) / T);
  const size_t smem = sizeof(float) * T * PITCH;
  cudaError_t e;
#define TEB_BQ(X)                                                                                              \
  e = cudaFuncSetAttribute(quantize_block128_kernel<X>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                           static_cast<int>(smem));                                                            \
  if (e != cudaSuccess) return e;                                                                              \
  quantize_block128_kernel<X><<<grid, NT, smem, s>>>(a)
  if (a.x_dtype == kBFloat16) { TEB_BQ(__nv_bfloat16); }
  else if (a.x_dtype == kFloat16) { TEB_BQ(__half); }
  else if (a.x_dtype == kFloat32) { TEB_BQ(float); }
  else return cudaErrorInvalidValue;
#undef TEB_BQ
  return cudaGetLastError();
}

}  // namespace teb200
