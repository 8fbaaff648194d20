// Launchers of the quantize / cast / activation+quantize / norm+quantize kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace teb200 {

// Element-wise producer fused in front of the quantizer.
enum Prologue : int {
  kProIdentity = 0,  // v = x[r,c]
  kProNorm = 1,      // v = (x[r,c] - mu[r]) * rs[r] * (gamma[c] + zc) + beta[c]   (mu/beta optional)
  kProAct = 2,       // v = act(x[r,c])
  kProGated = 3,     // v = act(x[r,c]) * x[r, n+c]            input [R,2n] -> output [R,n]
  kProDAct = 4,      // v = dy[r,c] * act'(x[r,c])
  kProDGated = 5,    // out [R,2n]: c<n: dy*x2*act'(x1); c>=n: dy*act(x1)
};

enum ActType : int { kActGelu = 0, kActSilu = 1, kActRelu = 2, kActQGelu = 3, kActSRelu = 4, kActIdentity = 5 };

struct QuantArgs {
  const void* x = nullptr;      // main input
  int x_dtype = 2;              // DType
  const void* dy = nullptr;     // upstream gradient for kProDAct / kProDGated (dtype = x_dtype)
  const float* mu = nullptr;    // [R] (LayerNorm) or null (RMSNorm)
  const float* rs = nullptr;    // [R]
  const void* gamma = nullptr;  // [C] dtype gamma_dtype
  const void* beta = nullptr;
  int gamma_dtype = 2;
  int zero_centered = 0;
  const float* row_scale = nullptr;  // optional per-row multiplier (MoE probabilities)
  int prologue = kProIdentity;
  int act = kActGelu;
  int R = 0, C = 0;             // OUTPUT rows / cols
  int64_t ldx = 0;              // input leading dim in elements
  // outputs (any may be null)
  void* y = nullptr;            // high-precision copy of the produced values, dtype y_dtype, [R,C]
  int y_dtype = 2;
  uint8_t* row_data = nullptr;  // [R,C] fp8
  uint8_t* row_scale_out = nullptr;  // swizzled ue8m0, scale matrix [R, C/32]
  uint8_t* col_data = nullptr;  // [C,R] fp8 (transposed)
  uint8_t* col_scale_out = nullptr;  // swizzled ue8m0, scale matrix [C, R/32]
  int fp8_e5m2 = 0;
  // per-tensor FP8 mode
  const float* scale = nullptr;  // [1] multiply before cast
  float* amax = nullptr;         // [1] atomic max of |v|
  float* scale_inv = nullptr;    // [1] written = 1/scale
  float* dbias = nullptr;        // [C] fp32, column sums of v accumulated atomically (optional)
};

cudaError_t quantize_mxfp8(const QuantArgs& a, cudaStream_t s);
// per-tensor scaled cast: row_data [R,C], col_data [C,R] (plain transpose), amax/scale_inv
cudaError_t quantize_fp8_tensor(const QuantArgs& a, cudaStream_t s);
// only produce y (and amax): fused norm-apply / activation without quantization
cudaError_t apply_prologue(const QuantArgs& a, cudaStream_t s);

cudaError_t dequantize_mxfp8(const uint8_t* q, const uint8_t* sf_swizzled, int R, int C, int e5m2, void* out,
                             int out_dtype, cudaStream_t s);
cudaError_t dequantize_fp8_tensor(const uint8_t* q, const float* scale_inv, int64_t n, int e5m2, void* out,
                                  int out_dtype, cudaStream_t s);
cudaError_t amax_abs(const void* x, int dtype, int64_t n, float* out /*zeroed by callee*/, cudaStream_t s);
cudaError_t swizzle_scales(const uint8_t* compact, int rows, int cols, uint8_t* out, cudaStream_t s);
cudaError_t unswizzle_scales(const uint8_t* swz, int rows, int cols, uint8_t* out, cudaStream_t s);

// delayed scaling: scales from the amax history [H, n], then roll the history and clear slot 0
cudaError_t delayed_scaling_update(float* history, float* scale, int H, int n, float fp8_max, int margin, int most_recent,
                                   cudaStream_t s);

// FP8 with one scale per 1 x 128 (dim = 1) or 128 x 128 (dim = 2) block.  Compact fp32 decode scales:
// row-wise [R, ceil(C/128)] or [ceil(R/128), ceil(C/128)]; column-wise (for the transposed copy [C, R])
// [C, ceil(R/128)] or [ceil(C/128), ceil(R/128)].  row_mx / col_mx (optional, power-of-two scales only):
// the same scales as UE8M0 bytes in the 128x4-tile GEMM layout of an operand with 32-element blocks,
// zero-initialised by the caller, padded to ru(rows,128) * ru(ceil(k/32),4) bytes.
struct BlockQuantArgs {
  const void* x = nullptr;
  int x_dtype = 2;
  int R = 0, C = 0;
  long long ld = 0;
  int dim = 1;
  int e5m2 = 0;
  int pow2 = 1;
  float eps = 0.f;
  uint8_t* row_data = nullptr;
  float* row_sinv = nullptr;
  uint8_t* row_mx = nullptr;
  uint8_t* col_data = nullptr;
  float* col_sinv = nullptr;
  uint8_t* col_mx = nullptr;
};
cudaError_t quantize_block128(const BlockQuantArgs& a, cudaStream_t s);

// NVFP4: 1x16 (or 16x16) blocks, E4M3 block scales (swizzled), global amax given.
struct Nvfp4Args {
  const void* x = nullptr;
  int x_dtype = 2;
  int R = 0, C = 0;
  const float* amax_row = nullptr;  // [1] global amax used for the rowwise copy
  const float* amax_col = nullptr;  // [1] global amax for the columnwise copy (post-RHT if with_rht)
  uint8_t* row_data = nullptr;      // [R, C/2]
  uint8_t* row_scale = nullptr;     // swizzled, matrix [R, C/16]
  uint8_t* col_data = nullptr;      // [C, R/2]
  uint8_t* col_scale = nullptr;     // swizzled, matrix [C, R/16]
  int with_rht = 0;                 // rotate 16-token blocks of the columnwise copy
  int with_2d = 0;                  // 16x16 block scales
  int stochastic = 0;
  uint64_t seed = 0, offset = 0;
  // optional device counter added to `offset` by the kernels: a launch recorded in a CUDA graph then draws
  // new random numbers on every replay (the caller advances the counter with a device op)
  const unsigned long long* offset_dev = nullptr;
};
cudaError_t quantize_nvfp4(const Nvfp4Args& a, cudaStream_t s);
// amax of x and of RHT(x^T) in one pass: out[0] = amax(x), out[1] = amax(RHT(x^T))
cudaError_t nvfp4_amax(const void* x, int dtype, int R, int C, int with_rht, float* out2, cudaStream_t s);
cudaError_t dequantize_nvfp4(const uint8_t* q, const uint8_t* sf_swizzled, const float* amax, int R, int C,
                             void* out, int out_dtype, cudaStream_t s);

}  // namespace teb200
