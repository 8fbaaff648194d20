// Shared pieces of the fused attention kernels (head dim 128, 16-bit inputs, fp32 softmax).
//
// All three kernels (forward, dQ, dK/dV) are warp-specialised: one TMA producer warp, one
// tcgen05 issuer warp and two groups of four softmax warps that work on two independent score
// tiles, so that the tensor pipe computes one tile's products while the other tile's
// exponentials run.  Score and output accumulators live in TMEM; probabilities go back to the
// tensor cores through 128-byte-swizzled shared-memory tiles.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "teb200/api.h"
#include "teb200/ptx.cuh"

namespace teb200 {
namespace attn {

constexpr int kHeadDim = 128;
constexpr int kThreads = 576;  // warp 0 TMA, warp 1 MMA, warps 2-9 tile (group) 0, warps 10-17 tile (group) 1

enum FlashStatus : int {
  kFlashOk = 0,
  kFlashTimeoutProducer = 21,
  kFlashTimeoutMma = 22,
  kFlashTimeoutSoftmax = 23,
};

struct FlashParams {
  int b, hq, hk, sq, sk;
  int causal;      // 1: key j visible to query i when j <= i + causal_off
  int causal_off;  // sk - sq for the bottom-right aligned mask, 0 for top-left
  float scale;       // softmax scale
  float scale_log2;  // scale * log2(e)
  int is_bf16;
  // outputs, addressed as [b, h, s, d] views with element strides (d contiguous)
  void* out;       // forward: O; dQ kernel: dQ
  long long o_sb, o_sh, o_ss;
  void* out2;      // dK/dV kernel: dV (out = dK), same strides
  float* lse;      // [b, hq, s_pad] natural-log LSE
  float* delta;    // [b, hq, s_pad] rowsum(dO * O)
  int s_pad;
  int* status;
  long long* timeline;  // optional [64][16] clock stamps of CTA 0 (profiling aid), else nullptr
  // packed variable-length sequences (nullptr: fixed lengths); then sq / sk above are the maxima
  const int* cu_q;
  const int* cu_k;
  const int* off_q;
  const int* off_k;
  int bottom_right;
  int gsplit;       // dK/dV pass: CTAs per group of query heads (partials o_sg elements apart)
  long long o_sg;
  // sliding window: with `causal` set, key j is visible to query i when j <= i + causal_off (which
  // includes the right extent win_right) and, when has_lo, j >= i + lo_off
  int win_left, win_right, has_lo, lo_off;
  int pair_balance;  // query-stationary kernels: a CTA takes 128-row tiles i and last - i (equal causal work)
};

// Where sequence b starts in the token dimension, and which batch coordinate the TMA maps take.
struct SeqView {
  int q_off, k_off, bt;
};

// Turn the launch-wide parameters into those of sequence b: with packed sequences the lengths come
// from the cumulative arrays (clamped to the launch's maxima, which sized the grid and lse/delta).
__device__ __forceinline__ SeqView localize(FlashParams& p, int b) {
  SeqView v = {0, 0, b};
  if (p.cu_q != nullptr) {
    int sq = p.cu_q[b + 1] - p.cu_q[b];
    int sk = p.cu_k[b + 1] - p.cu_k[b];
    sq = sq < 0 ? 0 : (sq > p.sq ? p.sq : sq);
    sk = sk < 0 ? 0 : (sk > p.sk ? p.sk : sk);
    p.sq = sq;
    p.sk = sk;
    p.causal_off = (p.bottom_right ? sk - sq : 0) + p.win_right;
    p.lo_off = (p.bottom_right ? sk - sq : 0) - p.win_left;
    v.q_off = p.off_q[b];
    v.k_off = p.off_k[b];
    v.bt = 0;
    p.o_sb = 0;
  }
  return v;
}

// 4-D tile load: coordinates (d, s, h, b)
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
      "%6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// instruction descriptor of a 16-bit MMA with fp32 accumulation, M = 128
__host__ __device__ constexpr uint32_t attn_idesc(bool bf16, int n, bool a_mn, bool b_mn) {
  uint32_t d = 0;
  const uint32_t fmt = bf16 ? 1u : 0u;
  d |= 1u << 4;
  d |= fmt << 7;
  d |= fmt << 10;
  d |= (a_mn ? 1u : 0u) << 15;
  d |= (b_mn ? 1u : 0u) << 16;
  d |= (uint32_t(n) >> 3) << 17;
  d |= (128u >> 4) << 24;
  return d;
}

// Write one row of a [128 x 64] 16-bit tile in the 128-byte-swizzled K-major layout the
// tensor core reads: row r starts at r * 128 bytes, its 16-byte chunk c sits at chunk c ^ (r % 8).
__device__ __forceinline__ void store_row_sw128(uint8_t* tile, int r, const uint32_t (&w)[32]) {
  uint8_t* row = tile + r * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = make_uint4(w[c * 4], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
  }
}

// tcgen05.mma with the A operand read from TMEM (16-bit elements packed two per 32-bit column,
// row = lane) and B from shared memory
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 16 columns: registers -> TMEM
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};\n" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Fill the mask fields of the launch parameters from the caller's arguments.
inline void set_mask_params(FlashParams& p, const FlashArgs& a) {
  const int base = a.bottom_right ? a.sk - a.sq : 0;
  p.bottom_right = a.bottom_right ? 1 : 0;
  p.win_right = a.causal ? 0 : (a.window_right >= 0 ? a.window_right : 0);
  p.causal = (a.causal || a.window_right >= 0) ? 1 : 0;
  p.causal_off = base + p.win_right;
  p.has_lo = a.window_left >= 0 ? 1 : 0;
  p.win_left = a.window_left >= 0 ? a.window_left : 0;
  p.lo_off = base - p.win_left;
}

// 4-D tensor map over a [b, h, s, d] view; strides in elements, box = [rows x 64 elements]
bool make_tensor_map_bhsd(CUtensorMap* map, const void* base, bool bf16, int b, int h, int s, long long sb,
                          long long sh, long long ss, int box_rows);

}  // namespace attn
}  // namespace teb200
