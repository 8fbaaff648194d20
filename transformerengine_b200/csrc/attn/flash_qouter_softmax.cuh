// Softmax / dS role of the query-stationary attention kernels (included by flash_qouter.cu).
//
// A tile has eight warps: two per TMEM lane quarter, each taking 32 of the block's 64 score
// columns.  Thread = (row, column half).  In the forward the two halves of a row agree on the
// running maximum through a small shared-memory exchange; their row sums stay separate until
// the epilogue.
#pragma once
#include "flash_common.cuh"

namespace teb200 {
namespace attn {

template <bool BF>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
  return BF ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}

// 16 packed words = 32 values = chunks [4*half, 4*half+4) of row r in a [128 x 64] swizzled tile
__device__ __forceinline__ void store_half_row_sw128(uint8_t* tile, int r, int half, const uint32_t (&w)[16]) {
  uint8_t* row = tile + r * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int ch = half * 4 + c;
    *reinterpret_cast<uint4*>(row + ((ch ^ (r & 7)) << 4)) = make_uint4(w[c * 4], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
  }
}

// Publish `v` for step `tag` and fetch the partner thread's value of the same step.
__device__ __forceinline__ bool xchg_pair(unsigned long long* slots, int mine, int theirs, uint32_t tag, float v,
                                          float& other) {
  volatile unsigned long long* vs = slots;
  vs[mine] = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
  const long long t0 = clock64();
  unsigned long long got = vs[theirs];
  while (static_cast<uint32_t>(got >> 32) != tag) {
    if (clock64() - t0 > kWaitCycles) return false;
    got = vs[theirs];
  }
  other = __uint_as_float(static_cast<uint32_t>(got));
  return true;
}

template <int MODE, bool BF, class C, bool WIN>
__device__ __forceinline__ void qouter_softmax_role(const FlashParams& p, uint8_t* smem, uint64_t* s_full,
                                                    uint64_t* p_ready, uint64_t* pv_done, unsigned long long* xchg,
                                                    uint32_t tmem_base, int warp, int lane, int q0, int h, int b,
                                                    int nt, int t, int jbase) {
  constexpr int kModeFwd = 0;
  const int wi = (warp - 2) & 7;
  const int half = wi >> 2;                // which 32 score columns / which 64 output columns
  const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
  const int r = quarter * 32 + lane;       // row inside the tile
  const int q_row = q0 + t * 128 + r;
  const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
  const float NEG_INF = -INFINITY;
  bool ok = true;
  float m_run = NEG_INF, l_run = 0.f;
  float lse2 = INFINITY, delta = 0.f;
  if (MODE != kModeFwd && q_row < p.sq) {
    const size_t off = (static_cast<size_t>(b) * p.hq + h) * p.s_pad + q_row;
    lse2 = p.lse[off] * 1.4426950408889634f;
    delta = p.delta[off];
  }
  constexpr int BK = C::kBlockKv;
  constexpr int HC = BK / 2;                 // score columns per thread
  const uint32_t col_s = lane_base + C::kColS + t * BK + half * HC;
  for (int j = 0; j < nt; ++j) {
    const bool stamp = p.timeline != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && t == 0 && half == 0 &&
                       quarter == 0 && lane == 0 && j < 64;
    if (stamp) p.timeline[j * 16 + 0] = clock64();
    if (!mbar_wait(&s_full[t * 2], j & 1)) { ok = false; break; }
    __syncwarp();
    tc_fence_after();
    if (stamp) p.timeline[j * 16 + 1] = clock64();
    const int kb0 = (jbase + j) * BK;     // first key of the block
    const int kv0 = kb0 + half * HC;      // first key of this thread's columns
    const bool need_mask = (kb0 + BK > p.sk) || (p.causal && kb0 + BK - 1 > q0 + t * 128 + p.causal_off) ||
                           (WIN && kb0 < q0 + t * 128 + 127 + p.lo_off);
    const int lim = p.causal ? min(p.sk - 1, q_row + p.causal_off) : p.sk - 1;  // last visible key
    const int lo = WIN ? q_row + p.lo_off : 0;                                 // first visible key
    if (MODE == kModeFwd) {
      // pass 1: block maximum of this thread's columns, 32 at a time
      float mx4[4] = {NEG_INF, NEG_INF, NEG_INF, NEG_INF};
#pragma unroll
      for (int c0 = 0; c0 < HC; c0 += 32) {
        uint32_t s[32];
        tmem_ld_32x32(col_s + c0, s);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (kv0 + c0 + c > lim || kv0 + c0 + c < lo) s[c] = __float_as_uint(NEG_INF);
        }
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], __uint_as_float(s[c + e]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the other half of the row: exchange block maxima through shared memory
      unsigned long long* slot = xchg + ((t * 2 + (j & 1)) * 2) * 128;
      float mx_other;
      if (!xchg_pair(slot, half * 128 + r, (half ^ 1) * 128 + r, j + 1, mx, mx_other)) { ok = false; break; }
      __syncwarp();
      const float mx_row = fmaxf(mx, mx_other);
      if (stamp) p.timeline[j * 16 + 2] = clock64();
      const float m_new = fmaxf(m_run, mx_row * p.scale_log2);
      const bool first = m_run == NEG_INF;
      const float m_use = (!first && m_new - m_run <= 8.f) ? m_run : m_new;
      const float m_eff = m_use == NEG_INF ? 0.f : m_use;
      const float alpha = first ? 1.f : fast_exp2(m_run - m_use);
      m_run = m_use;
      // pass 2: P = exp2(S*c - m) over the scores just read (each 32-column chunk of scores
      // becomes 16 packed columns at the start of this thread's region)
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c0 = 0; c0 < HC; c0 += 32) {
        uint32_t s[32];
        uint32_t w[16];
        tmem_ld_32x32(col_s + c0, s);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          float e4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float x = fmaf(__uint_as_float(s[c + e]), p.scale_log2, -m_eff);
            if (need_mask && (kv0 + c0 + c + e > lim || kv0 + c0 + c + e < lo)) x = NEG_INF;
            e4[e] = fast_exp2(x);
            sum4[e] += e4[e];
          }
          w[c / 2] = pack16<BF>(e4[0], e4[1]);
          w[c / 2 + 1] = pack16<BF>(e4[2], e4[3]);
        }
        tmem_st_32x16(col_s + c0 / 2, w);
      }
      l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      if (stamp) p.timeline[j * 16 + 3] = clock64();
      // the output accumulator is rescaled only when some row's maximum moved by more than 2^8;
      // block j-1's P V must have landed first
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!mbar_wait(&pv_done[t], (j - 1) & 1)) { ok = false; break; }
        __syncwarp();
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32(lane_base + C::kColO + t * 128 + half * 64 + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tmem_st_32x32(lane_base + C::kColO + t * 128 + half * 64 + c0, o);
        }
      }
      tmem_st_wait();
    } else {
      // dS = P * (dP - delta), P rebuilt from the saved log-sum-exp
      uint32_t s[32], dp[32];
      uint32_t w[16];
      tmem_ld_32x32(col_s, s);
      tmem_ld_32x32(lane_base + C::kColDp + t * BK + half * HC, dp);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float p0 = fast_exp2(fmaf(__uint_as_float(s[c]), p.scale_log2, -lse2));
        float p1 = fast_exp2(fmaf(__uint_as_float(s[c + 1]), p.scale_log2, -lse2));
        if (need_mask) {
          if (kv0 + c > lim || kv0 + c < lo) p0 = 0.f;
          if (kv0 + c + 1 > lim || kv0 + c + 1 < lo) p1 = 0.f;
        }
        const float d0 = p0 * (__uint_as_float(dp[c]) - delta);
        const float d1 = p1 * (__uint_as_float(dp[c + 1]) - delta);
        w[c / 2] = pack16<BF>(d0, d1);
      }
      // dS returns to the tensor core through TMEM over the scores this thread has just read
      tmem_st_32x16(col_s, w);
      tmem_st_wait();
    }
    if (stamp) p.timeline[j * 16 + 4] = clock64();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&p_ready[t]);
    if (stamp) p.timeline[j * 16 + 5] = clock64();
  }
  if (!ok && lane == 0) atomicCAS(p.status, 0, kFlashTimeoutSoftmax);
  // ------------------------------------------------------------------ epilogue
  if (ok && nt > 0) {
    if (!mbar_wait(&pv_done[t], (nt - 1) & 1)) {
      ok = false;
      if (lane == 0) atomicCAS(p.status, 0, kFlashTimeoutSoftmax);
    }
    tc_fence_after();
  }
  float l_row = l_run;
  if (MODE == kModeFwd && ok) {
    // total row sum = this half + the other half (both in the same reference maximum)
    unsigned long long* slot = xchg + ((t * 2 + (nt & 1)) * 2) * 128;
    float l_other = 0.f;
    ok = xchg_pair(slot, half * 128 + r, (half ^ 1) * 128 + r, nt + 1, l_run, l_other);
    l_row = l_run + l_other;
  }
  // TMEM loads are warp-wide: every lane takes part, only the stores depend on the row
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) return;
  const bool row_ok = q_row < p.sq;
  uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + b * p.o_sb + h * p.o_sh + static_cast<long long>(q_row) * p.o_ss +
                   half * 64;
  const float mul = MODE == kModeFwd ? (l_row > 0.f ? 1.f / l_row : 0.f) : p.scale;
#pragma unroll 1
  for (int c0 = 0; c0 < 64; c0 += 32) {
    uint32_t o[32];
    if (nt > 0) {
      tmem_ld_32x32(lane_base + C::kColO + t * 128 + half * 64 + c0, o);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c) o[c] = 0u;
    }
    if (row_ok) {
#pragma unroll
      for (int c = 0; c < 32; c += 8) {
        uint32_t q4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          q4[i] = pack16<BF>(__uint_as_float(o[c + 2 * i]) * mul, __uint_as_float(o[c + 2 * i + 1]) * mul);
        *reinterpret_cast<uint4*>(orow + c0 + c) = make_uint4(q4[0], q4[1], q4[2], q4[3]);
      }
    }
  }
  if (MODE == kModeFwd && row_ok && half == 0) {
    const size_t off = (static_cast<size_t>(b) * p.hq + h) * p.s_pad + q_row;
    p.lse[off] = l_row > 0.f ? m_run * 0.6931471805599453f + logf(l_row) : NEG_INF;
  }
}

}  // namespace attn
}  // namespace teb200
