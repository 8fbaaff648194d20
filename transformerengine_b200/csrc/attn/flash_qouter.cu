// Fused attention, query-stationary kernels: the forward pass and the dQ pass of the backward.
//
// One CTA owns 256 query rows of one head (two 128-row tiles) and walks the key/value sequence
// in blocks of 64.  Per block and tile:
//   forward : S = Q K^T            -> softmax warps: P = exp2(S*c - m), row sums, lazy rescale
//             O += P V                of the TMEM accumulator when the row max moved by > 8
//   dQ pass : S = Q K^T, dP = dO V^T -> dS = P * (dP - delta)   (P rebuilt from the saved LSE)
//             dQ += dS K
// K and V blocks arrive through separate TMA rings; a V block doubles as the MN-major B
// operand of P V, a K block as the MN-major B operand of dS K, so nothing is transposed.
// (Reference behaviour: common/fused_attn/fused_attn_f16_arbitrary_seqlen.cu, cuDNN graphs.)
#include "flash_common.cuh"

namespace teb200 {
namespace attn {

enum { kFwd = 0, kDq = 1 };

template <int MODE>
struct QCfg {
  static constexpr int kKvStages = MODE == kFwd ? 3 : 2;
  static constexpr int kQBytes = 2 * 32768;                       // two Q tiles
  static constexpr int kDoBytes = MODE == kFwd ? 0 : 2 * 32768;   // two dO tiles
  static constexpr int kPBytes = 2 * 16384;                       // P (or dS) tiles
  static constexpr int kKvBytes = 16384;                          // one K or V block
  static constexpr int kOffDo = kQBytes;
  static constexpr int kOffP = kOffDo + kDoBytes;
  static constexpr int kOffK = kOffP + kPBytes;
  static constexpr int kOffV = kOffK + kKvStages * kKvBytes;
  static constexpr int kOffBar = kOffV + kKvStages * kKvBytes;
  static constexpr int kNumBars = 1 + 4 * kKvStages + 6;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;
  // TMEM columns
  static constexpr int kColS = 0;                              // + t * 64
  static constexpr int kColDp = 128;                           // + t * 64 (dQ pass)
  static constexpr int kColO = MODE == kFwd ? 128 : 256;       // + t * 128
};

__device__ __forceinline__ int kv_blocks_of_tile(const FlashParams& p, int row0) {
  if (row0 >= p.sq) return 0;
  int kv_end = p.sk;
  if (p.causal) {
    const int lim = row0 + 128 + p.causal_off;  // exclusive bound for the tile's last row
    kv_end = lim < kv_end ? lim : kv_end;
  }
  return kv_end <= 0 ? 0 : (kv_end + 63) / 64;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
flash_qouter_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const FlashParams p) {
  using C = QCfg<MODE>;
  constexpr int KS = C::kKvStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;
  uint64_t* v_empty = v_full + KS;
  uint64_t* s_full = v_empty + KS;   // [2]
  uint64_t* p_ready = s_full + 2;    // [2]
  uint64_t* pv_done = p_ready + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // longest causal rows first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.hq / p.hk);
  const int q0 = qb * 256;
  int n[2];
  n[0] = kv_blocks_of_tile(p, q0);
  n[1] = kv_blocks_of_tile(p, q0 + 128);
  const int nmax = n[0] > n[1] ? n[0] : n[1];

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
    if (MODE == kDq) prefetch_tensormap(&tmap_do);
    mbar_init(q_full, 1);
    for (int i = 0; i < KS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_ready[t], 4);
      mbar_init(&pv_done[t], 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && nmax > 0) {
      mbar_expect_tx(q_full, C::kQBytes + C::kDoBytes);
      for (int t = 0; t < 2; ++t)
        for (int pn = 0; pn < 2; ++pn) {
          tma_load_4d(smem + t * 32768 + pn * 16384, &tmap_q, q_full, pn * 64, q0 + t * 128, h, b);
          if (MODE == kDq)
            tma_load_4d(smem + C::kOffDo + t * 32768 + pn * 16384, &tmap_do, q_full, pn * 64, q0 + t * 128, h, b);
        }
      for (int j = 0; j < nmax; ++j) {
        const int st = j % KS;
        const uint32_t par = ((j / KS) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par)) { atomicCAS(p.status, 0, kFlashTimeoutProducer); break; }
        mbar_expect_tx(&k_full[st], C::kKvBytes);
        for (int pn = 0; pn < 2; ++pn)
          tma_load_4d(smem + C::kOffK + st * C::kKvBytes + pn * 8192, &tmap_k, &k_full[st], pn * 64, j * 64, hk, b);
        if (!mbar_wait(&v_empty[st], par)) { atomicCAS(p.status, 0, kFlashTimeoutProducer); break; }
        mbar_expect_tx(&v_full[st], C::kKvBytes);
        for (int pn = 0; pn < 2; ++pn)
          tma_load_4d(smem + C::kOffV + st * C::kKvBytes + pn * 8192, &tmap_v, &v_full[st], pn * 64, j * 64, hk, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tcgen05 issuer
    if (lane == 0 && nmax > 0) {
      const bool bf = p.is_bf16 != 0;
      const uint32_t idesc_s = attn_idesc(bf, 64, false, false);
      const uint32_t idesc_o = attn_idesc(bf, 128, false, true);
      const uint32_t sQ = smem_u32(smem), sDo = smem_u32(smem + C::kOffDo), sP = smem_u32(smem + C::kOffP);
      const uint32_t sK = smem_u32(smem + C::kOffK), sV = smem_u32(smem + C::kOffV);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicCAS(p.status, 0, kFlashTimeoutMma);
      // S (and dP) of block j for tile t
      auto issue_s = [&](int t, int j) -> bool {
        const int st = j % KS;
        const uint32_t par = (j / KS) & 1;
        if (!mbar_wait(&k_full[st], par)) return false;
        if (MODE == kDq && !mbar_wait(&v_full[st], par)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t a = umma_desc_k_sw128(sQ + t * 32768 + (k >> 2) * 16384) + (k & 3) * 2;
          const uint64_t bd = umma_desc_k_sw128(sK + st * C::kKvBytes + (k >> 2) * 8192) + (k & 3) * 2;
          umma_f16(tmem_base + C::kColS + t * 64, a, bd, idesc_s, k != 0);
        }
        if (MODE == kDq) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t a = umma_desc_k_sw128(sDo + t * 32768 + (k >> 2) * 16384) + (k & 3) * 2;
            const uint64_t bd = umma_desc_k_sw128(sV + st * C::kKvBytes + (k >> 2) * 8192) + (k & 3) * 2;
            umma_f16(tmem_base + C::kColDp + t * 64, a, bd, idesc_s, k != 0);
          }
        }
        tc_commit(&s_full[t]);
        const bool last = (t == 1) || (j >= n[1]);
        if (last) {
          // forward: the K block is done; dQ pass: the V block is done (K is still needed by dS K)
          if (MODE == kFwd) tc_commit(&k_empty[st]);
          else tc_commit(&v_empty[st]);
        }
        return true;
      };
      for (int t = 0; ok && t < 2; ++t)
        if (n[t] > 0) ok = issue_s(t, 0);
      if (!ok) atomicCAS(p.status, 0, kFlashTimeoutMma);
      for (int j = 0; ok && j < nmax; ++j) {
        const int st = j % KS;
        const uint32_t par = (j / KS) & 1;
        for (int t = 0; ok && t < 2; ++t) {
          if (j >= n[t]) continue;
          if (!mbar_wait(&p_ready[t], j & 1)) { ok = false; break; }
          if (MODE == kFwd && !mbar_wait(&v_full[st], par)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sB = (MODE == kFwd ? sV : sK) + st * C::kKvBytes;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t a = umma_desc_k_sw128(sP + t * 16384) + k * 2;
            const uint64_t bd = umma_desc_mn_sw128(sB, 8192) + k * (2048 >> 4);
            umma_f16(tmem_base + C::kColO + t * 128, a, bd, idesc_o, (j | k) != 0);
          }
          tc_commit(&pv_done[t]);
          const bool last = (t == 1) || (j >= n[1]);
          if (last) {
            if (MODE == kFwd) tc_commit(&v_empty[st]);
            else tc_commit(&k_empty[st]);
          }
          if (j + 1 < n[t]) ok = issue_s(t, j + 1);
        }
        if (!ok) atomicCAS(p.status, 0, kFlashTimeoutMma);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / dS warps
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;       // row inside the tile
    const int q_row = q0 + t * 128 + r;
    const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
    uint8_t* sP = smem + C::kOffP + t * 16384;
    const int nt = n[t];
    const float NEG_INF = -INFINITY;
    bool ok = true;
    float m_run = NEG_INF, l_run = 0.f;
    float lse2 = INFINITY, delta = 0.f;
    if (MODE == kDq && q_row < p.sq) {
      const size_t off = (static_cast<size_t>(b) * p.hq + h) * p.s_pad + q_row;
      lse2 = p.lse[off] * 1.4426950408889634f;
      delta = p.delta[off];
    }
    for (int j = 0; j < nt; ++j) {
      if (!mbar_wait(&s_full[t], j & 1)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * 64;
      const bool need_mask = (kv0 + 64 > p.sk) || (p.causal && kv0 + 63 > q0 + t * 128 + p.causal_off);
      const int lim = p.causal ? min(p.sk - 1, q_row + p.causal_off) : p.sk - 1;  // last visible key
      uint32_t w[32];
      if (MODE == kFwd) {
        uint32_t s0[32], s1[32];
        tmem_ld_32x32(lane_base + C::kColS + t * 64, s0);
        tmem_ld_32x32(lane_base + C::kColS + t * 64 + 32, s1);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (kv0 + c > lim) s0[c] = __float_as_uint(NEG_INF);
            if (kv0 + 32 + c > lim) s1[c] = __float_as_uint(NEG_INF);
          }
        }
        float mx = NEG_INF;
#pragma unroll
        for (int c = 0; c < 32; ++c) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
        const float m_new = fmaxf(m_run, mx * p.scale_log2);
        const bool first = m_run == NEG_INF;
        const float m_use = (!first && m_new - m_run <= 8.f) ? m_run : m_new;
        const float m_eff = m_use == NEG_INF ? 0.f : m_use;
        const float alpha = first ? 1.f : fast_exp2(m_run - m_use);
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float a0 = fast_exp2(fmaf(__uint_as_float(s0[c]), p.scale_log2, -m_eff));
          const float a1 = fast_exp2(fmaf(__uint_as_float(s0[c + 1]), p.scale_log2, -m_eff));
          const float b0 = fast_exp2(fmaf(__uint_as_float(s1[c]), p.scale_log2, -m_eff));
          const float b1 = fast_exp2(fmaf(__uint_as_float(s1[c + 1]), p.scale_log2, -m_eff));
          sum += (a0 + a1) + (b0 + b1);
          w[c / 2] = p.is_bf16 ? pack_bf16x2(a0, a1) : pack_f16x2(a0, a1);
          w[16 + c / 2] = p.is_bf16 ? pack_bf16x2(b0, b1) : pack_f16x2(b0, b1);
        }
        l_run = l_run * alpha + sum;
        m_run = m_use;
        if (j > 0) {
          if (!mbar_wait(&pv_done[t], (j - 1) & 1)) { ok = false; break; }
          tc_fence_after();
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 32) {
              uint32_t o[32];
              tmem_ld_32x32(lane_base + C::kColO + t * 128 + c0, o);
              tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
              tmem_st_32x32(lane_base + C::kColO + t * 128 + c0, o);
            }
            tmem_st_wait();
          }
        }
      } else {
        // dS = P * (dP - delta), P rebuilt from the saved log-sum-exp
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t s[32], dp[32];
          tmem_ld_32x32(lane_base + C::kColS + t * 64 + half * 32, s);
          tmem_ld_32x32(lane_base + C::kColDp + t * 64 + half * 32, dp);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(s[c]), p.scale_log2, -lse2));
            float p1 = fast_exp2(fmaf(__uint_as_float(s[c + 1]), p.scale_log2, -lse2));
            if (need_mask) {
              if (kv0 + half * 32 + c > lim) p0 = 0.f;
              if (kv0 + half * 32 + c + 1 > lim) p1 = 0.f;
            }
            const float d0 = p0 * (__uint_as_float(dp[c]) - delta);
            const float d1 = p1 * (__uint_as_float(dp[c + 1]) - delta);
            w[half * 16 + c / 2] = p.is_bf16 ? pack_bf16x2(d0, d1) : pack_f16x2(d0, d1);
          }
        }
        if (j > 0) {
          if (!mbar_wait(&pv_done[t], (j - 1) & 1)) { ok = false; break; }
        }
      }
      store_row_sw128(sP, r, w);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, kFlashTimeoutSoftmax);
    // ---------------------------------------------------------------- epilogue
    if (ok && nt > 0) {
      if (!mbar_wait(&pv_done[t], (nt - 1) & 1)) {
        ok = false;
        if (lane == 0) atomicCAS(p.status, 0, kFlashTimeoutSoftmax);
      }
      tc_fence_after();
    }
    // TMEM loads are warp-wide: every lane takes part, only the stores depend on the row
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const bool row_ok = q_row < p.sq;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + b * p.o_sb + h * p.o_sh + static_cast<long long>(q_row) * p.o_ss;
      const float mul = MODE == kFwd ? (l_run > 0.f ? 1.f / l_run : 0.f) : p.scale;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t o[32];
        if (nt > 0) {
          tmem_ld_32x32(lane_base + C::kColO + t * 128 + c0, o);
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
            for (int i = 0; i < 4; ++i) {
              const float x0 = __uint_as_float(o[c + 2 * i]) * mul, x1 = __uint_as_float(o[c + 2 * i + 1]) * mul;
              q4[i] = p.is_bf16 ? pack_bf16x2(x0, x1) : pack_f16x2(x0, x1);
            }
            *reinterpret_cast<uint4*>(orow + c0 + c) = make_uint4(q4[0], q4[1], q4[2], q4[3]);
          }
        }
      }
      if (MODE == kFwd && row_ok) {
        const size_t off = (static_cast<size_t>(b) * p.hq + h) * p.s_pad + q_row;
        p.lse[off] = l_run > 0.f ? m_run * 0.6931471805599453f + logf(l_run) : NEG_INF;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------- host side
bool make_tensor_map_bhsd(CUtensorMap* map, const void* base, bool bf16, int b, int h, int s, long long sb,
                          long long sh, long long ss, int box_rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return false;
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (sb * 2) % 16 || (sh * 2) % 16 || (ss * 2) % 16) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(s), static_cast<cuuint64_t>(h),
                        static_cast<cuuint64_t>(b)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss * 2), static_cast<cuuint64_t>(sh * 2),
                           static_cast<cuuint64_t>(sb * 2)};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int MODE>
static cudaError_t launch_qouter(const FlashArgs& a, cudaStream_t stream) {
  using C = QCfg<MODE>;
  CUtensorMap tq, tk, tv, tdo;
  const bool bf = a.is_bf16;
  bool ok = make_tensor_map_bhsd(&tq, a.q, bf, a.b, a.hq, a.sq, a.q_sb, a.q_sh, a.q_ss, 128) &&
            make_tensor_map_bhsd(&tk, a.k, bf, a.b, a.hk, a.sk, a.k_sb, a.k_sh, a.k_ss, 64) &&
            make_tensor_map_bhsd(&tv, a.v, bf, a.b, a.hk, a.sk, a.v_sb, a.v_sh, a.v_ss, 64);
  if (MODE == kDq) ok = ok && make_tensor_map_bhsd(&tdo, a.dout, bf, a.b, a.hq, a.sq, a.do_sb, a.do_sh, a.do_ss, 128);
  else tdo = tq;
  if (!ok) return cudaErrorInvalidValue;
  FlashParams p = {};
  p.b = a.b; p.hq = a.hq; p.hk = a.hk; p.sq = a.sq; p.sk = a.sk;
  p.causal = a.causal ? 1 : 0;
  p.causal_off = a.bottom_right ? a.sk - a.sq : 0;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.is_bf16 = bf ? 1 : 0;
  if (MODE == kFwd) { p.out = a.out; p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_ss = a.o_ss; }
  else { p.out = a.dq; p.o_sb = a.dq_sb; p.o_sh = a.dq_sh; p.o_ss = a.dq_ss; }
  if ((reinterpret_cast<uintptr_t>(p.out) & 15) || p.o_sb % 8 || p.o_sh % 8 || p.o_ss % 8) return cudaErrorInvalidValue;
  p.lse = a.lse; p.delta = a.delta; p.s_pad = a.s_pad; p.status = a.status;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(flash_qouter_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  dim3 grid((a.sq + 255) / 256, a.hq, a.b);
  flash_qouter_kernel<MODE><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError();
}

}  // namespace attn

cudaError_t flash_fwd(const FlashArgs& a, cudaStream_t stream) { return attn::launch_qouter<attn::kFwd>(a, stream); }
cudaError_t flash_bwd_dq(const FlashArgs& a, cudaStream_t stream) { return attn::launch_qouter<attn::kDq>(a, stream); }

}  // namespace teb200
