// Fused attention backward, key-stationary kernel: dK and dV.
//
// One CTA owns 128 key rows of one K/V head and walks every 64-row query block that can see
// them, for every query head of the GQA group.  Per query block, on transposed tiles:
//   S^T = K Q^T, dP^T = V dO^T           (tensor cores, accumulators in TMEM)
//   P^T = exp2(S^T*c - lse), dS^T = P^T * (dP^T - delta)      (softmax warps, thread = key row)
//   dV += P^T dO,  dK += dS^T Q          (A operands from TMEM; dO and Q blocks reused as MN-major B)
// Two groups of softmax warps alternate over the query blocks so that the tensor pipe and the
// exponentials overlap.  dK/dV stay in TMEM for the whole walk and are written once.
#include "flash_common.cuh"
#include "flash_qouter_softmax.cuh"

namespace teb200 {
namespace attn {

struct KvCfg {
  static constexpr int kRing = 4;
  static constexpr int kKBytes = 32768, kVBytes = 32768;
  static constexpr int kQBlk = 16384;                       // [64 x 128] Q or dO block
  static constexpr int kVecBytes = 256;                     // 64 floats of lse / delta
  static constexpr int kStageBytes = 2 * kQBlk + 2 * kVecBytes + 512;  // keep 1024-byte alignment
  static constexpr int kOffV = kKBytes;
  static constexpr int kOffRing = kOffV + kVBytes;
  static constexpr int kOffBar = kOffRing + kRing * kStageBytes;
  static constexpr int kNumBars = 1 + 2 * kRing + 2 + 2 + 1;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;
  static constexpr int kColS = 0, kColDp = 128, kColDv = 256, kColDk = 384;
};
static_assert(KvCfg::kStageBytes % 1024 == 0, "ring stages must keep the swizzle alignment");

template <bool BF, bool WIN>
__global__ void __launch_bounds__(kThreads, 1)
flash_kvouter_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const FlashParams p_launch) {
  using C = KvCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint64_t* kv_full = bars;
  uint64_t* r_full = bars + 1;             // [kRing]
  uint64_t* r_empty = r_full + C::kRing;   // [kRing]
  uint64_t* s_full = r_empty + C::kRing;   // [2]
  uint64_t* p_ready = s_full + 2;          // [2]
  uint64_t* acc_done = p_ready + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heads vary fastest, so CTAs start in order of decreasing causal work over ALL heads
  const int kb = blockIdx.y;
  const int hk = static_cast<int>(blockIdx.x) / p_launch.gsplit;
  const int gs = static_cast<int>(blockIdx.x) % p_launch.gsplit;  // which part of the head group
  const int b = blockIdx.z;
  FlashParams p = p_launch;
  const SeqView sv = localize(p, b);
  p.out = reinterpret_cast<uint16_t*>(p.out) + static_cast<long long>(sv.k_off) * p.o_ss + gs * p.o_sg;
  p.out2 = reinterpret_cast<uint16_t*>(p.out2) + static_cast<long long>(sv.k_off) * p.o_ss + gs * p.o_sg;
  const int G = p.hq / p.hk;
  const int Gl = G / p.gsplit;  // query heads of this CTA
  const int kv0 = kb * 128;
  int nq = kv0 < p.sk ? (p.sq + 63) / 64 : 0;  // a key block past the sequence's end has no work
  if (WIN && nq > 0) {  // sliding window: the last query that still sees the block's last key
    const int q_last = min(kv0 + 127, p.sk - 1) - p.lo_off;
    nq = q_last < 0 ? 0 : min(nq, q_last / 64 + 1);
  }
  int i_start = 0;
  if (p.causal) {
    const int first_q = kv0 - p.causal_off;  // first query row that sees key kv0
    i_start = first_q <= 0 ? 0 : first_q / 64;
  }
  const int ni = nq > i_start ? nq - i_start : 0;
  const int N = Gl * ni;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
    prefetch_tensormap(&tmap_do);
    mbar_init(kv_full, 1);
    for (int i = 0; i < C::kRing; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 1);
    }
    for (int u = 0; u < 2; ++u) {
      mbar_init(&s_full[u], 1);
      mbar_init(&p_ready[u], 8);
    }
    mbar_init(acc_done, 1);
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
    if (lane == 0 && N > 0) {
      mbar_expect_tx(kv_full, C::kKBytes + C::kVBytes);
      for (int pn = 0; pn < 2; ++pn) {
        tma_load_4d(smem + pn * 16384, &tmap_k, kv_full, pn * 64, sv.k_off + kv0, hk, sv.bt);
        tma_load_4d(smem + C::kOffV + pn * 16384, &tmap_v, kv_full, pn * 64, sv.k_off + kv0, hk, sv.bt);
      }
      for (int it = 0; it < N; ++it) {
        const int st = it % C::kRing;
        const int h = hk * G + gs * Gl + it / ni;
        const int qr = (i_start + it % ni) * 64;
        if (!mbar_wait(&r_empty[st], ((it / C::kRing) & 1) ^ 1)) { atomicCAS(p.status, 0, kFlashTimeoutProducer); break; }
        uint8_t* base = smem + C::kOffRing + st * C::kStageBytes;
        mbar_expect_tx(&r_full[st], 2 * C::kQBlk + 2 * C::kVecBytes);
        for (int pn = 0; pn < 2; ++pn) {
          tma_load_4d(base + pn * 8192, &tmap_q, &r_full[st], pn * 64, sv.q_off + qr, h, sv.bt);
          tma_load_4d(base + C::kQBlk + pn * 8192, &tmap_do, &r_full[st], pn * 64, sv.q_off + qr, h, sv.bt);
        }
        const size_t off = (static_cast<size_t>(b) * p.hq + h) * p.s_pad + qr;
        bulk_load_1d(base + 2 * C::kQBlk, p.lse + off, C::kVecBytes, &r_full[st]);
        bulk_load_1d(base + 2 * C::kQBlk + C::kVecBytes, p.delta + off, C::kVecBytes, &r_full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tcgen05 issuer
    // Descriptors are precomputed and the whole warp walks the loop, so that every value stays
    // warp-uniform; one elected lane issues the tcgen05 instructions.
    if (N > 0) {
      constexpr uint32_t idesc_s = attn_idesc(BF, 64, false, false);
      constexpr uint32_t idesc_acc = attn_idesc(BF, 128, false, true);
      const uint64_t dK = umma_desc_k_sw128(smem_u32(smem));
      const uint64_t dV = umma_desc_k_sw128(smem_u32(smem + C::kOffV));
      const uint64_t dRk = umma_desc_k_sw128(smem_u32(smem + C::kOffRing));        // Q block, K-major view
      const uint64_t dRmn = umma_desc_mn_sw128(smem_u32(smem + C::kOffRing), 8192);  // Q block, MN-major view
      constexpr uint32_t kDoOff = C::kQBlk >> 4;                                    // dO block follows Q
      bool ok = __all_sync(0xffffffffu, mbar_wait(kv_full, 0));
      auto issue_s = [&](int it) -> bool {
        const int st = it % C::kRing, u = it & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&r_full[st], (it / C::kRing) & 1))) return false;
        tc_fence_after();
        const uint64_t q = dRk + static_cast<uint64_t>(st * (C::kStageBytes >> 4));
        const uint32_t cs = tmem_base + C::kColS + u * 64, cd = tmem_base + C::kColDp + u * 64;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16(cs, dK + (((k >> 2) * 16384) >> 4) + (k & 3) * 2, q + (((k >> 2) * 8192) >> 4) + (k & 3) * 2,
                     idesc_s, k != 0);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16(cd, dV + (((k >> 2) * 16384) >> 4) + (k & 3) * 2,
                     q + kDoOff + (((k >> 2) * 8192) >> 4) + (k & 3) * 2, idesc_s, k != 0);
          tc_commit(&s_full[u]);
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int it = 0; ok && it < N; ++it) {
        const int st = it % C::kRing, u = it & 1;
        if (it + 1 < N) ok = issue_s(it + 1);
        if (!ok) break;
        if (!__all_sync(0xffffffffu, mbar_wait(&p_ready[u], (it >> 1) & 1))) { ok = false; break; }
        tc_fence_after();
        const uint64_t q = dRmn + static_cast<uint64_t>(st * (C::kStageBytes >> 4));
        // A = P^T / dS^T from TMEM, left by the softmax halves at the start of their own columns
        const uint32_t cp = tmem_base + C::kColS + u * 64, cd = tmem_base + C::kColDp + u * 64;
        if (elect_one()) {
          umma_f16_ts(tmem_base + C::kColDv, cp, q + kDoOff, idesc_acc, it != 0);
#pragma unroll
          for (int k = 1; k < 4; ++k)
            umma_f16_ts(tmem_base + C::kColDv, cp + (k >> 1) * 32 + (k & 1) * 8, q + kDoOff + k * (2048 >> 4),
                        idesc_acc, 1);
          umma_f16_ts(tmem_base + C::kColDk, cd, q, idesc_acc, it != 0);
#pragma unroll
          for (int k = 1; k < 4; ++k)
            umma_f16_ts(tmem_base + C::kColDk, cd + (k >> 1) * 32 + (k & 1) * 8, q + k * (2048 >> 4), idesc_acc, 1);
            tc_commit(&r_empty[st]);
        }
        __syncwarp();
      }
      if (ok) {
        if (elect_one()) tc_commit(acc_done);
      } else if (lane == 0) {
        atomicCAS(p.status, 0, kFlashTimeoutMma);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / dS warps
    const int u = (warp - 2) >> 3;       // group u takes iterations it with it % 2 == u
    const int half = ((warp - 2) & 7) >> 2;  // which 32 query columns / which 64 output columns
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int kv_row = kv0 + r;
    const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
    bool ok = true;
    for (int it = u; it < N; it += 2) {
      const int st = it % C::kRing;
      const int qr = (i_start + it % ni) * 64;
      if (!mbar_wait(&s_full[u], (it >> 1) & 1)) { ok = false; break; }
      __syncwarp();
      tc_fence_after();
      const float* vec = reinterpret_cast<const float*>(smem + C::kOffRing + st * C::kStageBytes + 2 * C::kQBlk);
      const bool need_mask = (kv0 + 128 > p.sk) || (qr + 64 > p.sq) || (p.causal && kv0 + 127 > qr + p.causal_off) ||
                             (WIN && qr + 63 > kv0 - p.lo_off);
      // key kv_row is visible to query q iff q >= q_min (and the key exists)
      const int q_min = kv_row < p.sk ? (p.causal ? kv_row - p.causal_off : 0) : 0x7fffffff;
      const int q_max = WIN ? kv_row - p.lo_off : 0x7fffffff;
      uint32_t wp[16], wd[16];
      {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(lane_base + C::kColS + u * 64 + half * 32, s);
        tmem_ld_32x32(lane_base + C::kColDp + u * 64 + half * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(vec + half * 32 + c);
          const float4 d4 = *reinterpret_cast<const float4*>(vec + 64 + half * 32 + c);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
          const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float x = fast_exp2(fmaf(__uint_as_float(s[c + e]), p.scale_log2, -ls[e] * 1.4426950408889634f));
            float y = x * (__uint_as_float(dp[c + e]) - dl[e]);
            if (need_mask) {
              const int q = qr + half * 32 + c + e;
              const bool vis = q >= q_min && q <= q_max && q < p.sq;
              x = vis ? x : 0.f;
              y = vis ? y : 0.f;
            }
            pv[e] = x;
            dv[e] = y;
          }
          wp[c / 2] = pack16<BF>(pv[0], pv[1]);
          wp[c / 2 + 1] = pack16<BF>(pv[2], pv[3]);
          wd[c / 2] = pack16<BF>(dv[0], dv[1]);
          wd[c / 2 + 1] = pack16<BF>(dv[2], dv[3]);
        }
      }
      // no wait for block it-2's products here: this block's scores were written after them (the
      // tensor pipe runs in issue order), so their operands have been read
      // P^T and dS^T return through TMEM over the columns this thread has just read
      tmem_st_32x16(lane_base + C::kColS + u * 64 + half * 32, wp);
      tmem_st_32x16(lane_base + C::kColDp + u * 64 + half * 32, wd);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[u]);
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, kFlashTimeoutSoftmax);
    // ---------------------------------------------------------------- epilogue: group 0 -> dK, group 1 -> dV
    if (ok && N > 0) {
      if (!mbar_wait(acc_done, 0)) {
        ok = false;
        if (lane == 0) atomicCAS(p.status, 0, kFlashTimeoutSoftmax);
      }
      tc_fence_after();
    }
    // TMEM loads are warp-wide: every lane takes part, only the stores depend on the row
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const bool row_ok = kv_row < p.sk;
      uint16_t* orow = reinterpret_cast<uint16_t*>(u == 0 ? p.out : p.out2) + b * p.o_sb + hk * p.o_sh +
                       static_cast<long long>(kv_row) * p.o_ss + half * 64;
      const float mul = u == 0 ? p.scale : 1.f;
      const uint32_t col0 = (u == 0 ? C::kColDk : C::kColDv) + half * 64;
#pragma unroll 1
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t o[32];
        if (N > 0) {
          tmem_ld_32x32(lane_base + col0 + c0, o);
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
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d dO * O, one warp per row
__global__ void flash_delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ dout, float* delta,
                                   int b, int h, int s, int s_pad, long long o_sb, long long o_sh, long long o_ss,
                                   long long d_sb, long long d_sh, long long d_ss, int is_bf16,
                                   const int* __restrict__ cu_q, const int* __restrict__ off_q) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long rows = static_cast<long long>(b) * h * s;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int si = static_cast<int>(row % s);
  const int hi = static_cast<int>((row / s) % h);
  const int bi = static_cast<int>(row / (static_cast<long long>(s) * h));
  long long tok = si;   // row of the [.., s, d] views
  long long bo = bi;    // their batch index
  if (cu_q != nullptr) {  // packed sequences: s is the longest length, the views have one batch entry
    if (si >= cu_q[bi + 1] - cu_q[bi]) return;
    tok = off_q[bi] + si;
    bo = 0;
  }
  const uint2 a = *reinterpret_cast<const uint2*>(o + bo * o_sb + hi * o_sh + tok * o_ss + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(dout + bo * d_sb + hi * d_sh + tok * d_ss + lane * 4);
  float acc = 0.f;
  const uint32_t aw[2] = {a.x, a.y}, gw[2] = {g.x, g.y};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float a0, a1, g0, g1;
    if (is_bf16) {
      a0 = __uint_as_float(aw[i] << 16); a1 = __uint_as_float(aw[i] & 0xffff0000u);
      g0 = __uint_as_float(gw[i] << 16); g1 = __uint_as_float(gw[i] & 0xffff0000u);
    } else {
      const __half2 ah = *reinterpret_cast<const __half2*>(&aw[i]);
      const __half2 gh = *reinterpret_cast<const __half2*>(&gw[i]);
      a0 = __low2float(ah); a1 = __high2float(ah); g0 = __low2float(gh); g1 = __high2float(gh);
    }
    acc += a0 * g0 + a1 * g1;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[(static_cast<size_t>(bi) * h + hi) * s_pad + si] = acc;
}

}  // namespace attn

cudaError_t flash_bwd_dkdv(const FlashArgs& a, cudaStream_t stream) {
  using namespace attn;
  using C = KvCfg;
  CUtensorMap tq, tk, tv, tdo;
  const bool bf = a.is_bf16;
  const bool varlen = a.cu_q != nullptr;
  if (varlen && (a.cu_k == nullptr || a.off_q == nullptr || a.off_k == nullptr || a.tq <= 0 || a.tk <= 0))
    return cudaErrorInvalidValue;
  if (a.b <= 0 || a.sq <= 0 || a.sk <= 0) return cudaSuccess;
  const int mb = varlen ? 1 : a.b, msq = varlen ? a.tq : a.sq, msk = varlen ? a.tk : a.sk;
  const bool ok = make_tensor_map_bhsd(&tq, a.q, bf, mb, a.hq, msq, a.q_sb, a.q_sh, a.q_ss, 64) &&
                  make_tensor_map_bhsd(&tk, a.k, bf, mb, a.hk, msk, a.k_sb, a.k_sh, a.k_ss, 128) &&
                  make_tensor_map_bhsd(&tv, a.v, bf, mb, a.hk, msk, a.v_sb, a.v_sh, a.v_ss, 128) &&
                  make_tensor_map_bhsd(&tdo, a.dout, bf, mb, a.hq, msq, a.do_sb, a.do_sh, a.do_ss, 64);
  if (!ok) return cudaErrorInvalidValue;
  if (a.s_pad % 64 != 0 || a.s_pad < ((a.sq + 63) / 64) * 64) return cudaErrorInvalidValue;
  if (a.dk_sb != a.dv_sb || a.dk_sh != a.dv_sh || a.dk_ss != a.dv_ss) return cudaErrorInvalidValue;
  FlashParams p = {};
  p.b = a.b; p.hq = a.hq; p.hk = a.hk; p.sq = a.sq; p.sk = a.sk;
  set_mask_params(p, a);
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.is_bf16 = bf ? 1 : 0;
  p.out = a.dk; p.out2 = a.dv; p.o_sb = a.dk_sb; p.o_sh = a.dk_sh; p.o_ss = a.dk_ss;
  if ((reinterpret_cast<uintptr_t>(a.dk) & 15) || (reinterpret_cast<uintptr_t>(a.dv) & 15) || p.o_sb % 8 || p.o_sh % 8 ||
      p.o_ss % 8)
    return cudaErrorInvalidValue;
  p.lse = a.lse; p.delta = a.delta; p.s_pad = a.s_pad; p.status = a.status;
  p.cu_q = a.cu_q; p.cu_k = a.cu_k; p.off_q = a.off_q; p.off_k = a.off_k;
  p.gsplit = a.gsplit < 1 ? 1 : a.gsplit;
  p.o_sg = a.dk_sg;
  if ((a.hq / a.hk) % p.gsplit != 0 || p.o_sg % 8 != 0) return cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    const void* fns[4] = {reinterpret_cast<const void*>(flash_kvouter_kernel<true, false>),
                          reinterpret_cast<const void*>(flash_kvouter_kernel<false, false>),
                          reinterpret_cast<const void*>(flash_kvouter_kernel<true, true>),
                          reinterpret_cast<const void*>(flash_kvouter_kernel<false, true>)};
    for (const void* fn : fns) {
      cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return e;
    }
    attr_set = true;
  }
  dim3 grid(a.hk * p.gsplit, (a.sk + 127) / 128, a.b);
  const bool win = p.has_lo != 0;
  if (bf && !win) flash_kvouter_kernel<true, false><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  else if (!win) flash_kvouter_kernel<false, false><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  else if (bf) flash_kvouter_kernel<true, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  else flash_kvouter_kernel<false, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError();
}

cudaError_t flash_delta(const FlashArgs& a, cudaStream_t stream) {
  const long long rows = static_cast<long long>(a.b) * a.hq * a.sq;
  if (rows == 0) return cudaSuccess;
  if (a.o_ss % 4 || a.o_sh % 4 || a.o_sb % 4 || a.do_ss % 4 || a.do_sh % 4 || a.do_sb % 4) return cudaErrorInvalidValue;
  const int warps = 8;
  const unsigned grid = static_cast<unsigned>((rows + warps - 1) / warps);
  attn::flash_delta_kernel<<<grid, warps * 32, 0, stream>>>(
      reinterpret_cast<const uint16_t*>(a.out), reinterpret_cast<const uint16_t*>(a.dout), a.delta, a.b, a.hq, a.sq,
      a.s_pad, a.o_sb, a.o_sh, a.o_ss, a.do_sb, a.do_sh, a.do_ss, a.is_bf16 ? 1 : 0, a.cu_q, a.off_q);
  return cudaGetLastError();
}

}  // namespace teb200
