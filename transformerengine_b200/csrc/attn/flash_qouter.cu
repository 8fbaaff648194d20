// Fused attention, query-stationary kernels: the forward pass and the dQ pass of the backward.
//
// One CTA owns 256 query rows of one head (two 128-row tiles) and walks the key/value sequence
// in blocks.  Per block and tile:
//   forward : S = Q K^T            -> softmax warps: P = exp2(S*c - m), row sums, lazy rescale
//             O += P V                of the TMEM accumulator when the row max moved by > 8
//   dQ pass : S = Q K^T, dP = dO V^T -> dS = P * (dP - delta)   (P rebuilt from the saved LSE)
//             dQ += dS K
// Warp roles: warp 0 feeds K/V blocks through TMA rings, warp 1 issues tcgen05.mma, and each
// tile has eight softmax warps (two per TMEM lane quarter, each taking 32 of the 64 columns).
// The forward walks keys 128 at a time (one tcgen05.mma costs about 60 cycles whatever its N, so
// N = 128 doubles the score product's rate), the dQ pass 64 at a time (TMEM holds S, dP and dQ of
// both tiles).  P (and dS) return to the tensor core through TMEM as the A
// operand: each softmax thread overwrites the start of the score columns it has just read.  A V
// block doubles as the MN-major B operand of P V, a K block as the MN-major B operand of dS K,
// so nothing is transposed and shared memory holds only Q, dO and the K/V rings.
// (Reference behaviour: common/fused_attn/fused_attn_f16_arbitrary_seqlen.cu, cuDNN graphs.)
#include <cstdlib>

#include "flash_common.cuh"
#include "flash_qouter_softmax.cuh"

namespace teb200 {
namespace attn {

enum { kFwd = 0, kDq = 1 };

template <int V>
struct IC {
  static constexpr int value = V;
};

template <int MODE>
struct QCfg {
  static constexpr int kBlockKv = MODE == kFwd ? 128 : 64;        // keys per step (MMA N of the score product)
  static constexpr int kKvStages = MODE == kFwd ? 2 : 3;
  static constexpr int kSBufs = 1;                                // score accumulators per tile
  static constexpr int kQBytes = 2 * 32768;                       // two Q tiles
  static constexpr int kDoBytes = MODE == kFwd ? 0 : 2 * 32768;   // two dO tiles
  static constexpr int kKvBytes = kBlockKv * 256;                 // one K or V block
  static constexpr int kPanel = kBlockKv * 128;                   // one 64-column panel of it
  static constexpr int kOffDo = kQBytes;
  static constexpr int kOffK = kOffDo + kDoBytes;
  static constexpr int kOffV = kOffK + kKvStages * kKvBytes;
  static constexpr int kOffBar = kOffV + kKvStages * kKvBytes;
  static constexpr int kNumBars = 1 + 4 * kKvStages + 8;
  static constexpr int kOffXchg = kOffBar + kNumBars * 8 + 24;    // row max / row sum exchange
  static constexpr int kXchgBytes = MODE == kFwd ? 2 * 2 * 2 * 128 * 8 : 0;
  static constexpr int kSmemBytes = kOffXchg + kXchgBytes + 1024;
  // TMEM columns
  static constexpr int kColS = 0;                              // + t * kBlockKv
  static constexpr int kColDp = 128;                           // + t * 64 (dQ pass)
  static constexpr int kColO = 256;                            // + t * 128
};

__device__ __forceinline__ int kv_blocks_of_tile(const FlashParams& p, int row0, int bk) {
  if (row0 >= p.sq) return 0;
  int kv_end = p.sk;
  if (p.causal) {
    const int lim = row0 + 128 + p.causal_off;  // exclusive bound for the tile's last row
    kv_end = lim < kv_end ? lim : kv_end;
  }
  return kv_end <= 0 ? 0 : (kv_end + bk - 1) / bk;
}

// WIN: sliding-window lower bound compiled in (kept out of the plain causal kernels)
template <int MODE, bool BF, bool WIN>
__global__ void __launch_bounds__(kThreads, 1)
flash_qouter_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const FlashParams p_launch) {
  using C = QCfg<MODE>;
  constexpr int KS = C::kKvStages;
  constexpr int SB = C::kSBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;
  uint64_t* v_empty = v_full + KS;
  uint64_t* s_full = v_empty + KS;   // [2 tiles][2 buffers]
  uint64_t* p_ready = s_full + 4;    // [2]
  uint64_t* pv_done = p_ready + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  unsigned long long* xchg = reinterpret_cast<unsigned long long*>(smem + C::kOffXchg);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heaviest query blocks of every head first
  FlashParams p = p_launch;
  const int nqb = (p.sq + 255) / 256;
  const int qb = nqb - 1 - static_cast<int>(blockIdx.x) / p.hq;
  const int h = static_cast<int>(blockIdx.x) % p.hq;
  const int b = blockIdx.y;
  const SeqView sv = localize(p, b);
  p.out = reinterpret_cast<uint16_t*>(p.out) + static_cast<long long>(sv.q_off) * p.o_ss;
  const int hk = h / (p.hq / p.hk);
  // first query row of the CTA's two tiles: neighbours, or (few CTAs, causal mask) tile i with tile
  // last - i, so that every CTA walks the same number of key blocks in total
  int qrow[2] = {qb * 256, qb * 256 + 128};
  if (p_launch.pair_balance) {
    const int nqt = (p_launch.sq + 127) / 128;
    const int lo = static_cast<int>(blockIdx.x) / p.hq, hi = nqt - 1 - lo;
    qrow[0] = lo < hi ? lo * 128 : nqt * 128;  // the middle tile of an odd count runs alone
    qrow[1] = hi * 128;
  }
  int n[2];
  constexpr int BK = C::kBlockKv;
  n[0] = kv_blocks_of_tile(p, qrow[0], BK);
  n[1] = kv_blocks_of_tile(p, qrow[1], BK);
  // sliding window: both tiles start at the first key block that the earlier tile can see
  int jbase = 0;
  if (WIN) {
    int lo = 0x7fffffff;
    for (int t = 0; t < 2; ++t)
      if (n[t] > 0) {
        const int first = qrow[t] + p.lo_off;
        lo = min(lo, first > 0 ? first / BK : 0);
      }
    jbase = lo == 0x7fffffff ? 0 : lo;
    n[0] = n[0] > jbase ? n[0] - jbase : 0;
    n[1] = n[1] > jbase ? n[1] - jbase : 0;
  }
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
    for (int i = 0; i < 4; ++i) mbar_init(&s_full[i], 1);
    for (int t = 0; t < 2; ++t) {
      mbar_init(&p_ready[t], 8);
      mbar_init(&pv_done[t], 1);
    }
    mbar_fence_init();
  }
  if (MODE == kFwd)
    for (int i = threadIdx.x; i < C::kXchgBytes / 8; i += kThreads) xchg[i] = 0ull;  // tag 0 = nothing published
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
          tma_load_4d(smem + t * 32768 + pn * 16384, &tmap_q, q_full, pn * 64, sv.q_off + qrow[t], h, sv.bt);
          if (MODE == kDq)
            tma_load_4d(smem + C::kOffDo + t * 32768 + pn * 16384, &tmap_do, q_full, pn * 64, sv.q_off + qrow[t], h, sv.bt);
        }
      for (int j = 0; j < nmax; ++j) {
        const int st = j % KS;
        const uint32_t par = ((j / KS) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par)) { atomicCAS(p.status, 0, kFlashTimeoutProducer); break; }
        mbar_expect_tx(&k_full[st], C::kKvBytes);
        for (int pn = 0; pn < 2; ++pn)
          tma_load_4d(smem + C::kOffK + st * C::kKvBytes + pn * C::kPanel, &tmap_k, &k_full[st], pn * 64, sv.k_off + (jbase + j) * BK, hk, sv.bt);
        if (!mbar_wait(&v_empty[st], par)) { atomicCAS(p.status, 0, kFlashTimeoutProducer); break; }
        mbar_expect_tx(&v_full[st], C::kKvBytes);
        for (int pn = 0; pn < 2; ++pn)
          tma_load_4d(smem + C::kOffV + st * C::kKvBytes + pn * C::kPanel, &tmap_v, &v_full[st], pn * 64, sv.k_off + (jbase + j) * BK, hk, sv.bt);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tcgen05 issuer
    // One thread issues every MMA, so its instruction stream is the pipeline's clock: all
    // descriptors are precomputed (low words in registers, tile and step offsets folded at
    // compile time).  The whole warp walks the loop so that every value stays warp-uniform (the
    // descriptors live in uniform registers); one elected lane issues the tcgen05 instructions.
    if (nmax > 0) {
      constexpr uint32_t idesc_s = attn_idesc(BF, BK, false, false);
      constexpr uint32_t idesc_o = attn_idesc(BF, 128, false, true);
      const uint64_t dQ = umma_desc_k_sw128(smem_u32(smem));
      const uint64_t dDo = umma_desc_k_sw128(smem_u32(smem + C::kOffDo));
      const uint64_t dK = umma_desc_k_sw128(smem_u32(smem + C::kOffK));
      const uint64_t dVk = umma_desc_k_sw128(smem_u32(smem + C::kOffV));
      const uint64_t dBmn = umma_desc_mn_sw128(smem_u32(smem + (MODE == kFwd ? C::kOffV : C::kOffK)), C::kPanel);
      bool ok = __all_sync(0xffffffffu, mbar_wait(q_full, 0));
      // S (and dP) of block j for tile T
      auto issue_s = [&](auto tc, int j) -> bool {
        constexpr int T = decltype(tc)::value;
        const int st = j % KS;
        const uint32_t par = (j / KS) & 1;
        const int buf = j % SB;
        bool w = mbar_wait(&k_full[st], par);
        if (MODE == kDq) w = w && mbar_wait(&v_full[st], par);
        if (!__all_sync(0xffffffffu, w)) return false;
        tc_fence_after();
        const bool stamp = p.timeline && blockIdx.x == 0 && blockIdx.y == 0 && T == 0 && j >= SB && j - SB < 64 && lane == 0;
        if (stamp) p.timeline[(j - SB) * 16 + 10] = clock64();
        const uint32_t col_s = tmem_base + C::kColS + T * BK;
        const uint64_t kst = dK + static_cast<uint64_t>(st * (C::kKvBytes >> 4));
        const uint64_t vst = dVk + static_cast<uint64_t>(st * (C::kKvBytes >> 4));
        const bool last = T == 1 || j >= n[1];
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16(col_s, dQ + ((T * 32768 + (k >> 2) * 16384) >> 4) + (k & 3) * 2,
                     kst + (((k >> 2) * C::kPanel) >> 4) + (k & 3) * 2, idesc_s, k != 0);
          if (MODE == kDq) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_f16(tmem_base + C::kColDp + T * 64, dDo + ((T * 32768 + (k >> 2) * 16384) >> 4) + (k & 3) * 2,
                       vst + (((k >> 2) * C::kPanel) >> 4) + (k & 3) * 2, idesc_s, k != 0);
          }
          tc_commit(&s_full[T * 2 + buf]);
          // forward: the K block is done; dQ pass: the V block is done (K is still needed by dS K)
          if (last) tc_commit(MODE == kFwd ? &k_empty[st] : &v_empty[st]);
        }
        __syncwarp();
        if (stamp) p.timeline[(j - SB) * 16 + 11] = clock64();
        return true;
      };
      // O += P V (dQ += dS K) of block j for tile T, then the next score block into the freed buffer
      auto step = [&](auto tc, int j) -> bool {
        constexpr int T = decltype(tc)::value;
        const int st = j % KS;
        bool w = mbar_wait(&p_ready[T], j & 1);
        if (MODE == kFwd) w = w && mbar_wait(&v_full[st], (j / KS) & 1);
        if (!__all_sync(0xffffffffu, w)) return false;
        tc_fence_after();
        const bool stamp = p.timeline && blockIdx.x == 0 && blockIdx.y == 0 && T == 0 && j < 64 && lane == 0;
        if (stamp) p.timeline[j * 16 + 6] = clock64();
        const uint64_t bst = dBmn + static_cast<uint64_t>(st * (C::kKvBytes >> 4));
        // A = P (or dS) from TMEM: each softmax half left its BK/2 keys as BK/4 packed columns at
        // the start of its own BK/2 score columns; one step takes 16 keys = 8 columns
        const uint32_t col_p = tmem_base + C::kColS + T * BK;
        const uint32_t col_o = tmem_base + C::kColO + T * 128;
        const bool last = T == 1 || j >= n[1];
        if (elect_one()) {
          umma_f16_ts(col_o, col_p, bst, idesc_o, j != 0);
#pragma unroll
          for (int k = 1; k < BK / 16; ++k)
            umma_f16_ts(col_o, col_p + (k / (BK / 32)) * (BK / 2) + (k % (BK / 32)) * 8, bst + k * (2048 >> 4), idesc_o, 1);
          tc_commit(&pv_done[T]);
          if (last) tc_commit(MODE == kFwd ? &v_empty[st] : &k_empty[st]);
        }
        __syncwarp();
        if (stamp) p.timeline[j * 16 + 9] = clock64();
        bool r = true;
        if (j + SB < n[T]) r = issue_s(tc, j + SB);
        if (stamp) p.timeline[j * 16 + 7] = clock64();
        return r;
      };
      for (int jj = 0; ok && jj < SB; ++jj) {
        if (ok && jj < n[0]) ok = issue_s(IC<0>{}, jj);
        if (ok && jj < n[1]) ok = issue_s(IC<1>{}, jj);
      }
      for (int j = 0; ok && j < nmax; ++j) {
        if (j < n[0]) ok = step(IC<0>{}, j);
        if (ok && j < n[1]) ok = step(IC<1>{}, j);
      }
      if (!ok && lane == 0) atomicCAS(p.status, 0, kFlashTimeoutMma);
    }
  } else {
    const int t = (warp - 2) >> 3;
    qouter_softmax_role<MODE, BF, C, WIN>(p, smem, s_full, p_ready, pv_done, xchg, tmem_base, warp, lane, qrow[t] - t * 128, h, b, n[t], t, jbase);
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
  const bool varlen = a.cu_q != nullptr;
  if (varlen && (a.cu_k == nullptr || a.off_q == nullptr || a.off_k == nullptr || a.tq <= 0 || a.tk <= 0))
    return cudaErrorInvalidValue;
  const int mb = varlen ? 1 : a.b, msq = varlen ? a.tq : a.sq, msk = varlen ? a.tk : a.sk;
  bool ok = make_tensor_map_bhsd(&tq, a.q, bf, mb, a.hq, msq, a.q_sb, a.q_sh, a.q_ss, 128) &&
            make_tensor_map_bhsd(&tk, a.k, bf, mb, a.hk, msk, a.k_sb, a.k_sh, a.k_ss, C::kBlockKv) &&
            make_tensor_map_bhsd(&tv, a.v, bf, mb, a.hk, msk, a.v_sb, a.v_sh, a.v_ss, C::kBlockKv);
  if (MODE == kDq) ok = ok && make_tensor_map_bhsd(&tdo, a.dout, bf, mb, a.hq, msq, a.do_sb, a.do_sh, a.do_ss, 128);
  else tdo = tq;
  if (!ok) return cudaErrorInvalidValue;
  FlashParams p = {};
  p.b = a.b; p.hq = a.hq; p.hk = a.hk; p.sq = a.sq; p.sk = a.sk;
  set_mask_params(p, a);
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.is_bf16 = bf ? 1 : 0;
  if (MODE == kFwd) { p.out = a.out; p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_ss = a.o_ss; }
  else { p.out = a.dq; p.o_sb = a.dq_sb; p.o_sh = a.dq_sh; p.o_ss = a.dq_ss; }
  if ((reinterpret_cast<uintptr_t>(p.out) & 15) || p.o_sb % 8 || p.o_sh % 8 || p.o_ss % 8) return cudaErrorInvalidValue;
  p.lse = a.lse; p.delta = a.delta; p.s_pad = a.s_pad; p.status = a.status; p.timeline = a.timeline;
  p.cu_q = a.cu_q; p.cu_k = a.cu_k; p.off_q = a.off_q; p.off_k = a.off_k;
  p.gsplit = 1; p.o_sg = 0;
  if (a.sq <= 0 || a.b <= 0) return cudaSuccess;
  if (a.s_pad < a.sq) return cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    const void* fns[4] = {reinterpret_cast<const void*>(flash_qouter_kernel<MODE, true, false>),
                          reinterpret_cast<const void*>(flash_qouter_kernel<MODE, false, false>),
                          reinterpret_cast<const void*>(flash_qouter_kernel<MODE, true, true>),
                          reinterpret_cast<const void*>(flash_qouter_kernel<MODE, false, true>)};
    for (const void* fn : fns) {
      cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return e;
    }
    attr_set = true;
  }
  dim3 grid(((a.sq + 255) / 256) * a.hq, a.b);
  static const bool allow_pair = []() {
    const char* e = std::getenv("TEB200_ATTN_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  p.pair_balance = allow_pair && a.causal && a.window_left < 0 && static_cast<long long>(grid.x) * grid.y <= 148 ? 1 : 0;
  const bool win = p.has_lo != 0;
  if (bf && !win) flash_qouter_kernel<MODE, true, false><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  else if (!win) flash_qouter_kernel<MODE, false, false><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  else if (bf) flash_qouter_kernel<MODE, true, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  else flash_qouter_kernel<MODE, false, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError();
}

}  // namespace attn

cudaError_t flash_fwd(const FlashArgs& a, cudaStream_t stream) { return attn::launch_qouter<attn::kFwd>(a, stream); }
cudaError_t flash_bwd_dq(const FlashArgs& a, cudaStream_t stream) { return attn::launch_qouter<attn::kDq>(a, stream); }

}  // namespace teb200
