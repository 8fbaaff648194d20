// GEMM on CTA pairs (tcgen05 cta_group::2): D[M,N] = alpha * A[M,K] * B[N,K]^T with a 256x256
// tile per pair of SMs.  Each CTA of a pair loads its own 128 rows of A and only HALF of the
// B tile (128 rows); the tensor cores of both SMs read both halves, so bytes fetched from L2
// per flop drop by a third against one 128x256 tile per CTA, which is what limits the
// single-CTA kernel (its TMA feed is latency bound with all shared memory in use).
//
//   CTA rank 0 (leader): TMA producer, MMA issuer for the pair, epilogue of rows 0..127
//   CTA rank 1 (partner): TMA producer (signals the leader's barriers), epilogue of rows 128..255
//   (10 warps per CTA: producer, MMA issuer, eight epilogue warps)
//
// Epilogue: eight warps per CTA read the whole accumulator into registers (four back-to-back TMEM loads
// per thread, one wait), release it at once, then convert and stage the values in shared memory
// (128-byte-swizzled boxes); TMA stores (TMA reduce-adds when accumulating into fp32) carry the boxes to
// global memory while the next tile's MMAs already run.
//
// "Stage full" barriers live in the leader and count the bytes of both CTAs; "stage empty" and
// "accumulator full" are committed to the same-offset barrier of both CTAs; "accumulator empty"
// lives in the leader and is arrived on by the epilogue warps of both CTAs.  All loads fill
// only the issuing CTA's shared memory.  Every wait is bounded.
#include <cstdlib>
#include <teb200/api.h>
#include <teb200/gemm_common.cuh>
#include <teb200/ptx.cuh>

namespace teb200 {
namespace {

using namespace gemm_detail;

// producer warp, MMA warp and EW epilogue warps (4: each warp drains both column halves in turn; 8: one half
// per warp, the accumulator is released after a single round of loads)
constexpr int pair_threads(int ew) { return 64 + ew * 32; }
constexpr int PM = 256;   // rows per pair tile
constexpr int PN = 256;   // columns per pair tile

template <int KIND>
struct PairCfg {
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = (PN / 2) * 128;
  static constexpr int kSfaBytes = KIND == kKindMxf8 ? 512 : 0;
  static constexpr int kSfbBytes = KIND == kKindMxf8 ? 512 * (PN / 128) : 0;
  static constexpr int kStageBytes = ((kABytes + kBBytes + kSfaBytes + kSfbBytes + 1023) / 1024) * 1024;
  // epilogue staging: two boxes of 128 rows x 128 bytes (ping-pong), written by the epilogue warps and
  // read by TMA stores, so the accumulator is drained at shared-memory speed
  static constexpr int kBoxBytes = 128 * 128;
  static constexpr int kStagingBytes = 2 * kBoxBytes;
  static constexpr int kStages = (227 * 1024 - 2048 - kStagingBytes) / kStageBytes;
  static constexpr int kSfaCols = KIND == kKindMxf8 ? 4 : 0;
  static constexpr int kSfbCols = KIND == kKindMxf8 ? 4 * (PN / 128) : 0;
  static constexpr int kAccStages = (2 * PN + kSfaCols + kSfbCols <= 512) ? 2 : 1;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 2048;
  static constexpr int kBlockK = KIND == kKindF16 ? 64 : 128;
  // bytes that land per stage over BOTH CTAs (every CTA loads the whole B scale block)
  static constexpr uint32_t kTxBytes = 2u * (kABytes + kBBytes + kSfaBytes + kSfbBytes);
};

struct PairParams {
  KernelParams k;
  int num_m, num_n;  // pair tiles
};

__device__ __forceinline__ bool pair_tile(const PairParams& p, int t, int& mb, int& nb) {
  if (t >= p.num_m * p.num_n) return false;
  const int per_group = kGroupM * p.num_n;
  const int g = t / per_group;
  const int first = g * kGroupM;
  const int gsize = min(p.num_m - first, kGroupM);
  const int r = t - g * per_group;
  mb = first + r % gsize;
  nb = r / gsize;
  return true;
}

template <int KIND, int EW>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads(EW), 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                 const __grid_constant__ CUtensorMap tmap_d, const PairParams p) {
  using C = PairCfg<KIND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + C::kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::kStagingBytes);
  uint64_t* full_bar = bars;                       // used in the leader only
  uint64_t* empty_bar = bars + C::kStages;         // one copy per CTA
  uint64_t* tfull_bar = bars + 2 * C::kStages;     // one copy per CTA
  uint64_t* tempty_bar = tfull_bar + C::kAccStages;  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + C::kAccStages);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_k_blocks = (p.k.K + C::kBlockK - 1) / C::kBlockK;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    prefetch_tensormap(&tmap_d);
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < C::kAccStages; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 2 * EW);  // every epilogue warp of the two CTAs
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs exist before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sfa = tmem_base + C::kAccStages * PN;
  const uint32_t tmem_sfb = tmem_sfa + C::kSfaCols;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int mb, nb;
      for (int t = pair; ok && pair_tile(p, t, mb, nb); t += num_pairs) {
        const int m0 = mb * PM + static_cast<int>(rank) * 128;       // this CTA's rows of A
        const int nrow0 = nb * PN + static_cast<int>(rank) * (PN / 2);  // this CTA's half of B
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1)) {
            if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutProducer);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[stage]), 0);  // the leader's barrier
          if (leader) mbar_expect_tx(&full_bar[stage], C::kTxBytes);
          const int kc = KIND == kKindF16 ? kb * C::kBlockK : kb * 128;
          tma_load_2d_pair(sa, &tmap_a, fb, kc, m0);
          tma_load_2d_pair(sb, &tmap_b, fb, kc, nrow0);
          if constexpr (KIND == kKindMxf8) {
            uint8_t* ssfa = sb + C::kBBytes;
            uint8_t* ssfb = ssfa + C::kSfaBytes;
            // scale buffers are addressed as [tile][128 words]: tile = row_tile * k_tiles + k
            tma_load_2d_pair(ssfa, &tmap_sfa, fb, 0, (m0 / 128) * p.k.sf_k_tiles + kb);
#pragma unroll
            for (int j = 0; j < PN / 128; ++j)
              tma_load_2d_pair(ssfb + j * 512, &tmap_sfb, fb, 0, (nb * (PN / 128) + j) * p.k.sf_k_tiles + kb);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    // The whole warp walks the loop so that every value is warp-uniform (descriptors stay in
    // uniform registers); one elected lane issues the tcgen05 instructions.
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int mb, nb;
      const uint64_t adesc0 = umma_desc_k_sw128(smem_u32(smem));
      const uint32_t e_bar0 = map_to_cta(smem_u32(&empty_bar[0]), 0), e_bar1 = map_to_cta(smem_u32(&empty_bar[0]), 1);
      const uint32_t t_bar0 = map_to_cta(smem_u32(&tfull_bar[0]), 0), t_bar1 = map_to_cta(smem_u32(&tfull_bar[0]), 1);
      for (int t = pair; ok && pair_tile(p, t, mb, nb); t += num_pairs) {
        if (!__all_sync(0xffffffffu, mbar_wait_cluster(&tempty_bar[acc], acc_phase ^ 1))) {
          if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * PN;
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait_cluster(&full_bar[stage], phase))) {
            if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = adesc0 + static_cast<uint64_t>(stage * (C::kStageBytes >> 4));
          const uint64_t bdesc = adesc + (C::kABytes >> 4);
          if (elect_one()) {
            if constexpr (KIND == kKindF16) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_f16_pair(tmem_d, adesc + k * 2, bdesc + k * 2, p.k.idesc, (kb | k) != 0);
            } else {
              const uint32_t ssfa = smem_u32(smem + stage * C::kStageBytes) + C::kABytes + C::kBBytes;
              const uint32_t ssfb = ssfa + C::kSfaBytes;
              utccp_sf_pair(tmem_sfa, umma_desc_sf(ssfa));
#pragma unroll
              for (int j = 0; j < PN / 128; ++j) utccp_sf_pair(tmem_sfb + j * 4, umma_desc_sf(ssfb + j * 512));
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t idesc = p.k.idesc | (uint32_t(k) << 29) | (uint32_t(k) << 4);
                umma_mxf8_pair(tmem_d, adesc + k * 2, bdesc + k * 2, idesc, (kb | k) != 0, tmem_sfa, tmem_sfb);
              }
            }
            // the stage may be refilled in both CTAs once these MMAs have read it
            tc_commit_pair(e_bar0 + stage * 8);
            tc_commit_pair(e_bar1 + stage * 8);
          }
          __syncwarp();
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) {
          tc_commit_pair(t_bar0 + acc * 8);
          tc_commit_pair(t_bar1 + acc * 8);
        }
        __syncwarp();
        if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    // Eight warps: warp w reads the TMEM lanes of quarter w % 4 (its rows) and the column half (w - 2) / 4.
    // Each thread pulls its 128 accumulator columns with four back-to-back loads and ONE wait, releases the
    // accumulator, and only then converts and stages the values: the tensor core waits for loads, not stores.
    constexpr int kHalvesPerWarp = EW == 8 ? 1 : 2;
    const int quarter = warp & 3;
    const int half0 = EW == 8 ? (warp - 2) >> 2 : 0;   // 0: columns 0..127, 1: columns 128..255
    const int et = quarter * 32 + lane;        // row of this thread inside the CTA's 128 rows
    const bool issuer = quarter == 2 && lane == 0;     // lane 0 of the first warp of a group of four
    int acc = 0;
    uint32_t acc_phase = 0;
    const float alpha = p.k.alpha * (p.k.alpha_dev ? *p.k.alpha_dev : 1.0f);
    const int dt = p.k.d_dtype;
    const bool wide = dt == kFloat32;          // a box (128 bytes per row) holds 32 fp32 or 64 16-bit columns
    const int sw = et & 7;
    const uint32_t bar_id = 1 + (EW == 8 ? half0 : 0);   // the four warps that share a box buffer
    uint32_t in_flight = 0;                    // bit h: a TMA store may still be reading the buffer of half h
    int mb, nb;
    bool dead = false;  // a wait ran out: keep walking the loop (the named barriers need every warp), wait no more
    for (int t = pair; pair_tile(p, t, mb, nb); t += num_pairs) {
      if (!dead && !mbar_wait_cluster(&tfull_bar[acc], acc_phase)) {
        if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutEpilogue);
        dead = true;
      }
      tc_fence_after();
      const int row0 = mb * PM + static_cast<int>(rank) * 128;
#pragma unroll 1
      for (int hh = 0; hh < kHalvesPerWarp; ++hh) {
      const int half = half0 + hh;
      uint8_t* box = staging + half * C::kBoxBytes;   // one 16 KB box buffer per column half
      uint8_t* my_row = box + et * 128;
      const int n0 = nb * PN + half * 128;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * PN + half * 128;
      uint32_t r[4][32];
#pragma unroll
      for (int j = 0; j < 4; ++j) tmem_ld_32x32(taddr + j * 32, r[j]);
      tmem_ld_wait();
      if (hh == kHalvesPerWarp - 1) {
        // every column of the accumulator is in registers: the MMA warp may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      }
      if (p.k.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = n0 + j * 32 + i;
            float b = 0.f;
            if (col < p.k.N) {
              if (p.k.bias_dtype == kFloat32) b = reinterpret_cast<const float*>(p.k.bias)[col];
              else if (p.k.bias_dtype == kBFloat16) b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.k.bias)[col]);
              else b = __half2float(reinterpret_cast<const __half*>(p.k.bias)[col]);
            }
            r[j][i] = __float_as_uint(__uint_as_float(r[j][i]) * alpha + b);
          }
        }
      } else if (alpha != 1.0f) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int i = 0; i < 32; ++i) r[j][i] = __float_as_uint(__uint_as_float(r[j][i]) * alpha);
      }
      const int nboxes = wide ? 4 : 2;
#pragma unroll
      for (int bx = 0; bx < 4; ++bx) {
        if (bx < nboxes) {
          if (in_flight & (1u << half)) {
            if (issuer) tma_store_wait_read<0>();   // every earlier store has finished reading shared memory
            named_bar_sync(bar_id, 128);
          }
          if (wide) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(my_row + ((c ^ sw) << 4)) =
                  make_uint4(r[bx][4 * c], r[bx][4 * c + 1], r[bx][4 * c + 2], r[bx][4 * c + 3]);
          } else {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int j = (2 * bx + hh) & 3;   // bx < 2 on this path
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int i = 8 * c;
                const float v0 = __uint_as_float(r[j][i]), v1 = __uint_as_float(r[j][i + 1]);
                const float v2 = __uint_as_float(r[j][i + 2]), v3 = __uint_as_float(r[j][i + 3]);
                const float v4 = __uint_as_float(r[j][i + 4]), v5 = __uint_as_float(r[j][i + 5]);
                const float v6 = __uint_as_float(r[j][i + 6]), v7 = __uint_as_float(r[j][i + 7]);
                uint4 o;
                if (dt == kBFloat16)
                  o = make_uint4(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3), pack_bf16x2(v4, v5), pack_bf16x2(v6, v7));
                else
                  o = make_uint4(pack_f16x2(v0, v1), pack_f16x2(v2, v3), pack_f16x2(v4, v5), pack_f16x2(v6, v7));
                *reinterpret_cast<uint4*>(my_row + (((hh * 4 + c) ^ sw) << 4)) = o;
              }
            }
          }
          fence_proxy_async_smem();  // generic-proxy writes to shared memory -> TMA (async proxy) read
          named_bar_sync(bar_id, 128);
          if (issuer) {
            const int col = n0 + bx * (wide ? 32 : 64);
            if (col < p.k.N && row0 < p.k.M) {   // boxes wholly outside the matrix are skipped, the rest is clipped
              if (p.k.accumulate) tma_reduce_add_2d(&tmap_d, box, col, row0);
              else tma_store_2d(&tmap_d, box, col, row0);
            }
            tma_store_commit();
          }
          in_flight |= 1u << half;
        }
      }
      }
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) tma_store_wait<0>();  // shared memory stays valid until the last store has read it
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or exits while its partner may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int KIND, int EW>
cudaError_t launch_pair(const GemmArgs& a, cudaStream_t stream) {
  using C = PairCfg<KIND>;
  CUtensorMap ta, tb, tsa, tsb;
  bool ok;
  const int k_tiles = KIND == kKindMxf8 ? (a.sf_k_tiles > 0 ? a.sf_k_tiles : ((a.K + 31) / 32 + 3) / 4) : 0;
  if (KIND == kKindF16) {
    ok = make_tensor_map_2d(&ta, a.a, a.a_dtype, a.M, a.K, a.lda, 128, 64, true) &&
         make_tensor_map_2d(&tb, a.b, a.b_dtype, a.N, a.K, a.ldb, PN / 2, 64, true);
    tsa = ta;
    tsb = tb;
  } else {
    ok = make_tensor_map_2d(&ta, a.a, kByte, a.M, a.K, a.lda, 128, 128, true) &&
         make_tensor_map_2d(&tb, a.b, kByte, a.N, a.K, a.ldb, PN / 2, 128, true);
    // scale buffers as [number of 512-byte tiles][128 x 4-byte words]
    const uint64_t ta_tiles = static_cast<uint64_t>((a.M + 127) / 128) * k_tiles;
    const uint64_t tb_tiles = static_cast<uint64_t>((a.N + 127) / 128) * k_tiles;
    ok = ok && make_tensor_map_2d(&tsa, a.sfa, kFloat32, ta_tiles, 128, 128, 1, 128, false) &&
         make_tensor_map_2d(&tsb, a.sfb, kFloat32, tb_tiles, 128, 128, 1, 128, false);
  }
  // output boxes: 128 rows x 128 bytes, 128-byte swizzle (what the epilogue writes to shared memory)
  CUtensorMap td;
  const int d_es = a.d_dtype == kFloat32 ? 4 : 2;
  ok = ok && make_tensor_map_2d(&td, a.d, a.d_dtype, a.M, a.N, a.ldd, 128, 128 / d_es, true);
  if (!ok) return cudaErrorInvalidValue;
  PairParams p = {};
  KernelParams& k = p.k;
  k.d = a.d; k.bias = a.bias; k.aux = nullptr; k.sfa = a.sfa; k.sfb = a.sfb; k.alpha_dev = a.alpha_dev;
  k.group_offsets = nullptr; k.status = a.status; k.alpha = a.alpha;
  k.M = a.M; k.N = a.N; k.K = a.K; k.ldd = a.ldd;
  k.d_dtype = a.d_dtype; k.bias_dtype = a.bias_dtype; k.epilogue = a.epilogue;
  k.accumulate = a.accumulate ? 1 : 0; k.a_mn = 0; k.b_mn = 0;
  // instruction shape of the pair: M = 256, N = 256
  uint32_t idesc = make_idesc(KIND, a.a_dtype, a.b_dtype, PN, false, false);
  idesc &= ~(0x1Fu << 24);
  idesc |= (uint32_t(PM) >> 4) << 24;
  k.idesc = idesc;
  k.num_groups = 0;
  k.sf_k_tiles = k_tiles;
  p.num_m = (a.M + PM - 1) / PM;
  p.num_n = (a.N + PN - 1) / PN;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<KIND, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const long long tiles = static_cast<long long>(p.num_m) * p.num_n;
  const int sms = a.sm_count > 0 ? a.sm_count : device_sm_count();
  // pairs that can be resident at once (a pair must sit inside one GPC)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms - sms % 2);
    cfg.blockDim = dim3(pair_threads(EW));
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<KIND, EW>, &cfg) != cudaSuccess || n <= 0) n = sms / 2;
    max_pairs = n;
  }
  long long pairs = max_pairs < sms / 2 ? max_pairs : sms / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) pairs = 1;
  gemm_pair_kernel<KIND, EW><<<static_cast<int>(pairs * 2), pair_threads(EW), C::kSmemBytes, stream>>>(ta, tb, tsa, tsb, td, p);
  return cudaGetLastError();
}

}  // namespace

bool gemm_pair_supported(const GemmArgs& a, bool mxfp8) {
  if (a.num_groups > 0 || a.a_mn_major || a.b_mn_major) return false;
  if (a.epilogue != kEpiNone && a.epilogue != kEpiBias) return false;
  if (a.M < 256 || a.N < 256) return false;
  if (mxfp8 && a.K % 128 != 0) return false;
  // the epilogue leaves through TMA: 16-byte aligned output rows; accumulation is a TMA reduce-add (fp32 only)
  const int d_es = a.d_dtype == kFloat32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(a.d) & 15) != 0 || (a.ldd * d_es) % 16 != 0) return false;
  if (a.accumulate && a.d_dtype != kFloat32) return false;
  return true;
}

// TEB200_GEMM_EPI_WARPS=4 selects the four-warp epilogue (experiment knob; default eight)
static int epilogue_warps() {
  static const char* env = getenv("TEB200_GEMM_EPI_WARPS");
  return (env != nullptr && atoi(env) == 4) ? 4 : 8;
}

cudaError_t gemm_pair_bf16(const GemmArgs& a, cudaStream_t s) {
  return epilogue_warps() == 4 ? launch_pair<kKindF16, 4>(a, s) : launch_pair<kKindF16, 8>(a, s);
}
cudaError_t gemm_pair_mxfp8(const GemmArgs& a, cudaStream_t s) {
  return epilogue_warps() == 4 ? launch_pair<kKindMxf8, 4>(a, s) : launch_pair<kKindMxf8, 8>(a, s);
}

}  // namespace teb200
