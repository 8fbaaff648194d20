// Persistent warp-specialised GEMM for sm_100a: D[M,N] = alpha * A[M,K] * B[N,K]^T.
//
//   warp 0      TMA producer   (one elected lane): fills a ring of shared-memory stages
//   warp 1      MMA issuer     (one elected lane): tcgen05.mma into TMEM accumulators,
//                              tcgen05.commit releases stages / publishes accumulators
//   warps 2-5   epilogue       tcgen05.ld TMEM -> registers -> (alpha, bias, act, accumulate) -> global
//
// Kinds: 16-bit (bf16 / fp16, K- or MN-major operands), MXFP8 (e4m3/e5m2 with one
// UE8M0 scale per 32 values, tcgen05 kind::mxf8f6f4.block_scale) and NVFP4 (e2m1 with
// one E4M3 scale per 16 values, kind::mxf4nvf4.block_scale.block16).  Block scales
// are read from global memory in the 128x4-tile layout, so one 128-row x 4-scale tile is a
// contiguous 512-byte chunk that is bulk-copied to shared memory and moved to TMEM
// with tcgen05.cp.  Replaces the cuBLASLt adapter of the reference
// (common/gemm/cublaslt_gemm.cu:315-783) and its grouped variant
// (common/gemm/cublaslt_grouped_gemm.cu:1577).
//
// Every mbarrier wait is bounded; on a time-out the role writes a status code
// and leaves its loop, all roles meet at the final barrier and TMEM is freed.
#include <teb200/api.h>
#include <teb200/gemm_common.cuh>
#include <teb200/ptx.cuh>

#include <cstdlib>

namespace teb200 {

namespace {

using namespace gemm_detail;

struct TileInfo {
  int m0, n0;       // first row / column of the tile in D
  int m_end;        // rows >= m_end are not stored (group boundary or M)
  int b_row0;       // first row of the B panel
  int sfa_row_tile; // 128-row tile index into the A scale layout
  int sfb_row_tile;
};

// Static persistent schedule; grouped mode walks the per-group m-block counts.
__device__ __forceinline__ bool get_tile(const KernelParams& p, int BN, int tile, TileInfo& ti) {
  const int num_n = (p.N + BN - 1) / BN;
  if (p.num_groups == 0) {
    const int num_m = (p.M + kBlockM - 1) / kBlockM;
    if (tile >= num_m * num_n) return false;
    const int per_group = kGroupM * num_n;
    const int g = tile / per_group;
    const int first_m = g * kGroupM;
    const int gsize = min(num_m - first_m, kGroupM);
    const int r = tile - g * per_group;
    const int mb = first_m + r % gsize;
    const int nb = r / gsize;
    ti.m0 = mb * kBlockM;
    ti.n0 = nb * BN;
    ti.m_end = p.M;
    ti.b_row0 = ti.n0;
    ti.sfa_row_tile = mb;
    ti.sfb_row_tile = ti.n0 / 128;
    return true;
  }
  int t = tile;
  for (int g = 0; g < p.num_groups; ++g) {
    const int r0 = p.group_offsets[g], r1 = p.group_offsets[g + 1];
    const int nm = (r1 - r0 + kBlockM - 1) / kBlockM;
    if (t < nm * num_n) {
      const int mb = t % nm, nb = t / nm;
      ti.m0 = r0 + mb * kBlockM;
      ti.n0 = nb * BN;
      ti.m_end = r1;
      ti.b_row0 = g * p.N + ti.n0;
      ti.sfa_row_tile = ti.m0 / 128;
      ti.sfb_row_tile = ti.b_row0 / 128;
      return true;
    }
    t -= nm * num_n;
  }
  return false;
}

template <int KIND, int BN>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const KernelParams p) {
  using C = Cfg<KIND, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;                      // [kStages]
  uint64_t* empty_bar = bars + C::kStages;        // [kStages]
  uint64_t* tfull_bar = bars + 2 * C::kStages;    // [kAccStages]
  uint64_t* tempty_bar = tfull_bar + C::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + C::kAccStages);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k_blocks = (p.K + C::kBlockK - 1) / C::kBlockK;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < C::kAccStages; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sfa = tmem_base + C::kAccStages * BN;
  const uint32_t tmem_sfb = tmem_sfa + C::kSfaCols;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int tile = blockIdx.x; ok && get_tile(p, BN, tile, ti); tile += gridDim.x) {
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicCAS(p.status, 0, kTimeoutProducer);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          mbar_expect_tx(&full_bar[stage], C::kABytes + C::kBBytes + C::kSfaBytes + C::kSfbBytes);
          const int k0 = kb * C::kBlockK;
          if constexpr (KIND == kKindF16) {
            if (p.a_mn) {
              // A^T stored [K, M]: two 64-column panels, each [64 k-rows][128 bytes]
              tma_load_2d(sa, &tmap_a, &full_bar[stage], ti.m0, k0);
              tma_load_2d(sa + 8192, &tmap_a, &full_bar[stage], ti.m0 + 64, k0);
            } else {
              tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, ti.m0);
            }
            if (p.b_mn) {
#pragma unroll
              for (int pnl = 0; pnl < BN / 64; ++pnl)
                tma_load_2d(sb + pnl * 8192, &tmap_b, &full_bar[stage], ti.b_row0 + pnl * 64, k0);
            } else {
              tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, ti.b_row0);
            }
          } else {
            // byte coordinates: fp8 = 1 byte / element, fp4 = 2 elements / byte
            const int kbyte0 = kb * C::kBlockKBytes;
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kbyte0, ti.m0);
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kbyte0, ti.b_row0);
            if constexpr (KIND != kKindF8) {
            uint8_t* ssfa = sb + C::kBBytes;
            uint8_t* ssfb = ssfa + C::kSfaBytes;
            // one stage covers kSfTileBytes/512 consecutive 4-scale tiles along K
            constexpr int kTilesPerStage = C::kSfTileBytes / 512;
            const size_t kt = static_cast<size_t>(kb) * kTilesPerStage;
            bulk_load_1d(ssfa, p.sfa + (static_cast<size_t>(ti.sfa_row_tile) * p.sf_k_tiles + kt) * 512,
                         C::kSfTileBytes, &full_bar[stage]);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              bulk_load_1d(ssfb + j * C::kSfTileBytes,
                           p.sfb + (static_cast<size_t>(ti.sfb_row_tile + j) * p.sf_k_tiles + kt) * 512,
                           C::kSfTileBytes, &full_bar[stage]);
            }
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (values stay warp-uniform); one elected lane issues.
    {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int tile = blockIdx.x; ok && get_tile(p, BN, tile, ti); tile += gridDim.x) {
        if (!__all_sync(0xffffffffu, mbar_wait(&tempty_bar[acc], acc_phase ^ 1))) {
          if (lane == 0) atomicCAS(p.status, 0, kTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) {
            if (lane == 0) atomicCAS(p.status, 0, kTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          if (elect_one()) {
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
          if constexpr (KIND == kKindF16) {
            const uint64_t adesc = p.a_mn ? umma_desc_mn_sw128(sa, 8192) : umma_desc_k_sw128(sa);
            const uint64_t bdesc = p.b_mn ? umma_desc_mn_sw128(sb, 8192) : umma_desc_k_sw128(sb);
            // one MMA consumes K=16: 32 bytes along a K-major row, 16 rows (2048 bytes) MN-major
            const uint32_t astep = p.a_mn ? (2048 >> 4) : (32 >> 4);
            const uint32_t bstep = p.b_mn ? (2048 >> 4) : (32 >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16(tmem_d, adesc + k * astep, bdesc + k * bstep, p.idesc, (kb | k) != 0);
          } else if constexpr (KIND == kKindF8) {
            const uint64_t adesc = umma_desc_k_sw128(sa);
            const uint64_t bdesc = umma_desc_k_sw128(sb);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f8(tmem_d, adesc + k * 2, bdesc + k * 2, p.idesc, (kb | k) != 0);
          } else {
            const uint32_t ssfa = sb + C::kBBytes;
            const uint32_t ssfb = ssfa + C::kSfaBytes;
            constexpr int kTilesPerStage = C::kSfTileBytes / 512;
#pragma unroll
            for (int t = 0; t < kTilesPerStage; ++t) {
              utccp_sf(tmem_sfa + t * 4, umma_desc_sf(ssfa + t * 512));
#pragma unroll
              for (int j = 0; j < BN / 128; ++j)
                utccp_sf(tmem_sfb + (t * (BN / 128) + j) * 4, umma_desc_sf(ssfb + j * C::kSfTileBytes + t * 512));
            }
            const uint64_t adesc = umma_desc_k_sw128(sa);
            const uint64_t bdesc = umma_desc_k_sw128(sb);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if constexpr (KIND == kKindMxf8) {
                // scale id k selects byte k of each 32-bit scale column
                const uint32_t idesc = p.idesc | (uint32_t(k) << 29) | (uint32_t(k) << 4);
                umma_mxf8(tmem_d, adesc + k * 2, bdesc + k * 2, idesc, (kb | k) != 0, tmem_sfa, tmem_sfb);
              } else {
                // four scales per MMA (K=64): MMA k reads scale columns of K-tile k
                umma_nvf4(tmem_d, adesc + k * 2, bdesc + k * 2, p.idesc, (kb | k) != 0, tmem_sfa + k * 4,
                          tmem_sfb + k * (BN / 128) * 4);
              }
            }
          }
          tc_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          }
          __syncwarp();
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) tc_commit(&tfull_bar[acc]);
        __syncwarp();
        if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes a warp may touch: 32*(warp%4) ..
    int acc = 0;
    uint32_t acc_phase = 0;
    const float alpha = p.alpha * (p.alpha_dev ? *p.alpha_dev : 1.0f);
    TileInfo ti;
    for (int tile = blockIdx.x; get_tile(p, BN, tile, ti); tile += gridDim.x) {
      if (!mbar_wait(&tfull_bar[acc], acc_phase)) {
        if (lane == 0) atomicCAS(p.status, 0, kTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const int row = ti.m0 + quarter * 32 + lane;
      const bool row_ok = row < ti.m_end;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        if (c0 + 32 >= BN) {
          // all accumulator columns of this stage are in registers: hand TMEM back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        }
        const int col0 = ti.n0 + c0;
        if (!row_ok || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
        const int ncols = min(32, p.N - col0);
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i < ncols) {
              float b;
              if (p.bias_dtype == kFloat32) b = reinterpret_cast<const float*>(p.bias)[col0 + i];
              else if (p.bias_dtype == kBFloat16)
                b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + i]);
              else b = __half2float(reinterpret_cast<const __half*>(p.bias)[col0 + i]);
              v[i] += b;
            }
          }
        }
        const size_t off = static_cast<size_t>(row) * p.ldd + col0;
        if (p.epilogue == kEpiGelu || p.epilogue == kEpiDGelu) {
          // aux has the layout and dtype of D
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i < ncols) {
              if (p.epilogue == kEpiGelu) {
                if (p.d_dtype == kFloat32) reinterpret_cast<float*>(p.aux)[off + i] = v[i];
                else if (p.d_dtype == kBFloat16)
                  reinterpret_cast<__nv_bfloat16*>(p.aux)[off + i] = __float2bfloat16(v[i]);
                else reinterpret_cast<__half*>(p.aux)[off + i] = __float2half(v[i]);
                v[i] = gelu_tanh(v[i]);
              } else {
                float a;
                if (p.d_dtype == kFloat32) a = reinterpret_cast<const float*>(p.aux)[off + i];
                else if (p.d_dtype == kBFloat16)
                  a = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.aux)[off + i]);
                else a = __half2float(reinterpret_cast<const __half*>(p.aux)[off + i]);
                v[i] *= dgelu_tanh(a);
              }
            }
          }
        }
        if (p.d_dtype == kFloat32) {
          float* dp = reinterpret_cast<float*>(p.d) + off;
          if (ncols == 32 && (reinterpret_cast<uintptr_t>(dp) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
              if (p.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(dp + i);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(dp + i) = o;
            }
          } else {
            for (int i = 0; i < ncols; ++i) dp[i] = v[i] + (p.accumulate ? dp[i] : 0.f);
          }
        } else {
          uint16_t* dp = reinterpret_cast<uint16_t*>(p.d) + off;
          const bool bf = p.d_dtype == kBFloat16;
          if (ncols == 32 && (reinterpret_cast<uintptr_t>(dp) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (p.accumulate) {
                const uint4 old = *reinterpret_cast<const uint4*>(dp + i);
                const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float lo, hi;
                  if (bf) {
                    lo = __uint_as_float(ow[j] << 16);
                    hi = __uint_as_float(ow[j] & 0xFFFF0000u);
                  } else {
                    const __half2 h = *reinterpret_cast<const __half2*>(&ow[j]);
                    lo = __low2float(h);
                    hi = __high2float(h);
                  }
                  v[i + 2 * j] += lo;
                  v[i + 2 * j + 1] += hi;
                }
              }
              uint4 o;
              if (bf) {
                o.x = pack_bf16x2(v[i], v[i + 1]); o.y = pack_bf16x2(v[i + 2], v[i + 3]);
                o.z = pack_bf16x2(v[i + 4], v[i + 5]); o.w = pack_bf16x2(v[i + 6], v[i + 7]);
              } else {
                o.x = pack_f16x2(v[i], v[i + 1]); o.y = pack_f16x2(v[i + 2], v[i + 3]);
                o.z = pack_f16x2(v[i + 4], v[i + 5]); o.w = pack_f16x2(v[i + 6], v[i + 7]);
              }
              *reinterpret_cast<uint4*>(dp + i) = o;
            }
          } else {
            for (int i = 0; i < ncols; ++i) {
              float x = v[i];
              if (bf) {
                __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(dp) + i;
                if (p.accumulate) x += __bfloat162float(*q);
                *q = __float2bfloat16(x);
              } else {
                __half* q = reinterpret_cast<__half*>(dp) + i;
                if (p.accumulate) x += __half2float(*q);
                *q = __float2half(x);
              }
            }
          }
        }
      }
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int KIND, int BN>
cudaError_t launch(const GemmArgs& a, cudaStream_t stream) {
  using C = Cfg<KIND, BN>;
  static_assert(C::kStages >= 2, "not enough shared memory for a pipeline");
  CUtensorMap ta, tb;
  const int b_rows = a.num_groups > 0 ? a.N * a.num_groups : a.N;
  bool ok;
  if constexpr (KIND == kKindF16) {
    ok = a.a_mn_major ? make_tensor_map_2d(&ta, a.a, a.a_dtype, a.K, a.M, a.lda, 64, 64, true)
                      : make_tensor_map_2d(&ta, a.a, a.a_dtype, a.M, a.K, a.lda, kBlockM, 64, true);
    ok = ok && (a.b_mn_major ? make_tensor_map_2d(&tb, a.b, a.b_dtype, a.K, b_rows, a.ldb, 64, 64, true)
                             : make_tensor_map_2d(&tb, a.b, a.b_dtype, b_rows, a.K, a.ldb, BN, 64, true));
  } else {
    // operands addressed as bytes: fp8 K bytes per row, fp4 K/2 bytes per row
    const uint64_t kbytes = KIND == kKindNvf4 ? a.K / 2 : a.K;
    const uint64_t lda = KIND == kKindNvf4 ? a.lda / 2 : a.lda;
    const uint64_t ldb = KIND == kKindNvf4 ? a.ldb / 2 : a.ldb;
    ok = make_tensor_map_2d(&ta, a.a, kByte, a.M, kbytes, lda, kBlockM, 128, true) &&
         make_tensor_map_2d(&tb, a.b, kByte, b_rows, kbytes, ldb, BN, 128, true);
  }
  if (!ok) return cudaErrorInvalidValue;

  KernelParams p;
  p.d = a.d; p.bias = a.bias; p.aux = a.aux; p.sfa = a.sfa; p.sfb = a.sfb; p.alpha_dev = a.alpha_dev;
  p.group_offsets = a.group_offsets; p.status = a.status; p.alpha = a.alpha;
  p.M = a.M; p.N = a.N; p.K = a.K; p.ldd = a.ldd;
  p.d_dtype = a.d_dtype; p.bias_dtype = a.bias_dtype; p.epilogue = a.epilogue;
  p.accumulate = a.accumulate ? 1 : 0;
  p.a_mn = a.a_mn_major ? 1 : 0; p.b_mn = a.b_mn_major ? 1 : 0;
  p.idesc = make_idesc(KIND, a.a_dtype, a.b_dtype, BN, a.a_mn_major, a.b_mn_major);
  p.num_groups = a.num_groups;
  const int sf_per_elem = KIND == kKindMxf8 ? 32 : 16;
  p.sf_k_tiles = (KIND == kKindF16 || KIND == kKindF8) ? 0 : ((a.K + sf_per_elem - 1) / sf_per_elem + 3) / 4;
  if (a.sf_k_tiles > 0 && p.sf_k_tiles > 0) p.sf_k_tiles = a.sf_k_tiles;

  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int num_n = (a.N + BN - 1) / BN;
  long long tiles;
  if (a.num_groups > 0) {
    // upper bound: every group may add one partial m-block
    tiles = (static_cast<long long>(a.M + kBlockM - 1) / kBlockM + a.num_groups) * num_n;
  } else {
    tiles = static_cast<long long>((a.M + kBlockM - 1) / kBlockM) * num_n;
  }
  int sms = a.sm_count > 0 ? a.sm_count : device_sm_count();
  const int grid = static_cast<int>(tiles < sms ? (tiles > 0 ? tiles : 1) : sms);
  gemm_kernel<KIND, BN><<<grid, kNumThreads, C::kSmemBytes, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace

bool make_tensor_map_2d(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols,
                        uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  CUtensorMapDataType dt;
  size_t es;
  switch (dtype) {
    case kFloat32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; es = 4; break;
    case kFloat16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; es = 2; break;
    case kBFloat16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; es = 2; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; es = 1; break;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld_elems * es) % 16 != 0) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * es};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

static int pick_bn(int N, int M, bool block_scaled) {
  static const char* env = getenv("TEB200_GEMM_BN");  // experiment knob: force the tile width
  if (env != nullptr && atoi(env) == 128) return 128;
  // wide tiles need fewer shared-memory bytes per flop; narrow ones waste less on small N
  if (N <= 128) return 128;
  if (block_scaled) return 256;
  return 256;
}

static bool use_pairs() {
  static const char* env = getenv("TEB200_GEMM_2CTA");  // "0" selects the single-CTA kernels
  return env == nullptr || atoi(env) != 0;
}

cudaError_t gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return cudaSuccess;
  if (a.K <= 0) return cudaErrorInvalidValue;
  if (use_pairs() && gemm_pair_supported(a, false)) return gemm_pair_bf16(a, stream);
  return pick_bn(a.N, a.M, false) == 128 ? launch<kKindF16, 128>(a, stream) : launch<kKindF16, 256>(a, stream);
}

cudaError_t gemm_mxfp8(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return cudaSuccess;
  if (a.K <= 0 || a.K % 32 != 0) return cudaErrorInvalidValue;
  if (use_pairs() && gemm_pair_supported(a, true)) return gemm_pair_mxfp8(a, stream);
  return pick_bn(a.N, a.M, true) == 128 ? launch<kKindMxf8, 128>(a, stream) : launch<kKindMxf8, 256>(a, stream);
}

cudaError_t gemm_fp8(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return cudaSuccess;
  if (a.K <= 0 || a.K % 16 != 0) return cudaErrorInvalidValue;  // TMA row pitch of 16 bytes
  return pick_bn(a.N, a.M, false) == 128 ? launch<kKindF8, 128>(a, stream) : launch<kKindF8, 256>(a, stream);
}

cudaError_t gemm_nvfp4(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return cudaSuccess;
  if (a.K <= 0 || a.K % 256 != 0) return cudaErrorInvalidValue;  // one stage = 256 values = 4 scale tiles
  return pick_bn(a.N, a.M, true) == 128 ? launch<kKindNvf4, 128>(a, stream) : launch<kKindNvf4, 256>(a, stream);
}

}  // namespace teb200
