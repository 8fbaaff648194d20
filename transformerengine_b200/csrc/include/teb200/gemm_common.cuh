// Pieces shared by the dense GEMM (gemm_tcgen05.cu) and the GEMMs fused with a
// collective (comm/comm_gemm.cu): tile configuration, instruction descriptors,
// activation helpers and the TMA descriptor encoder lookup.
#pragma once
#include <teb200/api.h>
#include <teb200/ptx.cuh>

#include <cstdlib>

namespace teb200 {
namespace gemm_detail {

constexpr int kBlockM = 128;
constexpr int kNumThreads = 192;
constexpr int kGroupM = 8;  // m-blocks per scheduling group (L2 reuse of B panels)

enum Kind : int { kKindF16 = 0, kKindMxf8 = 1, kKindNvf4 = 2, kKindF8 = 3 };  // F8: per-tensor scaled e4m3/e5m2

struct KernelParams {
  void* d;
  const void* bias;
  void* aux;
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha_dev;
  const int32_t* group_offsets;
  int* status;
  float alpha;
  int M, N, K;
  long long ldd;
  int d_dtype, bias_dtype, epilogue;
  int accumulate;
  int a_mn, b_mn;
  uint32_t idesc;
  int num_groups;
  int sf_k_tiles;  // number of 4-scale tiles along K in the scale layout
};

template <int KIND, int BN>
struct Cfg {
  static constexpr int kBlockKBytes = 128;  // one 128-byte swizzle atom per row
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = BN * kBlockKBytes;
  static constexpr int kSfTileBytes = (KIND == kKindMxf8) ? 512 : (KIND == kKindNvf4 ? 2048 : 0);
  static constexpr int kSfaBytes = kSfTileBytes;
  static constexpr int kSfbBytes = kSfTileBytes * (BN / 128 > 0 ? BN / 128 : 1);
  static constexpr int kStageBytes = ((kABytes + kBBytes + kSfaBytes + kSfbBytes + 1023) / 1024) * 1024;
  static constexpr int kSfCols = (KIND == kKindMxf8) ? 4 : (KIND == kKindNvf4 ? 16 : 0);  // TMEM columns per 128 rows
  static constexpr int kSfaCols = kSfCols;
  static constexpr int kSfbCols = kSfCols * (BN / 128 > 0 ? BN / 128 : 1);
  // accumulator stages: two when they fit beside the scale columns in 512 TMEM columns
  static constexpr int kAccStages = (2 * BN + kSfaCols + kSfbCols <= 512) ? 2 : 1;
  static constexpr int kTmemCols = 512;
  static constexpr int kStages = (227 * 1024 - 2048) / kStageBytes > 8 ? 8 : (227 * 1024 - 2048) / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 1024 /*barriers*/;
  // elements of K covered by one stage / one MMA
  static constexpr int kBlockK = (KIND == kKindF16) ? 64 : (KIND == kKindNvf4 ? 256 : 128);
  static constexpr int kMmaPerStage = 4;
};

__device__ __forceinline__ float gelu_tanh(float x) {
  return x * (0.5f + 0.5f * tanhf(x * (0.79788456f + 0.03567741f * x * x)));
}
__device__ __forceinline__ float dgelu_tanh(float x) {
  const float t = tanhf(0.79788456f * x * (1.f + 0.044715f * x * x));
  return 0.5f * x * ((1.f - t * t) * (0.79788456f + 0.1070322243f * x * x)) + 0.5f * (1.f + t);
}


// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

inline int device_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

inline uint32_t make_idesc(int kind, int a_dtype, int b_dtype, int BN, bool a_mn, bool b_mn) {
  uint32_t d = 0;
  if (kind == kKindF16) {
    const uint32_t fmt = (a_dtype == kBFloat16) ? 1u : 0u;
    d |= 1u << 4;   // fp32 accumulator
    d |= fmt << 7;  // A format
    d |= fmt << 10; // B format
    d |= (a_mn ? 1u : 0u) << 15;
    d |= (b_mn ? 1u : 0u) << 16;
  } else if (kind == kKindF8) {
    d |= 1u << 4;  // fp32 accumulator
    d |= (a_dtype == kFloat8E5M2 ? 1u : 0u) << 7;
    d |= (b_dtype == kFloat8E5M2 ? 1u : 0u) << 10;
  } else if (kind == kKindMxf8) {
    d |= (a_dtype == kFloat8E5M2 ? 1u : 0u) << 7;
    d |= (b_dtype == kFloat8E5M2 ? 1u : 0u) << 10;
    d |= 1u << 23;  // UE8M0 scales
  } else {
    d |= 1u << 7;   // E2M1
    d |= 1u << 10;
    // bit 23 = 0: UE4M3 scales
  }
  d |= (uint32_t(BN) >> 3) << 17;
  d |= (uint32_t(kBlockM) >> 4) << 24;
  return d;
}


}  // namespace gemm_detail
}  // namespace teb200
