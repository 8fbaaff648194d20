// GEMMs fused with a tensor-parallel collective over NVLink peer memory.
//
//   kCommAllGather    : Y[M, N] = gather_rows(X)[M, K] * W[N, K]^T.  Every rank owns M/world rows of
//                       X inside a symmetric buffer; dedicated copy CTAs pull the peers' rows with
//                       plain peer loads into the local buffer and publish one flag per 128-row
//                       block; the TMA producer of the GEMM waits for the flag of the block it is
//                       about to read.  Rows cross NVLink once.
//   kCommReduceScatter: out[M/world, N] = sum_ranks (X_r[M, K_r] * W_r[N, K_r]^T)[my rows].  The
//                       epilogue stores every output tile straight into the owner rank's staging
//                       buffer (peer stores) and bumps a per-block counter there; after its own
//                       tiles each CTA reduces the blocks it owns as soon as all ranks delivered.
//
//   kCommAllReduce    : out[M, N] = sum_ranks (X_r * W_r^T) on EVERY rank (row-parallel layers without sequence
//                       parallelism).  The reduce-scatter kernel whose tail writes the reduced rows of this rank
//                       into the output buffer of every rank (peer stores) and returns once all ranks' rows have
//                       landed here (one counter per source rank).
//
// All waits on flags are bounded (status code kTimeoutPeerFlag, see ptx.cuh).  No load in
// these kernels is a cluster-wide broadcast.  Replaces the reference's Userbuffers
// pipelines (common/comm_gemm_overlap/comm_gemm_overlap.cpp:611-760, 1044-1217).
#pragma once
#include <teb200/api.h>

namespace teb200 {

constexpr int kCommMaxRanks = 8;
enum CommMode : int { kCommNone = 0, kCommAllGather = 1, kCommReduceScatter = 2, kCommAllReduce = 3 };

// Optional second all-gather carried out by copy CTAs of the same kernel while the GEMM runs (the
// operand of the weight-gradient GEMM that follows: bulk overlap).  Every rank stages a piece of
// `rows` rows x `row_bytes` bytes (contiguous) followed by `row_tiles` scale chunks of `sf_chunk`
// bytes; piece s lands at dst + s * dst_piece_off with row pitch dst_pitch, its scale chunk t at
// dst_sf + (t * world + s) * sf_chunk.  Consumers are later kernels of the stream (no flags).
struct SideGather {
  const uint8_t* src[kCommMaxRanks] = {};  // staged pieces of every rank (symmetric memory)
  uint8_t* dst = nullptr;
  uint8_t* dst_sf = nullptr;
  int rows = 0;                  // 0: no side gather
  int row_bytes = 0;             // multiple of 16, <= 32768
  long long dst_pitch = 0, dst_piece_off = 0;
  int row_tiles = 0, sf_chunk = 0;
};

struct CommGemmArgs {
  GemmArgs g;  // M = gathered rows; for all-gather g.a / g.sfa point at the LOCAL gathered buffer
  int mode = kCommNone;
  int rank = 0, world = 1;
  // three local device words: [0] calls completed so far on this (context, buffer slot), identical on all
  // ranks, advanced by the kernel itself (so launches recorded in a CUDA graph replay correctly);
  // [1] scratch counter of finished CTAs, [2] next unclaimed piece of the side gather; both zero between launches
  uint32_t* epoch_dev = nullptr;
  int copy_ctas = 8;

  // ---- all-gather: gathered buffers of every rank (index = rank), same layout everywhere
  const uint8_t* a_full[kCommMaxRanks] = {};
  const uint8_t* sfa_full[kCommMaxRanks] = {};
  long long a_row_bytes = 0;           // bytes per row of A
  long long sf_bytes_per_mblock = 0;   // bytes of scale tiles per 128-row block (0 for 16-bit kinds)
  uint32_t* ready[kCommMaxRanks] = {}; // ready[r][s] on rank r: epoch at which rank s published its rows
  uint32_t* chunk_flags = nullptr;     // local, one per 128-row block of the gathered matrix

  // ---- reduce-scatter
  uint8_t* stage[kCommMaxRanks] = {};       // stage[r] on rank r: [world][M/world][N] of d_dtype
  uint32_t* tile_flags[kCommMaxRanks] = {}; // tile_flags[r] on rank r: [world][M/world/128] counters
  void* out = nullptr;                      // local result [M/world, N], dtype d_dtype

  // ---- all-reduce (reduce-scatter fields above, `out` unused)
  uint8_t* out_all[kCommMaxRanks] = {};     // out_all[r]: the [M, N] result buffer of rank r (symmetric memory)
  uint32_t* ar_flags[kCommMaxRanks] = {};   // ar_flags[r] on rank r: [world] counters of CTAs whose rows have landed

  SideGather side;  // needs `ready` (both modes) and copy_ctas >= 1
};

cudaError_t comm_gemm(const CommGemmArgs& args, cudaStream_t stream);

// ---------------------------------------------------------------- expert-parallel token exchange
// ep ranks, L local experts per rank (E = ep * L experts).  Pointer arrays index the peer rank;
// flag arrays hold one epoch counter per source rank.
struct EpCountsArgs {
  int32_t* counts_all[kCommMaxRanks] = {};  // on rank r: [ep][E], row s published by rank s
  uint32_t* flags[kCommMaxRanks] = {};      // on rank r: [ep]
  const int32_t* my_counts = nullptr;       // [E] rows this rank sends to each expert
  int32_t* base = nullptr;                  // out [E]: first row of this rank's tokens in the owner's buffer
  int32_t* splits = nullptr;                // out [L+1]: padded rows per local expert, then the total
  int32_t* seg = nullptr;                   // out [L][ep+1]: start of each source's segment, then its end
  int ep = 0, L = 0, rank = 0, align = 1;
  uint32_t epoch = 0;
  int* status = nullptr;
};
struct EpPushArgs {
  const void* x = nullptr;                  // [T, H] rows of this rank
  const int32_t* within = nullptr;          // [T, E]: rank of token t among this rank's tokens of expert e, or -1
  const int32_t* base = nullptr;            // [E] from the counts kernel
  const float* scale = nullptr;             // optional [T, E] multiplier applied while copying
  const float* probs = nullptr;             // optional [T, E] routing weights sent along
  void* dst[kCommMaxRanks] = {};            // on rank r: [cap_rows, H]
  float* dst_probs[kCommMaxRanks] = {};     // on rank r: [cap_rows]
  uint32_t* flags[kCommMaxRanks] = {};      // on rank r: [ep]
  int32_t* rowmap = nullptr;                // out [T, E]: destination row of every pair, or -1
  unsigned* cta_counter = nullptr;          // zero-initialised scratch word
  int T = 0, ep = 0, L = 0, rank = 0, vec_per_row = 0, cap_rows = 0, is_bf16 = 1;
  uint32_t epoch = 0;
  int* status = nullptr;
};
struct EpSignalArgs {
  uint32_t* flags[kCommMaxRanks] = {};
  int ep = 0, rank = 0;
  uint32_t epoch = 0;
};
struct EpPullArgs {
  const void* src[kCommMaxRanks] = {};      // on rank r: [cap_rows, H] expert-major rows
  const int32_t* rowmap = nullptr;          // [T, E]
  const float* w = nullptr;                 // optional [T, E] weights
  void* out = nullptr;                      // [T, H]
  const void* g = nullptr;                  // optional [T, H]: with `dots`, dots[t,e] = <g[t], row(t,e)>
  float* dots = nullptr;                    // optional [T, E]
  const float* src_s[kCommMaxRanks] = {};   // optional per-row scalars on rank r: [cap_rows]
  float* out_s = nullptr;                   // optional [T, E]: the scalar of every pair's row
  int T = 0, ep = 0, L = 0, vec_per_row = 0, is_bf16 = 1;
};
// out[i] = sum_r src[r][i] over 16-byte vectors of 16-bit values (fp32 accumulation)
struct PeerSumArgs {
  const void* src[kCommMaxRanks] = {};
  void* out = nullptr;
  long long vecs = 0;
  int n = 0, is_bf16 = 1;
};
cudaError_t peer_sum(const PeerSumArgs& a, cudaStream_t s);
cudaError_t ep_counts(const EpCountsArgs& a, cudaStream_t s);
cudaError_t ep_push(const EpPushArgs& a, cudaStream_t s);
// waits (bounded by limit_cycles SM clock cycles; 0 = the library default of about one second) until the n
// flags reach `epoch`; on expiry *status becomes kTimeoutPeerFlag and the kernel returns
cudaError_t ep_wait(const uint32_t* flags, int n, uint32_t epoch, int* status, cudaStream_t s,
                    long long limit_cycles = 0);
cudaError_t ep_signal(const EpSignalArgs& a, cudaStream_t s);
cudaError_t ep_pull(const EpPullArgs& a, cudaStream_t s);

}  // namespace teb200
