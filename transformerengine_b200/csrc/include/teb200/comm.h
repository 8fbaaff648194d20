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
// All waits on flags are bounded (status code kTimeoutPeerFlag, see ptx.cuh).  No load in
// these kernels is a cluster-wide broadcast.  Replaces the reference's Userbuffers
// pipelines (common/comm_gemm_overlap/comm_gemm_overlap.cpp:611-760, 1044-1217).
#pragma once
#include <teb200/api.h>

namespace teb200 {

constexpr int kCommMaxRanks = 8;
enum CommMode : int { kCommNone = 0, kCommAllGather = 1, kCommReduceScatter = 2 };

struct CommGemmArgs {
  GemmArgs g;  // M = gathered rows; for all-gather g.a / g.sfa point at the LOCAL gathered buffer
  int mode = kCommNone;
  int rank = 0, world = 1;
  uint32_t epoch = 0;  // 1, 2, 3, ... per call on this context (identical on all ranks)
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
};

cudaError_t comm_gemm(const CommGemmArgs& args, cudaStream_t stream);

}  // namespace teb200
