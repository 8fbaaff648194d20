// Host-side launcher declarations of the teb200 kernels.  All launchers take
// raw device pointers and a stream; none allocates device memory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace teb200 {

enum DType : int { kFloat32 = 0, kFloat16 = 1, kBFloat16 = 2, kByte = 3, kFloat8E4M3 = 4, kFloat8E5M2 = 5 };

inline size_t dtype_size(int t) { return t == kFloat32 ? 4 : (t == kFloat16 || t == kBFloat16) ? 2 : 1; }

// Epilogue selector of the GEMM kernels.
enum Epilogue : int {
  kEpiNone = 0,
  kEpiBias = 1,        // D = acc + bias[n]
  kEpiGelu = 2,        // aux = acc (+bias); D = gelu(aux)
  kEpiDGelu = 3,       // D = acc * gelu'(aux)
  kEpiSwiGluPair = 4,  // reserved
};

struct GemmArgs {
  // D[M,N] (row-major, leading dim ldd) = alpha * A[M,K] * B[N,K]^T (+ D if accumulate) (+ bias)
  const void* a = nullptr;
  const void* b = nullptr;
  void* d = nullptr;
  const void* bias = nullptr;   // [N], dtype bias_dtype
  void* aux = nullptr;          // pre-activation output/input for gelu epilogues, same layout as D
  const uint8_t* sfa = nullptr; // block scales of A (128x4-tile swizzled), block-scaled kinds only
  const uint8_t* sfb = nullptr;
  const float* alpha_dev = nullptr;  // optional device scalar multiplied into the accumulator
  float alpha = 1.0f;
  int M = 0, N = 0, K = 0;
  int64_t lda = 0, ldb = 0, ldd = 0;  // in elements
  int a_dtype = kBFloat16, b_dtype = kBFloat16, d_dtype = kBFloat16, bias_dtype = kBFloat16;
  int epilogue = kEpiNone;
  bool accumulate = false;
  bool a_mn_major = false;  // A stored [K, M] (contraction dim slow); 16-bit kinds only
  bool b_mn_major = false;
  int* status = nullptr;    // device int, receives a Status code on failure
  int sm_count = 0;         // 0 = all SMs
  // grouped mode (MoE): rows of A/D are split in `num_groups` contiguous slabs; slab g uses
  // B rows [g*N, (g+1)*N).  `group_offsets` is a device array [num_groups+1] of row offsets.
  int num_groups = 0;
  const int32_t* group_offsets = nullptr;
  // Block-scaled kinds: k-tiles (of 4 scales) per row tile in the scale buffers of BOTH operands when they are
  // views of wider tensors (a slab of the contraction dim: data pointers and sfa / sfb point at the slab's
  // first column / first k-tile, the pitch stays that of the whole tensor).  0: derived from K.
  int sf_k_tiles = 0;
};

// dense / grouped tcgen05 GEMMs
cudaError_t gemm_bf16(const GemmArgs& args, cudaStream_t stream);    // fp16 or bf16 operands
cudaError_t gemm_mxfp8(const GemmArgs& args, cudaStream_t stream);   // e4m3/e5m2 + ue8m0 per 32
cudaError_t gemm_nvfp4(const GemmArgs& args, cudaStream_t stream);   // e2m1 + e4m3 per 16
cudaError_t gemm_fp8(const GemmArgs& args, cudaStream_t stream);     // e4m3/e5m2, per-tensor scales folded into alpha

// CTA-pair (cta_group::2) variants, 256x256 tile per pair of SMs
bool gemm_pair_supported(const GemmArgs& args, bool mxfp8);
cudaError_t gemm_pair_bf16(const GemmArgs& args, cudaStream_t stream);
cudaError_t gemm_pair_mxfp8(const GemmArgs& args, cudaStream_t stream);

// Fused attention (head dim 128, fp16/bf16).  Every tensor is a [b, h, s, d] VIEW described by
// element strides (d contiguous), so sbhd / bshd / packed-QKV layouts need no copy.
struct FlashArgs {
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  const void* dout = nullptr;
  void* out = nullptr;   // forward output (read by the delta pass in the backward)
  void* dq = nullptr;
  void* dk = nullptr;
  void* dv = nullptr;
  float* lse = nullptr;    // [b, hq, s_pad]
  float* delta = nullptr;  // [b, hq, s_pad]
  int b = 0, hq = 0, hk = 0, sq = 0, sk = 0, s_pad = 0;
  bool causal = false, bottom_right = true, is_bf16 = true;
  float scale = 1.0f;
  long long q_sb = 0, q_sh = 0, q_ss = 0, k_sb = 0, k_sh = 0, k_ss = 0, v_sb = 0, v_sh = 0, v_ss = 0;
  long long o_sb = 0, o_sh = 0, o_ss = 0, do_sb = 0, do_sh = 0, do_ss = 0;
  long long dq_sb = 0, dq_sh = 0, dq_ss = 0, dk_sb = 0, dk_sh = 0, dk_ss = 0, dv_sb = 0, dv_sh = 0, dv_ss = 0;
  int* status = nullptr;
  long long* timeline = nullptr;  // optional [64][16] clock stamps written by CTA 0 (profiling aid)
  // Packed variable-length sequences: when cu_q is set, q/out/dout/dq are [1, hq, tq, d] and k/v/dk/dv
  // [1, hk, tk, d] views of token-major tensors, b counts the sequences, sq / sk are the LONGEST
  // sequence lengths; sequence i has cu_q[i+1] - cu_q[i] queries that start at token off_q[i]
  // (same for keys).  All four are int32 device arrays of b + 1 entries.
  const int* cu_q = nullptr;
  const int* cu_k = nullptr;
  const int* off_q = nullptr;
  const int* off_k = nullptr;
  int tq = 0, tk = 0;
  // dK/dV pass: split every group of query heads that shares a key head over gsplit CTAs; CTA g writes
  // its partial sums at dk + g * dk_sg (elements), the caller adds the gsplit partials.  Fills the GPU
  // when key heads x key blocks are fewer than the SMs (tensor parallel shards).
  int gsplit = 1;
  long long dk_sg = 0;
  // Sliding window: query i (diagonal-aligned like the causal mask) sees keys in
  // [i - window_left, i + window_right]; -1 = unbounded.  causal forces window_right = 0.
  int window_left = -1, window_right = -1;
};
cudaError_t flash_fwd(const FlashArgs& args, cudaStream_t stream);
cudaError_t flash_delta(const FlashArgs& args, cudaStream_t stream);     // delta = rowsum(dO * O)
cudaError_t flash_bwd_dq(const FlashArgs& args, cudaStream_t stream);
cudaError_t flash_bwd_dkdv(const FlashArgs& args, cudaStream_t stream);

// build a 2-D row-major tensor map (TMA descriptor)
bool make_tensor_map_2d(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols,
                        uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, bool swizzle128);

}  // namespace teb200
