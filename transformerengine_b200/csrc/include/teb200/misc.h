// Launchers: multi-tensor optimizer kernels, cross entropy, RoPE, softmax, dropout,
// MoE router / permutation, padding helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace teb200 {

// ---------------------------------------------------------------- multi-tensor apply
// One launch covers up to kMtMaxTensors tensors of any size.  The work is cut in chunks of `chunk`
// elements; chunk c of the launch belongs to the tensor ti with chunk_start[ti] <= c < chunk_start[ti+1].
// A fixed grid (a few blocks per SM) strides over the chunks, so the number of launches depends on the
// number of tensors only and no launch ends in a part-filled wave of blocks.
constexpr int kMtMaxTensors = 56;
constexpr int kMtLists = 5;

struct MultiTensorTable {
  void* ptr[kMtLists][kMtMaxTensors];
  int64_t numel[kMtMaxTensors];
  int32_t chunk_start[kMtMaxTensors + 1];
  int32_t ntensors;
};

struct AdamArgs {
  float lr = 0, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, weight_decay = 0;
  float bias_correction1 = 1, bias_correction2 = 1;
  int adamw = 1;           // 1: decoupled weight decay, 0: L2 added to the gradient
  int grad_dtype = 2;      // lists: 0 = grad, 1 = param (model dtype), 2 = exp_avg, 3 = exp_avg_sq, 4 = master
  int param_dtype = 2;
  int state_dtype = 0;     // fp32 or bf16 moments
  int has_master = 1;      // 0: none, 1: fp32 master in list 4, 2: list 4 holds int16 remainders (the low 16 bits of
                           // the fp32 value whose rounded high half is the bf16 parameter)
  float grad_scale = 1.f;  // gradients are multiplied by this (1/loss_scale, 1/accumulation steps)
  const float* inv_scale_dev = nullptr;  // optional device scalar multiplied into the gradient
  const int* noop = nullptr;             // skip the update when *noop != 0
  // capturable mode: step count and learning rate live on the device, so a captured launch stays
  // valid across replays (bias corrections are then computed in the kernel from *step_dev)
  const int* step_dev = nullptr;
  const float* lr_dev = nullptr;
  int bias_correction = 1;
  int64_t chunk = 0;
};
cudaError_t multi_tensor_adam(const MultiTensorTable& t, int nchunks, const AdamArgs& a, cudaStream_t s);

struct SgdArgs {
  float lr = 0, momentum = 0, dampening = 0, weight_decay = 0, grad_scale = 1.f;
  int nesterov = 0, first_run = 0, wd_after_momentum = 0;
  int grad_dtype = 2, param_dtype = 2, has_master = 0;  // lists: 0 grad, 1 param, 2 momentum buf (fp32), 3 master
  const int* noop = nullptr;
  int64_t chunk = 0;
};
cudaError_t multi_tensor_sgd(const MultiTensorTable& t, int nchunks, const SgdArgs& a, cudaStream_t s);
// out (list 1) = in (list 0) * scale, dtype conversions allowed; sets *noop on non-finite input
cudaError_t multi_tensor_scale(const MultiTensorTable& t, int nchunks, int in_dtype, int out_dtype, float scale,
                               int* noop, int64_t chunk, cudaStream_t s);
// sum of squares of list 0 accumulated into out[0] (and per tensor into per_tensor[i] when not null)
cudaError_t multi_tensor_l2norm_sq(const MultiTensorTable& t, int nchunks, int dtype, float* out,
                                   float* per_tensor, int tensor_base, int64_t chunk, cudaStream_t s);

// ---------------------------------------------------------------- cross entropy
// logits [R, V] (bf16/fp16/fp32), targets int64 [R].  Writes loss[R] (fp32) and, when
// grad is not null, d(loss)/d(logits) * grad_scale into grad (may alias logits).
struct CrossEntropyArgs {
  const void* logits = nullptr;
  int dtype = 2;
  const int64_t* targets = nullptr;
  float* loss = nullptr;
  void* grad = nullptr;
  float* row_max = nullptr;  // optional [R]: statistics for vocab-parallel reduction
  float* row_sum = nullptr;
  float* row_tgt = nullptr;
  int R = 0, V = 0;
  int64_t ld = 0;
  int vocab_start = 0;  // first vocabulary id held by this rank
  float grad_scale = 1.f;
  const float* grad_scale_dev = nullptr;  // optional device scalar multiplied into grad_scale
  float label_smoothing = 0.f;
  int64_t ignore_index = -100;
};
cudaError_t cross_entropy_fwd_bwd(const CrossEntropyArgs& a, cudaStream_t s);
// vocab-parallel second stage: given the all-reduced max / sum / target logit, write the gradient
cudaError_t cross_entropy_parallel_bwd(const CrossEntropyArgs& a, const float* gmax, const float* gsum,
                                       cudaStream_t s);

// ---------------------------------------------------------------- RoPE
// x [s, b, h, d] (sbhd=1) or [b, s, h, d]; freqs [s_total, d_rot] fp32 angles.  In-place allowed.
struct RopeArgs {
  const void* x = nullptr;
  void* out = nullptr;
  const float* freqs = nullptr;
  int dtype = 2;
  int s = 0, b = 0, h = 0, d = 0, d_rot = 0;
  int64_t stride_s = 0, stride_b = 0, stride_h = 0;  // element strides of x / out
  int interleaved = 0;
  int backward = 0;
  int pos_offset = 0;  // added to the sequence index (context parallel / KV cache)
  int cp_size = 1, cp_rank = 0;  // dual-chunk position remap when cp_size > 1
  const int32_t* start_positions = nullptr;  // optional [b]
  // Packed QKV projection output: the h "heads" of a token are query, key and value heads of one tensor and
  // only the first two kinds are rotated (queries with freqs, keys with freqs_k), so that the split and both
  // rotations are ONE launch, in place.  qkv_mode 1: per key/value group [q_per_group query heads, 1 key, 1 value];
  // qkv_mode 2: [hq query heads | hk key heads | hk value heads].  16-bit types, d_rot % 16 == 0 only.
  int qkv_mode = 0;
  int q_per_group = 0, hq = 0, hk = 0;
  const float* freqs_k = nullptr;  // null: same angles as the queries
};
cudaError_t rope_apply(const RopeArgs& a, cudaStream_t s);

// ---------------------------------------------------------------- softmax (unfused attention path)
struct SoftmaxArgs {
  const void* x = nullptr;  // [rows, cols] scores, rows = b*h*sq
  void* y = nullptr;
  const uint8_t* mask = nullptr;  // optional [b, 1, sq, sk] bytes, non-zero = masked out
  int dtype = 2;
  int64_t rows = 0;
  int cols = 0, sq = 0, heads = 0;
  float scale = 1.f;
  int causal = 0;          // 1: upper-triangular mask aligned bottom-right
  const void* dy = nullptr;  // backward when not null: y holds probs, out = dx
};
cudaError_t softmax_fwd(const SoftmaxArgs& a, cudaStream_t s);
cudaError_t softmax_bwd(const SoftmaxArgs& a, cudaStream_t s);

// ---------------------------------------------------------------- dropout
cudaError_t dropout_fwd(const void* x, void* y, uint8_t* mask_bits, int64_t n, int dtype, float p, uint64_t seed,
                        uint64_t offset, cudaStream_t s);
cudaError_t dropout_bwd(const void* dy, const uint8_t* mask_bits, void* dx, int64_t n, int dtype, float p,
                        cudaStream_t s);

// ---------------------------------------------------------------- MoE router / permutation
struct RouterArgs {
  const void* logits = nullptr;  // [T, E]
  int dtype = 2;
  int T = 0, E = 0, topk = 0;
  int score_fn = 1;              // 0 sigmoid, 1 softmax, 2 sqrt-softplus
  int use_pre_softmax = 0;
  float scaling_factor = 1.f;
  const float* expert_bias = nullptr;
  int num_groups = 0, group_topk = 0;
  float* probs = nullptr;        // [T, E] dense, zero outside the top-k
  uint8_t* routing_map = nullptr;  // [T, E] bytes
  int32_t* topk_idx = nullptr;   // [T, topk]
  float* topk_w = nullptr;       // [T, topk]
  float* scores = nullptr;       // [T, E] optional: full score-function output (aux loss)
  int32_t* tokens_per_expert = nullptr;  // [E] optional, accumulated atomically (zeroed by callee)
};
cudaError_t router_topk_fwd(const RouterArgs& a, cudaStream_t s);
cudaError_t router_topk_bwd(const RouterArgs& a, const float* grad_probs, void* grad_logits, cudaStream_t s);

// rows of `in` [T, H] scattered to expert-major order.  `dest_row` [T, topk] gives the
// destination row of every (token, slot) or -1.
cudaError_t permute_rows(const void* in, void* out, const int32_t* dest_row, const float* probs, float* probs_out,
                         int T, int topk, int H, int dtype, cudaStream_t s);
// out[t] = sum_k w[t,k] * in[dest_row[t,k]]  (w may be null = plain sum)
cudaError_t unpermute_rows(const void* in, void* out, const int32_t* dest_row, const float* w, int T, int topk, int H,
                           int dtype, cudaStream_t s);
// dest_row from a routing of T tokens to E experts: stable expert-major order, per-expert
// row counts padded to `align`.  counts [E], offsets [E+1] written on device.
cudaError_t build_dest_rows(const int32_t* topk_idx, int T, int topk, int E, int align, int32_t* counts,
                            int32_t* offsets, int32_t* dest_row, cudaStream_t s);

// ---------------------------------------------------------------- column sums, offsets, padding
// out[c] = sum_r x[r, c] (bias gradient), deterministic two-stage reduction.  workspace: column_sum_parts(R, C) * C floats.
int column_sum_parts(int R, int C);
cudaError_t column_sum(const void* x, int x_dtype, int R, int C, long long ld, void* out, int out_dtype, float* workspace,
                       cudaStream_t s);
// per-slab column sums (bias gradients of a grouped linear layer): out[g][c] = sum of x[r][c] over the rows
// offsets[g] .. offsets[g+1]; offsets = int32 device array of groups + 1 entries
cudaError_t grouped_column_sum(const void* x, int x_dtype, const int* offsets, int groups, int C, long long ld, void* out,
                               int out_dtype, cudaStream_t s);
// x[r][c] += bias[g][c] for the rows of slab g, all slabs in one launch; max_rows bounds offsets[groups]
cudaError_t grouped_bias_add(void* x, const void* bias, int dtype, const int* offsets, int groups, int C, long long ld,
                             int max_rows, cudaStream_t s);
// out[r] = <a[r], b[r]> in fp32 (gradient of a per-row scale: routing probabilities of a scaled activation)
cudaError_t row_dot(const void* a, const void* b, int dtype, long long R, int C, long long lda, long long ldb, float* out,
                    cudaStream_t s);
// out[0] = 0, out[i + 1] = multiplier * (splits[0] + ... + splits[i]); int32 or int64 on either side, all on the device
cudaError_t splits_to_offsets(const void* splits, int splits_is_int64, int n, long long multiplier, void* out,
                              int out_is_int64, cudaStream_t s);
// Rows of `groups` slabs copied from in (slab g = rows [in_offsets[g], in_offsets[g+1])) to out (slab g =
// rows [out_offsets[g], out_offsets[g+1])): longer destination slabs are zero-filled (padding), shorter ones cut
// (unpadding).  Offsets are int32 device arrays of groups + 1 entries; max_out_rows bounds out_offsets[groups].
cudaError_t repad_rows(const void* in, void* out, const int* in_offsets, const int* out_offsets, int groups, int row_bytes,
                       int max_out_rows, cudaStream_t s);
// out [R, cp_bytes] = in [R, c_bytes] zero-padded (or cut) along the last dimension; byte counts multiples of 4
cudaError_t pad_last_dim(const void* in, void* out, long long R, int c_bytes, int cp_bytes, cudaStream_t s);

// ---------------------------------------------------------------- packed sequences ("thd") and KV cache
// cu: int32 cumulative sequence lengths [nb + 1] on the device.  dtype: 0 fp32, 1 fp16, 2 bf16.
// Context parallel layout: every sequence is cut into 2 * world chunks, rank r holds chunks r and
// 2 * world - 1 - r ("first half" and "second half" of its local tokens).
cudaError_t thd_partition_indices(int* out, const int* cu, int nb, int total_tokens, int world, int rank,
                                  cudaStream_t s);
// half [lead, t/2, row] <- the first (0) or second (1) half of every sequence of full [lead, t, row]
cudaError_t thd_read_half(void* half, const void* full, const int* cu, int nb, int t, int lead, int row_bytes,
                          int half_idx, cudaStream_t s);
// lse [heads, t], half [heads, t/2]; mode 0: lse(second halves) = logaddexp(lse, half); mode 1: half = lse(second halves)
cudaError_t thd_lse_half(float* lse, float* half, const int* cu, int nb, int heads, int t, int mode, cudaStream_t s);
// out [t, heads, d] += step [t or t/2, heads, d] * exp(lse_step - lse)
cudaError_t thd_out_correction(void* out, const void* step, const float* lse, const float* lse_step, const int* cu,
                               int nb, int heads, int d, int t, int only_second_half, int dtype, cudaStream_t s);
// grad [lead, t, row] (op)= step [lead, t_step, row] per half of every sequence; modes: 0 leave, 1 copy, 2 add
cudaError_t thd_grad_correction(void* grad, const void* step, const int* cu, int nb, int lead, int row, int t,
                                int t_step, int mode_first, int mode_second, int dtype, cudaStream_t s);
// packed [t, row] <-> padded [nb, s_max, row] (the destination must be zero-filled by the caller)
cudaError_t thd_bshd_convert(void* packed, void* padded, const int* cu, int nb, int t, int s_max, int row_bytes,
                             int to_bshd, cudaStream_t s);

// One decoding step of a (paged) KV cache: append every sequence's new tokens to the cache and gather
// all live sequences' keys / values, old and new, into packed [total, row] tensors.  A contiguous
// cache is the case page_size = max sequence length, width = 1, page_table[i] = slot of sequence i.
struct KvCacheArgs {
  const void* new_k = nullptr;  // [sum new, row]
  const void* new_v = nullptr;
  void* cache_k = nullptr;      // [num_pages, page_size, row]
  void* cache_v = nullptr;
  void* out_k = nullptr;        // [total, row]
  void* out_v = nullptr;
  const int* cu_new = nullptr;  // [nb + 1] cumulative new tokens
  const int* cu_kv = nullptr;   // [nb + 1] cumulative lengths after the step
  const int* page_table = nullptr;  // [nb, width]
  int nb = 0, width = 0, page_size = 0, num_pages = 0, total = 0;
  int row_bytes_k = 0, row_bytes_v = 0;
  int* status = nullptr;
};
cudaError_t kv_cache_step(const KvCacheArgs& a, cudaStream_t s);

}  // namespace teb200
