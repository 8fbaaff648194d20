// Bindings of the kernels that live outside the core translation unit
// (attention, softmax, dropout, MoE router / permutation, NVFP4, fused
// communication).  Kept separate so that touching one family does not rebuild
// the rest.
#include <cstdlib>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <teb200/api.h>
#include <teb200/nvtx.h>
#include <teb200/comm.h>
#include <teb200/misc.h>
#include <teb200/quant.h>
#include <torch/extension.h>

#include <optional>
#include <vector>

namespace py = pybind11;
using OptT = std::optional<at::Tensor>;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int dtype_code(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return teb200::kFloat32;
    case at::kHalf: return teb200::kFloat16;
    case at::kBFloat16: return teb200::kBFloat16;
    default: return teb200::kByte;
  }
}

// Fused collective GEMM.  `a` is the LOCAL gathered buffer [M, K] (all-gather) or the local
// operand [M, K_local] (reduce-scatter); peer buffers are passed as raw device addresses taken
// from the symmetric-memory rendezvous.
void comm_gemm(int64_t mode, int64_t rank, int64_t world, const at::Tensor& epoch_dev, int64_t copy_ctas, const at::Tensor& a,
               const OptT& sfa, const at::Tensor& b, const OptT& sfb, const OptT& d, const OptT& bias, bool a_e5m2,
               bool b_e5m2, std::vector<int64_t> a_ptrs, std::vector<int64_t> sfa_ptrs,
               std::vector<int64_t> ready_ptrs, int64_t chunk_flags_ptr, std::vector<int64_t> stage_ptrs,
               std::vector<int64_t> tile_flag_ptrs, const OptT& out, int64_t N, const at::Tensor& status,
               std::vector<int64_t> side_src_ptrs, const OptT& side_dst, const OptT& side_dst_sf,
               std::vector<int64_t> side_geom, std::vector<int64_t> out_all_ptrs, std::vector<int64_t> ar_flag_ptrs) {
  c10::cuda::CUDAGuard guard(a.device());
  teb200::CommGemmArgs c;
  teb200::GemmArgs& g = c.g;
  const bool mx = sfa.has_value() && sfa->defined();
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.M = static_cast<int>(a.size(0));
  g.K = static_cast<int>(a.size(1));
  g.N = static_cast<int>(N);
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  if (mx) {
    g.a_dtype = a_e5m2 ? teb200::kFloat8E5M2 : teb200::kFloat8E4M3;
    g.b_dtype = b_e5m2 ? teb200::kFloat8E5M2 : teb200::kFloat8E4M3;
    g.sfa = static_cast<const uint8_t*>(sfa->data_ptr());
    g.sfb = static_cast<const uint8_t*>(sfb->data_ptr());
  } else {
    g.a_dtype = g.b_dtype = dtype_code(a);
  }
  const at::Tensor& o = (mode == teb200::kCommAllGather) ? *d : *out;
  g.d_dtype = dtype_code(o);
  if (mode == teb200::kCommAllGather) {
    g.d = d->data_ptr();
    g.ldd = d->stride(0);
    if (out.has_value() && out->defined()) g.aux = out->data_ptr();  // optional timeline buffer, as below
  } else if (d.has_value() && d->defined()) {
    g.aux = d->data_ptr();  // optional int64 [ctas, 4] timeline buffer (profiling aid)
  }
  if (bias.has_value() && bias->defined()) {
    g.bias = bias->data_ptr();
    g.bias_dtype = dtype_code(*bias);
  }
  g.status = status.data_ptr<int>();
  c.mode = static_cast<int>(mode);
  c.rank = static_cast<int>(rank);
  c.world = static_cast<int>(world);
  TORCH_CHECK(epoch_dev.scalar_type() == at::kInt && epoch_dev.numel() >= 3 && epoch_dev.is_cuda(),
              "comm_gemm: the call counters must be three int32 words on the GPU");
  c.epoch_dev = reinterpret_cast<uint32_t*>(epoch_dev.data_ptr<int>());
  c.copy_ctas = static_cast<int>(copy_ctas);
  for (int r = 0; r < world && r < teb200::kCommMaxRanks; ++r) {
    if (!a_ptrs.empty()) c.a_full[r] = reinterpret_cast<const uint8_t*>(a_ptrs[r]);
    if (!sfa_ptrs.empty()) c.sfa_full[r] = reinterpret_cast<const uint8_t*>(sfa_ptrs[r]);
    if (!ready_ptrs.empty()) c.ready[r] = reinterpret_cast<uint32_t*>(ready_ptrs[r]);
    if (!stage_ptrs.empty()) c.stage[r] = reinterpret_cast<uint8_t*>(stage_ptrs[r]);
    if (!tile_flag_ptrs.empty()) c.tile_flags[r] = reinterpret_cast<uint32_t*>(tile_flag_ptrs[r]);
    if (!out_all_ptrs.empty()) c.out_all[r] = reinterpret_cast<uint8_t*>(out_all_ptrs[r]);
    if (!ar_flag_ptrs.empty()) c.ar_flags[r] = reinterpret_cast<uint32_t*>(ar_flag_ptrs[r]);
  }
  if (mode == teb200::kCommAllReduce)
    TORCH_CHECK(static_cast<int64_t>(out_all_ptrs.size()) >= world && static_cast<int64_t>(ar_flag_ptrs.size()) >= world &&
                    out.has_value() && out->defined() && out->size(0) == a.size(0),
                "comm_gemm: all-reduce needs the result buffer [M, N] and its address and counters on every rank");
  c.a_row_bytes = a.stride(0) * a.element_size();
  c.sf_bytes_per_mblock = mx ? static_cast<long long>(((g.K + 31) / 32 + 3) / 4) * 512 : 0;
  c.chunk_flags = reinterpret_cast<uint32_t*>(chunk_flags_ptr);
  c.out = (out.has_value() && out->defined()) ? out->data_ptr() : nullptr;
  if (!side_src_ptrs.empty()) {
    // side_geom = [rows, row_bytes, dst_pitch, dst_piece_off, row_tiles, sf_chunk]
    TORCH_CHECK(side_geom.size() == 6 && side_dst.has_value() && side_dst->defined(), "comm_gemm: bad side gather");
    TORCH_CHECK(static_cast<int64_t>(side_src_ptrs.size()) >= world, "comm_gemm: side gather needs one pointer per rank");
    for (int r = 0; r < world && r < teb200::kCommMaxRanks; ++r)
      c.side.src[r] = reinterpret_cast<const uint8_t*>(side_src_ptrs[r]);
    c.side.dst = static_cast<uint8_t*>(side_dst->data_ptr());
    c.side.dst_sf = (side_dst_sf.has_value() && side_dst_sf->defined()) ? static_cast<uint8_t*>(side_dst_sf->data_ptr()) : nullptr;
    c.side.rows = static_cast<int>(side_geom[0]);
    c.side.row_bytes = static_cast<int>(side_geom[1]);
    c.side.dst_pitch = side_geom[2];
    c.side.dst_piece_off = side_geom[3];
    c.side.row_tiles = static_cast<int>(side_geom[4]);
    c.side.sf_chunk = static_cast<int>(side_geom[5]);
    TORCH_CHECK(side_dst->numel() * side_dst->element_size() >=
                    (c.side.rows - 1) * c.side.dst_pitch + (world - 1) * c.side.dst_piece_off + c.side.row_bytes,
                "comm_gemm: side gather destination too small");
    if (c.side.sf_chunk > 0)
      TORCH_CHECK(c.side.dst_sf != nullptr && side_dst_sf->numel() * side_dst_sf->element_size() >=
                      static_cast<int64_t>(c.side.row_tiles) * world * c.side.sf_chunk,
                  "comm_gemm: side gather scale destination too small");
  }
  cudaError_t e = teb200::comm_gemm(c, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "comm_gemm failed: ", cudaGetErrorString(e));
}

// ---------------------------------------------------------------------------- fused attention
// Tensors are [b, h, s, d] views (any strides with d contiguous).
void fill_strides(const at::Tensor& t, long long& sb, long long& sh, long long& ss) {
  TORCH_CHECK(t.dim() == 4 && t.stride(3) == 1, "attention tensors must be [b, h, s, d] views with contiguous d");
  sb = t.stride(0);
  sh = t.stride(1);
  ss = t.stride(2);
}

teb200::FlashArgs flash_args(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& out,
                             const at::Tensor& lse, double scale, bool causal, bool bottom_right,
                             const at::Tensor& status) {
  TORCH_CHECK(q.size(3) == 128 && k.size(3) == 128 && v.size(3) == 128, "fused attention needs head dim 128");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf, "fused attention needs fp16/bf16");
  teb200::FlashArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.out = out.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.b = static_cast<int>(q.size(0)); a.hq = static_cast<int>(q.size(1)); a.hk = static_cast<int>(k.size(1));
  a.sq = static_cast<int>(q.size(2)); a.sk = static_cast<int>(k.size(2));
  a.s_pad = static_cast<int>(lse.size(2));
  a.causal = causal; a.bottom_right = bottom_right; a.is_bf16 = q.scalar_type() == at::kBFloat16;
  a.scale = static_cast<float>(scale);
  fill_strides(q, a.q_sb, a.q_sh, a.q_ss);
  fill_strides(k, a.k_sb, a.k_sh, a.k_ss);
  fill_strides(v, a.v_sb, a.v_sh, a.v_ss);
  fill_strides(out, a.o_sb, a.o_sh, a.o_ss);
  a.status = status.data_ptr<int>();
  return a;
}

void flash_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& out,
               const at::Tensor& lse, double scale, bool causal, bool bottom_right, const at::Tensor& status,
               const OptT& timeline, int64_t window_left, int64_t window_right) {
  c10::cuda::CUDAGuard guard(q.device());
  teb200::FlashArgs a = flash_args(q, k, v, out, lse, scale, causal, bottom_right, status);
  a.window_left = static_cast<int>(window_left); a.window_right = static_cast<int>(window_right);
  if (timeline.has_value() && timeline->defined()) {
    TORCH_CHECK(timeline->scalar_type() == at::kLong && timeline->numel() >= 1024, "timeline must be int64 [64, 16]");
    a.timeline = reinterpret_cast<long long*>(timeline->data_ptr());
  }
  cudaError_t e = teb200::flash_fwd(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "flash_fwd failed: ", cudaGetErrorString(e));
}


// dK/dV of a few key heads underfill the GPU (tensor-parallel shards): split every head group over
// several CTAs that write partial sums, and add the partials afterwards.
void run_dkdv(teb200::FlashArgs& a, const at::Tensor& k, const at::Tensor& dk, const at::Tensor& dv, bool zero_fill) {
  const int64_t ctas = static_cast<int64_t>((a.sk + 127) / 128) * a.hk * a.b;
  const int group = a.hq / a.hk;
  static const bool allow_split = []() {
    const char* e = std::getenv("TEB200_ATTN_GSPLIT");
    return e == nullptr || e[0] != '0';
  }();
  if (allow_split && group > 1 && ctas < 2 * 148) {
    auto opts = dk.options();
    std::vector<int64_t> shape = {group, k.size(0), k.size(1), k.size(2), 128};
    at::Tensor pk = zero_fill ? at::zeros(shape, opts) : at::empty(shape, opts);
    at::Tensor pv = zero_fill ? at::zeros(shape, opts) : at::empty(shape, opts);
    a.dk = pk.data_ptr(); a.dv = pv.data_ptr();
    a.dk_sb = a.dv_sb = pk.stride(1); a.dk_sh = a.dv_sh = pk.stride(2); a.dk_ss = a.dv_ss = pk.stride(3);
    a.gsplit = group; a.dk_sg = pk.stride(0);
    cudaError_t e = teb200::flash_bwd_dkdv(a, cur_stream());
    TORCH_CHECK(e == cudaSuccess, "flash_bwd_dkdv (split) failed: ", cudaGetErrorString(e));
    at::sum_out(const_cast<at::Tensor&>(dk), pk, at::IntArrayRef{0});
    at::sum_out(const_cast<at::Tensor&>(dv), pv, at::IntArrayRef{0});
    return;
  }
  cudaError_t e = teb200::flash_bwd_dkdv(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "flash_bwd_dkdv failed: ", cudaGetErrorString(e));
}

void flash_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
               const at::Tensor& out, const at::Tensor& lse, const at::Tensor& delta, const at::Tensor& dq,
               const at::Tensor& dk, const at::Tensor& dv, double scale, bool causal, bool bottom_right,
               const at::Tensor& status, int64_t window_left, int64_t window_right) {
  c10::cuda::CUDAGuard guard(q.device());
  teb200::FlashArgs a = flash_args(q, k, v, out, lse, scale, causal, bottom_right, status);
  a.window_left = static_cast<int>(window_left); a.window_right = static_cast<int>(window_right);
  a.dout = dout.data_ptr();
  a.delta = delta.data_ptr<float>();
  a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
  fill_strides(dout, a.do_sb, a.do_sh, a.do_ss);
  fill_strides(dq, a.dq_sb, a.dq_sh, a.dq_ss);
  fill_strides(dk, a.dk_sb, a.dk_sh, a.dk_ss);
  fill_strides(dv, a.dv_sb, a.dv_sh, a.dv_ss);
  cudaError_t e = teb200::flash_delta(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "flash_delta failed: ", cudaGetErrorString(e));
  run_dkdv(a, k, dk, dv, false);
  e = teb200::flash_bwd_dq(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "flash_bwd_dq failed: ", cudaGetErrorString(e));
}

// Packed variable-length sequences: q / out / dout / dq are [1, hq, tq, d] views, k / v / dk / dv
// [1, hk, tk, d]; cu_* hold cumulative lengths, off_* the first token of every sequence.
void set_varlen(teb200::FlashArgs& a, const at::Tensor& q, const at::Tensor& k, const at::Tensor& cu_q,
                const at::Tensor& cu_k, const at::Tensor& off_q, const at::Tensor& off_k, int64_t max_sq,
                int64_t max_sk) {
  for (const at::Tensor* t : {&cu_q, &cu_k, &off_q, &off_k})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous() && t->numel() == cu_q.numel(),
                "cumulative sequence lengths must be contiguous int32 CUDA tensors of equal length");
  TORCH_CHECK(q.size(0) == 1 && k.size(0) == 1 && cu_q.numel() >= 2, "packed attention takes [1, h, t, d] views");
  a.cu_q = cu_q.data_ptr<int>(); a.cu_k = cu_k.data_ptr<int>();
  a.off_q = off_q.data_ptr<int>(); a.off_k = off_k.data_ptr<int>();
  a.b = static_cast<int>(cu_q.numel() - 1);
  a.tq = static_cast<int>(q.size(2)); a.tk = static_cast<int>(k.size(2));
  a.sq = static_cast<int>(max_sq); a.sk = static_cast<int>(max_sk);
}

void flash_fwd_varlen(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& out,
                      const at::Tensor& lse, const at::Tensor& cu_q, const at::Tensor& cu_k, const at::Tensor& off_q,
                      const at::Tensor& off_k, int64_t max_sq, int64_t max_sk, double scale, bool causal,
                      bool bottom_right, const at::Tensor& status, int64_t window_left, int64_t window_right) {
  c10::cuda::CUDAGuard guard(q.device());
  teb200::FlashArgs a = flash_args(q, k, v, out, lse, scale, causal, bottom_right, status);
  a.window_left = static_cast<int>(window_left); a.window_right = static_cast<int>(window_right);
  set_varlen(a, q, k, cu_q, cu_k, off_q, off_k, max_sq, max_sk);
  TORCH_CHECK(lse.size(0) == a.b && lse.size(1) == a.hq && lse.size(2) >= max_sq, "lse must be [sequences, hq, >= max_sq]");
  cudaError_t e = teb200::flash_fwd(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "flash_fwd (packed) failed: ", cudaGetErrorString(e));
}

void flash_bwd_varlen(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                      const at::Tensor& out, const at::Tensor& lse, const at::Tensor& delta, const at::Tensor& dq,
                      const at::Tensor& dk, const at::Tensor& dv, const at::Tensor& cu_q, const at::Tensor& cu_k,
                      const at::Tensor& off_q, const at::Tensor& off_k, int64_t max_sq, int64_t max_sk, double scale,
                      bool causal, bool bottom_right, const at::Tensor& status, int64_t window_left,
                      int64_t window_right) {
  c10::cuda::CUDAGuard guard(q.device());
  teb200::FlashArgs a = flash_args(q, k, v, out, lse, scale, causal, bottom_right, status);
  a.window_left = static_cast<int>(window_left); a.window_right = static_cast<int>(window_right);
  set_varlen(a, q, k, cu_q, cu_k, off_q, off_k, max_sq, max_sk);
  TORCH_CHECK(lse.size(0) == a.b && lse.size(2) % 128 == 0 && lse.size(2) >= max_sq && delta.sizes() == lse.sizes(),
              "lse / delta must be [sequences, hq, s_pad] with s_pad a multiple of 128");
  a.dout = dout.data_ptr();
  a.delta = delta.data_ptr<float>();
  a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
  fill_strides(dout, a.do_sb, a.do_sh, a.do_ss);
  fill_strides(dq, a.dq_sb, a.dq_sh, a.dq_ss);
  fill_strides(dk, a.dk_sb, a.dk_sh, a.dk_ss);
  fill_strides(dv, a.dv_sb, a.dv_sh, a.dv_ss);
  cudaError_t e = teb200::flash_delta(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "flash_delta (packed) failed: ", cudaGetErrorString(e));
  run_dkdv(a, k, dk, dv, true);
  e = teb200::flash_bwd_dq(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "flash_bwd_dq (packed) failed: ", cudaGetErrorString(e));
}

// ---------------------------------------------------------------------------- packed sequences / KV cache
namespace {
const int* cu_ptr(const at::Tensor& cu) {
  TORCH_CHECK(cu.is_cuda() && cu.scalar_type() == at::kInt && cu.is_contiguous() && cu.numel() >= 2,
              "cumulative sequence lengths must be a contiguous int32 CUDA tensor of at least 2 entries");
  return cu.data_ptr<int>();
}
int thd_dtype(const at::Tensor& t) {
  if (t.scalar_type() == at::kFloat) return 0;
  if (t.scalar_type() == at::kHalf) return 1;
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, "expected fp32, fp16 or bf16");
  return 2;
}
void thd_check(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, " failed: ", cudaGetErrorString(e)); }
}  // namespace

at::Tensor thd_get_partitioned_indices(const at::Tensor& cu, int64_t total_tokens, int64_t world, int64_t rank) {
  c10::cuda::CUDAGuard guard(cu.device());
  at::Tensor out = at::empty({total_tokens / world}, cu.options());
  thd_check(teb200::thd_partition_indices(out.data_ptr<int>(), cu_ptr(cu), static_cast<int>(cu.numel() - 1),
                                          static_cast<int>(total_tokens), static_cast<int>(world),
                                          static_cast<int>(rank), cur_stream()), "thd_get_partitioned_indices");
  return out;
}

// tensor [t, ...] or [2, t, ...] (stacked K/V)
at::Tensor thd_read_half_tensor(const at::Tensor& tensor, const at::Tensor& cu, int64_t half_idx, bool stacked) {
  c10::cuda::CUDAGuard guard(tensor.device());
  at::Tensor x = tensor.contiguous();
  const int seq_dim = stacked ? 1 : 0;
  const int64_t t = x.size(seq_dim);
  const int64_t row_bytes = x.numel() / (t * (stacked ? x.size(0) : 1)) * x.element_size();
  auto shape = x.sizes().vec();
  shape[seq_dim] = t / 2;
  at::Tensor half = at::empty(shape, x.options());
  thd_check(teb200::thd_read_half(half.data_ptr(), x.data_ptr(), cu_ptr(cu), static_cast<int>(cu.numel() - 1),
                                  static_cast<int>(t), stacked ? static_cast<int>(x.size(0)) : 1,
                                  static_cast<int>(row_bytes), static_cast<int>(half_idx), cur_stream()),
            "thd_read_half_tensor");
  return half;
}

void thd_second_half_lse_correction(const at::Tensor& lse, const at::Tensor& lse_per_step, const at::Tensor& cu) {
  c10::cuda::CUDAGuard guard(lse.device());
  TORCH_CHECK(lse.dim() == 2 && lse.is_contiguous() && lse.scalar_type() == at::kFloat && lse_per_step.is_contiguous() &&
              lse_per_step.scalar_type() == at::kFloat && lse_per_step.size(0) == lse.size(0) &&
              lse_per_step.size(1) * 2 == lse.size(1), "lse must be fp32 [heads, t], lse_per_step [heads, t / 2]");
  thd_check(teb200::thd_lse_half(lse.data_ptr<float>(), lse_per_step.data_ptr<float>(), cu_ptr(cu),
                                 static_cast<int>(cu.numel() - 1), static_cast<int>(lse.size(0)),
                                 static_cast<int>(lse.size(1)), 0, cur_stream()), "thd_second_half_lse_correction");
}

at::Tensor thd_read_second_half_lse(const at::Tensor& lse, const at::Tensor& cu) {
  c10::cuda::CUDAGuard guard(lse.device());
  TORCH_CHECK(lse.dim() == 2 && lse.is_contiguous() && lse.scalar_type() == at::kFloat, "lse must be fp32 [heads, t]");
  at::Tensor half = at::empty({lse.size(0), lse.size(1) / 2}, lse.options());
  thd_check(teb200::thd_lse_half(lse.data_ptr<float>(), half.data_ptr<float>(), cu_ptr(cu),
                                 static_cast<int>(cu.numel() - 1), static_cast<int>(lse.size(0)),
                                 static_cast<int>(lse.size(1)), 1, cur_stream()), "thd_read_second_half_lse");
  return half;
}

void thd_out_correction(const at::Tensor& out, const at::Tensor& out_per_step, const at::Tensor& lse,
                        const at::Tensor& lse_per_step, const at::Tensor& cu, bool only_second_half) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.dim() == 3 && out.is_contiguous() && out_per_step.is_contiguous() &&
              out.scalar_type() == out_per_step.scalar_type(), "out / out_per_step must be contiguous [t, h, d] of one dtype");
  const int64_t t = out.size(0), ts = only_second_half ? t / 2 : t;
  TORCH_CHECK(out_per_step.size(0) == ts && lse.is_contiguous() && lse_per_step.is_contiguous() &&
              lse.scalar_type() == at::kFloat && lse_per_step.scalar_type() == at::kFloat && lse.size(0) == out.size(1) &&
              lse.size(1) == t && lse_per_step.size(0) == out.size(1) && lse_per_step.size(1) == ts,
              "lse must be fp32 [h, t] and the per-step tensors must cover t (or t / 2) tokens");
  thd_check(teb200::thd_out_correction(out.data_ptr(), out_per_step.data_ptr(), lse.data_ptr<float>(),
                                       lse_per_step.data_ptr<float>(), cu_ptr(cu), static_cast<int>(cu.numel() - 1),
                                       static_cast<int>(out.size(1)), static_cast<int>(out.size(2)),
                                       static_cast<int>(t), only_second_half ? 1 : 0, thd_dtype(out), cur_stream()),
            "thd_out_correction");
}

void thd_grad_correction(const at::Tensor& grad, const at::Tensor& grad_per_step, const at::Tensor& cu,
                         int64_t mode_first, int64_t mode_second, bool stacked) {
  c10::cuda::CUDAGuard guard(grad.device());
  TORCH_CHECK(grad.is_contiguous() && grad_per_step.is_contiguous() && grad.scalar_type() == grad_per_step.scalar_type(),
              "grad / grad_per_step must be contiguous and of one dtype");
  const int seq_dim = stacked ? 1 : 0;
  const int64_t t = grad.size(seq_dim), ts = grad_per_step.size(seq_dim);
  const int64_t lead = stacked ? grad.size(0) : 1;
  const int64_t row = grad.numel() / (t * lead);
  thd_check(teb200::thd_grad_correction(grad.data_ptr(), grad_per_step.data_ptr(), cu_ptr(cu),
                                        static_cast<int>(cu.numel() - 1), static_cast<int>(lead), static_cast<int>(row),
                                        static_cast<int>(t), static_cast<int>(ts), static_cast<int>(mode_first),
                                        static_cast<int>(mode_second), thd_dtype(grad), cur_stream()),
            "thd_grad_correction");
}

at::Tensor convert_thd_to_bshd(const at::Tensor& tensor, const at::Tensor& cu, int64_t b, int64_t max_seq_len) {
  c10::cuda::CUDAGuard guard(tensor.device());
  at::Tensor x = tensor.contiguous();
  auto shape = x.sizes().vec();
  shape[0] = max_seq_len;
  shape.insert(shape.begin(), b);
  at::Tensor out = at::zeros(shape, x.options());
  TORCH_CHECK(cu.numel() - 1 <= b, "more sequences than batch entries");
  const int64_t row_bytes = x.numel() / std::max<int64_t>(x.size(0), 1) * x.element_size();
  thd_check(teb200::thd_bshd_convert(x.data_ptr(), out.data_ptr(), cu_ptr(cu), static_cast<int>(cu.numel() - 1),
                                     static_cast<int>(x.size(0)), static_cast<int>(max_seq_len),
                                     static_cast<int>(row_bytes), 1, cur_stream()), "convert_thd_to_bshd");
  return out;
}

at::Tensor convert_bshd_to_thd(const at::Tensor& tensor, const at::Tensor& cu, int64_t t) {
  c10::cuda::CUDAGuard guard(tensor.device());
  at::Tensor x = tensor.contiguous();
  auto shape = x.sizes().vec();
  shape.erase(shape.begin());
  shape[0] = t;
  at::Tensor out = at::zeros(shape, x.options());
  TORCH_CHECK(cu.numel() - 1 <= x.size(0), "more sequences than batch entries");
  const int64_t row_bytes = x.numel() / std::max<int64_t>(x.size(0) * x.size(1), 1) * x.element_size();
  thd_check(teb200::thd_bshd_convert(out.data_ptr(), x.data_ptr(), cu_ptr(cu), static_cast<int>(cu.numel() - 1),
                                     static_cast<int>(t), static_cast<int>(x.size(1)), static_cast<int>(row_bytes), 0,
                                     cur_stream()), "convert_bshd_to_thd");
  return out;
}

// caches [num_pages, page_size, h, d]; new_k / new_v [sum new, h, d]; returns packed (k, v) of all live sequences
std::vector<at::Tensor> kv_cache_step(const at::Tensor& new_k, const at::Tensor& new_v, const at::Tensor& cache_k,
                                      const at::Tensor& cache_v, const at::Tensor& page_table, const at::Tensor& cu_new,
                                      const at::Tensor& cu_kv, int64_t total, const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(cache_k.device());
  TORCH_CHECK(cache_k.is_contiguous() && cache_v.is_contiguous() && cache_k.dim() == 4 && cache_v.dim() == 4,
              "caches must be contiguous [pages, page_size, h, d]");
  TORCH_CHECK(page_table.is_cuda() && page_table.scalar_type() == at::kInt && page_table.is_contiguous() &&
              page_table.dim() == 2 && page_table.size(0) == cu_kv.numel() - 1 && cu_new.numel() == cu_kv.numel(),
              "page_table must be int32 [sequences, width]");
  at::Tensor nk = new_k.contiguous(), nv = new_v.contiguous();
  TORCH_CHECK(nk.scalar_type() == cache_k.scalar_type() && nv.scalar_type() == cache_v.scalar_type(),
              "new tokens and cache must have one dtype");
  at::Tensor out_k = at::empty({total, cache_k.size(2), cache_k.size(3)}, cache_k.options());
  at::Tensor out_v = at::empty({total, cache_v.size(2), cache_v.size(3)}, cache_v.options());
  teb200::KvCacheArgs a;
  a.new_k = nk.data_ptr(); a.new_v = nv.data_ptr();
  a.cache_k = cache_k.data_ptr(); a.cache_v = cache_v.data_ptr();
  a.out_k = out_k.data_ptr(); a.out_v = out_v.data_ptr();
  a.cu_new = cu_ptr(cu_new); a.cu_kv = cu_ptr(cu_kv); a.page_table = page_table.data_ptr<int>();
  a.nb = static_cast<int>(cu_kv.numel() - 1); a.width = static_cast<int>(page_table.size(1));
  a.page_size = static_cast<int>(cache_k.size(1)); a.num_pages = static_cast<int>(cache_k.size(0));
  a.total = static_cast<int>(total);
  a.row_bytes_k = static_cast<int>(cache_k.size(2) * cache_k.size(3) * cache_k.element_size());
  a.row_bytes_v = static_cast<int>(cache_v.size(2) * cache_v.size(3) * cache_v.element_size());
  TORCH_CHECK(nk.numel() * nk.element_size() % a.row_bytes_k == 0, "new_k rows do not match the cache rows");
  a.status = status.data_ptr<int>();
  thd_check(teb200::kv_cache_step(a, cur_stream()), "kv_cache_step");
  return {out_k, out_v};
}

// ---------------------------------------------------------------------------- NVFP4
template <typename T = void>
T* optr(const OptT& t) {
  return t.has_value() && t->defined() ? static_cast<T*>(t->data_ptr()) : nullptr;
}

void nvfp4_amax(const at::Tensor& x, int64_t R, int64_t C, bool with_rht, const at::Tensor& out2) {
  c10::cuda::CUDAGuard guard(x.device());
  cudaError_t e = teb200::nvfp4_amax(x.data_ptr(), dtype_code(x), static_cast<int>(R), static_cast<int>(C),
                                     with_rht ? 1 : 0, out2.data_ptr<float>(), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "nvfp4_amax failed: ", cudaGetErrorString(e));
}

void quantize_nvfp4(const at::Tensor& x, int64_t R, int64_t C, const OptT& amax_row, const OptT& amax_col,
                    const OptT& row_data, const OptT& row_scale, const OptT& col_data, const OptT& col_scale,
                    bool with_rht, bool with_2d, bool stochastic, int64_t seed, int64_t offset,
                    const OptT& offset_dev) {
  c10::cuda::CUDAGuard guard(x.device());
  teb200::Nvfp4Args a;
  a.x = x.data_ptr();
  a.x_dtype = dtype_code(x);
  a.R = static_cast<int>(R);
  a.C = static_cast<int>(C);
  a.amax_row = optr<float>(amax_row);
  a.amax_col = optr<float>(amax_col);
  a.row_data = optr<uint8_t>(row_data);
  a.row_scale = optr<uint8_t>(row_scale);
  a.col_data = optr<uint8_t>(col_data);
  a.col_scale = optr<uint8_t>(col_scale);
  a.with_rht = with_rht;
  a.with_2d = with_2d;
  a.stochastic = stochastic;
  a.seed = static_cast<uint64_t>(seed);
  a.offset = static_cast<uint64_t>(offset);
  if (offset_dev.has_value() && offset_dev->defined()) {
    TORCH_CHECK(offset_dev->scalar_type() == at::kLong && offset_dev->is_cuda(), "the device RNG counter must be int64 on the GPU");
    a.offset_dev = reinterpret_cast<const unsigned long long*>(offset_dev->data_ptr<int64_t>());
  }
  TORCH_CHECK(a.row_data == nullptr || a.amax_row != nullptr, "row-wise NVFP4 needs its global amax");
  TORCH_CHECK(a.col_data == nullptr || a.amax_col != nullptr, "column-wise NVFP4 needs its global amax");
  cudaError_t e = teb200::quantize_nvfp4(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "quantize_nvfp4 failed: ", cudaGetErrorString(e));
}

void dequantize_nvfp4(const at::Tensor& q, const at::Tensor& sf, const at::Tensor& amax, int64_t R, int64_t C,
                      const at::Tensor& out) {
  c10::cuda::CUDAGuard guard(q.device());
  cudaError_t e = teb200::dequantize_nvfp4(static_cast<const uint8_t*>(q.data_ptr()),
                                           static_cast<const uint8_t*>(sf.data_ptr()), amax.data_ptr<float>(),
                                           static_cast<int>(R), static_cast<int>(C), out.data_ptr(), dtype_code(out),
                                           cur_stream());
  TORCH_CHECK(e == cudaSuccess, "dequantize_nvfp4 failed: ", cudaGetErrorString(e));
}

// ---------------------------------------------------------------------------- MoE router / permutation
teb200::RouterArgs router_args(const at::Tensor& logits, int64_t topk, bool pre_softmax, double scaling,
                               int64_t score_fn, const OptT& expert_bias) {
  teb200::RouterArgs a;
  a.logits = logits.data_ptr();
  a.dtype = dtype_code(logits);
  a.T = static_cast<int>(logits.size(0));
  a.E = static_cast<int>(logits.size(1));
  a.topk = static_cast<int>(topk);
  a.score_fn = static_cast<int>(score_fn);
  a.use_pre_softmax = pre_softmax ? 1 : 0;
  a.scaling_factor = static_cast<float>(scaling);
  a.expert_bias = optr<float>(expert_bias);
  return a;
}

std::vector<at::Tensor> router_topk(const at::Tensor& logits, int64_t topk, bool pre_softmax, double scaling,
                                    int64_t score_fn, const OptT& expert_bias, bool want_scores) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous(), "router logits must be a contiguous [T, E] tensor");
  teb200::RouterArgs a = router_args(logits, topk, pre_softmax, scaling, score_fn, expert_bias);
  auto f32 = logits.options().dtype(at::kFloat);
  at::Tensor probs = at::empty({a.T, a.E}, f32);
  at::Tensor rmap = at::empty({a.T, a.E}, logits.options().dtype(at::kByte));
  at::Tensor idx = at::empty({a.T, a.topk}, logits.options().dtype(at::kInt));
  at::Tensor tpe = at::empty({a.E}, logits.options().dtype(at::kInt));
  at::Tensor scores = want_scores ? at::empty({a.T, a.E}, f32) : at::Tensor();
  a.probs = probs.data_ptr<float>();
  a.routing_map = rmap.data_ptr<uint8_t>();
  a.topk_idx = idx.data_ptr<int32_t>();
  a.tokens_per_expert = tpe.data_ptr<int32_t>();
  a.scores = want_scores ? scores.data_ptr<float>() : nullptr;
  cudaError_t e = teb200::router_topk_fwd(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "router_topk failed: ", cudaGetErrorString(e));
  return {probs, rmap, idx, tpe, scores};
}

at::Tensor router_topk_bwd(const at::Tensor& logits, const at::Tensor& rmap, const at::Tensor& grad_probs, int64_t topk,
                           bool pre_softmax, double scaling, int64_t score_fn) {
  c10::cuda::CUDAGuard guard(logits.device());
  teb200::RouterArgs a = router_args(logits, topk, pre_softmax, scaling, score_fn, OptT());
  a.routing_map = rmap.data_ptr<uint8_t>();
  at::Tensor g = at::empty_like(logits);
  cudaError_t e = teb200::router_topk_bwd(a, grad_probs.data_ptr<float>(), g.data_ptr(), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "router_topk_bwd failed: ", cudaGetErrorString(e));
  return g;
}

std::vector<at::Tensor> permute_rows(const at::Tensor& inp, const at::Tensor& dest_row, const OptT& probs, int64_t n_out) {
  c10::cuda::CUDAGuard guard(inp.device());
  TORCH_CHECK(inp.dim() == 2 && inp.is_contiguous() && dest_row.is_contiguous() && dest_row.scalar_type() == at::kInt);
  at::Tensor out = at::zeros({n_out, inp.size(1)}, inp.options());
  at::Tensor pout;
  const float* pp = nullptr;
  float* po = nullptr;
  if (probs.has_value() && probs->defined()) {
    TORCH_CHECK(probs->scalar_type() == at::kFloat && probs->is_contiguous());
    pout = at::zeros({n_out}, probs->options());
    pp = probs->data_ptr<float>();
    po = pout.data_ptr<float>();
  }
  cudaError_t e = teb200::permute_rows(inp.data_ptr(), out.data_ptr(), dest_row.data_ptr<int32_t>(), pp, po,
                                       static_cast<int>(inp.size(0)), static_cast<int>(dest_row.size(1)),
                                       static_cast<int>(inp.size(1)), dtype_code(inp), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "permute_rows failed: ", cudaGetErrorString(e));
  return {out, pout};
}

at::Tensor unpermute_rows(const at::Tensor& inp, const at::Tensor& dest_row, const OptT& w) {
  c10::cuda::CUDAGuard guard(inp.device());
  TORCH_CHECK(inp.dim() == 2 && inp.is_contiguous() && dest_row.is_contiguous() && dest_row.scalar_type() == at::kInt);
  const int T = static_cast<int>(dest_row.size(0));
  at::Tensor out = at::empty({T, inp.size(1)}, inp.options());
  cudaError_t e = teb200::unpermute_rows(inp.data_ptr(), out.data_ptr(), dest_row.data_ptr<int32_t>(), optr<float>(w), T,
                                         static_cast<int>(dest_row.size(1)), static_cast<int>(inp.size(1)),
                                         dtype_code(inp), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "unpermute_rows failed: ", cudaGetErrorString(e));
  return out;
}

std::vector<at::Tensor> build_dest_rows(const at::Tensor& topk_idx, int64_t E, int64_t align) {
  c10::cuda::CUDAGuard guard(topk_idx.device());
  TORCH_CHECK(topk_idx.dim() == 2 && topk_idx.is_contiguous() && topk_idx.scalar_type() == at::kInt);
  at::Tensor counts = at::empty({E}, topk_idx.options());
  at::Tensor offsets = at::empty({E + 1}, topk_idx.options());
  at::Tensor dest = at::empty_like(topk_idx);
  cudaError_t e = teb200::build_dest_rows(topk_idx.data_ptr<int32_t>(), static_cast<int>(topk_idx.size(0)),
                                          static_cast<int>(topk_idx.size(1)), static_cast<int>(E),
                                          static_cast<int>(align), counts.data_ptr<int32_t>(),
                                          offsets.data_ptr<int32_t>(), dest.data_ptr<int32_t>(), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "build_dest_rows failed: ", cudaGetErrorString(e));
  return {dest, counts, offsets};
}

// ---------------------------------------------------------------------------- expert-parallel exchange
void ep_counts(std::vector<int64_t> counts_ptrs, std::vector<int64_t> flag_ptrs, const at::Tensor& my_counts,
               const at::Tensor& base, const at::Tensor& splits, const at::Tensor& seg, int64_t L, int64_t rank,
               int64_t align, int64_t epoch, const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(my_counts.device());
  teb200::EpCountsArgs a;
  a.ep = static_cast<int>(counts_ptrs.size());
  for (int r = 0; r < a.ep; ++r) {
    a.counts_all[r] = reinterpret_cast<int32_t*>(counts_ptrs[r]);
    a.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  a.my_counts = my_counts.data_ptr<int32_t>();
  a.base = base.data_ptr<int32_t>();
  a.splits = splits.data_ptr<int32_t>();
  a.seg = seg.data_ptr<int32_t>();
  a.L = static_cast<int>(L);
  a.rank = static_cast<int>(rank);
  a.align = static_cast<int>(align);
  a.epoch = static_cast<uint32_t>(epoch);
  a.status = status.data_ptr<int>();
  cudaError_t e = teb200::ep_counts(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "ep_counts failed: ", cudaGetErrorString(e));
}

void ep_push(const at::Tensor& x, const at::Tensor& within, const at::Tensor& base, const OptT& scale, const OptT& probs,
             std::vector<int64_t> dst_ptrs, std::vector<int64_t> dst_prob_ptrs, std::vector<int64_t> flag_ptrs,
             const at::Tensor& rowmap, const at::Tensor& counter, int64_t L, int64_t rank, int64_t cap_rows, int64_t epoch,
             const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && (x.size(1) * x.element_size()) % 16 == 0);
  teb200::EpPushArgs a;
  a.ep = static_cast<int>(dst_ptrs.size());
  for (int r = 0; r < a.ep; ++r) {
    a.dst[r] = reinterpret_cast<void*>(dst_ptrs[r]);
    a.dst_probs[r] = dst_prob_ptrs.empty() ? nullptr : reinterpret_cast<float*>(dst_prob_ptrs[r]);
    a.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  a.x = x.data_ptr();
  a.within = within.data_ptr<int32_t>();
  a.base = base.data_ptr<int32_t>();
  a.scale = optr<float>(scale);
  a.probs = optr<float>(probs);
  a.rowmap = rowmap.data_ptr<int32_t>();
  a.cta_counter = reinterpret_cast<unsigned*>(counter.data_ptr<int32_t>());
  a.T = static_cast<int>(x.size(0));
  a.L = static_cast<int>(L);
  a.rank = static_cast<int>(rank);
  a.vec_per_row = static_cast<int>(x.size(1) * x.element_size() / 16);
  a.cap_rows = static_cast<int>(cap_rows);
  a.is_bf16 = x.scalar_type() == at::kBFloat16;
  a.epoch = static_cast<uint32_t>(epoch);
  a.status = status.data_ptr<int>();
  cudaError_t e = teb200::ep_push(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "ep_push failed: ", cudaGetErrorString(e));
}

void ep_wait(int64_t flags_ptr, int64_t n, int64_t epoch, const at::Tensor& status, int64_t limit_cycles) {
  c10::cuda::CUDAGuard guard(status.device());
  cudaError_t e = teb200::ep_wait(reinterpret_cast<const uint32_t*>(flags_ptr), static_cast<int>(n),
                                  static_cast<uint32_t>(epoch), status.data_ptr<int>(), cur_stream(), limit_cycles);
  TORCH_CHECK(e == cudaSuccess, "ep_wait failed: ", cudaGetErrorString(e));
}

void ep_signal(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t epoch, const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  teb200::EpSignalArgs a;
  a.ep = static_cast<int>(flag_ptrs.size());
  for (int r = 0; r < a.ep; ++r) a.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  a.rank = static_cast<int>(rank);
  a.epoch = static_cast<uint32_t>(epoch);
  cudaError_t e = teb200::ep_signal(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "ep_signal failed: ", cudaGetErrorString(e));
}

void ep_pull(std::vector<int64_t> src_ptrs, const at::Tensor& rowmap, const OptT& w, const at::Tensor& out, const OptT& g,
             const OptT& dots, int64_t L, std::vector<int64_t> src_scalar_ptrs, const OptT& out_scalars) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.dim() == 2 && out.is_contiguous() && (out.size(1) * out.element_size()) % 16 == 0);
  teb200::EpPullArgs a;
  a.ep = static_cast<int>(src_ptrs.size());
  for (int r = 0; r < a.ep; ++r) a.src[r] = reinterpret_cast<const void*>(src_ptrs[r]);
  a.rowmap = rowmap.data_ptr<int32_t>();
  a.w = optr<float>(w);
  a.out = out.data_ptr();
  a.g = g.has_value() && g->defined() ? g->data_ptr() : nullptr;
  a.dots = optr<float>(dots);
  if (!src_scalar_ptrs.empty()) {
    for (int r = 0; r < a.ep; ++r) a.src_s[r] = reinterpret_cast<const float*>(src_scalar_ptrs[r]);
    a.out_s = optr<float>(out_scalars);
  }
  a.T = static_cast<int>(out.size(0));
  a.L = static_cast<int>(L);
  a.vec_per_row = static_cast<int>(out.size(1) * out.element_size() / 16);
  a.is_bf16 = out.scalar_type() == at::kBFloat16;
  cudaError_t e = teb200::ep_pull(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "ep_pull failed: ", cudaGetErrorString(e));
}

void peer_sum(std::vector<int64_t> src_ptrs, const at::Tensor& out) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous() && (out.numel() * out.element_size()) % 16 == 0);
  teb200::PeerSumArgs a;
  a.n = static_cast<int>(src_ptrs.size());
  for (int r = 0; r < a.n; ++r) a.src[r] = reinterpret_cast<const void*>(src_ptrs[r]);
  a.out = out.data_ptr();
  a.vecs = static_cast<long long>(out.numel() * out.element_size() / 16);
  a.is_bf16 = out.scalar_type() == at::kBFloat16;
  cudaError_t e = teb200::peer_sum(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "peer_sum failed: ", cudaGetErrorString(e));
}

// ---------------------------------------------------------------------------- softmax / dropout
at::Tensor softmax_fwd(const at::Tensor& x, const OptT& mask, double scale, bool causal, int64_t sq, int64_t heads) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous());
  at::Tensor y = at::empty_like(x);
  teb200::SoftmaxArgs a;
  a.x = x.data_ptr(); a.y = y.data_ptr();
  a.mask = optr<uint8_t>(mask);
  a.dtype = dtype_code(x);
  a.cols = static_cast<int>(x.size(-1));
  a.rows = x.numel() / a.cols;
  a.sq = static_cast<int>(sq); a.heads = static_cast<int>(heads);
  a.scale = static_cast<float>(scale);
  a.causal = causal ? 1 : 0;
  cudaError_t e = teb200::softmax_fwd(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "softmax_fwd failed: ", cudaGetErrorString(e));
  return y;
}

at::Tensor softmax_bwd(const at::Tensor& probs, const at::Tensor& dprobs, double scale) {
  c10::cuda::CUDAGuard guard(probs.device());
  TORCH_CHECK(probs.is_contiguous() && dprobs.is_contiguous() && probs.scalar_type() == dprobs.scalar_type());
  at::Tensor dx = at::empty_like(probs);
  teb200::SoftmaxArgs a;
  a.x = probs.data_ptr(); a.dy = dprobs.data_ptr(); a.y = dx.data_ptr();
  a.dtype = dtype_code(probs);
  a.cols = static_cast<int>(probs.size(-1));
  a.rows = probs.numel() / a.cols;
  a.scale = static_cast<float>(scale);
  cudaError_t e = teb200::softmax_bwd(a, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "softmax_bwd failed: ", cudaGetErrorString(e));
  return dx;
}

std::vector<at::Tensor> dropout_fwd(const at::Tensor& x, double p, int64_t seed, int64_t offset) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous());
  at::Tensor y = at::empty_like(x);
  at::Tensor bits = at::empty({(x.numel() + 7) / 8}, x.options().dtype(at::kByte));
  cudaError_t e = teb200::dropout_fwd(x.data_ptr(), y.data_ptr(), bits.data_ptr<uint8_t>(), x.numel(), dtype_code(x),
                                      static_cast<float>(p), static_cast<uint64_t>(seed), static_cast<uint64_t>(offset),
                                      cur_stream());
  TORCH_CHECK(e == cudaSuccess, "dropout_fwd failed: ", cudaGetErrorString(e));
  return {y, bits};
}

at::Tensor dropout_bwd(const at::Tensor& dy, const at::Tensor& bits, double p) {
  c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(dy.is_contiguous());
  at::Tensor dx = at::empty_like(dy);
  cudaError_t e = teb200::dropout_bwd(dy.data_ptr(), bits.data_ptr<uint8_t>(), dx.data_ptr(), dy.numel(), dtype_code(dy),
                                      static_cast<float>(p), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "dropout_bwd failed: ", cudaGetErrorString(e));
  return dx;
}

void delayed_scaling_update(const at::Tensor& history, const at::Tensor& scale, double fp8_max, int64_t margin,
                            bool most_recent) {
  c10::cuda::CUDAGuard guard(history.device());
  TORCH_CHECK(history.dim() == 2 && history.is_contiguous() && scale.is_contiguous() &&
              history.scalar_type() == at::kFloat && scale.scalar_type() == at::kFloat && history.size(1) == scale.numel());
  cudaError_t e = teb200::delayed_scaling_update(history.data_ptr<float>(), scale.data_ptr<float>(),
                                                 static_cast<int>(history.size(0)), static_cast<int>(history.size(1)),
                                                 static_cast<float>(fp8_max), static_cast<int>(margin), most_recent ? 1 : 0,
                                                 cur_stream());
  TORCH_CHECK(e == cudaSuccess, "delayed_scaling_update failed: ", cudaGetErrorString(e));
}

// ---------------------------------------------------------------------------- column sums, offsets, padding
at::Tensor column_sum(const at::Tensor& x, at::ScalarType out_dtype) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "column_sum expects a [R, C] matrix with contiguous rows");
  const int R = static_cast<int>(x.size(0)), C = static_cast<int>(x.size(1));
  at::Tensor out = at::empty({C}, x.options().dtype(out_dtype));
  if (R == 0) return out.zero_();
  at::Tensor ws = at::empty({teb200::column_sum_parts(R, C), C}, x.options().dtype(at::kFloat));
  cudaError_t e = teb200::column_sum(x.data_ptr(), dtype_code(x), R, C, x.stride(0), out.data_ptr(), dtype_code(out),
                                     ws.data_ptr<float>(), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "column_sum failed: ", cudaGetErrorString(e));
  return out;
}

at::Tensor grouped_column_sum(const at::Tensor& x, const at::Tensor& offsets, at::ScalarType out_dtype) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "grouped_column_sum expects a [R, C] matrix with contiguous rows");
  TORCH_CHECK(offsets.scalar_type() == at::kInt && offsets.is_cuda() && offsets.numel() >= 2, "offsets: int32 device tensor");
  const int G = static_cast<int>(offsets.numel() - 1), C = static_cast<int>(x.size(1));
  at::Tensor out = at::empty({G, C}, x.options().dtype(out_dtype));
  cudaError_t e = teb200::grouped_column_sum(x.data_ptr(), dtype_code(x), offsets.data_ptr<int>(), G, C, x.stride(0),
                                             out.data_ptr(), dtype_code(out), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "grouped_column_sum failed: ", cudaGetErrorString(e));
  return out;
}

void grouped_bias_add(at::Tensor& x, const at::Tensor& bias, const at::Tensor& offsets) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && bias.dim() == 2 && bias.is_contiguous() && bias.size(1) == x.size(1) &&
                  bias.scalar_type() == x.scalar_type() && bias.size(0) == offsets.numel() - 1,
              "grouped_bias_add: x [R, C], bias [G, C] of the same dtype, offsets [G + 1]");
  TORCH_CHECK(offsets.scalar_type() == at::kInt && offsets.is_cuda(), "offsets: int32 device tensor");
  cudaError_t e = teb200::grouped_bias_add(x.data_ptr(), bias.data_ptr(), dtype_code(x), offsets.data_ptr<int>(),
                                           static_cast<int>(bias.size(0)), static_cast<int>(x.size(1)), x.stride(0),
                                           static_cast<int>(x.size(0)), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "grouped_bias_add failed: ", cudaGetErrorString(e));
}

at::Tensor row_dot(const at::Tensor& a, const at::Tensor& b) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.sizes() == b.sizes() && a.stride(1) == 1 && b.stride(1) == 1 &&
                  a.scalar_type() == b.scalar_type(), "row_dot expects two [R, C] matrices of one dtype");
  at::Tensor out = at::empty({a.size(0)}, a.options().dtype(at::kFloat));
  cudaError_t e = teb200::row_dot(a.data_ptr(), b.data_ptr(), dtype_code(a), a.size(0), static_cast<int>(a.size(1)),
                                  a.stride(0), b.stride(0), out.data_ptr<float>(), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "row_dot failed: ", cudaGetErrorString(e));
  return out;
}

at::Tensor splits_to_offsets(const at::Tensor& splits, int64_t multiplier, bool out_int64) {
  c10::cuda::CUDAGuard guard(splits.device());
  TORCH_CHECK(splits.dim() == 1 && splits.is_contiguous() &&
                  (splits.scalar_type() == at::kInt || splits.scalar_type() == at::kLong),
              "splits_to_offsets expects a 1-D int32 / int64 tensor");
  const int n = static_cast<int>(splits.numel());
  at::Tensor out = at::empty({n + 1}, splits.options().dtype(out_int64 ? at::kLong : at::kInt));
  cudaError_t e = teb200::splits_to_offsets(splits.data_ptr(), splits.scalar_type() == at::kLong, n, multiplier,
                                            out.data_ptr(), out_int64, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "splits_to_offsets failed: ", cudaGetErrorString(e));
  return out;
}

// in [rows_in, C], offsets: int32 device tensors of groups + 1 entries; out has out_rows rows
at::Tensor repad_rows(const at::Tensor& in, const at::Tensor& in_offsets, const at::Tensor& out_offsets, int64_t out_rows) {
  c10::cuda::CUDAGuard guard(in.device());
  TORCH_CHECK(in.dim() == 2 && in.is_contiguous(), "repad_rows expects a contiguous [rows, C] matrix");
  TORCH_CHECK(in_offsets.scalar_type() == at::kInt && out_offsets.scalar_type() == at::kInt &&
                  in_offsets.numel() == out_offsets.numel() && in_offsets.numel() >= 2,
              "repad_rows: offsets are int32 tensors of groups + 1 entries");
  at::Tensor out = at::empty({out_rows, in.size(1)}, in.options());
  const int row_bytes = static_cast<int>(in.size(1) * in.element_size());
  cudaError_t e = teb200::repad_rows(in.data_ptr(), out.data_ptr(), in_offsets.data_ptr<int>(), out_offsets.data_ptr<int>(),
                                     static_cast<int>(in_offsets.numel() - 1), row_bytes, static_cast<int>(out_rows),
                                     cur_stream());
  TORCH_CHECK(e == cudaSuccess, "repad_rows failed: ", cudaGetErrorString(e));
  return out;
}

at::Tensor pad_last_dim(const at::Tensor& in, int64_t new_cols) {
  c10::cuda::CUDAGuard guard(in.device());
  TORCH_CHECK(in.dim() >= 1 && in.is_contiguous(), "pad_last_dim expects a contiguous tensor");
  const int64_t C = in.size(-1);
  const int64_t R = C > 0 ? in.numel() / C : 0;
  auto shape = in.sizes().vec();
  shape.back() = new_cols;
  at::Tensor out = at::empty(shape, in.options());
  cudaError_t e = teb200::pad_last_dim(in.data_ptr(), out.data_ptr(), R, static_cast<int>(C * in.element_size()),
                                       static_cast<int>(new_cols * in.element_size()), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "pad_last_dim failed: ", cudaGetErrorString(e));
  return out;
}

}  // namespace

void register_extra(py::module_& m) {
  m.def("column_sum", teb200::traced("teb200.column_sum", &column_sum));
  m.def("splits_to_offsets", teb200::traced("teb200.splits_to_offsets", &splits_to_offsets));
  m.def("grouped_column_sum", teb200::traced("teb200.grouped_column_sum", &grouped_column_sum));
  m.def("grouped_bias_add", teb200::traced("teb200.grouped_bias_add", &grouped_bias_add));
  m.def("row_dot", teb200::traced("teb200.row_dot", &row_dot));
  m.def("repad_rows", teb200::traced("teb200.repad_rows", &repad_rows));
  m.def("pad_last_dim", teb200::traced("teb200.pad_last_dim", &pad_last_dim));
  m.def("delayed_scaling_update", teb200::traced("teb200.delayed_scaling_update", &delayed_scaling_update));
  m.def("softmax_fwd", teb200::traced("teb200.softmax_fwd", &softmax_fwd));
  m.def("softmax_bwd", teb200::traced("teb200.softmax_bwd", &softmax_bwd));
  m.def("dropout_fwd", teb200::traced("teb200.dropout_fwd", &dropout_fwd));
  m.def("dropout_bwd", teb200::traced("teb200.dropout_bwd", &dropout_bwd));
  m.def("peer_sum", teb200::traced("teb200.peer_sum", &peer_sum));
  m.def("ep_counts", teb200::traced("teb200.ep_counts", &ep_counts));
  m.def("ep_push", teb200::traced("teb200.ep_push", &ep_push));
  m.def("ep_wait", teb200::traced("teb200.ep_wait", &ep_wait), py::arg("flags_ptr"), py::arg("n"), py::arg("epoch"), py::arg("status"),
        py::arg("limit_cycles") = 0);
  m.def("ep_signal", teb200::traced("teb200.ep_signal", &ep_signal));
  m.def("ep_pull", teb200::traced("teb200.ep_pull", &ep_pull));
  m.def("router_topk", teb200::traced("teb200.router_topk", &router_topk));
  m.def("router_topk_bwd", teb200::traced("teb200.router_topk_bwd", &router_topk_bwd));
  m.def("permute_rows", teb200::traced("teb200.permute_rows", &permute_rows));
  m.def("unpermute_rows", teb200::traced("teb200.unpermute_rows", &unpermute_rows));
  m.def("build_dest_rows", teb200::traced("teb200.build_dest_rows", &build_dest_rows));
  m.def("nvfp4_amax", teb200::traced("teb200.nvfp4_amax", &nvfp4_amax));
  m.def("quantize_nvfp4", teb200::traced("teb200.quantize_nvfp4", &quantize_nvfp4));
  m.def("dequantize_nvfp4", teb200::traced("teb200.dequantize_nvfp4", &dequantize_nvfp4));
  m.def("comm_gemm", teb200::traced("teb200.comm_gemm", &comm_gemm), py::arg("mode"), py::arg("rank"), py::arg("world"), py::arg("epoch_dev"),
        py::arg("copy_ctas"), py::arg("a"), py::arg("sfa"), py::arg("b"), py::arg("sfb"), py::arg("d"), py::arg("bias"),
        py::arg("a_e5m2"), py::arg("b_e5m2"), py::arg("a_ptrs"), py::arg("sfa_ptrs"), py::arg("ready_ptrs"),
        py::arg("chunk_flags_ptr"), py::arg("stage_ptrs"), py::arg("tile_flag_ptrs"), py::arg("out"), py::arg("N"),
        py::arg("status"), py::arg("side_src_ptrs") = std::vector<int64_t>(), py::arg("side_dst") = py::none(),
        py::arg("side_dst_sf") = py::none(), py::arg("side_geom") = std::vector<int64_t>(),
        py::arg("out_all_ptrs") = std::vector<int64_t>(), py::arg("ar_flag_ptrs") = std::vector<int64_t>());
  m.def("flash_fwd", teb200::traced("teb200.flash_fwd", &flash_fwd), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"),
        py::arg("scale"), py::arg("causal"), py::arg("bottom_right"), py::arg("status"),
        py::arg("timeline") = py::none(), py::arg("window_left") = -1, py::arg("window_right") = -1);
  m.def("flash_bwd", teb200::traced("teb200.flash_bwd", &flash_bwd), py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"),
        py::arg("lse"), py::arg("delta"), py::arg("dq"), py::arg("dk"), py::arg("dv"), py::arg("scale"),
        py::arg("causal"), py::arg("bottom_right"), py::arg("status"), py::arg("window_left") = -1,
        py::arg("window_right") = -1);
  m.def("thd_get_partitioned_indices", teb200::traced("teb200.thd_get_partitioned_indices", &thd_get_partitioned_indices));
  m.def("thd_read_half_tensor", teb200::traced("teb200.thd_read_half_tensor", &thd_read_half_tensor));
  m.def("thd_second_half_lse_correction", teb200::traced("teb200.thd_second_half_lse_correction", &thd_second_half_lse_correction));
  m.def("thd_read_second_half_lse", teb200::traced("teb200.thd_read_second_half_lse", &thd_read_second_half_lse));
  m.def("thd_out_correction", teb200::traced("teb200.thd_out_correction", &thd_out_correction));
  m.def("thd_grad_correction", teb200::traced("teb200.thd_grad_correction", &thd_grad_correction));
  m.def("convert_thd_to_bshd", teb200::traced("teb200.convert_thd_to_bshd", &convert_thd_to_bshd));
  m.def("convert_bshd_to_thd", teb200::traced("teb200.convert_bshd_to_thd", &convert_bshd_to_thd));
  m.def("kv_cache_step", teb200::traced("teb200.kv_cache_step", &kv_cache_step));
  m.def("flash_fwd_varlen", teb200::traced("teb200.flash_fwd_varlen", &flash_fwd_varlen), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"),
        py::arg("lse"), py::arg("cu_q"), py::arg("cu_k"), py::arg("off_q"), py::arg("off_k"), py::arg("max_sq"),
        py::arg("max_sk"), py::arg("scale"), py::arg("causal"), py::arg("bottom_right"), py::arg("status"),
        py::arg("window_left") = -1, py::arg("window_right") = -1);
  m.def("flash_bwd_varlen", teb200::traced("teb200.flash_bwd_varlen", &flash_bwd_varlen), py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"),
        py::arg("out"), py::arg("lse"), py::arg("delta"), py::arg("dq"), py::arg("dk"), py::arg("dv"), py::arg("cu_q"),
        py::arg("cu_k"), py::arg("off_q"), py::arg("off_k"), py::arg("max_sq"), py::arg("max_sk"), py::arg("scale"),
        py::arg("causal"), py::arg("bottom_right"), py::arg("status"), py::arg("window_left") = -1,
        py::arg("window_right") = -1);
}

