// Python bindings: thin glue from at::Tensor to the raw-pointer launchers.
// Output tensors are allocated by the Python callers; nothing here allocates
// except the per-device status word.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <teb200/api.h>
#include <teb200/nvtx.h>
#include <teb200/misc.h>
#include <teb200/norm.h>
#include <teb200/quant.h>
#include <torch/extension.h>

#include <optional>
#include <vector>

namespace py = pybind11;
using teb200::DType;
using OptT = std::optional<at::Tensor>;

namespace {

int to_dtype(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return teb200::kFloat32;
    case at::kHalf: return teb200::kFloat16;
    case at::kBFloat16: return teb200::kBFloat16;
    case at::kByte: return teb200::kByte;
    case at::kFloat8_e4m3fn: return teb200::kFloat8E4M3;
    case at::kFloat8_e5m2: return teb200::kFloat8E5M2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
}
template <typename T = void>
T* ptr(const OptT& t) {
  return t.has_value() && t->defined() ? static_cast<T*>(t->data_ptr()) : nullptr;
}
cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
// number of kernel launches issued through this module (one per launcher call)
long long g_launches = 0;
void check(cudaError_t e, const char* what) {
  ++g_launches;
  TORCH_CHECK(e == cudaSuccess, what, " failed: ", cudaGetErrorString(e));
}
long long launch_count() { return g_launches; }

// One int per device; kernels write a Status code there when a bounded wait expires.
at::Tensor& status_tensor(int device) {
  static std::vector<at::Tensor> st(64);
  if (!st[device].defined())
    st[device] = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  return st[device];
}

at::Tensor status(int device) { return status_tensor(device); }

// kind: 0 = 16-bit, 1 = mxfp8, 2 = nvfp4, 3 = per-tensor fp8.  a [M,K] (or [K,M] when a_mn), b [N,K] (or [K,N]); d [M,N].
void gemm(int kind, const at::Tensor& a, const at::Tensor& b, at::Tensor& d, const OptT& sfa, const OptT& sfb,
          const OptT& bias, const OptT& aux, int epilogue, bool accumulate, bool a_e5m2, bool b_e5m2, bool a_mn,
          bool b_mn, double alpha, const OptT& alpha_dev, const OptT& group_offsets, int num_groups, int sm_count,
          int64_t K_override, int64_t sf_k_tiles) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2, "gemm operands must be 2-D");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "gemm operands must be row-major");
  teb200::GemmArgs g;
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.d = d.data_ptr();
  g.M = static_cast<int>(d.size(0));
  g.N = static_cast<int>(d.size(1));
  if (kind == 0) {
    g.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
    g.a_dtype = to_dtype(a);
    g.b_dtype = to_dtype(b);
    TORCH_CHECK(g.a_dtype == g.b_dtype && (g.a_dtype == teb200::kBFloat16 || g.a_dtype == teb200::kFloat16),
                "16-bit gemm needs matching bf16/fp16 operands");
    g.lda = a.stride(0);
    g.ldb = b.stride(0);
  } else if (kind == 1 || kind == 3) {
    g.K = static_cast<int>(a.size(1));
    g.a_dtype = a_e5m2 ? teb200::kFloat8E5M2 : teb200::kFloat8E4M3;
    g.b_dtype = b_e5m2 ? teb200::kFloat8E5M2 : teb200::kFloat8E4M3;
    g.lda = a.stride(0);
    g.ldb = b.stride(0);
  } else {
    g.K = static_cast<int>(a.size(1)) * 2;
    g.lda = a.stride(0) * 2;
    g.ldb = b.stride(0) * 2;
  }
  if (K_override > 0) g.K = static_cast<int>(K_override);
  if (num_groups > 0) g.N = static_cast<int>(b.size(a_mn || b_mn ? 1 : 0)) / num_groups;
  g.ldd = d.stride(0);
  g.d_dtype = to_dtype(d);
  g.sfa = ptr<uint8_t>(sfa);
  g.sfb = ptr<uint8_t>(sfb);
  if (bias.has_value() && bias->defined()) {
    g.bias = bias->data_ptr();
    g.bias_dtype = to_dtype(*bias);
  }
  g.aux = ptr<void>(aux);
  g.epilogue = epilogue;
  g.accumulate = accumulate;
  g.a_mn_major = a_mn;
  g.b_mn_major = b_mn;
  g.alpha = static_cast<float>(alpha);
  g.alpha_dev = ptr<float>(alpha_dev);
  g.num_groups = num_groups;
  g.group_offsets = ptr<int32_t>(group_offsets);
  g.sm_count = sm_count;
  g.sf_k_tiles = static_cast<int>(sf_k_tiles);
  g.status = status_tensor(a.get_device()).data_ptr<int>();
  cudaError_t e = kind == 0   ? teb200::gemm_bf16(g, stream())
                  : kind == 1 ? teb200::gemm_mxfp8(g, stream())
                  : kind == 3 ? teb200::gemm_fp8(g, stream())
                              : teb200::gemm_nvfp4(g, stream());
  check(e, "gemm");
}

// FP8 with 128-wide block scales; returns nothing, fills the given outputs (any of the two copies may be absent)
void quantize_block128(const at::Tensor& x, int64_t dim, bool e5m2, bool pow2, double eps, const OptT& row_data,
                       const OptT& row_sinv, const OptT& row_mx, const OptT& col_data, const OptT& col_sinv,
                       const OptT& col_mx) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "quantize_block128 expects a row-major matrix");
  teb200::BlockQuantArgs a;
  a.x = x.data_ptr();
  a.x_dtype = to_dtype(x);
  a.R = static_cast<int>(x.size(0));
  a.C = static_cast<int>(x.size(1));
  a.ld = x.stride(0);
  a.dim = static_cast<int>(dim);
  a.e5m2 = e5m2;
  a.pow2 = pow2;
  a.eps = static_cast<float>(eps);
  a.row_data = ptr<uint8_t>(row_data);
  a.row_sinv = ptr<float>(row_sinv);
  a.row_mx = ptr<uint8_t>(row_mx);
  a.col_data = ptr<uint8_t>(col_data);
  a.col_sinv = ptr<float>(col_sinv);
  a.col_mx = ptr<uint8_t>(col_mx);
  TORCH_CHECK((a.row_data == nullptr) == (a.row_sinv == nullptr) && (a.col_data == nullptr) == (a.col_sinv == nullptr),
              "quantize_block128: data and scales of a copy go together");
  check(teb200::quantize_block128(a, stream()), "quantize_block128");
}

// mode: 0 = mxfp8, 1 = per-tensor fp8, 2 = no quantization (produce y only)
void quantize(int mode, int prologue, int act, const at::Tensor& x, const OptT& dy, int64_t R, int64_t C,
              const OptT& y, const OptT& row_data, const OptT& row_scale, const OptT& col_data, const OptT& col_scale,
              bool e5m2, const OptT& mu, const OptT& rs, const OptT& gamma, const OptT& beta, bool zero_centered,
              const OptT& row_mul, const OptT& scale, const OptT& amax, const OptT& scale_inv, const OptT& dbias) {
  c10::cuda::CUDAGuard guard(x.device());
  teb200::QuantArgs q;
  q.x = x.data_ptr();
  q.x_dtype = to_dtype(x);
  q.ldx = x.dim() >= 2 ? x.stride(-2) : x.size(-1);
  q.dy = ptr<void>(dy);
  q.mu = ptr<float>(mu);
  q.rs = ptr<float>(rs);
  if (gamma.has_value() && gamma->defined()) {
    q.gamma = gamma->data_ptr();
    q.gamma_dtype = to_dtype(*gamma);
  }
  q.beta = ptr<void>(beta);
  q.zero_centered = zero_centered;
  q.row_scale = ptr<float>(row_mul);
  q.prologue = prologue;
  q.act = act;
  q.R = static_cast<int>(R);
  q.C = static_cast<int>(C);
  if (y.has_value() && y->defined()) {
    q.y = y->data_ptr();
    q.y_dtype = to_dtype(*y);
  }
  q.row_data = ptr<uint8_t>(row_data);
  q.row_scale_out = ptr<uint8_t>(row_scale);
  q.col_data = ptr<uint8_t>(col_data);
  q.col_scale_out = ptr<uint8_t>(col_scale);
  q.fp8_e5m2 = e5m2;
  q.scale = ptr<float>(scale);
  q.amax = ptr<float>(amax);
  q.scale_inv = ptr<float>(scale_inv);
  q.dbias = ptr<float>(dbias);
  cudaError_t e = mode == 0 ? teb200::quantize_mxfp8(q, stream())
                            : (mode == 1 ? teb200::quantize_fp8_tensor(q, stream()) : teb200::apply_prologue(q, stream()));
  check(e, "quantize");
}

void dequantize_mxfp8(const at::Tensor& q, const at::Tensor& sf, int64_t R, int64_t C, bool e5m2, at::Tensor& out) {
  c10::cuda::CUDAGuard guard(q.device());
  check(teb200::dequantize_mxfp8(static_cast<const uint8_t*>(q.data_ptr()), static_cast<const uint8_t*>(sf.data_ptr()),
                                 static_cast<int>(R), static_cast<int>(C), e5m2, out.data_ptr(), to_dtype(out), stream()),
        "dequantize_mxfp8");
}
void dequantize_fp8(const at::Tensor& q, const at::Tensor& scale_inv, bool e5m2, at::Tensor& out) {
  c10::cuda::CUDAGuard guard(q.device());
  check(teb200::dequantize_fp8_tensor(static_cast<const uint8_t*>(q.data_ptr()), scale_inv.data_ptr<float>(), q.numel(),
                                      e5m2, out.data_ptr(), to_dtype(out), stream()),
        "dequantize_fp8");
}
void amax(const at::Tensor& x, at::Tensor& out) {
  c10::cuda::CUDAGuard guard(x.device());
  check(teb200::amax_abs(x.data_ptr(), to_dtype(x), x.numel(), out.data_ptr<float>(), stream()), "amax");
}
void swizzle(const at::Tensor& in, int64_t rows, int64_t cols, at::Tensor& out, bool to_swizzled) {
  c10::cuda::CUDAGuard guard(in.device());
  auto* i = static_cast<const uint8_t*>(in.data_ptr());
  auto* o = static_cast<uint8_t*>(out.data_ptr());
  check(to_swizzled ? teb200::swizzle_scales(i, rows, cols, o, stream()) : teb200::unswizzle_scales(i, rows, cols, o, stream()),
        "swizzle");
}

void norm_fwd(bool layernorm, const at::Tensor& x, const at::Tensor& gamma, const OptT& beta, const OptT& y,
              const OptT& mu, at::Tensor& rs, double eps, bool zero_centered) {
  c10::cuda::CUDAGuard guard(x.device());
  teb200::NormArgs n;
  n.layernorm = layernorm;
  n.C = static_cast<int>(x.size(-1));
  n.R = static_cast<int>(x.numel() / x.size(-1));
  n.x_dtype = to_dtype(x);
  n.w_dtype = to_dtype(gamma);
  n.eps = static_cast<float>(eps);
  n.zero_centered = zero_centered;
  n.x = x.data_ptr();
  n.gamma = gamma.data_ptr();
  n.beta = ptr<void>(beta);
  n.y = ptr<void>(y);
  n.mu = ptr<float>(mu);
  n.rs = rs.data_ptr<float>();
  check(teb200::norm_fwd(n, stream()), "norm_fwd");
}
int64_t norm_bwd_workspace(int64_t R, int64_t C) { return static_cast<int64_t>(teb200::norm_bwd_parts(R)) * 2 * C; }
void norm_bwd(bool layernorm, const at::Tensor& dy, const at::Tensor& x, const OptT& mu, const at::Tensor& rs,
              const at::Tensor& gamma, const OptT& add, at::Tensor& dx, at::Tensor& dgamma, const OptT& dbeta,
              at::Tensor& workspace, bool zero_centered) {
  c10::cuda::CUDAGuard guard(x.device());
  teb200::NormArgs n;
  n.layernorm = layernorm;
  n.C = static_cast<int>(x.size(-1));
  n.R = static_cast<int>(x.numel() / x.size(-1));
  n.x_dtype = to_dtype(x);
  n.w_dtype = to_dtype(gamma);
  n.zero_centered = zero_centered;
  n.x = x.data_ptr();
  n.dy = dy.data_ptr();
  n.gamma = gamma.data_ptr();
  n.mu = ptr<float>(mu);
  n.rs = rs.data_ptr<float>();
  n.add = ptr<void>(add);
  n.dx = dx.data_ptr();
  n.dgamma = dgamma.data_ptr();
  n.dbeta = ptr<void>(dbeta);
  n.workspace = workspace.data_ptr<float>();
  TORCH_CHECK(workspace.numel() >= norm_bwd_workspace(n.R, n.C), "norm_bwd workspace too small");
  ++g_launches;  // statistics kernel + finalize kernel
  check(teb200::norm_bwd(n, stream()), "norm_bwd");
}

// lists[k][i]: tensor i of list k.  Splits into launches of <= kMtMaxTensors tensors / kMtMaxBlocks blocks.
// The kernels index raw pointers with 16-byte vector accesses: every entry must be dense, as long as its
// partner in list 0, of one dtype per list and 16-byte aligned.
template <typename Launch>
void multi_tensor_apply(const std::vector<std::vector<at::Tensor>>& lists, int64_t chunk, Launch&& launch) {
  const size_t nt = lists[0].size();
  for (size_t k = 0; k < lists.size(); ++k) {
    TORCH_CHECK(lists[k].size() == nt, "multi_tensor_apply: list ", k, " has ", lists[k].size(), " tensors, list 0 has ", nt);
    for (size_t i = 0; i < nt; ++i) {
      const at::Tensor& x = lists[k][i];
      TORCH_CHECK(x.is_cuda(), "multi_tensor_apply: tensor ", i, " of list ", k, " is not on a GPU");
      TORCH_CHECK(x.is_contiguous(), "multi_tensor_apply: tensor ", i, " of list ", k,
                  " is not contiguous (an expanded or strided view; call .contiguous() first)");
      TORCH_CHECK(x.numel() == lists[0][i].numel(), "multi_tensor_apply: tensor ", i, " of list ", k, " has ",
                  x.numel(), " elements, its partner in list 0 has ", lists[0][i].numel());
      TORCH_CHECK(x.scalar_type() == lists[k][0].scalar_type(), "multi_tensor_apply: list ", k, " mixes dtypes");
      TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0 || x.numel() == 0, "multi_tensor_apply: tensor ",
                  i, " of list ", k, " is not 16-byte aligned (a sliced view; clone it)");
    }
  }
  teb200::MultiTensorTable tab;
  int nten = 0, base = 0;
  int64_t nchunks = 0;
  tab.chunk_start[0] = 0;
  auto flush = [&]() {
    if (nten == 0) return;
    tab.ntensors = nten;
    launch(tab, static_cast<int>(nchunks), base);
    base += nten;
    nten = 0;
    nchunks = 0;
  };
  for (size_t i = 0; i < nt; ++i) {
    const int64_t n = lists[0][i].numel();
    if (n == 0) continue;
    const int64_t c = (n + chunk - 1) / chunk;
    if (nten == teb200::kMtMaxTensors || nchunks + c > (int64_t{1} << 30)) flush();
    for (size_t k = 0; k < lists.size(); ++k) tab.ptr[k][nten] = lists[k][i].data_ptr();
    tab.numel[nten] = n;
    nchunks += c;
    ++nten;
    tab.chunk_start[nten] = static_cast<int32_t>(nchunks);
  }
  flush();
}

void multi_tensor_adam(std::vector<std::vector<at::Tensor>> lists, double lr, double beta1, double beta2, double eps,
                       int64_t step, bool adamw, bool bias_correction, double weight_decay, double grad_scale,
                       const OptT& inv_scale, const OptT& noop, int64_t chunk, const OptT& step_dev,
                       const OptT& lr_dev, bool remainders) {
  TORCH_CHECK(lists.size() == 4 || lists.size() == 5, "adam expects [g, p, m, v] or [g, p, m, v, master]");
  if (lists[0].empty()) return;
  c10::cuda::CUDAGuard guard(lists[0][0].device());
  teb200::AdamArgs a;
  a.lr = static_cast<float>(lr);
  a.beta1 = static_cast<float>(beta1);
  a.beta2 = static_cast<float>(beta2);
  a.eps = static_cast<float>(eps);
  a.weight_decay = static_cast<float>(weight_decay);
  a.bias_correction1 = bias_correction ? static_cast<float>(1.0 - std::pow(beta1, static_cast<double>(step))) : 1.f;
  a.bias_correction2 = bias_correction ? static_cast<float>(1.0 - std::pow(beta2, static_cast<double>(step))) : 1.f;
  a.adamw = adamw;
  a.grad_dtype = to_dtype(lists[0][0]);
  a.param_dtype = to_dtype(lists[1][0]);
  a.state_dtype = to_dtype(lists[2][0]);
  a.has_master = lists.size() == 5 ? (remainders ? 2 : 1) : 0;
  if (remainders) {
    TORCH_CHECK(lists.size() == 5 && lists[4][0].scalar_type() == at::kShort && lists[1][0].scalar_type() == at::kBFloat16,
                "parameter remainders need bf16 parameters and an int16 list");
  } else if (lists.size() == 5) {
    TORCH_CHECK(lists[4][0].scalar_type() == at::kFloat, "master weights must be fp32");
  }
  a.bias_correction = bias_correction;
  if (step_dev.has_value()) {
    TORCH_CHECK(step_dev->scalar_type() == at::kInt && step_dev->is_cuda(), "device step counter must be int32 on the GPU");
    a.step_dev = step_dev->data_ptr<int>();
  }
  if (lr_dev.has_value()) {
    TORCH_CHECK(lr_dev->scalar_type() == at::kFloat && lr_dev->is_cuda(), "device learning rate must be fp32 on the GPU");
    a.lr_dev = lr_dev->data_ptr<float>();
  }
  a.grad_scale = static_cast<float>(grad_scale);
  a.inv_scale_dev = ptr<float>(inv_scale);
  a.noop = ptr<int>(noop);
  a.chunk = chunk;
  auto s = stream();
  multi_tensor_apply(lists, chunk, [&](const teb200::MultiTensorTable& t, int nblk, int) {
    check(teb200::multi_tensor_adam(t, nblk, a, s), "multi_tensor_adam");
  });
}

void multi_tensor_sgd(std::vector<std::vector<at::Tensor>> lists, double lr, double momentum, double dampening,
                      double weight_decay, bool nesterov, bool first_run, bool wd_after_momentum, double grad_scale,
                      const OptT& noop, int64_t chunk) {
  if (lists[0].empty()) return;
  c10::cuda::CUDAGuard guard(lists[0][0].device());
  teb200::SgdArgs a;
  a.lr = lr; a.momentum = momentum; a.dampening = dampening; a.weight_decay = weight_decay;
  a.nesterov = nesterov; a.first_run = first_run; a.wd_after_momentum = wd_after_momentum;
  a.grad_scale = grad_scale;
  a.grad_dtype = to_dtype(lists[0][0]);
  a.param_dtype = to_dtype(lists[1][0]);
  a.has_master = lists.size() == 4;
  a.noop = ptr<int>(noop);
  a.chunk = chunk;
  auto s = stream();
  multi_tensor_apply(lists, chunk, [&](const teb200::MultiTensorTable& t, int nblk, int) {
    check(teb200::multi_tensor_sgd(t, nblk, a, s), "multi_tensor_sgd");
  });
}

void multi_tensor_scale(std::vector<std::vector<at::Tensor>> lists, double scale, const OptT& noop, int64_t chunk) {
  if (lists[0].empty()) return;
  c10::cuda::CUDAGuard guard(lists[0][0].device());
  const int in_dt = to_dtype(lists[0][0]), out_dt = to_dtype(lists[1][0]);
  auto s = stream();
  multi_tensor_apply(lists, chunk, [&](const teb200::MultiTensorTable& t, int nblk, int) {
    check(teb200::multi_tensor_scale(t, nblk, in_dt, out_dt, static_cast<float>(scale), ptr<int>(noop), chunk, s),
          "multi_tensor_scale");
  });
}

void multi_tensor_l2norm_sq(std::vector<std::vector<at::Tensor>> lists, at::Tensor& out, const OptT& per_tensor,
                            int64_t chunk) {
  if (lists[0].empty()) return;
  c10::cuda::CUDAGuard guard(lists[0][0].device());
  const int dt = to_dtype(lists[0][0]);
  auto s = stream();
  multi_tensor_apply(lists, chunk, [&](const teb200::MultiTensorTable& t, int nblk, int base) {
    check(teb200::multi_tensor_l2norm_sq(t, nblk, dt, out.data_ptr<float>(), ptr<float>(per_tensor), base, chunk, s),
          "multi_tensor_l2norm");
  });
}

void cross_entropy(const at::Tensor& logits, const at::Tensor& targets, const OptT& loss, const OptT& grad,
                   const OptT& row_max, const OptT& row_sum, const OptT& row_tgt, int64_t vocab_start,
                   double grad_scale, double label_smoothing, int64_t ignore_index, const OptT& gmax,
                   const OptT& gsum, const OptT& grad_scale_dev) {
  c10::cuda::CUDAGuard guard(logits.device());
  teb200::CrossEntropyArgs a;
  a.logits = logits.data_ptr();
  a.dtype = to_dtype(logits);
  a.targets = targets.data_ptr<int64_t>();
  a.loss = ptr<float>(loss);
  a.grad = ptr<void>(grad);
  a.row_max = ptr<float>(row_max);
  a.row_sum = ptr<float>(row_sum);
  a.row_tgt = ptr<float>(row_tgt);
  a.V = static_cast<int>(logits.size(-1));
  a.R = static_cast<int>(logits.numel() / logits.size(-1));
  a.ld = logits.stride(-2);
  a.vocab_start = static_cast<int>(vocab_start);
  a.grad_scale = static_cast<float>(grad_scale);
  a.grad_scale_dev = ptr<float>(grad_scale_dev);
  a.label_smoothing = static_cast<float>(label_smoothing);
  a.ignore_index = ignore_index;
  if (gmax.has_value() && gmax->defined())
    check(teb200::cross_entropy_parallel_bwd(a, gmax->data_ptr<float>(), gsum->data_ptr<float>(), stream()),
          "cross_entropy_parallel_bwd");
  else
    check(teb200::cross_entropy_fwd_bwd(a, stream()), "cross_entropy");
}

// x, out: 4-D views [s, b, h, d] (any strides with unit stride on d)
void rope(const at::Tensor& x, at::Tensor& out, const at::Tensor& freqs, int64_t d_rot, bool interleaved,
          bool backward, int64_t pos_offset, int64_t cp_size, int64_t cp_rank, const OptT& start_positions,
          int64_t qkv_mode, int64_t q_per_group, int64_t hq, int64_t hk, const OptT& freqs_k) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 4 && x.stride(3) == 1 && out.strides() == x.strides(), "rope expects [s,b,h,d] views");
  teb200::RopeArgs a;
  a.x = x.data_ptr();
  a.out = out.data_ptr();
  a.freqs = freqs.data_ptr<float>();
  a.dtype = to_dtype(x);
  a.s = x.size(0); a.b = x.size(1); a.h = x.size(2); a.d = x.size(3);
  a.d_rot = static_cast<int>(d_rot);
  a.stride_s = x.stride(0); a.stride_b = x.stride(1); a.stride_h = x.stride(2);
  a.interleaved = interleaved;
  a.backward = backward;
  a.pos_offset = static_cast<int>(pos_offset);
  a.cp_size = static_cast<int>(cp_size);
  a.cp_rank = static_cast<int>(cp_rank);
  a.start_positions = ptr<int32_t>(start_positions);
  a.qkv_mode = static_cast<int>(qkv_mode);
  a.q_per_group = static_cast<int>(q_per_group);
  a.hq = static_cast<int>(hq);
  a.hk = static_cast<int>(hk);
  if (qkv_mode != 0) {
    TORCH_CHECK(qkv_mode == 1 ? (q_per_group > 0 && a.h % (q_per_group + 2) == 0) : (qkv_mode == 2 && hq + 2 * hk == a.h),
                "rope: the packed QKV head layout does not match the tensor");
    if (freqs_k.has_value() && freqs_k->defined()) {
      TORCH_CHECK(freqs_k->sizes() == freqs.sizes(), "rope: key angles must have the shape of the query angles");
      a.freqs_k = freqs_k->data_ptr<float>();
    }
  }
  check(teb200::rope_apply(a, stream()), "rope");
}

}  // namespace

void register_extra(py::module_& m);  // bindings of kernels added in other translation units

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("status", teb200::traced("teb200.status", &status));
  m.def("launch_count", teb200::traced("teb200.launch_count", &launch_count));
  m.def("gemm", teb200::traced("teb200.gemm", &gemm), py::arg("kind"), py::arg("a"), py::arg("b"), py::arg("d"), py::arg("sfa"), py::arg("sfb"),
        py::arg("bias"), py::arg("aux"), py::arg("epilogue"), py::arg("accumulate"), py::arg("a_e5m2"),
        py::arg("b_e5m2"), py::arg("a_mn"), py::arg("b_mn"), py::arg("alpha"), py::arg("alpha_dev"),
        py::arg("group_offsets"), py::arg("num_groups"), py::arg("sm_count"), py::arg("K_override") = 0,
        py::arg("sf_k_tiles") = 0);
  m.def("quantize", teb200::traced("teb200.quantize", &quantize));
  m.def("quantize_block128", teb200::traced("teb200.quantize_block128", &quantize_block128));
  m.def("dequantize_mxfp8", teb200::traced("teb200.dequantize_mxfp8", &dequantize_mxfp8));
  m.def("dequantize_fp8", teb200::traced("teb200.dequantize_fp8", &dequantize_fp8));
  m.def("amax", teb200::traced("teb200.amax", &amax));
  m.def("swizzle", teb200::traced("teb200.swizzle", &swizzle));
  m.def("norm_fwd", teb200::traced("teb200.norm_fwd", &norm_fwd));
  m.def("norm_bwd", teb200::traced("teb200.norm_bwd", &norm_bwd));
  m.def("norm_bwd_workspace", teb200::traced("teb200.norm_bwd_workspace", &norm_bwd_workspace));
  m.def("multi_tensor_adam", teb200::traced("teb200.multi_tensor_adam", &multi_tensor_adam));
  m.def("multi_tensor_sgd", teb200::traced("teb200.multi_tensor_sgd", &multi_tensor_sgd));
  m.def("multi_tensor_scale", teb200::traced("teb200.multi_tensor_scale", &multi_tensor_scale));
  m.def("multi_tensor_l2norm_sq", teb200::traced("teb200.multi_tensor_l2norm_sq", &multi_tensor_l2norm_sq));
  m.def("cross_entropy", teb200::traced("teb200.cross_entropy", &cross_entropy));
  m.def("rope", teb200::traced("teb200.rope", &rope), py::arg("x"), py::arg("out"), py::arg("freqs"), py::arg("d_rot"),
        py::arg("interleaved"), py::arg("backward"), py::arg("pos_offset"), py::arg("cp_size"), py::arg("cp_rank"),
        py::arg("start_positions"), py::arg("qkv_mode") = 0, py::arg("q_per_group") = 0, py::arg("hq") = 0,
        py::arg("hk") = 0, py::arg("freqs_k") = py::none());
  register_extra(m);
}
