// C interface over the native launchers (see teb200/c_api.h).  Handles are small host structs that
// describe caller-owned device buffers; every entry point checks shapes, dtypes and alignment on the
// host and only then builds the launcher's argument struct.
#include <teb200/c_api.h>

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>

#include <teb200/api.h>
#include <teb200/norm.h>
#include <teb200/quant.h>

namespace {

constexpr uint32_t kTensorMagic = 0x7eb200a1u;
constexpr uint32_t kConfigMagic = 0x7eb200c2u;
constexpr int kMaxDims = 8;

struct Buffer {
  void* ptr = nullptr;
  teb200_dtype_t dtype = TEB200_BYTE;
  int ndim = 0;
  int64_t shape[kMaxDims] = {};
  bool set() const { return ptr != nullptr; }
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    return n;
  }
  int64_t last() const { return ndim > 0 ? shape[ndim - 1] : 1; }
  int64_t lead() const { return ndim > 0 ? numel() / (last() > 0 ? last() : 1) : 1; }
};

thread_local std::string g_error;

teb200_status_t fail(teb200_status_t code, const std::string& msg) {
  g_error = msg;
  return code;
}

teb200_status_t cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return TEB200_OK;
  return fail(TEB200_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

bool is_fp8(teb200_dtype_t d) { return d == TEB200_FLOAT8_E4M3 || d == TEB200_FLOAT8_E5M2; }
bool is_hp(teb200_dtype_t d) { return d == TEB200_FLOAT32 || d == TEB200_FLOAT16 || d == TEB200_BFLOAT16; }
bool is_16bit(teb200_dtype_t d) { return d == TEB200_FLOAT16 || d == TEB200_BFLOAT16; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

struct teb200_tensor_s {
  uint32_t magic = kTensorMagic;
  teb200_scaling_t scaling = TEB200_SCALING_NONE;
  Buffer params[TEB200_NUM_PARAMS];
};

struct teb200_quant_config_s {
  uint32_t magic = kConfigMagic;
  int force_pow2 = 1;
  float amax_epsilon = 0.f;
  int stochastic = 0;
  int hadamard = 0;
  int nvfp4_2d = 0;
  uint64_t seed = 0, offset = 0;
};

namespace {

bool valid(teb200_tensor_t t) { return t != nullptr && t->magic == kTensorMagic; }
bool valid(teb200_quant_config_t c) { return c != nullptr && c->magic == kConfigMagic; }

// logical [rows, cols] of a tensor from its data copies
bool matrix_shape(const teb200_tensor_s& t, int64_t& rows, int64_t& cols) {
  const Buffer& r = t.params[TEB200_ROWWISE_DATA];
  const Buffer& c = t.params[TEB200_COLUMNWISE_DATA];
  const int pack = t.scaling == TEB200_SCALING_NVFP4 ? 2 : 1;  // two E2M1 values per byte
  if (r.set()) {
    rows = r.lead();
    cols = r.last() * pack;
    return true;
  }
  if (c.set()) {
    cols = c.lead();
    rows = c.last() * pack;
    return true;
  }
  return false;
}

}  // namespace

extern "C" {

const char* teb200_version(void) { return "teb200 C API 1"; }
const char* teb200_last_error(void) { return g_error.c_str(); }

teb200_status_t teb200_tensor_create(teb200_scaling_t scaling, teb200_tensor_t* out) {
  if (out == nullptr) return fail(TEB200_ERR_INVALID, "tensor_create: null result pointer");
  if (scaling < TEB200_SCALING_NONE || scaling > TEB200_SCALING_BLOCK_2D)
    return fail(TEB200_ERR_INVALID, "tensor_create: unknown scaling mode");
  teb200_tensor_s* t = new (std::nothrow) teb200_tensor_s();
  if (t == nullptr) return fail(TEB200_ERR_INVALID, "tensor_create: out of host memory");
  t->scaling = scaling;
  *out = t;
  return TEB200_OK;
}

teb200_status_t teb200_tensor_destroy(teb200_tensor_t t) {
  if (t == nullptr) return TEB200_OK;
  if (!valid(t)) return fail(TEB200_ERR_INVALID, "tensor_destroy: not a live tensor handle");
  t->magic = 0;  // a second destroy of the same pointer is then caught, not a double free of live data
  delete t;
  return TEB200_OK;
}

teb200_status_t teb200_tensor_set_param(teb200_tensor_t t, teb200_param_t which, void* ptr, teb200_dtype_t dtype,
                                        const int64_t* shape, int ndim) {
  if (!valid(t)) return fail(TEB200_ERR_INVALID, "tensor_set_param: not a live tensor handle");
  if (which < 0 || which >= TEB200_NUM_PARAMS) return fail(TEB200_ERR_INVALID, "tensor_set_param: unknown parameter");
  if (ndim < 0 || ndim > kMaxDims || (ndim > 0 && shape == nullptr))
    return fail(TEB200_ERR_INVALID, "tensor_set_param: between 0 and 8 dimensions");
  if (dtype < TEB200_FLOAT32 || dtype > TEB200_FLOAT4_E2M1) return fail(TEB200_ERR_INVALID, "tensor_set_param: unknown dtype");
  for (int i = 0; i < ndim; ++i)
    if (shape[i] < 0) return fail(TEB200_ERR_INVALID, "tensor_set_param: negative extent");
  const bool data = which == TEB200_ROWWISE_DATA || which == TEB200_COLUMNWISE_DATA;
  if (data && ptr != nullptr) {
    if (t->scaling == TEB200_SCALING_NONE && !is_hp(dtype))
      return fail(TEB200_ERR_INVALID, "tensor_set_param: an unscaled tensor holds fp32, fp16 or bf16");
    if (t->scaling == TEB200_SCALING_NVFP4 && dtype != TEB200_FLOAT4_E2M1 && dtype != TEB200_BYTE)
      return fail(TEB200_ERR_INVALID, "tensor_set_param: NVFP4 data is E2M1 (two values per byte)");
    if (t->scaling != TEB200_SCALING_NONE && t->scaling != TEB200_SCALING_NVFP4 && !is_fp8(dtype))
      return fail(TEB200_ERR_INVALID, "tensor_set_param: FP8 scaling modes hold E4M3 or E5M2 data");
    if (!aligned16(ptr)) return fail(TEB200_ERR_INVALID, "tensor_set_param: data must be 16-byte aligned");
  }
  if ((which == TEB200_SCALE || which == TEB200_AMAX || which == TEB200_COLUMNWISE_AMAX) && ptr != nullptr &&
      dtype != TEB200_FLOAT32)
    return fail(TEB200_ERR_INVALID, "tensor_set_param: scale and amax are fp32");
  Buffer& b = t->params[which];
  b.ptr = ptr;
  b.dtype = dtype;
  b.ndim = ndim;
  for (int i = 0; i < kMaxDims; ++i) b.shape[i] = i < ndim ? shape[i] : 0;
  return TEB200_OK;
}

teb200_status_t teb200_tensor_get_param(teb200_tensor_t t, teb200_param_t which, void** ptr, teb200_dtype_t* dtype,
                                        int64_t* shape, int* ndim) {
  if (!valid(t)) return fail(TEB200_ERR_INVALID, "tensor_get_param: not a live tensor handle");
  if (which < 0 || which >= TEB200_NUM_PARAMS) return fail(TEB200_ERR_INVALID, "tensor_get_param: unknown parameter");
  const Buffer& b = t->params[which];
  if (ptr) *ptr = b.ptr;
  if (dtype) *dtype = b.dtype;
  if (ndim) *ndim = b.ndim;
  if (shape)
    for (int i = 0; i < b.ndim; ++i) shape[i] = b.shape[i];
  return TEB200_OK;
}

teb200_status_t teb200_tensor_scaling(teb200_tensor_t t, teb200_scaling_t* out) {
  if (!valid(t) || out == nullptr) return fail(TEB200_ERR_INVALID, "tensor_scaling: bad handle or null result");
  *out = t->scaling;
  return TEB200_OK;
}

teb200_status_t teb200_tensor_matrix_shape(teb200_tensor_t t, int64_t* rows, int64_t* cols) {
  if (!valid(t) || rows == nullptr || cols == nullptr) return fail(TEB200_ERR_INVALID, "tensor_matrix_shape: bad arguments");
  if (!matrix_shape(*t, *rows, *cols)) return fail(TEB200_ERR_INVALID, "tensor_matrix_shape: no data copy is set");
  return TEB200_OK;
}

int64_t teb200_scale_inv_bytes(teb200_scaling_t scaling, int64_t rows, int64_t cols, int columnwise) {
  const int64_t r = columnwise ? cols : rows, c = columnwise ? rows : cols;  // the copy's own [r, c]
  switch (scaling) {
    case TEB200_SCALING_TENSOR: return 4;
    case TEB200_SCALING_MXFP8: return round_up(r, 128) * round_up((c + 31) / 32, 4);          // UE8M0, swizzled tiles
    case TEB200_SCALING_NVFP4: return round_up(r, 128) * round_up((c + 15) / 16, 4);          // E4M3, swizzled tiles
    case TEB200_SCALING_BLOCK_1D: return r * ((c + 127) / 128) * 4;                            // fp32 [r, ceil(c/128)]
    case TEB200_SCALING_BLOCK_2D: return ((r + 127) / 128) * ((c + 127) / 128) * 4;
    default: return 0;
  }
}

teb200_status_t teb200_quant_config_create(teb200_quant_config_t* out) {
  if (out == nullptr) return fail(TEB200_ERR_INVALID, "quant_config_create: null result pointer");
  teb200_quant_config_s* c = new (std::nothrow) teb200_quant_config_s();
  if (c == nullptr) return fail(TEB200_ERR_INVALID, "quant_config_create: out of host memory");
  *out = c;
  return TEB200_OK;
}

teb200_status_t teb200_quant_config_destroy(teb200_quant_config_t c) {
  if (c == nullptr) return TEB200_OK;
  if (!valid(c)) return fail(TEB200_ERR_INVALID, "quant_config_destroy: not a live config handle");
  c->magic = 0;
  delete c;
  return TEB200_OK;
}

namespace {
struct AttrSlot {
  void* p;
  size_t size;
};
bool attr_slot(teb200_quant_config_s* c, teb200_quant_attr_t a, AttrSlot& s) {
  switch (a) {
    case TEB200_QCFG_FORCE_POW2_SCALES: s = {&c->force_pow2, sizeof(int)}; return true;
    case TEB200_QCFG_AMAX_EPSILON: s = {&c->amax_epsilon, sizeof(float)}; return true;
    case TEB200_QCFG_STOCHASTIC_ROUNDING: s = {&c->stochastic, sizeof(int)}; return true;
    case TEB200_QCFG_RANDOM_HADAMARD: s = {&c->hadamard, sizeof(int)}; return true;
    case TEB200_QCFG_NVFP4_2D: s = {&c->nvfp4_2d, sizeof(int)}; return true;
    case TEB200_QCFG_RNG_SEED: s = {&c->seed, sizeof(uint64_t)}; return true;
    case TEB200_QCFG_RNG_OFFSET: s = {&c->offset, sizeof(uint64_t)}; return true;
    default: return false;
  }
}
}  // namespace

teb200_status_t teb200_quant_config_set(teb200_quant_config_t c, teb200_quant_attr_t attr, const void* value, size_t size) {
  AttrSlot s;
  if (!valid(c) || value == nullptr) return fail(TEB200_ERR_INVALID, "quant_config_set: bad handle or null value");
  if (!attr_slot(c, attr, s)) return fail(TEB200_ERR_INVALID, "quant_config_set: unknown attribute");
  if (size != s.size) return fail(TEB200_ERR_INVALID, "quant_config_set: value has the wrong size for this attribute");
  std::memcpy(s.p, value, size);
  return TEB200_OK;
}

teb200_status_t teb200_quant_config_get(teb200_quant_config_t c, teb200_quant_attr_t attr, void* value, size_t size) {
  AttrSlot s;
  if (!valid(c) || value == nullptr) return fail(TEB200_ERR_INVALID, "quant_config_get: bad handle or null value");
  if (!attr_slot(c, attr, s)) return fail(TEB200_ERR_INVALID, "quant_config_get: unknown attribute");
  if (size != s.size) return fail(TEB200_ERR_INVALID, "quant_config_get: value has the wrong size for this attribute");
  std::memcpy(value, s.p, size);
  return TEB200_OK;
}

teb200_status_t teb200_quantize(teb200_tensor_t in, teb200_tensor_t out, teb200_quant_config_t cfg, teb200_stream_t stream) {
  if (!valid(in) || !valid(out)) return fail(TEB200_ERR_INVALID, "quantize: not a live tensor handle");
  if (cfg != nullptr && !valid(cfg)) return fail(TEB200_ERR_INVALID, "quantize: not a live config handle");
  teb200_quant_config_s defaults;
  const teb200_quant_config_s& q = cfg ? *cfg : defaults;
  if (in->scaling != TEB200_SCALING_NONE || !in->params[TEB200_ROWWISE_DATA].set())
    return fail(TEB200_ERR_INVALID, "quantize: the input is an unscaled tensor with row-wise data");
  const Buffer& x = in->params[TEB200_ROWWISE_DATA];
  const int64_t R = x.lead(), C = x.last();
  const Buffer& rd = out->params[TEB200_ROWWISE_DATA];
  const Buffer& cd = out->params[TEB200_COLUMNWISE_DATA];
  const Buffer& rs = out->params[TEB200_ROWWISE_SCALE_INV];
  const Buffer& cs = out->params[TEB200_COLUMNWISE_SCALE_INV];
  if (!rd.set() && !cd.set()) return fail(TEB200_ERR_INVALID, "quantize: the output has no data copy to fill");
  int64_t oR = 0, oC = 0;
  matrix_shape(*out, oR, oC);
  if (oR != R || oC != C) return fail(TEB200_ERR_INVALID, "quantize: output shape differs from the input's");
  if (rd.set() && cd.set() && (cd.lead() != C || cd.last() * (out->scaling == TEB200_SCALING_NVFP4 ? 2 : 1) != R))
    return fail(TEB200_ERR_INVALID, "quantize: the column-wise copy must be [cols, rows]");
  if (R > INT32_MAX || C > INT32_MAX) return fail(TEB200_ERR_INVALID, "quantize: extent above 2^31");
  if (R == 0 || C == 0) return TEB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool e5m2 = (rd.set() ? rd.dtype : cd.dtype) == TEB200_FLOAT8_E5M2;
  switch (out->scaling) {
    case TEB200_SCALING_TENSOR: {
      const Buffer& scale = out->params[TEB200_SCALE];
      if (!scale.set() || !rs.set()) return fail(TEB200_ERR_INVALID, "quantize: per-tensor scaling needs scale and scale_inv");
      teb200::QuantArgs a;
      a.x = x.ptr; a.x_dtype = x.dtype; a.R = static_cast<int>(R); a.C = static_cast<int>(C); a.ldx = C;
      a.row_data = static_cast<uint8_t*>(rd.ptr); a.col_data = static_cast<uint8_t*>(cd.ptr);
      a.fp8_e5m2 = e5m2; a.scale = static_cast<const float*>(scale.ptr);
      a.amax = static_cast<float*>(out->params[TEB200_AMAX].ptr); a.scale_inv = static_cast<float*>(rs.ptr);
      return cuda_status(teb200::quantize_fp8_tensor(a, s), "quantize (per-tensor FP8)");
    }
    case TEB200_SCALING_MXFP8: {
      if (C % 32 != 0 || (cd.set() && R % 32 != 0))
        return fail(TEB200_ERR_INVALID, "quantize: MXFP8 needs the scaled dimension to be a multiple of 32");
      if ((rd.set() && !rs.set()) || (cd.set() && !cs.set()))
        return fail(TEB200_ERR_INVALID, "quantize: every MXFP8 data copy needs its scale_inv buffer");
      if (rd.set() && rs.numel() * 1 < teb200_scale_inv_bytes(out->scaling, R, C, 0))
        return fail(TEB200_ERR_INVALID, "quantize: row-wise scale_inv buffer too small (see teb200_scale_inv_bytes)");
      if (cd.set() && cs.numel() * 1 < teb200_scale_inv_bytes(out->scaling, R, C, 1))
        return fail(TEB200_ERR_INVALID, "quantize: column-wise scale_inv buffer too small (see teb200_scale_inv_bytes)");
      teb200::QuantArgs a;
      a.x = x.ptr; a.x_dtype = x.dtype; a.R = static_cast<int>(R); a.C = static_cast<int>(C); a.ldx = C;
      a.row_data = static_cast<uint8_t*>(rd.ptr); a.row_scale_out = static_cast<uint8_t*>(rs.ptr);
      a.col_data = static_cast<uint8_t*>(cd.ptr); a.col_scale_out = static_cast<uint8_t*>(cs.ptr);
      a.fp8_e5m2 = e5m2;
      return cuda_status(teb200::quantize_mxfp8(a, s), "quantize (MXFP8)");
    }
    case TEB200_SCALING_NVFP4: {
      const Buffer& amax = out->params[TEB200_AMAX];
      if (C % 16 != 0 || R % 16 != 0)
        return fail(TEB200_ERR_INVALID, "quantize: NVFP4 needs rows and columns to be multiples of 16");
      if (!amax.set() || amax.numel() < 2)
        return fail(TEB200_ERR_INVALID, "quantize: NVFP4 needs an amax buffer of two floats (row-wise, column-wise)");
      if ((rd.set() && !rs.set()) || (cd.set() && !cs.set()))
        return fail(TEB200_ERR_INVALID, "quantize: every NVFP4 data copy needs its scale_inv buffer");
      float* am = static_cast<float*>(amax.ptr);
      cudaError_t e = teb200::nvfp4_amax(x.ptr, x.dtype, static_cast<int>(R), static_cast<int>(C), q.hadamard, am, s);
      if (e != cudaSuccess) return cuda_status(e, "quantize (NVFP4 amax)");
      teb200::Nvfp4Args a;
      a.x = x.ptr; a.x_dtype = x.dtype; a.R = static_cast<int>(R); a.C = static_cast<int>(C);
      a.amax_row = am; a.amax_col = am + 1;
      a.row_data = static_cast<uint8_t*>(rd.ptr); a.row_scale = static_cast<uint8_t*>(rs.ptr);
      a.col_data = static_cast<uint8_t*>(cd.ptr); a.col_scale = static_cast<uint8_t*>(cs.ptr);
      a.with_rht = q.hadamard; a.with_2d = q.nvfp4_2d; a.stochastic = q.stochastic; a.seed = q.seed; a.offset = q.offset;
      return cuda_status(teb200::quantize_nvfp4(a, s), "quantize (NVFP4)");
    }
    case TEB200_SCALING_BLOCK_1D:
    case TEB200_SCALING_BLOCK_2D: {
      if ((rd.set() && !rs.set()) || (cd.set() && !cs.set()))
        return fail(TEB200_ERR_INVALID, "quantize: every block-scaled data copy needs its scale_inv buffer");
      teb200::BlockQuantArgs a;
      a.x = x.ptr; a.x_dtype = x.dtype; a.R = static_cast<int>(R); a.C = static_cast<int>(C); a.ld = C;
      a.dim = out->scaling == TEB200_SCALING_BLOCK_1D ? 1 : 2;
      a.e5m2 = e5m2; a.pow2 = q.force_pow2; a.eps = q.amax_epsilon;
      a.row_data = static_cast<uint8_t*>(rd.ptr); a.row_sinv = static_cast<float*>(rs.ptr);
      a.col_data = static_cast<uint8_t*>(cd.ptr); a.col_sinv = static_cast<float*>(cs.ptr);
      return cuda_status(teb200::quantize_block128(a, s), "quantize (FP8 block scaling)");
    }
    default:
      return fail(TEB200_ERR_INVALID, "quantize: the output has no scaling mode");
  }
}

teb200_status_t teb200_dequantize(teb200_tensor_t in, teb200_tensor_t out, teb200_stream_t stream) {
  if (!valid(in) || !valid(out)) return fail(TEB200_ERR_INVALID, "dequantize: not a live tensor handle");
  const Buffer& y = out->params[TEB200_ROWWISE_DATA];
  const Buffer& d = in->params[TEB200_ROWWISE_DATA];
  const Buffer& sc = in->params[TEB200_ROWWISE_SCALE_INV];
  if (out->scaling != TEB200_SCALING_NONE || !y.set()) return fail(TEB200_ERR_INVALID, "dequantize: the output is an unscaled tensor");
  if (!d.set() || !sc.set()) return fail(TEB200_ERR_INVALID, "dequantize: the input needs row-wise data and scale_inv");
  int64_t R = 0, C = 0;
  matrix_shape(*in, R, C);
  if (y.lead() != R || y.last() != C) return fail(TEB200_ERR_INVALID, "dequantize: output shape differs from the input's");
  if (R > INT32_MAX || C > INT32_MAX) return fail(TEB200_ERR_INVALID, "dequantize: extent above 2^31");
  if (R == 0 || C == 0) return TEB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int e5m2 = d.dtype == TEB200_FLOAT8_E5M2;
  switch (in->scaling) {
    case TEB200_SCALING_TENSOR:
      return cuda_status(teb200::dequantize_fp8_tensor(static_cast<const uint8_t*>(d.ptr), static_cast<const float*>(sc.ptr),
                                                       R * C, e5m2, y.ptr, y.dtype, s), "dequantize (per-tensor FP8)");
    case TEB200_SCALING_MXFP8:
      return cuda_status(teb200::dequantize_mxfp8(static_cast<const uint8_t*>(d.ptr), static_cast<const uint8_t*>(sc.ptr),
                                                  static_cast<int>(R), static_cast<int>(C), e5m2, y.ptr, y.dtype, s),
                         "dequantize (MXFP8)");
    case TEB200_SCALING_NVFP4: {
      const Buffer& amax = in->params[TEB200_AMAX];
      if (!amax.set()) return fail(TEB200_ERR_INVALID, "dequantize: NVFP4 needs the amax it was quantized with");
      return cuda_status(teb200::dequantize_nvfp4(static_cast<const uint8_t*>(d.ptr), static_cast<const uint8_t*>(sc.ptr),
                                                  static_cast<const float*>(amax.ptr), static_cast<int>(R),
                                                  static_cast<int>(C), y.ptr, y.dtype, s), "dequantize (NVFP4)");
    }
    default:
      return fail(TEB200_ERR_UNSUPPORTED, "dequantize: block-scaled FP8 is dequantized by the framework layer");
  }
}

teb200_status_t teb200_gemm(teb200_tensor_t a, teb200_tensor_t b, teb200_tensor_t d, teb200_tensor_t bias, int accumulate,
                            float alpha, int* status_dev, teb200_stream_t stream) {
  if (!valid(a) || !valid(b) || !valid(d)) return fail(TEB200_ERR_INVALID, "gemm: not a live tensor handle");
  if (bias != nullptr && !valid(bias)) return fail(TEB200_ERR_INVALID, "gemm: bias is not a live tensor handle");
  if (status_dev == nullptr) return fail(TEB200_ERR_INVALID, "gemm: status_dev (a zeroed device int) is required");
  if (a->scaling != b->scaling) return fail(TEB200_ERR_INVALID, "gemm: A and B must share a scaling mode");
  const Buffer& ad = a->params[TEB200_ROWWISE_DATA];
  const Buffer& bd = b->params[TEB200_ROWWISE_DATA];
  const Buffer& dd = d->params[TEB200_ROWWISE_DATA];
  if (!ad.set() || !bd.set() || !dd.set()) return fail(TEB200_ERR_INVALID, "gemm: A, B and D need row-wise data");
  if (d->scaling != TEB200_SCALING_NONE) return fail(TEB200_ERR_UNSUPPORTED, "gemm: the output is an unscaled tensor");
  const int64_t M = ad.lead(), K = ad.last(), N = bd.lead();
  if (bd.last() != K) return fail(TEB200_ERR_INVALID, "gemm: A is [M, K] and B is [N, K]: contraction lengths differ");
  if (dd.lead() != M || dd.last() != N) return fail(TEB200_ERR_INVALID, "gemm: D must be [M, N]");
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(TEB200_ERR_INVALID, "gemm: extent above 2^31");
  if (accumulate && dd.dtype != TEB200_FLOAT32 && !is_16bit(dd.dtype)) return fail(TEB200_ERR_INVALID, "gemm: bad output dtype");
  teb200::GemmArgs g;
  g.a = ad.ptr; g.b = bd.ptr; g.d = dd.ptr;
  g.M = static_cast<int>(M); g.N = static_cast<int>(N); g.K = static_cast<int>(K);
  g.lda = K; g.ldb = K; g.ldd = N;
  g.a_dtype = ad.dtype; g.b_dtype = bd.dtype; g.d_dtype = dd.dtype;
  g.alpha = alpha; g.accumulate = accumulate != 0; g.status = status_dev;
  if (bias != nullptr) {
    const Buffer& bb = bias->params[TEB200_ROWWISE_DATA];
    if (bias->scaling != TEB200_SCALING_NONE || !bb.set() || bb.numel() != N)
      return fail(TEB200_ERR_INVALID, "gemm: bias is an unscaled tensor of N values");
    g.bias = bb.ptr; g.bias_dtype = bb.dtype; g.epilogue = teb200::kEpiBias;
  }
  if (M == 0 || N == 0) return TEB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (a->scaling) {
    case TEB200_SCALING_NONE:
      if (!is_16bit(ad.dtype) || ad.dtype != bd.dtype)
        return fail(TEB200_ERR_UNSUPPORTED, "gemm: unscaled operands are both fp16 or both bf16");
      if (K % 8 != 0) return fail(TEB200_ERR_INVALID, "gemm: K must be a multiple of 8 for 16-bit operands (16-byte rows)");
      return cuda_status(teb200::gemm_bf16(g, s), "gemm (16-bit)");
    case TEB200_SCALING_MXFP8: {
      const Buffer& sa = a->params[TEB200_ROWWISE_SCALE_INV];
      const Buffer& sb = b->params[TEB200_ROWWISE_SCALE_INV];
      if (!sa.set() || !sb.set()) return fail(TEB200_ERR_INVALID, "gemm: MXFP8 operands need row-wise scale_inv");
      if (K % 32 != 0) return fail(TEB200_ERR_INVALID, "gemm: MXFP8 needs K to be a multiple of 32");
      g.sfa = static_cast<const uint8_t*>(sa.ptr);
      g.sfb = static_cast<const uint8_t*>(sb.ptr);
      return cuda_status(teb200::gemm_mxfp8(g, s), "gemm (MXFP8)");
    }
    case TEB200_SCALING_TENSOR:
    case TEB200_SCALING_NVFP4:
      return fail(TEB200_ERR_UNSUPPORTED,
                  "gemm: per-tensor FP8 and NVFP4 products need a device-side alpha that the framework layer computes");
    default:
      return fail(TEB200_ERR_UNSUPPORTED, "gemm: block-scaled FP8 operands go through their MXFP8 scale copies");
  }
}

teb200_status_t teb200_norm_forward(teb200_tensor_t x, teb200_tensor_t gamma, teb200_tensor_t beta, float eps,
                                    int zero_centered_gamma, teb200_tensor_t y, float* mu, float* rsigma,
                                    teb200_stream_t stream) {
  if (!valid(x) || !valid(gamma) || !valid(y)) return fail(TEB200_ERR_INVALID, "norm_forward: not a live tensor handle");
  if (beta != nullptr && !valid(beta)) return fail(TEB200_ERR_INVALID, "norm_forward: beta is not a live tensor handle");
  const Buffer& xb = x->params[TEB200_ROWWISE_DATA];
  const Buffer& gb = gamma->params[TEB200_ROWWISE_DATA];
  const Buffer& yb = y->params[TEB200_ROWWISE_DATA];
  if (x->scaling != TEB200_SCALING_NONE || y->scaling != TEB200_SCALING_NONE || gamma->scaling != TEB200_SCALING_NONE)
    return fail(TEB200_ERR_UNSUPPORTED, "norm_forward: unscaled tensors only (quantize the result with teb200_quantize)");
  if (!xb.set() || !gb.set() || !yb.set() || rsigma == nullptr) return fail(TEB200_ERR_INVALID, "norm_forward: missing buffer");
  const int64_t R = xb.lead(), C = xb.last();
  if (gb.numel() != C || yb.lead() != R || yb.last() != C || yb.dtype != xb.dtype)
    return fail(TEB200_ERR_INVALID, "norm_forward: gamma is [cols], y matches x in shape and dtype");
  if (C % 8 != 0) return fail(TEB200_ERR_INVALID, "norm_forward: the normalized dimension must be a multiple of 8");
  if (R > INT32_MAX || C > INT32_MAX) return fail(TEB200_ERR_INVALID, "norm_forward: extent above 2^31");
  const bool layernorm = beta != nullptr;
  if (layernorm && mu == nullptr) return fail(TEB200_ERR_INVALID, "norm_forward: LayerNorm needs the mu buffer");
  teb200::NormArgs a;
  a.layernorm = layernorm; a.R = static_cast<int>(R); a.C = static_cast<int>(C);
  a.x_dtype = xb.dtype; a.w_dtype = gb.dtype; a.eps = eps; a.zero_centered = zero_centered_gamma;
  a.x = xb.ptr; a.gamma = gb.ptr; a.y = yb.ptr; a.mu = mu; a.rs = rsigma;
  if (layernorm) {
    const Buffer& bb = beta->params[TEB200_ROWWISE_DATA];
    if (!bb.set() || bb.numel() != C || bb.dtype != gb.dtype) return fail(TEB200_ERR_INVALID, "norm_forward: beta is [cols], dtype of gamma");
    a.beta = bb.ptr;
  }
  return cuda_status(teb200::norm_fwd(a, static_cast<cudaStream_t>(stream)), "norm_forward");
}

}  // extern "C"
