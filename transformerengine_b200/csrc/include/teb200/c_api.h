// Framework-agnostic C interface: opaque tensor handles over caller-owned device memory, a
// quantization-config object and the entry points a non-PyTorch host needs (quantize, dequantize,
// GEMM, normalization).  Nothing here allocates device memory or depends on a tensor library; every
// call validates its arguments before it launches anything and returns a teb200_status_t, with a
// human-readable message kept per thread (teb200_last_error).
// (Reference counterpart: common/include/transformer_engine/transformer_engine.h, the NVTETensor
// handle API; the handle layout and the functions here are this library's own.)
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct teb200_tensor_s* teb200_tensor_t;
typedef struct teb200_quant_config_s* teb200_quant_config_t;
typedef void* teb200_stream_t;  // a cudaStream_t

typedef enum {
  TEB200_OK = 0,
  TEB200_ERR_INVALID = 1,      // bad handle, shape, dtype, alignment or missing buffer
  TEB200_ERR_UNSUPPORTED = 2,  // a valid request that no kernel covers
  TEB200_ERR_CUDA = 3,         // the launch failed; teb200_last_error names the CUDA error
} teb200_status_t;

// Same numbering as the native launchers.
typedef enum {
  TEB200_FLOAT32 = 0,
  TEB200_FLOAT16 = 1,
  TEB200_BFLOAT16 = 2,
  TEB200_BYTE = 3,
  TEB200_FLOAT8_E4M3 = 4,
  TEB200_FLOAT8_E5M2 = 5,
  TEB200_FLOAT4_E2M1 = 6,  // two values per byte
} teb200_dtype_t;

typedef enum {
  TEB200_SCALING_NONE = 0,      // plain fp32 / fp16 / bf16 data
  TEB200_SCALING_TENSOR = 1,    // FP8 with one scale per tensor (delayed or current scaling)
  TEB200_SCALING_MXFP8 = 2,     // FP8 with a UE8M0 scale per 32 values, 128x4-tile swizzled
  TEB200_SCALING_NVFP4 = 3,     // E2M1 with an E4M3 scale per 16 values plus a tensor amax
  TEB200_SCALING_BLOCK_1D = 4,  // FP8 with an fp32 scale per 1 x 128 block
  TEB200_SCALING_BLOCK_2D = 5,  // FP8 with an fp32 scale per 128 x 128 block
} teb200_scaling_t;

typedef enum {
  TEB200_ROWWISE_DATA = 0,       // [rows, cols]
  TEB200_COLUMNWISE_DATA = 1,    // [cols, rows] (transposed copy, scales along the rows)
  TEB200_SCALE = 2,              // fp32 [1], multiply-before-cast (per-tensor scaling)
  TEB200_AMAX = 3,               // fp32 [1]
  TEB200_ROWWISE_SCALE_INV = 4,  // decode scales of the row-wise copy (layout depends on the scaling mode)
  TEB200_COLUMNWISE_SCALE_INV = 5,
  TEB200_COLUMNWISE_AMAX = 6,    // fp32 [1], NVFP4 column-wise copy (after the Hadamard rotation)
  TEB200_NUM_PARAMS = 7,
} teb200_param_t;

typedef enum {
  TEB200_QCFG_FORCE_POW2_SCALES = 0,   // int
  TEB200_QCFG_AMAX_EPSILON = 1,        // float
  TEB200_QCFG_STOCHASTIC_ROUNDING = 2, // int
  TEB200_QCFG_RANDOM_HADAMARD = 3,     // int: rotate 16-token blocks of the NVFP4 column-wise copy
  TEB200_QCFG_NVFP4_2D = 4,            // int: 16 x 16 block scales
  TEB200_QCFG_RNG_SEED = 5,            // uint64
  TEB200_QCFG_RNG_OFFSET = 6,          // uint64
  TEB200_QCFG_NUM_ATTRS = 7,
} teb200_quant_attr_t;

const char* teb200_version(void);
const char* teb200_last_error(void);  // message of the calling thread's last failing call ("" if none)

// ---- tensors.  A handle only DESCRIBES memory: destroy never frees a buffer.
teb200_status_t teb200_tensor_create(teb200_scaling_t scaling, teb200_tensor_t* out);
teb200_status_t teb200_tensor_destroy(teb200_tensor_t t);
// shape: up to 8 dims; data params flatten to 2-D as (product of the leading dims, last dim)
teb200_status_t teb200_tensor_set_param(teb200_tensor_t t, teb200_param_t which, void* ptr, teb200_dtype_t dtype,
                                        const int64_t* shape, int ndim);
teb200_status_t teb200_tensor_get_param(teb200_tensor_t t, teb200_param_t which, void** ptr, teb200_dtype_t* dtype,
                                        int64_t* shape, int* ndim);
teb200_status_t teb200_tensor_scaling(teb200_tensor_t t, teb200_scaling_t* out);
// logical 2-D shape of the tensor (from whichever data copy is set; the column-wise copy counts transposed)
teb200_status_t teb200_tensor_matrix_shape(teb200_tensor_t t, int64_t* rows, int64_t* cols);
// bytes a scale_inv buffer of this mode must hold for a [rows, cols] tensor (row-wise or column-wise copy)
int64_t teb200_scale_inv_bytes(teb200_scaling_t scaling, int64_t rows, int64_t cols, int columnwise);

// ---- quantization config
teb200_status_t teb200_quant_config_create(teb200_quant_config_t* out);
teb200_status_t teb200_quant_config_destroy(teb200_quant_config_t c);
teb200_status_t teb200_quant_config_set(teb200_quant_config_t c, teb200_quant_attr_t attr, const void* value, size_t size);
teb200_status_t teb200_quant_config_get(teb200_quant_config_t c, teb200_quant_attr_t attr, void* value, size_t size);

// ---- operations (asynchronous on `stream`)
// out = quantize(in).  `in` is a SCALING_NONE tensor; which copies are produced follows from the data
// params set on `out`.  cfg may be NULL (defaults).
teb200_status_t teb200_quantize(teb200_tensor_t in, teb200_tensor_t out, teb200_quant_config_t cfg, teb200_stream_t stream);
// out (SCALING_NONE) = dequantize(in), from the row-wise copy
teb200_status_t teb200_dequantize(teb200_tensor_t in, teb200_tensor_t out, teb200_stream_t stream);
// D[M, N] = alpha * A[M, K] * B[N, K]^T (+ D if accumulate) (+ bias[N]); A and B use their row-wise copies
// and must share a scaling mode (NONE: fp16 / bf16, TENSOR, MXFP8, NVFP4).  status_dev: a zero-initialised
// int in device memory that receives a non-zero code if a bounded wait inside the kernel runs out.
teb200_status_t teb200_gemm(teb200_tensor_t a, teb200_tensor_t b, teb200_tensor_t d, teb200_tensor_t bias, int accumulate,
                            float alpha, int* status_dev, teb200_stream_t stream);
// y = norm(x) * gamma (+ beta): LayerNorm when beta and mu are given, RMSNorm otherwise.  mu / rsigma: fp32 [rows].
teb200_status_t teb200_norm_forward(teb200_tensor_t x, teb200_tensor_t gamma, teb200_tensor_t beta, float eps,
                                    int zero_centered_gamma, teb200_tensor_t y, float* mu, float* rsigma,
                                    teb200_stream_t stream);

#ifdef __cplusplus
}
#endif
