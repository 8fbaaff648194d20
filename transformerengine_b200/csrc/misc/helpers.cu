// Small memory-bound helpers: column sums (bias gradient), splits -> offsets, multi-slab row padding
// (FP8 alignment of MoE expert slabs) and last-dimension padding.
// (Reference behaviour: common/util/padding.cu:46,130; common/util/splits_to_offsets.cu:61;
// fused_attn/flash_attn.cu pad-last-dim helper; the dbias reductions of common/cast/**.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <teb200/api.h>
#include <teb200/misc.h>

namespace teb200 {
namespace {

constexpr int CS_COLS = 256;  // columns per block: 32 lanes x 8 values (one 16-byte load of a 16-bit type)
constexpr int CS_ROWS = 8;    // row lanes per block

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = static_cast<float>(p[i]);
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(u[i] << 16);
    v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __low2float(h[i]);
    v[2 * i + 1] = __high2float(h[i]);
  }
}

// stage 1: partial[part][c] = sum over the rows of the part.  Needs C % 8 == 0 and 16-byte aligned rows.
template <typename T>
__global__ void __launch_bounds__(32 * CS_ROWS)
colsum_partial_kernel(const T* __restrict__ x, int R, int C, long long ld, int rows_per_part, float* __restrict__ partial) {
  __shared__ float sm[CS_ROWS][CS_COLS + 8];
  const int lane = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c0 = blockIdx.x * CS_COLS + lane * 8;
  const int part = blockIdx.y;
  const int r0 = part * rows_per_part, r1 = min(R, r0 + rows_per_part);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < C) {
    for (int r = r0 + ry; r < r1; r += CS_ROWS) {
      float v[8];
      load8<T>(x + static_cast<long long>(r) * ld + c0, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sm[ry][lane * 8 + i] = acc[i];
  __syncthreads();
  for (int c = threadIdx.x; c < CS_COLS; c += 32 * CS_ROWS) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < CS_ROWS; ++r) s += sm[r][c];
    const int col = blockIdx.x * CS_COLS + c;
    if (col < C) partial[static_cast<size_t>(part) * C + col] = s;
  }
}

template <typename O>
__global__ void colsum_final_kernel(const float* __restrict__ partial, int parts, int C, O* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<size_t>(p) * C + c];
  out[c] = static_cast<O>(s);
}

template <typename I, typename O>
__global__ void splits_to_offsets_kernel(const I* __restrict__ splits, int n, long long mult, O* __restrict__ out) {
  // one block; n is small (experts, sequences): a serial scan per 1024-element chunk by thread 0 would do,
  // a warp scan keeps it a few hundred nanoseconds for n in the thousands
  __shared__ long long carry;
  if (threadIdx.x == 0) {
    carry = 0;
    out[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    long long v = i < n ? static_cast<long long>(splits[i]) * mult : 0;
    // inclusive scan inside the block through shared memory
    __shared__ long long buf[1024];
    buf[threadIdx.x] = v;
    __syncthreads();
    for (int off = 1; off < blockDim.x; off <<= 1) {
      const long long add = threadIdx.x >= off ? buf[threadIdx.x - off] : 0;
      __syncthreads();
      buf[threadIdx.x] += add;
      __syncthreads();
    }
    if (i < n) out[i + 1] = static_cast<O>(carry + buf[threadIdx.x]);
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry += buf[threadIdx.x];
    __syncthreads();
  }
}

// out row r of slab g (out_off[g] <= r < out_off[g+1]) = in row in_off[g] + (r - out_off[g]) when that row
// exists in the source slab, zero otherwise.  Covers padding (out slabs longer) and unpadding (shorter).
__global__ void repad_rows_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, const int* __restrict__ in_off,
                                  const int* __restrict__ out_off, int groups, int vec_per_row) {
  const int total = out_off[groups];
  for (int r = blockIdx.x; r < total; r += gridDim.x) {
    int lo = 0, hi = groups;  // largest g with out_off[g] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (out_off[mid] <= r) lo = mid;
      else hi = mid;
    }
    const int local = r - out_off[lo];
    const int src_rows = in_off[lo + 1] - in_off[lo];
    uint4* o = out + static_cast<size_t>(r) * vec_per_row;
    if (local < src_rows) {
      const uint4* s = in + static_cast<size_t>(in_off[lo] + local) * vec_per_row;
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) o[v] = s[v];
    } else {
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) o[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// out [R, Cp] = in [R, C] padded with zeros (Cp >= C) or cut (Cp < C); element size es bytes
__global__ void pad_last_dim_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, long long R, int c_bytes,
                                    int cp_bytes) {
  const long long total = R * (cp_bytes / 4);
  const int words_out = cp_bytes / 4, words_in = c_bytes / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / words_out;
    const int w = static_cast<int>(i - r * words_out);
    uint32_t v = 0;
    if (w < words_in) v = reinterpret_cast<const uint32_t*>(in + r * c_bytes)[w];
    reinterpret_cast<uint32_t*>(out + r * cp_bytes)[w] = v;
  }
}

// out[g][c] = sum over the rows of slab g (offsets[g] .. offsets[g+1]) of x[r][c]; one block per (256 columns, slab)
template <typename T, typename O>
__global__ void __launch_bounds__(32 * CS_ROWS)
grouped_colsum_kernel(const T* __restrict__ x, const int* __restrict__ offsets, int C, long long ld, O* __restrict__ out) {
  __shared__ float sm[CS_ROWS][CS_COLS + 8];
  const int lane = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c0 = blockIdx.x * CS_COLS + lane * 8;
  const int g = blockIdx.y;
  const int r0 = offsets[g], r1 = offsets[g + 1];
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < C) {
    for (int r = r0 + ry; r < r1; r += CS_ROWS) {
      float v[8];
      load8<T>(x + static_cast<long long>(r) * ld + c0, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sm[ry][lane * 8 + i] = acc[i];
  __syncthreads();
  for (int c = threadIdx.x; c < CS_COLS; c += 32 * CS_ROWS) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < CS_ROWS; ++r) s += sm[r][c];
    const int col = blockIdx.x * CS_COLS + c;
    if (col < C) out[static_cast<size_t>(g) * C + col] = static_cast<O>(s);
  }
}

// x[r][c] += bias[g(r)][c] for the rows of every slab; one block per row, the slab found by binary search
template <typename T>
__global__ void grouped_bias_add_kernel(T* __restrict__ x, const T* __restrict__ bias, const int* __restrict__ offsets,
                                        int groups, int C, long long ld) {
  const int total = offsets[groups];
  for (int r = blockIdx.x; r < total; r += gridDim.x) {
    int lo = 0, hi = groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= r) lo = mid;
      else hi = mid;
    }
    T* row = x + static_cast<long long>(r) * ld;
    const T* b = bias + static_cast<size_t>(lo) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) row[c] = static_cast<T>(static_cast<float>(row[c]) + static_cast<float>(b[c]));
  }
}

// out[r] = sum_c a[r][c] * b[r][c] in fp32; one warp per row, 8 values per load
template <typename T>
__global__ void row_dot_kernel(const T* __restrict__ a, const T* __restrict__ b, long long R, int C, long long lda,
                               long long ldb, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < R; r += nwarps) {
    float acc = 0.f;
    for (int c = lane * 8; c < C; c += 256) {
      float va[8], vb[8];
      load8<T>(a + r * lda + c, va);
      load8<T>(b + r * ldb + c, vb);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += va[i] * vb[i];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) out[r] = acc;
  }
}

}  // namespace

int column_sum_parts(int R, int C) {
  const int col_blocks = (C + CS_COLS - 1) / CS_COLS;
  int parts = (148 * 4 + col_blocks - 1) / col_blocks;  // about four blocks per SM
  const int max_parts = (R + 63) / 64;                  // at least 64 rows per part
  if (parts > max_parts) parts = max_parts;
  return parts < 1 ? 1 : parts;
}

cudaError_t column_sum(const void* x, int x_dtype, int R, int C, long long ld, void* out, int out_dtype, float* workspace,
                       cudaStream_t s) {
  if (R <= 0 || C <= 0) return cudaSuccess;
  if (C % 8 != 0 || workspace == nullptr) return cudaErrorInvalidValue;
  const size_t es = dtype_size(x_dtype);
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (ld * es) % 16 != 0) return cudaErrorInvalidValue;
  const int parts = column_sum_parts(R, C);
  const int rows_per_part = (R + parts - 1) / parts;
  dim3 grid((C + CS_COLS - 1) / CS_COLS, parts);
  if (x_dtype == kBFloat16)
    colsum_partial_kernel<__nv_bfloat16><<<grid, 32 * CS_ROWS, 0, s>>>(static_cast<const __nv_bfloat16*>(x), R, C, ld, rows_per_part, workspace);
  else if (x_dtype == kFloat16)
    colsum_partial_kernel<__half><<<grid, 32 * CS_ROWS, 0, s>>>(static_cast<const __half*>(x), R, C, ld, rows_per_part, workspace);
  else if (x_dtype == kFloat32)
    colsum_partial_kernel<float><<<grid, 32 * CS_ROWS, 0, s>>>(static_cast<const float*>(x), R, C, ld, rows_per_part, workspace);
  else return cudaErrorInvalidValue;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int fg = (C + 255) / 256;
  if (out_dtype == kFloat32) colsum_final_kernel<float><<<fg, 256, 0, s>>>(workspace, parts, C, static_cast<float*>(out));
  else if (out_dtype == kBFloat16) colsum_final_kernel<__nv_bfloat16><<<fg, 256, 0, s>>>(workspace, parts, C, static_cast<__nv_bfloat16*>(out));
  else if (out_dtype == kFloat16) colsum_final_kernel<__half><<<fg, 256, 0, s>>>(workspace, parts, C, static_cast<__half*>(out));
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t grouped_column_sum(const void* x, int x_dtype, const int* offsets, int groups, int C, long long ld, void* out,
                               int out_dtype, cudaStream_t s) {
  if (groups <= 0 || C <= 0) return cudaSuccess;
  const size_t es = dtype_size(x_dtype);
  if (C % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 || (ld * es) % 16 != 0) return cudaErrorInvalidValue;
  dim3 grid((C + CS_COLS - 1) / CS_COLS, groups);
#define TEB_GCS(T, O) grouped_colsum_kernel<T, O><<<grid, 32 * CS_ROWS, 0, s>>>(static_cast<const T*>(x), offsets, C, ld, static_cast<O*>(out))
  if (x_dtype == kBFloat16 && out_dtype == kBFloat16) TEB_GCS(__nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == kBFloat16 && out_dtype == kFloat32) TEB_GCS(__nv_bfloat16, float);
  else if (x_dtype == kFloat16 && out_dtype == kFloat16) TEB_GCS(__half, __half);
  else if (x_dtype == kFloat16 && out_dtype == kFloat32) TEB_GCS(__half, float);
  else if (x_dtype == kFloat32 && out_dtype == kFloat32) TEB_GCS(float, float);
  else return cudaErrorInvalidValue;
#undef TEB_GCS
  return cudaGetLastError();
}

cudaError_t grouped_bias_add(void* x, const void* bias, int dtype, const int* offsets, int groups, int C, long long ld,
                             int max_rows, cudaStream_t s) {
  if (groups <= 0 || C <= 0 || max_rows <= 0) return cudaSuccess;
  const int grid = max_rows < 148 * 16 ? max_rows : 148 * 16;
  if (dtype == kBFloat16)
    grouped_bias_add_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(bias), offsets, groups, C, ld);
  else if (dtype == kFloat16)
    grouped_bias_add_kernel<__half><<<grid, 256, 0, s>>>(static_cast<__half*>(x), static_cast<const __half*>(bias), offsets, groups, C, ld);
  else if (dtype == kFloat32)
    grouped_bias_add_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(x), static_cast<const float*>(bias), offsets, groups, C, ld);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t row_dot(const void* a, const void* b, int dtype, long long R, int C, long long lda, long long ldb, float* out,
                    cudaStream_t s) {
  if (R <= 0) return cudaSuccess;
  const size_t es = dtype_size(dtype);
  if (C % 8 != 0 || (reinterpret_cast<uintptr_t>(a) & 15) != 0 || (reinterpret_cast<uintptr_t>(b) & 15) != 0 ||
      (lda * es) % 16 != 0 || (ldb * es) % 16 != 0)
    return cudaErrorInvalidValue;
  const long long blocks = (R + 7) / 8;  // eight warps (rows) per block
  const int grid = static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16);
  if (dtype == kBFloat16)
    row_dot_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), R, C, lda, ldb, out);
  else if (dtype == kFloat16)
    row_dot_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(a), static_cast<const __half*>(b), R, C, lda, ldb, out);
  else if (dtype == kFloat32)
    row_dot_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(a), static_cast<const float*>(b), R, C, lda, ldb, out);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t splits_to_offsets(const void* splits, int splits_is_int64, int n, long long multiplier, void* out,
                              int out_is_int64, cudaStream_t s) {
  if (n < 0) return cudaErrorInvalidValue;
  const int threads = n >= 1024 ? 1024 : (n > 32 ? ((n + 31) / 32) * 32 : 32);
  if (splits_is_int64 && out_is_int64)
    splits_to_offsets_kernel<long long, long long><<<1, threads, 0, s>>>(static_cast<const long long*>(splits), n, multiplier, static_cast<long long*>(out));
  else if (splits_is_int64)
    splits_to_offsets_kernel<long long, int><<<1, threads, 0, s>>>(static_cast<const long long*>(splits), n, multiplier, static_cast<int*>(out));
  else if (out_is_int64)
    splits_to_offsets_kernel<int, long long><<<1, threads, 0, s>>>(static_cast<const int*>(splits), n, multiplier, static_cast<long long*>(out));
  else
    splits_to_offsets_kernel<int, int><<<1, threads, 0, s>>>(static_cast<const int*>(splits), n, multiplier, static_cast<int*>(out));
  return cudaGetLastError();
}

cudaError_t repad_rows(const void* in, void* out, const int* in_offsets, const int* out_offsets, int groups, int row_bytes,
                       int max_out_rows, cudaStream_t s) {
  if (groups <= 0 || max_out_rows <= 0) return cudaSuccess;
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return cudaErrorInvalidValue;
  const int grid = max_out_rows < 148 * 16 ? max_out_rows : 148 * 16;
  const int vec = row_bytes / 16;
  repad_rows_kernel<<<grid, vec >= 256 ? 256 : (vec >= 128 ? 128 : 64), 0, s>>>(
      static_cast<const uint4*>(in), static_cast<uint4*>(out), in_offsets, out_offsets, groups, vec);
  return cudaGetLastError();
}

cudaError_t pad_last_dim(const void* in, void* out, long long R, int c_bytes, int cp_bytes, cudaStream_t s) {
  if (R <= 0 || cp_bytes <= 0) return cudaSuccess;
  if (c_bytes % 4 != 0 || cp_bytes % 4 != 0) return cudaErrorInvalidValue;
  const long long total = R * (cp_bytes / 4);
  const int grid = static_cast<int>(total / 256 + 1 < 148 * 8 ? total / 256 + 1 : 148 * 8);
  pad_last_dim_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), R, c_bytes, cp_bytes);
  return cudaGetLastError();
}

}  // namespace teb200
