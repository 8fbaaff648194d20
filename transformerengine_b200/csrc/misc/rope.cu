// Rotary position embedding, forward and backward, strided SBHD / BSHD input so it
// can run in place on the Q and K slices of a fused QKV projection output.
// out = x*cos + rot(x)*sin over the first d_rot dims, the rest is copied
// (reference: common/fused_rope/fused_rope.cu:39-92; context-parallel position
// remap for the dual-chunk split at :181-191).
#include <teb200/api.h>
#include <teb200/misc.h>
#include <teb200/ptx.cuh>

namespace teb200 {
namespace {

template <typename T>
__global__ void rope_kernel(const RopeArgs a) {
  extern __shared__ float cs[];  // cos[d_rot], sin[d_rot]
  const int si = blockIdx.x, bi = blockIdx.y;
  int pos = si;
  if (a.cp_size > 1) {
    const int half = a.s / 2;
    pos = si < half ? si + a.cp_rank * half : si + a.s * a.cp_size - (a.cp_rank + 1) * half - half;
  }
  pos += a.pos_offset + (a.start_positions ? a.start_positions[bi] : 0);
  for (int j = threadIdx.x; j < a.d_rot; j += blockDim.x) {
    float sn, c;
    sincosf(a.freqs[static_cast<size_t>(pos) * a.d_rot + j], &sn, &c);
    cs[j] = c;
    cs[a.d_rot + j] = sn;
  }
  __syncthreads();
  const T* x = static_cast<const T*>(a.x) + si * a.stride_s + bi * a.stride_b;
  T* out = static_cast<T*>(a.out) + si * a.stride_s + bi * a.stride_b;
  const int half = a.d_rot / 2;
  for (int idx = threadIdx.x; idx < a.h * a.d; idx += blockDim.x) {
    const int hi = idx / a.d, j = idx % a.d;
    const T* xh = x + hi * a.stride_h;
    float v = static_cast<float>(xh[j]);
    if (j < a.d_rot) {
      int jp;
      float sign;
      if (a.interleaved) {
        jp = (j & 1) ? j - 1 : j + 1;
        sign = (j & 1) ? 1.f : -1.f;
      } else {
        jp = j < half ? j + half : j - half;
        sign = j < half ? -1.f : 1.f;
      }
      const float other = static_cast<float>(xh[jp]);
      if (!a.backward) v = v * cs[j] + sign * other * cs[a.d_rot + j];
      else v = v * cs[j] - sign * other * cs[a.d_rot + jp];
    }
    // in-place: every thread reads both operands before any thread of this (s,b) writes
    reinterpret_cast<float*>(cs)[2 * a.d_rot + idx] = v;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < a.h * a.d; idx += blockDim.x) {
    const int hi = idx / a.d, j = idx % a.d;
    out[hi * a.stride_h + j] = static_cast<T>(cs[2 * a.d_rot + idx]);
  }
}

// Vector path (16-bit types, d_rot % 16 == 0, 16-byte aligned rows): one block per token, one
// thread per (head, 8-element group); both operands of a rotation pair are read by the thread
// that writes them, so the kernel is safe in place and needs no staging.
// kind of head `hi` of a packed QKV tensor: 0 query, 1 key, 2 value (plain tensors: always 0)
__device__ __forceinline__ int qkv_role(const RopeArgs& a, int hi) {
  if (a.qkv_mode == 1) {
    const int r = hi % (a.q_per_group + 2);
    return r < a.q_per_group ? 0 : (r == a.q_per_group ? 1 : 2);
  }
  if (a.qkv_mode == 2) return hi < a.hq ? 0 : (hi < a.hq + a.hk ? 1 : 2);
  return 0;
}

template <bool BF>
__global__ void rope_vec_kernel(const RopeArgs a) {
  extern __shared__ float cs_all[];  // cos[d_rot], sin[d_rot] of the queries, then (packed QKV, own key angles) of the keys
  const int si = blockIdx.x, bi = blockIdx.y;
  int pos = si;
  if (a.cp_size > 1) {
    const int half = a.s / 2;
    pos = si < half ? si + a.cp_rank * half : si + a.s * a.cp_size - (a.cp_rank + 1) * half - half;
  }
  pos += a.pos_offset + (a.start_positions ? a.start_positions[bi] : 0);
  const bool own_k = a.qkv_mode != 0 && a.freqs_k != nullptr && a.freqs_k != a.freqs;
  for (int j = threadIdx.x; j < a.d_rot; j += blockDim.x) {
    float sn, c;
    sincosf(a.freqs[static_cast<size_t>(pos) * a.d_rot + j], &sn, &c);
    cs_all[j] = c;
    cs_all[a.d_rot + j] = sn;
    if (own_k) {
      sincosf(a.freqs_k[static_cast<size_t>(pos) * a.d_rot + j], &sn, &c);
      cs_all[2 * a.d_rot + j] = c;
      cs_all[3 * a.d_rot + j] = sn;
    }
  }
  __syncthreads();
  const uint16_t* x = static_cast<const uint16_t*>(a.x) + si * a.stride_s + bi * a.stride_b;
  uint16_t* out = static_cast<uint16_t*>(a.out) + si * a.stride_s + bi * a.stride_b;
  const int half = a.d_rot / 2;
  auto unpack = [](uint32_t w, float& lo, float& hi) {
    if (BF) {
      lo = __uint_as_float(w << 16);
      hi = __uint_as_float(w & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w);
      lo = __low2float(h);
      hi = __high2float(h);
    }
  };
  auto pack = [](float lo, float hi) { return BF ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi); };
  if (!a.interleaved) {
    // out[j] = x[j] cos[j] - x[j+half] sin[j];  out[j+half] = x[j+half] cos[j+half] + x[j] sin[j+half]
    const int groups = half / 8;
    for (int it = threadIdx.x; it < a.h * groups; it += blockDim.x) {
      const int hi = it / groups, j0 = (it % groups) * 8;
      const uint16_t* xh = x + hi * a.stride_h;
      uint16_t* oh = out + hi * a.stride_h;
      const int role = qkv_role(a, hi);
      const uint4 va = *reinterpret_cast<const uint4*>(xh + j0);
      const uint4 vb = *reinterpret_cast<const uint4*>(xh + j0 + half);
      if (role == 2) {  // value head: untouched in place, copied otherwise
        if (a.out != a.x) {
          *reinterpret_cast<uint4*>(oh + j0) = va;
          *reinterpret_cast<uint4*>(oh + j0 + half) = vb;
        }
        continue;
      }
      const float* cs = cs_all + ((role == 1 && own_k) ? 2 * a.d_rot : 0);
      const uint32_t* wa = reinterpret_cast<const uint32_t*>(&va);
      const uint32_t* wb = reinterpret_cast<const uint32_t*>(&vb);
      uint4 oa, ob;
      uint32_t* pa = reinterpret_cast<uint32_t*>(&oa);
      uint32_t* pb = reinterpret_cast<uint32_t*>(&ob);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a0, a1, b0, b1;
        unpack(wa[k], a0, a1);
        unpack(wb[k], b0, b1);
        const int j = j0 + 2 * k;
        const float* sn = cs + a.d_rot;
        if (!a.backward) {
          pa[k] = pack(a0 * cs[j] - b0 * sn[j], a1 * cs[j + 1] - b1 * sn[j + 1]);
          pb[k] = pack(b0 * cs[j + half] + a0 * sn[j + half], b1 * cs[j + half + 1] + a1 * sn[j + half + 1]);
        } else {  // transpose of the forward map
          pa[k] = pack(a0 * cs[j] + b0 * sn[j + half], a1 * cs[j + 1] + b1 * sn[j + half + 1]);
          pb[k] = pack(b0 * cs[j + half] - a0 * sn[j], b1 * cs[j + half + 1] - a1 * sn[j + 1]);
        }
      }
      *reinterpret_cast<uint4*>(oh + j0) = oa;
      *reinterpret_cast<uint4*>(oh + j0 + half) = ob;
    }
  } else {
    // pairs (2i, 2i+1): out[2i] = x[2i] cos - x[2i+1] sin;  out[2i+1] = x[2i+1] cos + x[2i] sin
    const int groups = a.d_rot / 8;
    for (int it = threadIdx.x; it < a.h * groups; it += blockDim.x) {
      const int hi = it / groups, j0 = (it % groups) * 8;
      const uint16_t* xh = x + hi * a.stride_h;
      uint16_t* oh = out + hi * a.stride_h;
      const int role = qkv_role(a, hi);
      const uint4 va = *reinterpret_cast<const uint4*>(xh + j0);
      if (role == 2) {
        if (a.out != a.x) *reinterpret_cast<uint4*>(oh + j0) = va;
        continue;
      }
      const float* cs = cs_all + ((role == 1 && own_k) ? 2 * a.d_rot : 0);
      const uint32_t* wa = reinterpret_cast<const uint32_t*>(&va);
      uint4 oa;
      uint32_t* pa = reinterpret_cast<uint32_t*>(&oa);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float e, o;
        unpack(wa[k], e, o);
        const int j = j0 + 2 * k;
        const float* sn = cs + a.d_rot;
        if (!a.backward) pa[k] = pack(e * cs[j] - o * sn[j], o * cs[j + 1] + e * sn[j + 1]);
        else pa[k] = pack(e * cs[j] + o * sn[j + 1], o * cs[j + 1] - e * sn[j]);
      }
      *reinterpret_cast<uint4*>(oh + j0) = oa;
    }
  }
  if (a.out != a.x && a.d_rot < a.d) {  // the part that is not rotated is copied
    const int rest = a.d - a.d_rot;
    for (int it = threadIdx.x; it < a.h * rest; it += blockDim.x) {
      const int hi = it / rest, j = a.d_rot + it % rest;
      out[hi * a.stride_h + j] = x[hi * a.stride_h + j];
    }
  }
}

}  // namespace

cudaError_t rope_apply(const RopeArgs& a, cudaStream_t s) {
  if (a.s <= 0 || a.b <= 0) return cudaSuccess;
  const bool vec = (a.dtype == kBFloat16 || a.dtype == kFloat16) && a.d_rot % 16 == 0 && a.stride_s % 8 == 0 &&
                   a.stride_b % 8 == 0 && a.stride_h % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
  if (a.qkv_mode != 0 && !vec) return cudaErrorInvalidValue;  // the packed-QKV form exists in the vector kernel only
  if (vec) {
    dim3 grid(a.s, a.b);
    const size_t sm = (a.qkv_mode != 0 ? 4 : 2) * static_cast<size_t>(a.d_rot) * sizeof(float);
    const int work = a.h * (a.interleaved ? a.d_rot / 8 : a.d_rot / 16);
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    if (a.dtype == kBFloat16) rope_vec_kernel<true><<<grid, threads, sm, s>>>(a);
    else rope_vec_kernel<false><<<grid, threads, sm, s>>>(a);
    return cudaGetLastError();
  }
  const size_t smem = (2 * static_cast<size_t>(a.d_rot) + static_cast<size_t>(a.h) * a.d) * sizeof(float);
  dim3 grid(a.s, a.b);
  cudaError_t e = cudaSuccess;
#define TEB_ROPE(T)                                                                                       \
  do {                                                                                                    \
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(rope_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
    if (e != cudaSuccess) return e;                                                                       \
    rope_kernel<T><<<grid, 256, smem, s>>>(a);                                                            \
  } while (0)
  if (a.dtype == kBFloat16) TEB_ROPE(__nv_bfloat16);
  else if (a.dtype == kFloat16) TEB_ROPE(__half);
  else if (a.dtype == kFloat32) TEB_ROPE(float);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace teb200
