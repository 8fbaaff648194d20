// Expert-parallel token exchange fused with the permutation, over NVLink peer memory.
//
//   counts : every rank publishes its per-expert token counts into every peer's table and
//            waits for all tables; each rank then derives, on the device, where its rows go.
//   push   : dispatch = permute + all-to-all in one kernel: the row of token t for expert e is
//            stored straight into the owner rank's expert-major buffer (16-byte peer stores),
//            optionally scaled per (token, expert); the last CTA raises a flag on every peer.
//   pull   : combine = all-to-all + unpermute in one kernel: out[t] = sum_e w[t,e] * peer row,
//            read with 16-byte peer loads; optionally also the per-pair dot products needed for
//            the routing-weight gradient.
// Flags are epoch counters in symmetric memory; every wait is bounded and reports through the
// status word.  (Reference: pytorch/ep.py dispatch/combine over a closed NCCL extension plus
// separate permutation kernels.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "teb200/api.h"
#include "teb200/comm.h"
#include "teb200/ptx.cuh"

namespace teb200 {
namespace {

// ---- counts exchange ---------------------------------------------------------------------------
// counts_all on every rank: [ep][E] int32, row s = counts published by rank s.
// Outputs (local): base[E]   first row of MY tokens for expert e inside the owner's buffer
//                  splits[L] padded row count of each local expert, splits[L] = total rows
//                  seg[L][ep+1] start row of each source's segment inside my buffer (+ end)
__global__ void ep_counts_kernel(EpCountsArgs a) {
  const int E = a.ep * a.L;
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  // publish my counts to every peer (including myself)
  for (int i = threadIdx.x; i < a.ep * E; i += blockDim.x) {
    const int r = i / E, e = i % E;
    a.counts_all[r][a.rank * E + e] = a.my_counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.ep) st_release_sys(a.flags[threadIdx.x] + a.rank, a.epoch);
  // wait for every source's table
  if (threadIdx.x < a.ep) {
    if (!wait_flag_ge(a.flags[a.rank] + threadIdx.x, a.epoch)) {
      atomicCAS(a.status, 0, kTimeoutPeerFlag);
      ok = 0;
    }
  }
  __syncthreads();
  if (!ok) return;
  const volatile int32_t* tab = a.counts_all[a.rank];
  if (threadIdx.x == 0) {
    // my own buffer layout
    int row = 0;
    for (int el = 0; el < a.L; ++el) {
      const int e = a.rank * a.L + el;
      int tot = 0;
      for (int s = 0; s < a.ep; ++s) {
        a.seg[el * (a.ep + 1) + s] = row + tot;
        tot += tab[s * E + e];
      }
      a.seg[el * (a.ep + 1) + a.ep] = row + tot;
      const int padded = (tot + a.align - 1) / a.align * a.align;
      a.splits[el] = padded;
      row += padded;
    }
    a.splits[a.L] = row;
  }
  // where my rows start inside every owner's buffer
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int r = e / a.L, el = e % a.L;
    int row = 0;
    for (int el2 = 0; el2 < el; ++el2) {
      int tot = 0;
      for (int s = 0; s < a.ep; ++s) tot += tab[s * E + r * a.L + el2];
      row += (tot + a.align - 1) / a.align * a.align;
    }
    for (int s = 0; s < a.rank; ++s) row += tab[s * E + e];
    a.base[e] = row;
  }
}

// ---- push ------------------------------------------------------------------------------------------
// CTAs stride over the (token, expert) pairs; a pair with within[t][e] >= 0 is one row copy
__global__ void ep_push_kernel(EpPushArgs a) {
  const int E = a.ep * a.L;
  const long long npairs = static_cast<long long>(a.T) * E;
  for (long long pair = blockIdx.x; pair < npairs; pair += gridDim.x) {
    const int t = static_cast<int>(pair / E), e = static_cast<int>(pair % E);
    const int w = a.within[pair];
    if (w < 0) {
      if (threadIdx.x == 0) a.rowmap[pair] = -1;
      continue;
    }
    const int r = e / a.L;
    const int row = a.base[e] + w;
    if (threadIdx.x == 0) a.rowmap[pair] = row;
    if (row >= a.cap_rows) {
      if (threadIdx.x == 0) atomicCAS(a.status, 0, kBadArgument);  // destination buffer too small for this routing
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(a.x) + static_cast<size_t>(t) * a.vec_per_row;
    uint4* dst = reinterpret_cast<uint4*>(a.dst[r]) + static_cast<size_t>(row) * a.vec_per_row;
    if (a.scale == nullptr) {
      for (int i = threadIdx.x; i < a.vec_per_row; i += blockDim.x) dst[i] = src[i];
    } else {
      const float sc = a.scale[pair];
      for (int i = threadIdx.x; i < a.vec_per_row; i += blockDim.x) {
        uint4 v = src[i];
        uint32_t* w32 = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (a.is_bf16) {
            const float lo = __uint_as_float(w32[k] << 16) * sc, hi = __uint_as_float(w32[k] & 0xffff0000u) * sc;
            w32[k] = pack_bf16x2(lo, hi);
          } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&w32[k]);
            w32[k] = pack_f16x2(__low2float(h) * sc, __high2float(h) * sc);
          }
        }
        dst[i] = v;
      }
    }
    if (a.probs != nullptr && threadIdx.x == 0) a.dst_probs[r][row] = a.probs[pair];
  }
  // completion: the last CTA tells every peer that this rank's rows have landed
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(a.cta_counter, 1u);
    if (done == gridDim.x - 1) {
      *a.cta_counter = 0;
      __threadfence_system();
      for (int r = 0; r < a.ep; ++r) st_release_sys(a.flags[r] + a.rank, a.epoch);
    }
  }
}

// ---- wait / signal ------------------------------------------------------------------------------------
__global__ void ep_wait_kernel(const uint32_t* flags, int n, uint32_t epoch, int* status, long long limit) {
  if (threadIdx.x < n && !wait_flag_ge(flags + threadIdx.x, epoch, limit)) atomicCAS(status, 0, kTimeoutPeerFlag);
}
__global__ void ep_signal_kernel(EpSignalArgs a) {
  __threadfence_system();
  if (threadIdx.x < a.ep) st_release_sys(a.flags[threadIdx.x] + a.rank, a.epoch);
}

// ---- pull ------------------------------------------------------------------------------------------
// one CTA per token: out[t] = sum_e w[t,e] * src[owner(e)][rowmap[t,e]];  dots[t,e] = <g[t], row>
template <bool BF>
__global__ void ep_pull_kernel(EpPullArgs a) {
  const int E = a.ep * a.L;
  const int t = blockIdx.x;
  extern __shared__ float red[];
  for (int i = threadIdx.x; i < a.vec_per_row; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int e = 0; e < E; ++e) {
      const int row = a.rowmap[static_cast<size_t>(t) * E + e];
      if (row < 0) continue;
      const float wk = a.w != nullptr ? a.w[static_cast<size_t>(t) * E + e] : 1.f;
      const uint4 v = reinterpret_cast<const uint4*>(a.src[e / a.L])[static_cast<size_t>(row) * a.vec_per_row + i];
      const uint32_t* w32 = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float lo, hi;
        if (BF) {
          lo = __uint_as_float(w32[k] << 16);
          hi = __uint_as_float(w32[k] & 0xffff0000u);
        } else {
          const __half2 h = *reinterpret_cast<const __half2*>(&w32[k]);
          lo = __low2float(h);
          hi = __high2float(h);
        }
        acc[2 * k] += wk * lo;
        acc[2 * k + 1] += wk * hi;
      }
    }
    uint4 o;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) o32[k] = BF ? pack_bf16x2(acc[2 * k], acc[2 * k + 1]) : pack_f16x2(acc[2 * k], acc[2 * k + 1]);
    reinterpret_cast<uint4*>(a.out)[static_cast<size_t>(t) * a.vec_per_row + i] = o;
  }
  if (a.out_s != nullptr && threadIdx.x < E) {
    const int row = a.rowmap[static_cast<size_t>(t) * E + threadIdx.x];
    a.out_s[static_cast<size_t>(t) * E + threadIdx.x] = row >= 0 ? a.src_s[threadIdx.x / a.L][row] : 0.f;
  }
  if (a.dots == nullptr) return;
  // per-pair dot products with g[t] (gradient of the routing weights)
  for (int e = 0; e < E; ++e) {
    const int row = a.rowmap[static_cast<size_t>(t) * E + e];
    float part = 0.f;
    if (row >= 0) {
      for (int i = threadIdx.x; i < a.vec_per_row; i += blockDim.x) {
        const uint4 v = reinterpret_cast<const uint4*>(a.src[e / a.L])[static_cast<size_t>(row) * a.vec_per_row + i];
        const uint4 g = reinterpret_cast<const uint4*>(a.g)[static_cast<size_t>(t) * a.vec_per_row + i];
        const uint32_t* v32 = reinterpret_cast<const uint32_t*>(&v);
        const uint32_t* g32 = reinterpret_cast<const uint32_t*>(&g);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (BF) {
            part += __uint_as_float(v32[k] << 16) * __uint_as_float(g32[k] << 16) +
                    __uint_as_float(v32[k] & 0xffff0000u) * __uint_as_float(g32[k] & 0xffff0000u);
          } else {
            const __half2 hv = *reinterpret_cast<const __half2*>(&v32[k]);
            const __half2 hg = *reinterpret_cast<const __half2*>(&g32[k]);
            part += __low2float(hv) * __low2float(hg) + __high2float(hv) * __high2float(hg);
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int wi = 0; wi < (blockDim.x >> 5); ++wi) tot += red[wi];
      a.dots[static_cast<size_t>(t) * E + e] = row >= 0 ? tot : 0.f;
    }
    __syncthreads();
  }
}

}  // namespace

cudaError_t ep_counts(const EpCountsArgs& a, cudaStream_t s) {
  if (a.ep > kCommMaxRanks || a.ep * a.L > 1024) return cudaErrorInvalidValue;
  ep_counts_kernel<<<1, 256, 0, s>>>(a);
  return cudaGetLastError();
}
cudaError_t ep_push(const EpPushArgs& a, cudaStream_t s) {
  const long long pairs = static_cast<long long>(a.T) * a.ep * a.L;
  if (pairs == 0) {
    // nothing to send: still raise the flags so that peers do not wait
    EpSignalArgs sg;
    for (int r = 0; r < a.ep; ++r) sg.flags[r] = a.flags[r];
    sg.ep = a.ep; sg.rank = a.rank; sg.epoch = a.epoch;
    ep_signal_kernel<<<1, 32, 0, s>>>(sg);
    return cudaGetLastError();
  }
  // a few CTAs per SM: every CTA ends with one system-scope fence and one atomic on the completion counter
  const long long want = 148LL * 16;
  ep_push_kernel<<<static_cast<unsigned>(pairs < want ? pairs : want), 256, 0, s>>>(a);
  return cudaGetLastError();
}
cudaError_t ep_wait(const uint32_t* flags, int n, uint32_t epoch, int* status, cudaStream_t s, long long limit_cycles) {
  ep_wait_kernel<<<1, 32, 0, s>>>(flags, n, epoch, status, limit_cycles > 0 ? limit_cycles : kWaitCycles);
  return cudaGetLastError();
}
cudaError_t ep_signal(const EpSignalArgs& a, cudaStream_t s) {
  ep_signal_kernel<<<1, 32, 0, s>>>(a);
  return cudaGetLastError();
}
cudaError_t ep_pull(const EpPullArgs& a, cudaStream_t s) {
  if (a.T == 0) return cudaSuccess;
  if (a.is_bf16) ep_pull_kernel<true><<<a.T, 256, 8 * sizeof(float), s>>>(a);
  else ep_pull_kernel<false><<<a.T, 256, 8 * sizeof(float), s>>>(a);
  return cudaGetLastError();
}

}  // namespace teb200
