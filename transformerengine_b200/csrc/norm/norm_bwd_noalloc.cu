// Allocation-free norm backward: the two-stage weight-gradient reduction of
// norm_bwd() runs with its scratch in a file-scope device array instead of a
// caller- or framework-allocated buffer.  See teb200/noalloc.h for who needs this
// and for the rules of use.
#include <teb200/noalloc.h>
#include <teb200/norm.h>

#include <cstdio>
#include <mutex>

namespace {

// Lives in the library image on every GPU that loads it, until process exit.
static __device__ __align__(256) float g_noalloc_scratch[TEB200_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_mutex;

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device
// address: the address has to be asked for, once per device, with that device current.
cudaError_t scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" long long teb200_norm_bwd_noalloc_scratch_floats(int R, int C) {
  return static_cast<long long>(teb200::norm_bwd_parts(R)) * 2LL * C;
}

extern "C" int teb200_norm_bwd_noalloc(int layernorm, int R, int C, int x_dtype, int w_dtype, int zero_centered_gamma,
                                       const void* dy, const void* x, const float* mu, const float* rsigma,
                                       const void* gamma, const void* add, void* dx, void* dgamma, void* dbeta,
                                       cudaStream_t stream) {
  if (R <= 0 || C <= 0) return static_cast<int>(cudaSuccess);
  const long long need = teb200_norm_bwd_noalloc_scratch_floats(R, C);
  if (need > static_cast<long long>(TEB200_NOALLOC_SCRATCH_FLOATS)) {
    std::fprintf(stderr,
                 "teb200_norm_bwd_noalloc: problem [%d x %d] needs %lld scratch floats, the built-in array holds %d; "
                 "use the allocating entry point for this size\n",
                 R, C, need, TEB200_NOALLOC_SCRATCH_FLOATS);
    return static_cast<int>(cudaErrorInvalidValue);
  }
  float* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return static_cast<int>(e);
  teb200::NormArgs a;
  a.layernorm = layernorm;
  a.R = R;
  a.C = C;
  a.x_dtype = x_dtype;
  a.w_dtype = w_dtype;
  a.zero_centered = zero_centered_gamma;
  a.x = x;
  a.dy = dy;
  a.mu = const_cast<float*>(mu);
  a.rs = const_cast<float*>(rsigma);
  a.gamma = gamma;
  a.add = add;
  a.dx = dx;
  a.dgamma = dgamma;
  a.dbeta = dbeta;
  a.workspace = scratch;  // every word read by the finalize stage is written by the first stage of this call
  return static_cast<int>(teb200::norm_bwd(a, stream));
}
