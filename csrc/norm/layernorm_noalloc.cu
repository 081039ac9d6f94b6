// Allocation-free LayerNorm backward: the two-stage weight/bias-gradient reduction of
// layernorm.cu, with its partial rows kept in a fixed array that is part of the library image
// instead of a buffer the caller provides. See norm_noalloc.h for who needs this and for the
// rules of use (capacity, first call before stream capture, no overlapping calls).
#include "norm_noalloc.h"

#include <cstdio>
#include <mutex>

#include "norm.h"

namespace z2h {
namespace {

// The scratch area itself. In host code this name is only a handle for the runtime, not a
// device address: the address the kernels need comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_ln_bwd_scratch[kLayerNormNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch area on the current device (looked up once per device).
int scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 5;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_ln_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "z2h_layernorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return 5;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

int layernorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean,
                          const float* rstd, const void* dresid, void* dx, float* dw, float* db,
                          int M, int C, int accumulate, cudaStream_t stream) {
  if (M < 0 || C <= 0 || C % 8 != 0) return 1;
  const long long need = (long long)layernorm_bwd_num_partials(M) * 2 * C;
  // C beyond 2048 is refused whatever M is (a small M could still fit the area, but the kernels
  // underneath are not built for wider rows): the documented limit holds for every call
  if (C > kLayerNormNoAllocMaxColumns || need > kLayerNormNoAllocScratchFloats) {
    fprintf(stderr,
            "z2h_layernorm_bwd_noalloc: M=%d C=%d needs %lld floats of scratch, the built-in area holds "
            "%lld (C up to 2048); use z2h_layernorm_bwd with a caller-provided buffer\n",
            M, C, need, kLayerNormNoAllocScratchFloats);
    return 4;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  return layernorm_bwd(dy, x, w, mean, rstd, dresid, dx, dw, db, scratch, M, C, accumulate, stream);
}

}  // namespace z2h

extern "C" {
int z2h_layernorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean,
                              const float* rstd, const void* dresid, void* dx, float* dw, float* db,
                              int M, int C, int accumulate, void* stream) {
  return z2h::layernorm_bwd_noalloc(dy, x, w, mean, rstd, dresid, dx, dw, db, M, C, accumulate,
                                    (cudaStream_t)stream);
}
long long z2h_layernorm_bwd_noalloc_capacity(void) { return z2h::kLayerNormNoAllocScratchFloats; }
}
