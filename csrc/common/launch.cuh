// Kernel launch helper with programmatic dependent launch.
//
// Every kernel of the training step starts with pdl_launch_dependents() and runs pdl_wait() before
// its first access to global memory. Launched through launch_kernel(..., /*pdl=*/true), the next
// kernel in the stream may then be scheduled onto SMs as the CTAs of the current one retire, run
// its prologue (barrier initialisation, tensor-memory allocation, descriptor prefetch) and park in
// pdl_wait() until the current kernel has completed and its memory is visible. Inside a captured
// CUDA graph the launches become programmatic dependency edges. What is gained is the launch
// latency and the prologue of every kernel at each of the ~310 boundaries of a micro-step.
// Measured on GPT-2 124M (B200, CUDA-graph replay, two runs each): 841.9 k / 840.0 k tokens/s with
// the attribute, 847.9 k / 848.5 k without: inside a graph the boundaries are already short and
// the early-resident CTAs of the next kernel cost more than they hide. The attribute is therefore
// off unless Z2H_PDL=1 is set in the environment; the kernels keep the two instructions, which
// are no-ops in plain stream order.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdlib>

namespace z2h {

// cudaFuncAttributeMaxDynamicSharedMemorySize (and the SM count) belong to a (kernel, device)
// pair, not to the process: a host program that drives several GPUs from one process must set
// them once per device. `seen` is a per-call-site bit mask of devices already configured; the
// function returns true exactly once per device (devices 64 and up are configured every time).
inline bool first_use_on_current_device(std::atomic<unsigned long long>& seen, int* device = nullptr) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (device != nullptr) *device = dev;
  if (dev < 0 || dev >= 64) return true;
  const unsigned long long bit = 1ull << dev;
  return (seen.fetch_or(bit) & bit) == 0;
}

// Number of SMs of the current device (cached per device).
inline int sm_count_current_device() {
  static std::atomic<int> cache[64];
  int dev = 0;
  cudaGetDevice(&dev);
  const bool cached = dev >= 0 && dev < 64;
  int n = cached ? cache[dev].load(std::memory_order_relaxed) : 0;
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (cached) cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("Z2H_PDL");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int n = 0;
  if (pdl && pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace z2h
