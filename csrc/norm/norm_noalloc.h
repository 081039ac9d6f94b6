// LayerNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for host programs that use
// this library without an allocator at hand: a plain C/C++ application that links libz2h.so
// without PyTorch, or a long-running server that has already handed all device memory to its
// own pools and forbids any further cudaMalloc (there an allocation can fail outright, or
// synchronise the whole device in the middle of serving). The regular entry point
// (z2h_layernorm_bwd) asks the caller for a scratch buffer; this one brings its own.
#pragma once
#include <cuda_runtime.h>

namespace z2h {

// Capacity of the built-in scratch area, in floats: 296 partial rows x 2 (dw, db) x 2048
// columns = 1,212,416 floats (about 4.6 MiB). Every GPU whose context loads the library
// holds this much until the process exits, whether or not the function is ever called.
constexpr long long kLayerNormNoAllocScratchFloats = 296LL * 2 * 2048;
// Widest row accepted; wider problems get return code 4 whatever their row count.
constexpr int kLayerNormNoAllocMaxColumns = 2048;

// Same computation and arguments as layernorm_bwd() minus the scratch pointer.
// Returns 0 on success, 1 for a bad argument, 3 if a launch failed, 4 if the problem needs more
// scratch than the built-in area holds (C > 2048), 5 if the address of the scratch area could
// not be obtained on the current device. Nothing is allocated or freed, by this function or by
// anything it calls.
//
// Set-up: the first call on each device looks up the device address of the scratch area
// (cudaGetSymbolAddress, with that device current) and caches it; make that first call before
// any stream capture begins on that device.
// Sharing: all calls on a device use the same scratch area. Calls that may overlap on the GPU
// (different streams without ordering between them) race on it; order them on one stream or
// with events. The area keeps the previous call's contents, which is harmless here: every
// partial row the second kernel reads is written by the first kernel of the same call, so
// nothing has to start at zero.
int layernorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean,
                          const float* rstd, const void* dresid, void* dx, float* dw, float* db,
                          int M, int C, int accumulate, cudaStream_t stream);

}  // namespace z2h

extern "C" {
// C ABI of the above (stream is a cudaStream_t).
int z2h_layernorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean,
                              const float* rstd, const void* dresid, void* dx, float* dw, float* db,
                              int M, int C, int accumulate, void* stream);
// Capacity of the built-in scratch area in floats.
long long z2h_layernorm_bwd_noalloc_capacity(void);
}
