// Elementwise dropout host API.
#pragma once
#include <cuda_runtime.h>
namespace z2h {
// out[i] = (keep(i) ? x[i] * scale : 0) + (residual ? residual[i] : 0) over n contiguous bf16
// elements (n a multiple of 8, pointers 16-byte aligned, out may alias x). The mask depends on
// (*seed_ptr, site, i) only; see csrc/common/dropout.cuh.
int dropout_apply(const void* x, const void* residual, void* out, long long n, float p,
                  const unsigned long long* seed_ptr, unsigned int site, cudaStream_t stream);
}  // namespace z2h
