// Embedding host API: bf16 tables / activations, fp32 gradients (accumulated into).
#pragma once
#include <cuda_runtime.h>
namespace z2h {
int embed_fwd(const void* idx, int idx_is_64, const void* wte, const void* wpe, void* out, int M,
              int T, int C, int V, int* status, cudaStream_t stream);
// ordered != 0: the token-embedding gradient is summed in ascending position by one writer per
// vocabulary row (bitwise reproducible; slower).
int embed_bwd_ordered(const void* idx, int idx_is_64, const void* dx, float* dwte, float* dwpe, int B, int T,
                      int C, int V, int ordered, cudaStream_t stream);
int embed_bwd(const void* idx, int idx_is_64, const void* dx, float* dwte, float* dwpe, int B, int T,
              int C, int V, cudaStream_t stream);
}  // namespace z2h
