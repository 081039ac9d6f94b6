// Flash attention host API (causal, head_dim 64, bf16; qkv packed as [B*T, 3*H*64]).
#pragma once
#include <cuda_runtime.h>
namespace z2h {
// out: bf16 [B*T, H*64]; lse: fp32 [B, H, T] (natural log of the scaled-score partition sum).
int flash_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int* status,
              cudaStream_t stream);
// dqkv: bf16 [B*T, 3*H*64]; dq_accum: fp32 scratch [B*T, H*64];
// stats: fp32 scratch of 2 * B * H * roundup(T, 128) elements.
int flash_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
              float* dq_accum, float* stats, int B, int T, int H, int* status, cudaStream_t stream);
}  // namespace z2h
