// Flash attention host API (causal, head_dim 64, bf16; qkv packed as [B*T, 3*H*64]).
#pragma once
#include <cuda_runtime.h>
namespace z2h {
// out: bf16 [B*T, H*64]; lse: fp32 [B, H, T] (natural log of the scaled-score partition sum).
int flash_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int* status,
              cudaStream_t stream);
// dqkv: bf16 [B*T, 3*H*64]; dq_accum: fp32 scratch of roundup(B*T, 32) * H*64 elements (the kernels
// keep dQ there in a blocked layout, see flash_bwd.cu);
// stats: fp32 scratch of 2 * B * H * roundup(T, 128) elements.
int flash_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
              float* dq_accum, float* stats, int B, int T, int H, int* status, cudaStream_t stream);
// The same with attention-probability dropout (nn/gpt2/modules.py:36 of the reference passes
// dropout_p to SDPA). drop_p in [0, 1) is quantised to 1/256; the mask is a function of
// (*seed_ptr, site, b, h, q, k) (csrc/common/dropout.cuh), so forward and backward agree when
// they are given the same seed and site. drop_p == 0 runs the plain kernels.
int flash_fwd_dropout(const void* qkv, void* out, float* lse, int B, int T, int H, float drop_p,
                      const unsigned long long* seed_ptr, unsigned int site, int* status,
                      cudaStream_t stream);
int flash_bwd_dropout(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                      float* dq_accum, float* stats, int B, int T, int H, float drop_p,
                      const unsigned long long* seed_ptr, unsigned int site, int* status,
                      cudaStream_t stream);
// The same again (drop_p may be 0, seed_ptr then unused) with a by-product: dbias, fp32 [3*H*64] or
// null, receives += the column sums of dqkv as stored, which is the gradient of the bias of the
// projection that produced qkv (nn/gpt2/modules.py:19 of the reference: c_attn has a bias).
int flash_bwd_dbias(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                    float* dq_accum, float* stats, int B, int T, int H, float drop_p,
                    const unsigned long long* seed_ptr, unsigned int site, float* dbias, int* status,
                    cudaStream_t stream);
// ordered != 0: the KV tiles are launched one after the other so that the fp32 dQ accumulation happens
// in a fixed order (bitwise reproducible results; dbias must be null).
int flash_bwd_ex(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                 float* dq_accum, float* stats, int B, int T, int H, float drop_p,
                 const unsigned long long* seed_ptr, unsigned int site, float* dbias, int ordered, int* status,
                 cudaStream_t stream);
}  // namespace z2h
