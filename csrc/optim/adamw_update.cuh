// The per-element AdamW update shared by the single-GPU optimizer kernel and the fused
// reduce-scatter + AdamW + all-gather kernel.
#pragma once
#include "optim.h"

namespace z2h {

struct AdamConsts {
  float lr, beta1, beta2, eps, wd, step_size, inv_sqrt_bc2, gscale;
};

__device__ __forceinline__ AdamConsts load_adam_consts(const float* hyper, float gscale) {
  AdamConsts k;
  k.lr = hyper[kHyLr];
  k.beta1 = hyper[kHyBeta1];
  k.beta2 = hyper[kHyBeta2];
  k.eps = hyper[kHyEps];
  k.wd = hyper[kHyWeightDecay];
  k.step_size = k.lr / hyper[kHyBiasCorr1];
  k.inv_sqrt_bc2 = rsqrtf(hyper[kHyBiasCorr2]);
  k.gscale = gscale;
  return k;
}

// torch.optim.AdamW order: decay the parameter, update the moments, then take the step with
// denom = sqrt(v) / sqrt(1 - beta2^t) + eps and step size lr / (1 - beta1^t).
__device__ __forceinline__ void adamw_update(float& p, float& m, float& v, float g_raw,
                                             const AdamConsts& k, bool decay) {
  const float g = g_raw * k.gscale;
  if (decay) p *= (1.f - k.lr * k.wd);
  m = k.beta1 * m + (1.f - k.beta1) * g;
  v = k.beta2 * v + (1.f - k.beta2) * g * g;
  const float denom = sqrtf(v) * k.inv_sqrt_bc2 + k.eps;
  p -= k.step_size * (m / denom);
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float s, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) t += sh[w];
  return t;
}

}  // namespace z2h
