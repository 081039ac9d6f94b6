// Softmax cross-entropy over bf16 logits, fused with its own backward.
//
// One CTA per row. Pass 1 streams the row once (16-byte loads) keeping a running
// (max, sum-exp) per thread, folds them across the CTA, and writes the row loss
// lse - logit[target]. Pass 2 re-reads the row, which is still in L2, and overwrites it in
// place with dlogits = (softmax - onehot) * grad_scale, so the lm_head data- and
// weight-gradient GEMMs can consume the same buffer. Columns >= V_real (vocabulary padding)
// never enter the softmax and get a zero gradient.
//
// Semantics: F.cross_entropy(logits.view(B*T, V), Y.view(B*T)) as in nn/gpt2/modules.py:115-117
// (mean over rows is applied through grad_scale and by the caller for the loss); the fused
// backward is the identity derived by hand in nn/makemore/3_1_backprop.py:222-231.
#include "../common/ptx.cuh"
#include "ce.h"

namespace z2h {
namespace {

constexpr int kThreads = 512;

__device__ __forceinline__ void online_add(float& m, float& s, float x) {
  if (x > m) {
    s = s * __expf(m - x) + 1.f;
    m = x;
  } else {
    s += __expf(x - m);
  }
}

template <typename IdxT>
__global__ void __launch_bounds__(kThreads)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const IdxT* __restrict__ targets,
                  float* __restrict__ losses, int V_real, int V_pad, long long ld, float grad_scale,
                  int write_grad, int ignore_index) {
  __shared__ float sm[kThreads / 32], ss[kThreads / 32];
  __shared__ float row_max, row_lse;
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (long long)row * ld;
  const int nvec = V_pad / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kThreads) {
    uint4 u = *reinterpret_cast<const uint4*>(lr + i * 8);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(w[j]);
      const int c = i * 8 + j * 2;
      if (c < V_real) online_add(m, s, f.x);
      if (c + 1 < V_real) online_add(m, s, f.y);
    }
  }
  for (int c = nvec * 8 + threadIdx.x; c < V_real; c += kThreads)
    online_add(m, s, __bfloat162float(lr[c]));
  // fold (m, s) pairs: warp, then CTA
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
    m = mn;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sm[warp] = m;
    ss[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < kThreads / 32 ? sm[lane] : -INFINITY;
    s = lane < kThreads / 32 ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      float mn = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
      m = mn;
    }
    if (lane == 0) {
      row_max = m;
      row_lse = m + __logf(s);
    }
  }
  __syncthreads();
  const float lse = row_lse;
  long long tgt = (long long)targets[row];
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V_real;
  if (threadIdx.x == 0 && losses != nullptr)
    losses[row] = ignored ? 0.f : lse - __bfloat162float(lr[tgt]);
  if (!write_grad) return;
  const float gs = ignored ? 0.f : grad_scale;
  for (int i = threadIdx.x; i < nvec; i += kThreads) {
    uint4 u = *reinterpret_cast<const uint4*>(lr + i * 8);
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(w[j]);
      const int c = i * 8 + j * 2;
      float g0 = c < V_real ? (__expf(f.x - lse) - (c == tgt ? 1.f : 0.f)) * gs : 0.f;
      float g1 = c + 1 < V_real ? (__expf(f.y - lse) - (c + 1 == tgt ? 1.f : 0.f)) * gs : 0.f;
      w[j] = pack_bf16x2(g0, g1);
    }
    *reinterpret_cast<uint4*>(lr + i * 8) = u;
  }
  for (int c = nvec * 8 + threadIdx.x; c < V_pad; c += kThreads) {
    float g = c < V_real ? (__expf(__bfloat162float(lr[c]) - lse) - (c == tgt ? 1.f : 0.f)) * gs : 0.f;
    lr[c] = __float2bfloat16(g);
  }
}

// Sum of n floats into *out (scaled); single CTA, fixed order.
__global__ void reduce_sum_kernel(const float* __restrict__ x, int n, float scale, float* out,
                                  int accumulate) {
  __shared__ float sh[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) *out = accumulate ? *out + s * scale : s * scale;
  }
}

}  // namespace

int ce_fwd_bwd(void* logits, const void* targets, int idx_is_64, float* losses, int M, int V_real,
               int V_pad, long long ld, float grad_scale, int write_grad, int ignore_index,
               cudaStream_t stream) {
  if (M <= 0) return 0;
  if (ld % 8 != 0 || (reinterpret_cast<uintptr_t>(logits) & 15)) return 1;
  if (idx_is_64)
    ce_fwd_bwd_kernel<long long><<<M, kThreads, 0, stream>>>((__nv_bfloat16*)logits,
                                                            (const long long*)targets, losses, V_real,
                                                            V_pad, ld, grad_scale, write_grad,
                                                            ignore_index);
  else
    ce_fwd_bwd_kernel<int><<<M, kThreads, 0, stream>>>((__nv_bfloat16*)logits, (const int*)targets,
                                                      losses, V_real, V_pad, ld, grad_scale,
                                                      write_grad, ignore_index);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int reduce_sum(const float* x, int n, float scale, float* out, int accumulate, cudaStream_t stream) {
  reduce_sum_kernel<<<1, 1024, 0, stream>>>(x, n, scale, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace z2h

extern "C" {
int z2h_ce_fwd_bwd(void* logits, const void* targets, int idx_is_64, float* losses, int M, int V_real,
                   int V_pad, long long ld, float grad_scale, int write_grad, int ignore_index,
                   void* stream) {
  return z2h::ce_fwd_bwd(logits, targets, idx_is_64, losses, M, V_real, V_pad, ld, grad_scale,
                         write_grad, ignore_index, (cudaStream_t)stream);
}
int z2h_reduce_sum(const float* x, int n, float scale, float* out, int accumulate, void* stream) {
  return z2h::reduce_sum(x, n, scale, out, accumulate, (cudaStream_t)stream);
}
}
