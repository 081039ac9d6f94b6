// Softmax cross-entropy over bf16 logits, fused with its own backward.
//
// One CTA per row. Rows of up to 112 KiB are copied into shared memory by one bulk copy
// (cp.async.bulk + mbarrier), the maximum, the sum of exponentials and the gradient are taken
// from there, and one bulk copy writes the row back: the row is read from memory exactly once,
// written once, and two CTAs per SM overlap one row's copies with the other's arithmetic. The row loss is
// lse - logit[target]; the row is overwritten in place with dlogits = (softmax - onehot) *
// grad_scale, so the lm_head data- and weight-gradient GEMMs can consume the same buffer.
// Columns >= V_real (vocabulary padding) never enter the softmax and get a zero gradient.
// Longer rows take a streaming kernel with a running (max, sum-exp) pair and a second read.
//
// Semantics: F.cross_entropy(logits.view(B*T, V), Y.view(B*T)) as in nn/gpt2/modules.py:115-117
// (mean over rows is applied through grad_scale and by the caller for the loss); the fused
// backward is the identity derived by hand in nn/makemore/3_1_backprop.py:222-231.
#include "../common/launch.cuh"
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

constexpr int kRowThreads = 1024;
constexpr int kRowMaxBytes = 112 * 1024;  // two CTAs of this size share an SM
constexpr float kLog2e = 1.4426950408889634f;

// blockDim.x == kRowThreads; returns the maximum (IS_MAX) or the sum of v over the CTA
template <bool IS_MAX>
__device__ __forceinline__ float cta_reduce(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, t) : v + t;
  }
  __syncthreads();  // sh may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  v = (threadIdx.x & 31) < kRowThreads / 32 ? sh[threadIdx.x & 31] : (IS_MAX ? -INFINITY : 0.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, t) : v + t;
  }
  return v;
}

// One CTA per row, the row held in shared memory: one bulk copy brings it in, three passes over
// shared memory take the maximum, the sum of exponentials and the gradient (written in place),
// one bulk copy writes it back. Two CTAs fit on an SM, so one row's copies overlap the other
// row's arithmetic and ~200 KB per SM are in flight.
template <typename IdxT>
__global__ void __launch_bounds__(kRowThreads)
ce_row_in_smem_kernel(__nv_bfloat16* __restrict__ logits, const IdxT* __restrict__ targets,
                      float* __restrict__ losses, int V_real, int V_pad, long long ld, float grad_scale,
                      int write_grad, int ignore_index, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float sh[32];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (long long)row * ld;
  const uint32_t row_bytes = (uint32_t)V_pad * 2;  // a multiple of 16
  const int nvec = V_pad / 8;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
    mbar_arrive_expect_tx(&bar, row_bytes);
    bulk_load_1d(smem, lr, row_bytes, &bar);
  }
  __syncthreads();
  const long long tgt = (long long)targets[row];
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V_real;
  if (!mbar_wait_bounded(&bar, 0, &abort_flag, status, kTimeoutFull)) return;
  const uint4* sv = reinterpret_cast<const uint4*>(smem);
  const int vlast = V_real / 8;  // first vector that may contain padding columns
  // ---- maximum (padding columns are skipped)
  float m = -INFINITY;
  for (int v = threadIdx.x; v < nvec; v += kRowThreads) {
    const uint4 u = sv[v];
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
    if (v < vlast) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        m = max3(m, f.x, f.y);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        const int c = v * 8 + 2 * j;
        if (c < V_real) m = fmaxf(m, f.x);
        if (c + 1 < V_real) m = fmaxf(m, f.y);
      }
    }
  }
  m = cta_reduce<true>(m, sh);
  const float m2 = m * kLog2e;
  // The target logit is needed for the loss and the row is about to be overwritten in place.
  const float tgt_logit =
      ignored ? 0.f : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(smem)[tgt]);
  __syncthreads();
  // ---- sum of exponentials; e = exp(x - max) replaces x in shared memory as bf16, so that the
  // gradient pass needs no second exponential (its result is rounded to bf16 anyway)
  float s = 0.f;
  uint4* sw = reinterpret_cast<uint4*>(smem);
  for (int v = threadIdx.x; v < nvec; v += kRowThreads) {
    uint4 u = sw[v];
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      float e0 = ex2_fast(fmaf(f.x, kLog2e, -m2)), e1 = ex2_fast(fmaf(f.y, kLog2e, -m2));
      if (v >= vlast) {
        const int c = v * 8 + 2 * j;
        if (c >= V_real) e0 = 0.f;
        if (c + 1 >= V_real) e1 = 0.f;
      }
      s += e0 + e1;
      w[j] = pack_bf16x2(e0, e1);
    }
    if (write_grad) sw[v] = u;
  }
  s = cta_reduce<false>(s, sh);
  const float lse = m + __logf(s);
  if (threadIdx.x == 0 && losses != nullptr) losses[row] = ignored ? 0.f : lse - tgt_logit;
  if (!write_grad) return;
  // ---- gradient, in place: e * (grad_scale / sum) - onehot * grad_scale
  // (cta_reduce ended with a barrier after every thread's writes above)
  const float gs = ignored ? 0.f : grad_scale;
  const float k = gs / s;
  const int vt = ignored ? -1 : (int)(tgt >> 3), jt = (int)(tgt & 7);
  for (int v = threadIdx.x; v < nvec; v += kRowThreads) {
    uint4 u = sw[v];
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
    float g[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 e = unpack_bf16x2(w[j]);
      g[2 * j] = e.x * k;
      g[2 * j + 1] = e.y * k;
    }
    if (v == vt) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j == jt) g[j] -= gs;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = pack_bf16x2(g[2 * j], g[2 * j + 1]);
    sw[v] = u;
  }
  fence_proxy_async();  // make the generic-proxy writes visible to the bulk copy
  __syncthreads();
  if (threadIdx.x == 0) {
    bulk_store_1d(lr, smem, row_bytes);
    tma_store_commit();
    tma_store_wait_read<0>();  // shared memory must stay alive until the copy has read it
  }
}

template <typename IdxT>
__global__ void __launch_bounds__(kThreads)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const IdxT* __restrict__ targets,
                  float* __restrict__ losses, int V_real, int V_pad, long long ld, float grad_scale,
                  int write_grad, int ignore_index) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sm[kThreads / 32], ss[kThreads / 32];
  __shared__ float row_max, row_lse;
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (long long)row * ld;
  const int nvec = V_pad / 8;
  const long long tgt = (long long)targets[row];
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V_real;
  // taken now: the row is overwritten in place further down
  const float tgt_logit = (threadIdx.x == 0 && !ignored) ? __bfloat162float(lr[tgt]) : 0.f;
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
  if (threadIdx.x == 0 && losses != nullptr) losses[row] = ignored ? 0.f : lse - tgt_logit;
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
  pdl_launch_dependents();
  pdl_wait();
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
  // rows that fit in shared memory twice per SM (the usual case: GPT-2's 50,304 columns are 98 KiB)
  const size_t row_bytes = (size_t)V_pad * 2;
  if (V_pad % 8 == 0 && row_bytes <= (size_t)kRowMaxBytes) {
    static std::atomic<unsigned long long> attr_seen{0};
    if (first_use_on_current_device(attr_seen)) {
      cudaFuncSetAttribute(ce_row_in_smem_kernel<long long>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kRowMaxBytes);
      cudaFuncSetAttribute(ce_row_in_smem_kernel<int>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kRowMaxBytes);
    }
    if (idx_is_64)
      launch_kernel(ce_row_in_smem_kernel<long long>, dim3(M), dim3(kRowThreads), row_bytes, stream, true, 
          (__nv_bfloat16*)logits, (const long long*)targets, losses, V_real, V_pad, ld, grad_scale,
          write_grad, ignore_index, nullptr);
    else
      launch_kernel(ce_row_in_smem_kernel<int>, dim3(M), dim3(kRowThreads), row_bytes, stream, true, 
          (__nv_bfloat16*)logits, (const int*)targets, losses, V_real, V_pad, ld, grad_scale, write_grad,
          ignore_index, nullptr);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
  }
  if (idx_is_64)
    launch_kernel(ce_fwd_bwd_kernel<long long>, dim3(M), dim3(kThreads), 0, stream, true, (__nv_bfloat16*)logits,
                                                            (const long long*)targets, losses, V_real,
                                                            V_pad, ld, grad_scale, write_grad,
                                                            ignore_index);
  else
    launch_kernel(ce_fwd_bwd_kernel<int>, dim3(M), dim3(kThreads), 0, stream, true, (__nv_bfloat16*)logits, (const int*)targets,
                                                      losses, V_real, V_pad, ld, grad_scale,
                                                      write_grad, ignore_index);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int reduce_sum(const float* x, int n, float scale, float* out, int accumulate, cudaStream_t stream) {
  launch_kernel(reduce_sum_kernel, dim3(1), dim3(1024), 0, stream, true, x, n, scale, out, accumulate);
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
