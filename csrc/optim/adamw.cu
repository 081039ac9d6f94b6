// Global grad-norm clipping + AdamW as two passes over flat fp32 buffers (single-GPU path;
// the multi-GPU path in comm/ar_adamw.cu reuses adamw_update()).
//
// Replaces torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW(fused=True) of the reference
// trainers (nn/gpt2/train.py:73-84,126-127, nn/gpt2/train_ddp.py:92-103,142-143): the update
// rule, the eps placement and the decoupled weight decay match torch's AdamW.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "optim.h"
#include "../gemm/gemm.h"  // gemm_fold_slices: ordered sum of partial vectors
#include "adamw_update.cuh"

namespace z2h {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
gradnorm_partials_kernel(const float* __restrict__ g, long long n, float* __restrict__ partials) {
  __shared__ float sh[kThreads / 32];
  float s = 0.f;
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * kThreads) {
    float4 x = reinterpret_cast<const float4*>(g)[i];
    s += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * 4 + threadIdx.x; i < n; i += kThreads) s += g[i] * g[i];
  s = block_sum<kThreads>(s, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void __launch_bounds__(kThreads)
adamw_step_kernel(float* __restrict__ p32, float* __restrict__ g, float* __restrict__ m,
                  float* __restrict__ v, __nv_bfloat16* __restrict__ p16, long long n,
                  long long n_decay, const float* __restrict__ hyper,
                  const float* __restrict__ partials, int num_partials, float* norm_out,
                  int zero_grad) {
  __shared__ float sh[kThreads / 32];
  __shared__ float s_clip;
  float t = 0.f;
  for (int i = threadIdx.x; i < num_partials; i += kThreads) t += partials[i];
  t = block_sum<kThreads>(t, sh);
  if (threadIdx.x == 0) {
    const float gs = hyper[kHyGradScale];
    const float norm = sqrtf(t) * gs;
    const float max_norm = hyper[kHyMaxNorm];
    float clip = 1.f;
    if (max_norm > 0.f) clip = fminf(1.f, max_norm / (norm + 1e-6f));
    s_clip = clip * gs;
    if (blockIdx.x == 0 && norm_out != nullptr) *norm_out = norm;
  }
  __syncthreads();
  AdamConsts k = load_adam_consts(hyper, s_clip);
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * kThreads) {
    float4 gp = reinterpret_cast<float4*>(g)[i];
    float4 pp = reinterpret_cast<float4*>(p32)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const long long e = i * 4;
    adamw_update(pp.x, mm.x, vv.x, gp.x, k, e + 0 < n_decay);
    adamw_update(pp.y, mm.y, vv.y, gp.y, k, e + 1 < n_decay);
    adamw_update(pp.z, mm.z, vv.z, gp.z, k, e + 2 < n_decay);
    adamw_update(pp.w, mm.w, vv.w, gp.w, k, e + 3 < n_decay);
    reinterpret_cast<float4*>(p32)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p16 != nullptr) {
      uint2 o;
      o.x = pack_bf16x2(pp.x, pp.y);
      o.y = pack_bf16x2(pp.z, pp.w);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (blockIdx.x == 0) {
    for (long long e = nvec * 4 + threadIdx.x; e < n; e += kThreads) {
      float pp = p32[e], mm = m[e], vv = v[e];
      adamw_update(pp, mm, vv, g[e], k, e < n_decay);
      p32[e] = pp; m[e] = mm; v[e] = vv;
      if (p16 != nullptr) p16[e] = __float2bfloat16(pp);
      if (zero_grad) g[e] = 0.f;
    }
  }
}

// block = 32 column-vectors (256 columns) x 8 row lanes
__global__ void __launch_bounds__(256)
colsum_bf16_kernel(const __nv_bfloat16* __restrict__ dy, int M, int N, long long ld,
                   float* __restrict__ db, int rows_per_slab, int store_partials) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[8][256];
  const int cv = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c = blockIdx.x * 256 + cv * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const int r0 = blockIdx.y * rows_per_slab;
  const int r1 = min(M, r0 + rows_per_slab);
  if (c < N) {
    // four rows per trip: four independent 16-byte loads in flight per thread
    int r = r0 + rl;
    for (; r + 24 < r1; r += 32) {
      uint4 u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) u[k] = *reinterpret_cast<const uint4*>(dy + (long long)(r + 8 * k) * ld + c);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&u[k]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(w[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
    }
    for (; r < r1; r += 8) {
      uint4 u = *reinterpret_cast<const uint4*>(dy + (long long)r * ld + c);
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(w[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sh[rl][cv * 8 + j] = acc[j];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < N) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) s += sh[r][threadIdx.x];
    if (store_partials) db[(long long)blockIdx.y * N + col] = s;  // db is the [slabs][N] scratch here
    else atomicAdd(db + col, s);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                        long long n) {
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 x = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    o.x = pack_bf16x2(x.x, x.y);
    o.y = pack_bf16x2(x.z, x.w);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
  if (blockIdx.x == 0)
    for (long long e = nvec * 4 + threadIdx.x; e < n; e += blockDim.x) dst[e] = __float2bfloat16(src[e]);
}

int grid_for(long long nvec, int threads, int cap) {
  long long b = (nvec + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b < cap ? b : cap);
}

}  // namespace

int gradnorm_partials(const float* g, long long n, float* partials, cudaStream_t stream) {
  if (reinterpret_cast<uintptr_t>(g) & 15) return -1;
  const int grid = grid_for(n / 4, kThreads, kGradNormMaxPartials);
  gradnorm_partials_kernel<<<grid, kThreads, 0, stream>>>(g, n, partials);
  return cudaGetLastError() == cudaSuccess ? grid : -3;
}

int adamw_step(float* p32, float* g, float* m, float* v, void* p16, long long n, long long n_decay,
               const float* hyper, const float* partials, int num_partials, float* norm_out,
               int zero_grad, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(p32) | reinterpret_cast<uintptr_t>(g) |
       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15)
    return 1;
  if (p16 != nullptr && (reinterpret_cast<uintptr_t>(p16) & 7)) return 1;
  const int grid = grid_for(n / 4, kThreads, 148 * 8);
  adamw_step_kernel<<<grid, kThreads, 0, stream>>>(p32, g, m, v, (__nv_bfloat16*)p16, n, n_decay, hyper,
                                                  partials, num_partials, norm_out, zero_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int colsum_bf16(const void* dy, int M, int N, long long ld, float* db, int accumulate,
                cudaStream_t stream) {
  return colsum_bf16_ordered(dy, M, N, ld, db, accumulate, 0, nullptr, stream);
}

// ordered != 0: the result does not depend on the order in which CTAs finish. With a scratch buffer of
// colsum_scratch_elems(M, N) floats the row slabs store their partial sums there and a second kernel
// adds them to db in slab order; without one a single slab is used (every column summed by one CTA:
// N / 256 CTAs stream the whole matrix, slow).
long long colsum_scratch_elems(int M, int N) {
  int slabs = (M + 127) / 128;
  if (slabs > 128) slabs = 128;
  if (slabs < 1) slabs = 1;
  return (long long)slabs * N;
}

int colsum_bf16_ordered(const void* dy, int M, int N, long long ld, float* db, int accumulate, int ordered,
                        float* scratch, cudaStream_t stream) {
  if (N % 8 != 0 || ld % 8 != 0) return 1;
  if (!accumulate) cudaMemsetAsync(db, 0, sizeof(float) * N, stream);
  const bool two_stage = ordered && scratch != nullptr;
  int slabs = (ordered && !two_stage) ? 1 : (M + 127) / 128;
  if (slabs > 128) slabs = 128;
  if (slabs < 1) slabs = 1;
  if (two_stage) {
    const int rows = (M + slabs - 1) / slabs;
    dim3 g2((N + 255) / 256, slabs);
    launch_kernel(colsum_bf16_kernel, dim3(g2), dim3(256), 0, stream, true, (const __nv_bfloat16*)dy, M, N, ld, scratch,
                  rows, 1);
    return gemm_fold_slices(scratch, slabs, N, db, stream);
  }
  const int rows_per_slab = (M + slabs - 1) / slabs;
  dim3 grid((N + 255) / 256, slabs);
  launch_kernel(colsum_bf16_kernel, dim3(grid), dim3(256), 0, stream, true, (const __nv_bfloat16*)dy, M, N, ld, db, rows_per_slab, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int cast_f32_to_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  const int grid = grid_for(n / 4, 256, 148 * 8);
  cast_f32_to_bf16_kernel<<<grid, 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace z2h

extern "C" {
int z2h_gradnorm_partials(const float* g, long long n, float* partials, void* stream) {
  return z2h::gradnorm_partials(g, n, partials, (cudaStream_t)stream);
}
int z2h_adamw_step(float* p32, float* g, float* m, float* v, void* p16, long long n, long long n_decay,
                   const float* hyper, const float* partials, int num_partials, float* norm_out,
                   int zero_grad, void* stream) {
  return z2h::adamw_step(p32, g, m, v, p16, n, n_decay, hyper, partials, num_partials, norm_out,
                         zero_grad, (cudaStream_t)stream);
}
int z2h_colsum_bf16_ordered(const void* dy, int M, int N, long long ld, float* db, int accumulate, int ordered,
                            float* scratch, void* stream) {
  return z2h::colsum_bf16_ordered(dy, M, N, ld, db, accumulate, ordered, scratch, (cudaStream_t)stream);
}
long long z2h_colsum_scratch_elems(int M, int N) { return z2h::colsum_scratch_elems(M, N); }
int z2h_colsum_bf16(const void* dy, int M, int N, long long ld, float* db, int accumulate,
                    void* stream) {
  return z2h::colsum_bf16(dy, M, N, ld, db, accumulate, (cudaStream_t)stream);
}
int z2h_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream) {
  return z2h::cast_f32_to_bf16(src, dst, n, (cudaStream_t)stream);
}
}
