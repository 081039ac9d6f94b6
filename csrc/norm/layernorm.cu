// LayerNorm forward / backward over bf16 activations with fp32 statistics.
//
// forward : y = (x - mean) * rstd * w (+ b); one warp per row, the row is read once with
//           16-byte loads and kept in registers; mean / rstd are saved for the backward pass.
// backward: dx = dresid + rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * w
//           dw += sum_rows dy * xhat,  db += sum_rows dy
//           The weight/bias gradients are reduced without atomics in two stages: every CTA
//           sums its rows per column and writes one partial row to a scratch buffer
//           [num_ctas, 2, C]; a second kernel folds the partials in a fixed order and adds the
//           result to the fp32 gradient, so the result does not depend on scheduling.
//
// Semantics follow nn.LayerNorm(bias=False) of the reference model (nn/gpt2/modules.py:62-69,81)
// and the hand-written weight+bias LayerNorm of the char-level model (nn/gpt/3_gpt.py:79-91):
// biased variance, eps inside the square root.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "norm.h"

namespace z2h {
namespace {

constexpr int kMaxVec = 8;  // per-lane 8-element vectors: rows up to 32 * 8 * 8 = 2048 wide
constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
         d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

template <int NVEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int M, int C,
                     float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + warp;
  if (row >= M) return;
  const __nv_bfloat16* xr = x + (long long)row * C;
  float v[NVEC][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
      load8(xr + c, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
  }
  const float mean = warp_sum(s) / C;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / C + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  __nv_bfloat16* yr = y + (long long)row * C;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
      float wv[8], o[8];
      load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * wv[j];
      if (b != nullptr) {
        float bv[8];
        load8(b + c, bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += bv[j];
      }
      store8(yr + c, o);
    }
  }
}

// scratch layout: [gridDim.x][NSEG][C] fp32: dw partials, db partials and, with HAS_DXSUM, the
// column sums of the OUTPUT dx (NSEG = 3). dx is the gradient of the residual stream, i.e. the
// gradient of the output of the projection that wrote into it, so its column sums are that
// projection's bias gradient: producing them here saves the separate pass over dx.
template <int NVEC, bool HAS_DB, bool HAS_DXSUM>
__global__ void __launch_bounds__(kWarpsPerCta * 32, NVEC <= 4 ? 2 : 1)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dresid,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ scratch, int M, int C) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NSEG = HAS_DXSUM ? 3 : 2;
  extern __shared__ float sh[];  // [kWarpsPerCta][NSEG][C]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float dw_acc[NVEC][8];
  float db_acc[HAS_DB ? NVEC : 1][8];
  float dxs_acc[HAS_DXSUM ? NVEC : 1][8];
  uint4 wraw[NVEC];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * 32 + lane) * 8;
    wraw[i] = make_uint4(0, 0, 0, 0);
    if (c < C) wraw[i] = *reinterpret_cast<const uint4*>(w + c);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dw_acc[i][j] = 0.f;
      if (HAS_DB) db_acc[i][j] = 0.f;
      if (HAS_DXSUM) dxs_acc[i][j] = 0.f;
    }
  }
  for (int row = blockIdx.x * kWarpsPerCta + warp; row < M; row += gridDim.x * kWarpsPerCta) {
    const long long off = (long long)row * C;
    const float mean = mean_in[row], rstd = rstd_in[row];
    uint4 dyraw[NVEC], xraw[NVEC], rraw[NVEC];
    // every load of this row is issued before the first use, and the lines of the warp's next
    // row are requested into L2 meanwhile
    const int next_row = row + gridDim.x * kWarpsPerCta;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < C) {
        dyraw[i] = *reinterpret_cast<const uint4*>(dy + off + c);
        xraw[i] = *reinterpret_cast<const uint4*>(x + off + c);
        if (dresid != nullptr) rraw[i] = *reinterpret_cast<const uint4*>(dresid + off + c);
        if (next_row < M && (lane & 7) == 0) {  // one request per 128-byte line
          const long long noff = (long long)next_row * C + c;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(dy + noff));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(x + noff));
          if (dresid != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(dresid + noff));
        }
      }
    }
    // packed fp32 pairs throughout (one instruction per two columns): the kernel's 16 warps per SM
    // were issuing 55 % of the time, and the per-row chain is latency-bound on top of that
    const float2 rstd2 = make_float2(rstd, rstd);
    const float2 shift2 = make_float2(-mean * rstd, -mean * rstd);
    float2 s1p = make_float2(0.f, 0.f), s2p = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < C) {
        const uint32_t* dyu = reinterpret_cast<const uint32_t*>(&dyraw[i]);
        const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xraw[i]);
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wraw[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 d = unpack_bf16x2(dyu[j]);
          const float2 xh = fma2(unpack_bf16x2(xu[j]), rstd2, shift2);  // (x - mean) * rstd
          const float2 g = mul2(d, unpack_bf16x2(wu[j]));
          s1p = add2(s1p, g);
          s2p = fma2(g, xh, s2p);
          const float2 dwp = fma2(d, xh, make_float2(dw_acc[i][2 * j], dw_acc[i][2 * j + 1]));
          dw_acc[i][2 * j] = dwp.x;
          dw_acc[i][2 * j + 1] = dwp.y;
          if (HAS_DB) {
            db_acc[i][2 * j] += d.x;
            db_acc[i][2 * j + 1] += d.y;
          }
        }
      }
    }
    const float s1 = warp_sum(s1p.x + s1p.y) / C;
    const float s2 = warp_sum(s2p.x + s2p.y) / C;
    const float2 ms1 = make_float2(-s1, -s1), ms2 = make_float2(-s2, -s2);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < C) {
        const uint32_t* dyu = reinterpret_cast<const uint32_t*>(&dyraw[i]);
        const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xraw[i]);
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wraw[i]);
        float o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xh = fma2(unpack_bf16x2(xu[j]), rstd2, shift2);
          // rstd * (dy * w - s1 - xhat * s2)
          float2 t = fma2(unpack_bf16x2(dyu[j]), unpack_bf16x2(wu[j]), ms1);
          t = mul2(fma2(xh, ms2, t), rstd2);
          if (dresid != nullptr) {
            const uint32_t* ru = reinterpret_cast<const uint32_t*>(&rraw[i]);
            t = add2(t, unpack_bf16x2(ru[j]));
          }
          o[2 * j] = t.x;
          o[2 * j + 1] = t.y;
        }
        if (HAS_DXSUM) {
#pragma unroll
          for (int j = 0; j < 8; ++j) dxs_acc[i][j] += o[j];
        }
        store8(dx + off + c, o);
      }
    }
  }
  // fold the 8 warps of this CTA, then write one partial row
  float* my = sh + warp * NSEG * C;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        my[c + j] = dw_acc[i][j];
        my[C + c + j] = HAS_DB ? db_acc[i][j] : 0.f;
        if (HAS_DXSUM) my[2 * C + c + j] = dxs_acc[i][j];
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < NSEG * C; c += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int wi = 0; wi < kWarpsPerCta; ++wi) t += sh[wi * NSEG * C + c];
    scratch[(long long)blockIdx.x * NSEG * C + c] = t;
  }
}

// Folds the per-CTA partial rows in a fixed order: a CTA owns 32 columns of the [2, C] row
// (dw then db) and its 32 warps-worth of threads split the partials 32 ways, then a shared-memory
// tree in fixed order finishes the sum.
__global__ void __launch_bounds__(1024)
layernorm_bwd_reduce_kernel(const float* __restrict__ scratch, int num_partials,
                            float* __restrict__ dw, float* __restrict__ db, float* __restrict__ dxsum,
                            int nseg, int C, int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32][33];
  const int col_in = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int c2 = blockIdx.x * 32 + col_in;  // column of the [nseg * C] partial row
  float s = 0.f;
  if (c2 < nseg * C)
    for (int p = part; p < num_partials; p += 32) s += scratch[(long long)p * nseg * C + c2];
  sh[part][col_in] = s;
  __syncthreads();
  if (part == 0 && c2 < nseg * C) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += sh[k][col_in];
    const int seg = c2 / C, c = c2 - seg * C;
    float* dst = seg == 0 ? dw : (seg == 1 ? db : dxsum);
    // the column sums of dx always accumulate: they are a bias gradient in the flat buffer
    if (dst != nullptr) dst[c] = (accumulate || seg == 2) ? dst[c] + t : t;
  }
}

}  // namespace

int layernorm_bwd_num_partials(int M) {
  int rows_ctas = (M + kWarpsPerCta - 1) / kWarpsPerCta;
  return rows_ctas < kLayerNormBwdMaxCtas ? rows_ctas : kLayerNormBwdMaxCtas;
}

int layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                  int M, int C, float eps, cudaStream_t stream) {
  if (C % 8 != 0 || C > 32 * 8 * kMaxVec) return 1;
  if (M <= 0) return 0;
  const int grid = (M + kWarpsPerCta - 1) / kWarpsPerCta;
#define Z2H_LN_FWD(NV)                                                                         \
  launch_kernel(layernorm_fwd_kernel<NV>, dim3(grid), dim3(kWarpsPerCta * 32), 0, stream, true,                              \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, \
      mean, rstd, M, C, eps)
  if (C <= 768) Z2H_LN_FWD(3);
  else if (C <= 1024) Z2H_LN_FWD(4);
  else Z2H_LN_FWD(8);
#undef Z2H_LN_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                  const void* dresid, void* dx, float* dw, float* db, float* scratch, int M, int C,
                  int accumulate, cudaStream_t stream) {
  return layernorm_bwd_dxsum(dy, x, w, mean, rstd, dresid, dx, dw, db, nullptr, scratch, M, C, accumulate,
                             stream);
}

int layernorm_bwd_dxsum(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                        const void* dresid, void* dx, float* dw, float* db, float* dxsum, float* scratch,
                        int M, int C, int accumulate, cudaStream_t stream) {
  if (C % 8 != 0 || C > 32 * 8 * kMaxVec) return 1;
  if (M <= 0) return 0;
  const int grid = layernorm_bwd_num_partials(M);
  const int nseg = dxsum != nullptr ? 3 : 2;
  const size_t smem = (size_t)kWarpsPerCta * nseg * C * sizeof(float);
  if (smem > 227 * 1024) return 1;
#define Z2H_LN_BWD(NV, DB)                                                                     \
  do {                                                                                         \
    if (dxsum != nullptr) Z2H_LN_BWD_X(NV, DB, true); else Z2H_LN_BWD_X(NV, DB, false);       \
  } while (0)
#define Z2H_LN_BWD_X(NV, DB, DXS)                                                              \
  do {                                                                                         \
    auto kern = layernorm_bwd_kernel<NV, DB, DXS>;                                             \
    static std::atomic<unsigned long long> attr_seen{0};                                       \
    if (first_use_on_current_device(attr_seen))                                                \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                           kWarpsPerCta * (DXS ? 3 : 2) * 32 * 8 * NV * (int)sizeof(float));   \
    launch_kernel(kern, dim3(grid), dim3(kWarpsPerCta * 32), smem, stream, true,                                            \
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, mean, rstd, \
        (const __nv_bfloat16*)dresid, (__nv_bfloat16*)dx, scratch, M, C);                      \
  } while (0)
  const bool has_db = db != nullptr;
  if (C <= 768) { if (has_db) Z2H_LN_BWD(3, true); else Z2H_LN_BWD(3, false); }
  else if (C <= 1024) { if (has_db) Z2H_LN_BWD(4, true); else Z2H_LN_BWD(4, false); }
  else { if (has_db) Z2H_LN_BWD(8, true); else Z2H_LN_BWD(8, false); }
#undef Z2H_LN_BWD
#undef Z2H_LN_BWD_X
  launch_kernel(layernorm_bwd_reduce_kernel, dim3((nseg * C + 31) / 32), dim3(1024), 0, stream, true, scratch,
                grid, dw, db, dxsum, nseg, C, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace z2h

extern "C" {
int z2h_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                      int M, int C, float eps, void* stream) {
  return z2h::layernorm_fwd(x, w, b, y, mean, rstd, M, C, eps, (cudaStream_t)stream);
}
int z2h_layernorm_bwd_num_partials(int M) { return z2h::layernorm_bwd_num_partials(M); }
// As z2h_layernorm_bwd; additionally dxsum[C] += column sums of dx (scratch: partials * 3 * C).
int z2h_layernorm_bwd_dxsum(const void* dy, const void* x, const void* w, const float* mean,
                            const float* rstd, const void* dresid, void* dx, float* dw, float* db,
                            float* dxsum, float* scratch, int M, int C, int accumulate, void* stream) {
  return z2h::layernorm_bwd_dxsum(dy, x, w, mean, rstd, dresid, dx, dw, db, dxsum, scratch, M, C,
                                  accumulate, (cudaStream_t)stream);
}
int z2h_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                      const float* rstd, const void* dresid, void* dx, float* dw, float* db,
                      float* scratch, int M, int C, int accumulate, void* stream) {
  return z2h::layernorm_bwd(dy, x, w, mean, rstd, dresid, dx, dw, db, scratch, M, C, accumulate,
                            (cudaStream_t)stream);
}
}
