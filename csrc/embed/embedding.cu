// Token + position embedding for the GPT models.
//
// forward : out[m, :] = wte[idx[m], :] + wpe[m % T, :]                    (bf16)
// backward: dwte[idx[m], :] += dx[m, :]   (fp32, vector red.global.add: rows of one token that
//                                           occur in several positions are summed by the L2)
//           dwpe[t, :]     += sum_b dx[b*T + t, :]  (fp32, one thread per column, fixed order)
//
// Out-of-range token ids are clamped into the table and counted in the status word instead
// of faulting (the reference kernel bounds-checks ids as well, gpu-mojo/problems/p21/op/
// embedding.mojo:13-60); the model-level semantics are nn/gpt2/modules.py:104-107.
#include "../common/checked.cuh"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "embed.h"

namespace z2h {
namespace {

template <typename IdxT>
__global__ void embed_fwd_kernel(const IdxT* __restrict__ idx, const __nv_bfloat16* __restrict__ wte,
                                 const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out,
                                 int M, int T, int C, int V, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec_per_row = C / 8;
  const long long total = (long long)M * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / vec_per_row);
    const int c = (int)(i % vec_per_row) * 8;
    long long tok = (long long)idx[m];
    if (tok < 0 || tok >= V) {
      if (status != nullptr) atomicCAS(status, 0, (int)kBadArgument);
      tok = tok < 0 ? 0 : V - 1;
    }
    const int t = m % T;
    if (!in_bounds(tok * C + c + 7, (long long)V * C, status, kSiteEmbedTable) ||
        !in_bounds((long long)m * C + c + 7, (long long)M * C, status, kSiteEmbedOut))
      continue;
    uint4 a = *reinterpret_cast<const uint4*>(wte + tok * C + c);
    float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z),
           a3 = unpack_bf16x2(a.w);
    if (wpe != nullptr) {
      uint4 b = *reinterpret_cast<const uint4*>(wpe + (long long)t * C + c);
      float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z),
             b3 = unpack_bf16x2(b.w);
      a0.x += b0.x; a0.y += b0.y; a1.x += b1.x; a1.y += b1.y;
      a2.x += b2.x; a2.y += b2.y; a3.x += b3.x; a3.y += b3.y;
    }
    uint4 o;
    o.x = pack_bf16x2(a0.x, a0.y); o.y = pack_bf16x2(a1.x, a1.y);
    o.z = pack_bf16x2(a2.x, a2.y); o.w = pack_bf16x2(a3.x, a3.y);
    *reinterpret_cast<uint4*>(out + (long long)m * C + c) = o;
  }
}

template <typename IdxT>
__global__ void embed_bwd_wte_kernel(const IdxT* __restrict__ idx, const __nv_bfloat16* __restrict__ dx,
                                     float* __restrict__ dwte, int M, int C, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec_per_row = C / 4;
  const long long total = (long long)M * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / vec_per_row);
    const int c = (int)(i % vec_per_row) * 4;
    long long tok = (long long)idx[m];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    uint2 a = *reinterpret_cast<const uint2*>(dx + (long long)m * C + c);
    float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y);
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dwte + tok * C + c),
                 "f"(a0.x), "f"(a0.y), "f"(a1.x), "f"(a1.y)
                 : "memory");
  }
}

// The same sums in a fixed order, for bitwise reproducible training: one warp per vocabulary row scans
// the token ids (staged through shared memory, 2048 at a time, for the CTA's eight rows) and adds the
// rows of dx whose token is its own in ascending position; one writer per row, no atomics. Most rows
// have no occurrence and cost only the scan (M / 32 ballots). Slower than the scatter above (the ids
// are read V / 8 times), which is why it is a mode, not the default.
constexpr int kOrderedChunk = 2048;
template <typename IdxT>
__global__ void __launch_bounds__(256)
embed_bwd_wte_ordered_kernel(const IdxT* __restrict__ idx, const __nv_bfloat16* __restrict__ dx,
                             float* __restrict__ dwte, int M, int C, int V) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int sidx[kOrderedChunk];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int v = blockIdx.x * 8 + warp;  // this warp's vocabulary row (may be past the end)
  for (int c0 = 0; c0 < C; c0 += 32 * 8) {  // 256 columns per pass: 8 per lane
    const int c = c0 + lane * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    bool any = false;
    for (int base = 0; base < M; base += kOrderedChunk) {
      __syncthreads();
      for (int i = threadIdx.x; i < kOrderedChunk && base + i < M; i += blockDim.x) {
        long long tok = (long long)idx[base + i];
        sidx[i] = (int)(tok < 0 ? 0 : (tok >= V ? V - 1 : tok));
      }
      __syncthreads();
      const int n = min(kOrderedChunk, M - base);
      for (int i0 = 0; i0 < n; i0 += 32) {
        const bool mine = (i0 + lane < n) && sidx[i0 + lane] == v;
        unsigned hits = __ballot_sync(0xffffffffu, mine);
        while (hits != 0u) {  // ascending position: the order of the additions is fixed
          const int b = __ffs(hits) - 1;
          hits &= hits - 1u;
          any = true;
          if (c < C) {
            const uint4 a = *reinterpret_cast<const uint4*>(dx + (long long)(base + i0 + b) * C + c);
            const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z),
                         a3 = unpack_bf16x2(a.w);
            acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y;
            acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
          }
        }
      }
    }
    if (any && v < V && c < C) {
      float* dst = dwte + (long long)v * C + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] += acc[j];
    }
  }
}

__global__ void embed_bwd_wpe_kernel(const __nv_bfloat16* __restrict__ dx, float* __restrict__ dwpe,
                                     int B, int T, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)T * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int b = 0; b < B; ++b) s += __bfloat162float(dx[(long long)b * T * C + i]);
    dwpe[i] += s;
  }
}

}  // namespace

int embed_fwd(const void* idx, int idx_is_64, const void* wte, const void* wpe, void* out, int M,
              int T, int C, int V, int* status, cudaStream_t stream) {
  if (C % 8 != 0) return 1;
  if (M <= 0) return 0;
  const long long total = (long long)M * (C / 8);
  const int grid = (int)((total + 255) / 256 < sm_count_current_device() * 16 ? (total + 255) / 256 : sm_count_current_device() * 16);
  if (idx_is_64)
    launch_kernel(embed_fwd_kernel<long long>, dim3(grid), dim3(256), 0, stream, true, (const long long*)idx, (const __nv_bfloat16*)wte,
                                                         (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out,
                                                         M, T, C, V, status);
  else
    launch_kernel(embed_fwd_kernel<int>, dim3(grid), dim3(256), 0, stream, true, (const int*)idx, (const __nv_bfloat16*)wte,
                                                   (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, M,
                                                   T, C, V, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int embed_bwd(const void* idx, int idx_is_64, const void* dx, float* dwte, float* dwpe, int B, int T,
              int C, int V, cudaStream_t stream) {
  return embed_bwd_ordered(idx, idx_is_64, dx, dwte, dwpe, B, T, C, V, 0, stream);
}

int embed_bwd_ordered(const void* idx, int idx_is_64, const void* dx, float* dwte, float* dwpe, int B, int T,
                      int C, int V, int ordered, cudaStream_t stream) {
  if (C % 8 != 0) return 1;
  const int M = B * T;
  if (M <= 0) return 0;
  const long long total = (long long)M * (C / 4);
  const int grid = (int)((total + 255) / 256 < sm_count_current_device() * 16 ? (total + 255) / 256 : sm_count_current_device() * 16);
  if (ordered) {
    const int g = (V + 7) / 8;
    if (idx_is_64)
      launch_kernel(embed_bwd_wte_ordered_kernel<long long>, dim3(g), dim3(256), 0, stream, true, (const long long*)idx,
                    (const __nv_bfloat16*)dx, dwte, M, C, V);
    else
      launch_kernel(embed_bwd_wte_ordered_kernel<int>, dim3(g), dim3(256), 0, stream, true, (const int*)idx,
                    (const __nv_bfloat16*)dx, dwte, M, C, V);
  } else if (idx_is_64)
    launch_kernel(embed_bwd_wte_kernel<long long>, dim3(grid), dim3(256), 0, stream, true, (const long long*)idx,
                                                             (const __nv_bfloat16*)dx, dwte, M, C, V);
  else
    launch_kernel(embed_bwd_wte_kernel<int>, dim3(grid), dim3(256), 0, stream, true, (const int*)idx, (const __nv_bfloat16*)dx,
                                                       dwte, M, C, V);
  if (dwpe != nullptr) {
    const long long tc = (long long)T * C;
    const int g2 = (int)((tc + 255) / 256 < sm_count_current_device() * 16 ? (tc + 255) / 256 : sm_count_current_device() * 16);
    launch_kernel(embed_bwd_wpe_kernel, dim3(g2), dim3(256), 0, stream, true, (const __nv_bfloat16*)dx, dwpe, B, T, C);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace z2h

extern "C" {
int z2h_embed_fwd(const void* idx, int idx_is_64, const void* wte, const void* wpe, void* out, int M,
                  int T, int C, int V, int* status, void* stream) {
  return z2h::embed_fwd(idx, idx_is_64, wte, wpe, out, M, T, C, V, status, (cudaStream_t)stream);
}
int z2h_embed_bwd_ordered(const void* idx, int idx_is_64, const void* dx, float* dwte, float* dwpe, int B,
                          int T, int C, int V, int ordered, void* stream) {
  return z2h::embed_bwd_ordered(idx, idx_is_64, dx, dwte, dwpe, B, T, C, V, ordered, (cudaStream_t)stream);
}
int z2h_embed_bwd(const void* idx, int idx_is_64, const void* dx, float* dwte, float* dwpe, int B,
                  int T, int C, int V, void* stream) {
  return z2h::embed_bwd(idx, idx_is_64, dx, dwte, dwpe, B, T, C, V, (cudaStream_t)stream);
}
}
