// Parameter block and fused epilogue shared by the one-CTA and the CTA-pair GEMM kernels.
#pragma once
#include "../common/ptx.cuh"
#include "gemm.h"

namespace z2h {
namespace gemm_detail {

struct KernelParams {
  int M, N, K;
  int split_k;
  int epi;
  int out_fp32;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* aux_out;
  const __nv_bfloat16* aux_in;
  long long ldaux;
  int* status;
};

// Epilogue for 32 consecutive columns of one output row.
__device__ __forceinline__ void epilogue_chunk(const KernelParams& p, float (&v)[32], long long grow,
                                               int gcol, const float* sbias) {
  const int ncols = min(32, p.N - gcol);
  if (ncols <= 0) return;
  const bool full = (ncols == 32);
  if (sbias != nullptr) {  // bias of these 32 columns, staged in shared memory (zero past N)
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 b = *reinterpret_cast<const float4*>(sbias + j);
      v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
    }
  }
  if (p.epi == kEpiResidual) {
    const __nv_bfloat16* rp = p.residual + grow * p.ldr + gcol;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 b = *reinterpret_cast<const uint4*>(rp + q * 8);
        float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z),
               f3 = unpack_bf16x2(b.w);
        v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
        v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
      }
    } else {
      #pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) v[j] += __bfloat162float(rp[j]);
    }
  } else if (p.epi == kEpiGelu) {
    // keep the pre-activation for the backward pass, output the activation
    __nv_bfloat16* ap = p.aux_out + grow * p.ldaux + gcol;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        *reinterpret_cast<uint4*>(ap + q * 8) = o;
      }
    } else {
      #pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) ap[j] = __float2bfloat16(v[j]);
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      // the activation is taken of the bf16-rounded pre-activation, as the backward pass sees it
      float x = __bfloat162float(__float2bfloat16(v[j]));
      v[j] = gelu_tanh(x);
    }
  } else if (p.epi == kEpiGeluGrad) {
    const __nv_bfloat16* ap = p.aux_in + grow * p.ldaux + gcol;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 b = *reinterpret_cast<const uint4*>(ap + q * 8);
        float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z),
               f3 = unpack_bf16x2(b.w);
        v[q * 8 + 0] *= gelu_tanh_grad(f0.x); v[q * 8 + 1] *= gelu_tanh_grad(f0.y);
        v[q * 8 + 2] *= gelu_tanh_grad(f1.x); v[q * 8 + 3] *= gelu_tanh_grad(f1.y);
        v[q * 8 + 4] *= gelu_tanh_grad(f2.x); v[q * 8 + 5] *= gelu_tanh_grad(f2.y);
        v[q * 8 + 6] *= gelu_tanh_grad(f3.x); v[q * 8 + 7] *= gelu_tanh_grad(f3.y);
      }
    } else {
      #pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) v[j] *= gelu_tanh_grad(__bfloat162float(ap[j]));
    }
  }

  if (p.out_fp32) {
    float* cp = reinterpret_cast<float*>(p.C) + grow * p.ldc + gcol;
    if (p.epi == kEpiAtomicAdd) {
      if (full) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + q * 4),
                       "f"(v[q * 4 + 0]), "f"(v[q * 4 + 1]), "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3])
                       : "memory");
        }
      } else {
        #pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) atomicAdd(cp + j, v[j]);
      }
    } else if (p.epi == kEpiAccumulate) {
      if (full) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float4 o = *reinterpret_cast<float4*>(cp + q * 4);
          o.x += v[q * 4 + 0]; o.y += v[q * 4 + 1]; o.z += v[q * 4 + 2]; o.w += v[q * 4 + 3];
          *reinterpret_cast<float4*>(cp + q * 4) = o;
        }
      } else {
        #pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) cp[j] += v[j];
      }
    } else {
      if (full) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          *reinterpret_cast<float4*>(cp + q * 4) =
              make_float4(v[q * 4 + 0], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        }
      } else {
        #pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) cp[j] = v[j];
      }
    }
  } else {
    __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + grow * p.ldc + gcol;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        *reinterpret_cast<uint4*>(cp + q * 8) = o;
      }
    } else {
      #pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) cp[j] = __float2bfloat16(v[j]);
    }
  }
}


// Each epilogue warp copies the bias of the 128 columns it will drain into its own 128-float
// slice of shared memory (lane l takes columns 4l..4l+3), so that the per-chunk epilogue reads
// it with broadcast loads instead of waiting on global memory. Only a warp-level sync is needed.
__device__ __forceinline__ void stage_bias(const KernelParams& p, float* my_sbias, int gcol0, int lane) {
  if (p.bias == nullptr) return;
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = gcol0 + lane * 4 + j;
    my_sbias[lane * 4 + j] = c < p.N ? __bfloat162float(p.bias[c]) : 0.f;
  }
  __syncwarp();
}

inline KernelParams make_kernel_params(const GemmArgs& g) {
  KernelParams p;
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.split_k = g.split_k < 1 ? 1 : g.split_k;
  p.epi = g.epi;
  p.out_fp32 = g.out_fp32;
  p.C = g.C; p.ldc = g.ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(g.bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(g.residual);
  p.ldr = g.ldr;
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(g.aux_out);
  p.aux_in = reinterpret_cast<const __nv_bfloat16*>(g.aux_in);
  p.ldaux = g.ldaux;
  p.status = g.status;
  return p;
}

}  // namespace gemm_detail
}  // namespace z2h
