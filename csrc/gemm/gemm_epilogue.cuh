// Parameter block and fused epilogue shared by the one-CTA and the CTA-pair GEMM kernels.
#pragma once
#include "../common/checked.cuh"
#include "../common/ptx.cuh"
#include "../common/warp_colsum.cuh"
#include "gemm.h"
#include <cstdlib>

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
  float* colsum;  // fp32 [N] or null: column sums of the (bf16-rounded) output are added here
  long long slice_stride;  // kEpiSliceStore: elements between the outputs of consecutive K-slices
  int wide;      // every row segment the epilogue touches is 32-byte aligned
  // 0: whole tiles / split-K slices. 1: stream-K, work cut into equal runs of k-blocks, every
  // piece added atomically (fp32 output). 2: stream-K with fix-up (any epilogue, CTA-pair kernel):
  // the piece of a tile that STARTS a worker's run goes to a workspace as fp32, the worker whose run
  // ENDS in that tile adds it to its own accumulator and runs the epilogue once.
  int stream_k;
  // Order in which whole tiles are dealt to the workers that run at the same time: 0 = M fastest
  // (a wave shares one or two B panels and touches every A panel: right when A fits L2 or N is
  // wide), 1 = N fastest (a wave holds all N tiles of a few A panels, so A streams from DRAM once:
  // right for narrow outputs over a long K, e.g. 16384 x 768 with K = 3072, whose A is 100 MB).
  int raster_n;
  float* sk_ws;   // mode 2: [pairs][2 CTAs][8 warps][4 blocks][32 columns][32 lanes] fp32
  int* sk_flags;  // mode 2: [pairs][2][8], 1 = that warp's piece is in the workspace
};

constexpr int kSkWarpFloats = 4 * 32 * 32;           // what one epilogue warp parks: 16 KiB
constexpr int kSkPairFloats = 2 * 8 * kSkWarpFloats;  // 256 KiB per CTA pair

// One unit of work of a CTA (or CTA pair): k-blocks [kb0, kb1) of output tile (mt, nt).
struct Segment {
  int mt, nt, kb0, kb1;
};

// Static work distribution, the same sequence for every role of a worker (a CTA or CTA pair).
//   tiles / split-K: items (tile, k-slice) are dealt round-robin, M fastest, so the workers that
//     run at the same time share one B panel out of L2;
//   stream-K: the tiles x k-blocks units are cut into `workers` equal contiguous runs, a run is
//     walked tile by tile, and every piece is added to the output atomically. No worker idles in
//     a last partial wave, which is what the weight-gradient GEMMs (few tiles, very long K) need.
struct TileScheduler {
  int tiles_m, tiles_n, num_kb, kb_per_split, total_items, item, stride, stream_k, raster_n;
  long long u, u_end;
  __device__ TileScheduler(const KernelParams& p, int bm, int bn, int bk, int worker, int workers) {
    tiles_m = (p.M + bm - 1) / bm;
    tiles_n = (p.N + bn - 1) / bn;
    num_kb = (p.K + bk - 1) / bk;
    stream_k = p.stream_k;
    raster_n = p.raster_n;
    kb_per_split = (num_kb + p.split_k - 1) / p.split_k;
    total_items = tiles_m * tiles_n * p.split_k;
    item = worker;
    stride = workers;
    const long long total = (long long)tiles_m * tiles_n * num_kb;
    const long long per = (total + workers - 1) / workers;
    u = per * worker;
    u_end = u + per < total ? u + per : total;
  }
  __device__ bool next(Segment& s) {
    if (stream_k) {
      if (u >= u_end) return false;
      const long long tile = u / num_kb;
      s.kb0 = (int)(u - tile * num_kb);
      const long long left = u_end - u;
      s.kb1 = left < (long long)(num_kb - s.kb0) ? s.kb0 + (int)left : num_kb;
      s.mt = (int)(tile % tiles_m);
      s.nt = (int)(tile / tiles_m);
      u += s.kb1 - s.kb0;
      return true;
    }
    if (item >= total_items) return false;
    int ks;
    if (raster_n) {
      s.nt = item % tiles_n;
      const int rest = item / tiles_n;
      s.mt = rest % tiles_m;
      ks = rest / tiles_m;
    } else {
      s.mt = item % tiles_m;
      const int rest = item / tiles_m;
      s.nt = rest % tiles_n;
      ks = rest / tiles_n;
    }
    s.kb0 = ks * kb_per_split;
    s.kb1 = min(num_kb, s.kb0 + kb_per_split);  // may be empty for the last slices
    item += stride;
    return true;
  }
};

__device__ __forceinline__ float4 load_bf16x4(const __nv_bfloat16* ptr) {
  const uint2 u = *reinterpret_cast<const uint2*>(ptr);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}

// Shared memory of one epilogue warp: 4 KiB, used either for the bias of its 128 columns (first
// 512 bytes) or as the 32 x 32 fp32 transposition buffer of the atomic-accumulate epilogue
// (the two never occur in the same GEMM call path at the same time: staging happens per block).
constexpr int kEpiWarpBytes = 32 * 32 * 4;
constexpr int kEpiBiasFloats = kEpiWarpBytes / 4;  // stride between the warps' regions, in floats

// ---- 16-byte and 32-byte global accesses -------------------------------------------------
// A thread owns one accumulator row, i.e. 32 consecutive output columns: 64 contiguous bytes
// as bf16, 128 as fp32. With 32-byte vectors every request a lane makes is one whole sector,
// so rows that lie far apart (one row per lane) cost no partial-sector writes; 16-byte
// vectors remain for pointers or pitches that are only 16-byte aligned.
__device__ __forceinline__ void ld_global_b128(const void* ptr, uint32_t* w) {
  asm volatile("ld.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
               : "l"(ptr));
}
__device__ __forceinline__ void st_global_b128(void* ptr, const uint32_t* w) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3])
               : "memory");
}
__device__ __forceinline__ void ld_global_b256(const void* ptr, uint32_t* w) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]),
                 "=r"(w[7])
               : "l"(ptr));
}
__device__ __forceinline__ void st_global_b256(void* ptr, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(w[0]),
               "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
// N_WORDS 32-bit words (a multiple of 8) from / to consecutive addresses
template <int N_WORDS>
__device__ __forceinline__ void ld_row(const void* ptr, uint32_t (&w)[N_WORDS], bool wide) {
  const uint8_t* b = reinterpret_cast<const uint8_t*>(ptr);
  if (wide) {
#pragma unroll
    for (int i = 0; i < N_WORDS / 8; ++i) ld_global_b256(b + i * 32, &w[i * 8]);
  } else {
#pragma unroll
    for (int i = 0; i < N_WORDS / 4; ++i) ld_global_b128(b + i * 16, &w[i * 4]);
  }
}
template <int N_WORDS>
__device__ __forceinline__ void st_row(void* ptr, const uint32_t (&w)[N_WORDS], bool wide) {
  uint8_t* b = reinterpret_cast<uint8_t*>(ptr);
  if (wide) {
#pragma unroll
    for (int i = 0; i < N_WORDS / 8; ++i) st_global_b256(b + i * 32, &w[i * 8]);
  } else {
#pragma unroll
    for (int i = 0; i < N_WORDS / 4; ++i) st_global_b128(b + i * 16, &w[i * 4]);
  }
}

// Epilogue of 32 consecutive columns of one output row, all of which exist; one instantiation
// per epilogue kind and output type keeps each kernel's hot path short.
//   r: the accumulator values (fp32 bit patterns); sbias: bias of these columns in shared memory.
//   pre: for kEpiResidual / kEpiGeluGrad, the 32 bf16 values of the second operand (residual or
//        pre-activation) of these columns, loaded by the caller ahead of time; unused otherwise.
template <int EPI, bool OUT_FP32>
__device__ __forceinline__ void epilogue_row(const KernelParams& p, const uint32_t (&r)[32], long long grow,
                                             int gcol, const float* sbias, const uint32_t (&pre)[16]) {
  if (!in_bounds_2d(grow, 1, p.M, gcol, 32, p.N, p.status, kSiteGemmRow)) return;
  const bool wide = p.wide != 0;
  // two columns per step with packed fp32 arithmetic: the epilogue warps (two per scheduler) are
  // bound by the instructions they issue, and the packed forms halve those
  float2 v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
  if (sbias != nullptr) {
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      const float4 b = *reinterpret_cast<const float4*>(sbias + 2 * j);  // same address in all lanes
      v[j] = add2(v[j], make_float2(b.x, b.y));
      v[j + 1] = add2(v[j + 1], make_float2(b.z, b.w));
    }
  }
  if (EPI == kEpiResidual) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = add2(v[j], unpack_bf16x2(pre[j]));
  } else if (EPI == kEpiGelu) {
    // keep the pre-activation for the backward pass, output the activation of its bf16 rounding
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = pack_bf16x2(v[j].x, v[j].y);
    st_row(p.aux_out + grow * p.ldaux + gcol, w, wide);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = gelu_tanh2(unpack_bf16x2(w[j]));
  } else if (EPI == kEpiGeluGrad) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = mul2(v[j], gelu_tanh_grad2(unpack_bf16x2(pre[j])));
  } else if (EPI == kEpiGeluSaveGrad) {
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float2 act, grad;
      gelu_tanh_with_grad2(v[j], act, grad);
      w[j] = pack_bf16x2(grad.x, grad.y);
      v[j] = act;
    }
    st_row(p.aux_out + grow * p.ldaux + gcol, w, wide);
  } else if (EPI == kEpiMulAux) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = mul2(v[j], unpack_bf16x2(pre[j]));
  }
  if (OUT_FP32) {
    float* cp = reinterpret_cast<float*>(p.C) + grow * p.ldc + gcol;
    if (EPI == kEpiAtomicAdd) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + q * 4), "f"(v[2 * q].x),
                     "f"(v[2 * q].y), "f"(v[2 * q + 1].x), "f"(v[2 * q + 1].y)
                     : "memory");
      }
    } else {
      uint32_t w[32];
      if (EPI == kEpiAccumulate) {
        ld_row(cp, w, wide);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 s2 = add2(v[j], make_float2(__uint_as_float(w[2 * j]), __uint_as_float(w[2 * j + 1])));
          w[2 * j] = __float_as_uint(s2.x);
          w[2 * j + 1] = __float_as_uint(s2.y);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          w[2 * j] = __float_as_uint(v[j].x);
          w[2 * j + 1] = __float_as_uint(v[j].y);
        }
      }
      st_row(cp, w, wide);
    }
  } else {
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = pack_bf16x2(v[j].x, v[j].y);
    st_row(reinterpret_cast<__nv_bfloat16*>(p.C) + grow * p.ldc + gcol, w, wide);
    if (p.colsum != nullptr) {
      // bias gradient of the layer whose output gradient this GEMM produces: sum what was stored
      // (the rounded values, as a separate pass over C would). The launcher admits this only when
      // M is a multiple of 32, so all 32 lanes of the warp are here.
      float t[32];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        t[2 * j] = f.x; t[2 * j + 1] = f.y;
      }
      const float sum = warp_column_sums<32>(t, (int)(threadIdx.x & 31));
      asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p.colsum + gcol + (threadIdx.x & 31)), "f"(sum) : "memory");
    }
  }
}

// The same for a block at the right edge (fewer than 32 columns exist) or for a combination of
// kind and output type that has no instantiation above: one element at a time, loop kept
// rolled so that this seldom-run code stays small.
static __device__ __noinline__ void epilogue_row_edge(int epi, int out_fp32, void* C, long long ldc,
                                               const __nv_bfloat16* residual, long long ldr,
                                               __nv_bfloat16* aux_out, const __nv_bfloat16* aux_in,
                                               long long ldaux, const uint32_t* r, long long grow,
                                               int gcol, int ncols, const float* sbias
#ifdef Z2H_BOUNDS
                                               , long long bounds_m, long long bounds_n, int* bounds_status
#endif
                                               ) {
#pragma unroll 1
  for (int j = 0; j < ncols; ++j) {
#ifdef Z2H_BOUNDS
    if (!in_bounds_2d(grow, 1, bounds_m, gcol + j, 1, bounds_n, bounds_status, kSiteGemmEdge)) continue;
#endif
    float v = __uint_as_float(r[j]);
    if (sbias != nullptr) v += sbias[j];
    const long long col = gcol + j;
    if (epi == kEpiResidual) {
      v += __bfloat162float(residual[grow * ldr + col]);
    } else if (epi == kEpiGelu) {
      const __nv_bfloat16 pre = __float2bfloat16(v);
      aux_out[grow * ldaux + col] = pre;
      v = gelu_tanh(__bfloat162float(pre));
    } else if (epi == kEpiGeluGrad) {
      v *= gelu_tanh_grad(__bfloat162float(aux_in[grow * ldaux + col]));
    } else if (epi == kEpiGeluSaveGrad) {
      aux_out[grow * ldaux + col] = __float2bfloat16(gelu_tanh_grad(v));
      v = gelu_tanh(v);
    } else if (epi == kEpiMulAux) {
      v *= __bfloat162float(aux_in[grow * ldaux + col]);
    }
    if (out_fp32) {
      float* cp = reinterpret_cast<float*>(C) + grow * ldc + col;
      if (epi == kEpiAtomicAdd) atomicAdd(cp, v);
      else if (epi == kEpiAccumulate) *cp += v;
      else *cp = v;
    } else {
      reinterpret_cast<__nv_bfloat16*>(C)[grow * ldc + col] = __float2bfloat16(v);
    }
  }
}

// Epilogue of the four 32-column blocks a warp owns in one tile: r[c] holds block c of the row
// `grow` (one row per lane), gcol0 is the first column of block 0, sbias the warp's staged bias
// (128 floats, zero past N) or null.
//
// The residual / pre-activation operand of block c + 1 is loaded before block c is worked on. One
// row per lane means every such load is a long-latency access of its own (32 rows, 32 sectors), the
// eight epilogue warps of a CTA cannot hide it, and with short main loops (K = 768) the epilogue,
// not the tensor pipe, then sets the tile time: the GELU-gradient GEMM of the MLP ran at 128 us
// against 66 us for the same product with a plain epilogue.
template <int EPI, bool OUT_FP32>
__device__ __forceinline__ void epilogue_blocks(const KernelParams& p, const uint32_t (&r)[4][32],
                                                long long grow, int gcol0, const float* sbias) {
  constexpr bool kSecondOperand = EPI == kEpiResidual || EPI == kEpiGeluGrad || EPI == kEpiMulAux;
  const __nv_bfloat16* src = nullptr;
  if (EPI == kEpiResidual) src = p.residual + grow * p.ldr;
  if (EPI == kEpiGeluGrad || EPI == kEpiMulAux) src = p.aux_in + grow * p.ldaux;
  const bool wide = p.wide != 0;
  uint32_t pre[2][16] = {};
  if (kSecondOperand && gcol0 + 32 <= p.N) ld_row(src + gcol0, pre[0], wide);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int gcol = gcol0 + c * 32;
    if (kSecondOperand && c + 1 < 4 && gcol + 64 <= p.N) ld_row(src + gcol + 32, pre[(c + 1) & 1], wide);
    if (gcol + 32 <= p.N) {
      epilogue_row<EPI, OUT_FP32>(p, r[c], grow, gcol, sbias != nullptr ? sbias + c * 32 : nullptr, pre[c & 1]);
    } else if (gcol < p.N) {
      uint32_t tmp[32];  // addressable copy for the rolled loop
#pragma unroll
      for (int j = 0; j < 32; ++j) tmp[j] = r[c][j];
      epilogue_row_edge(p.epi, p.out_fp32, p.C, p.ldc, p.residual, p.ldr, p.aux_out, p.aux_in, p.ldaux,
                        tmp, grow, gcol, p.N - gcol, sbias != nullptr ? sbias + c * 32 : nullptr
#ifdef Z2H_BOUNDS
                        , p.M, p.N, p.status
#endif
                        );
    }
  }
}

// Atomic accumulation (split-K / stream-K weight gradients) of a 32 x 32 block with coalesced
// reductions. One accumulator row per lane would make every red.global.add touch 32 rows, i.e.
// 32 memory transactions per instruction; the block is therefore transposed through a swizzled
// 4 KiB shared-memory buffer so that 8 neighbouring lanes share a row and each instruction covers
// 4 rows with one contiguous 128-byte segment each.
//   row_base: global row of lane 0's accumulator row; stage: the warp's buffer (shared address).
__device__ __forceinline__ void epilogue_block_atomic(const KernelParams& p, const uint32_t (&r)[32],
                                                      long long row_base, int gcol, int lane,
                                                      uint32_t stage) {
  if (!in_bounds_2d(row_base, 32, p.M, gcol, 32, p.N, p.status, kSiteGemmAtomic)) return;
  __syncwarp();  // the previous block's reads of the buffer are done
#pragma unroll
  for (int c4 = 0; c4 < 8; ++c4) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                     stage + lane * 128 + ((c4 ^ (lane & 7)) << 4)),
                 "r"(r[c4 * 4 + 0]), "r"(r[c4 * 4 + 1]), "r"(r[c4 * 4 + 2]), "r"(r[c4 * 4 + 3])
                 : "memory");
  }
  __syncwarp();
  const int sub = lane >> 3, c4 = lane & 7;
  float* cp = reinterpret_cast<float*>(p.C) + (row_base + sub) * p.ldc + gcol + c4 * 4;
  const long long cstep = 4 * p.ldc;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int lr = i * 4 + sub;
    uint32_t x0, x1, x2, x3;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                 : "r"(stage + lr * 128 + ((c4 ^ (lr & 7)) << 4))
                 : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + i * cstep),
                 "f"(__uint_as_float(x0)), "f"(__uint_as_float(x1)), "f"(__uint_as_float(x2)),
                 "f"(__uint_as_float(x3))
                 : "memory");
  }
}

//   stage: shared address of the warp's 4 KiB buffer (used by the atomic epilogue only)
__device__ __forceinline__ void epilogue_tile(const KernelParams& p, const uint32_t (&r)[4][32],
                                              long long grow, int gcol0, const float* sbias, int lane,
                                              uint32_t stage) {
  if (p.out_fp32 && p.epi == kEpiAtomicAdd && sbias == nullptr) {
    const long long row_base = grow - lane;
    if (row_base + 32 <= p.M && gcol0 + 128 <= p.N) {  // interior: the same for the whole warp
#pragma unroll
      for (int c = 0; c < 4; ++c) epilogue_block_atomic(p, r[c], row_base, gcol0 + c * 32, lane, stage);
      return;
    }
  }
  if (grow >= p.M) return;
  if (p.out_fp32) {
    if (p.epi == kEpiAtomicAdd) return epilogue_blocks<kEpiAtomicAdd, true>(p, r, grow, gcol0, sbias);
    if (p.epi == kEpiAccumulate) return epilogue_blocks<kEpiAccumulate, true>(p, r, grow, gcol0, sbias);
    if (p.epi == kEpiNone) return epilogue_blocks<kEpiNone, true>(p, r, grow, gcol0, sbias);
  } else {
    if (p.epi == kEpiNone) return epilogue_blocks<kEpiNone, false>(p, r, grow, gcol0, sbias);
    if (p.epi == kEpiResidual) return epilogue_blocks<kEpiResidual, false>(p, r, grow, gcol0, sbias);
    if (p.epi == kEpiGelu) return epilogue_blocks<kEpiGelu, false>(p, r, grow, gcol0, sbias);
    if (p.epi == kEpiGeluGrad) return epilogue_blocks<kEpiGeluGrad, false>(p, r, grow, gcol0, sbias);
  }
  // remaining combinations (e.g. residual with an fp32 output): element by element
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int gcol = gcol0 + c * 32;
    if (gcol < p.N) {
      uint32_t tmp[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) tmp[j] = r[c][j];
      epilogue_row_edge(p.epi, p.out_fp32, p.C, p.ldc, p.residual, p.ldr, p.aux_out, p.aux_in, p.ldaux,
                        tmp, grow, gcol, min(32, p.N - gcol), sbias != nullptr ? sbias + c * 32 : nullptr
#ifdef Z2H_BOUNDS
                        , p.M, p.N, p.status
#endif
                        );
    }
  }
}

// ---- the tile epilogue, streamed over the warp's four 32-column blocks --------------------------
// Waits for the outstanding tensor-memory load and tells the compiler that r is written HERE (the
// load itself is asynchronous: a copy of r made between the load and this wait would hold garbage).
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                 "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                 "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

constexpr int kEpiGeneric = -1;  // any kind / output type without an instantiation: element by element

// One 32 x 32 block: r = accumulator row of this lane, pre = its second operand (if the kind has one).
template <int EPI, bool OUT_FP32>
__device__ __forceinline__ void epilogue_block(const KernelParams& p, const uint32_t (&r)[32],
                                               const uint32_t (&pre)[16], long long grow, int gcol,
                                               const float* sbias, int lane, uint32_t stage, bool row_ok,
                                               bool atomic_interior) {
  if (OUT_FP32 && EPI == kEpiAtomicAdd) {
    if (atomic_interior) {  // the same for the whole warp
      epilogue_block_atomic(p, r, grow - lane, gcol, lane, stage);
      return;
    }
  }
  if (!row_ok || gcol >= p.N) return;
  if (EPI != kEpiGeneric && gcol + 32 <= p.N) {
    epilogue_row<EPI == kEpiGeneric ? kEpiNone : EPI, OUT_FP32>(p, r, grow, gcol, sbias, pre);
  } else {
    uint32_t tmp[32];  // addressable copy for the rolled loop
#pragma unroll
    for (int j = 0; j < 32; ++j) tmp[j] = r[j];
    epilogue_row_edge(p.epi, p.out_fp32, p.C, p.ldc, p.residual, p.ldr, p.aux_out, p.aux_in, p.ldaux, tmp,
                      grow, gcol, min(32, p.N - gcol), sbias
#ifdef Z2H_BOUNDS
                      , p.M, p.N, p.status
#endif
                      );
  }
}

// The warp's four blocks, two register buffers: while block c is worked on, the tensor-memory load
// of block c + 1 and the load of its second operand (residual or pre-activation) are in flight. A
// tensor-memory load issued while MMAs are queued takes around a thousand cycles and one row per
// lane makes every global load a long-latency access of its own; with all four blocks loaded up
// front (128 registers) nothing was left to overlap either with, and the GELU-gradient GEMM of the
// MLP (K = 768, a short main loop) took 128 us against 66 us with a plain epilogue. The accumulator
// is handed back (release()) when its last block is in registers.
//   taddr: tensor-memory address of the warp's first block; active: false for a tile that has no
//   k-blocks in this worker's share (the accumulator protocol still runs).
//   k_slice: which K-slice of the tile this is (kEpiSliceStore only; 0 otherwise)
template <int EPI, bool OUT_FP32, class Release>
__device__ __forceinline__ void epilogue_stream(const KernelParams& p_in, uint32_t taddr, long long grow,
                                                int gcol0, const float* sbias, int lane, uint32_t stage,
                                                bool active, int k_slice, Release release) {
  constexpr bool kSecondOperand = EPI == kEpiResidual || EPI == kEpiGeluGrad || EPI == kEpiMulAux;
  // a K-slice stores to its own copy of the output; a slice without k-blocks stores zeros there
  KernelParams p_slice = p_in;
  if (EPI == kEpiSliceStore)
    p_slice.C = reinterpret_cast<float*>(p_in.C) + (long long)k_slice * p_in.slice_stride;
  const KernelParams& p = EPI == kEpiSliceStore ? p_slice : p_in;
  const bool zero_fill = EPI == kEpiSliceStore && !active;
  if (EPI == kEpiSliceStore) active = true;
  const bool row_ok = active && grow < p.M;
  const bool atomic_interior = OUT_FP32 && EPI == kEpiAtomicAdd && active && sbias == nullptr &&
                               (grow - lane) + 32 <= p.M && gcol0 + 128 <= p.N;
  const __nv_bfloat16* src = nullptr;
  if (EPI == kEpiResidual) src = p.residual + grow * p.ldr + gcol0;
  if (EPI == kEpiGeluGrad || EPI == kEpiMulAux) src = p.aux_in + grow * p.ldaux + gcol0;
  const bool wide = p.wide != 0;
  uint32_t r[2][32];
  uint32_t pre[2][16] = {};
  tmem_ld_32x32b_x32(taddr, r[0]);
  if (kSecondOperand && row_ok && gcol0 + 32 <= p.N) ld_row(src, pre[0], wide);
#pragma unroll 1
  for (int c = 0; c < 4; c += 2) {
    tmem_ld_wait_for(r[0]);
    if (zero_fill) {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[0][j] = 0u;
    }
    tmem_ld_32x32b_x32(taddr + (c + 1) * 32, r[1]);
    if (kSecondOperand && row_ok && gcol0 + (c + 2) * 32 <= p.N) ld_row(src + (c + 1) * 32, pre[1], wide);
    epilogue_block<EPI, OUT_FP32>(p, r[0], pre[0], grow, gcol0 + c * 32,
                                  sbias != nullptr ? sbias + c * 32 : nullptr, lane, stage, row_ok, atomic_interior);
    tmem_ld_wait_for(r[1]);
    if (zero_fill) {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[1][j] = 0u;
    }
    if (c + 2 < 4) {
      tmem_ld_32x32b_x32(taddr + (c + 2) * 32, r[0]);
      if (kSecondOperand && row_ok && gcol0 + (c + 3) * 32 <= p.N) ld_row(src + (c + 2) * 32, pre[0], wide);
    } else {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release();
    }
    epilogue_block<EPI, OUT_FP32>(p, r[1], pre[1], grow, gcol0 + (c + 1) * 32,
                                  sbias != nullptr ? sbias + (c + 1) * 32 : nullptr, lane, stage, row_ok,
                                  atomic_interior);
  }
}

//   stage: shared address of the warp's 4 KiB buffer (used by the atomic epilogue only)
// EXTRA selects which kinds a kernel instantiation carries. The kinds added for the MLP's activation
// pair and for split-K without atomics live in kernel instantiations of their own: compiled into the
// same kernel as the others they changed nothing in the other kinds' code, yet the register allocation
// and scheduling of the whole kernel came out 10 % slower for every plain GEMM (M16384 N3072 K768
// 63.5 -> 71.7 us, lm_head 932 -> 1020 us).
template <bool EXTRA, class Release>
__device__ __forceinline__ void epilogue_tile_streamed(const KernelParams& p, uint32_t taddr, long long grow,
                                                       int gcol0, const float* sbias, int lane, uint32_t stage,
                                                       bool active, int k_slice, Release release) {
  if (EXTRA) {
    if (p.out_fp32)
      return epilogue_stream<kEpiSliceStore, true>(p, taddr, grow, gcol0, sbias, lane, stage, active, k_slice, release);
    if (p.epi == kEpiGeluSaveGrad)
      return epilogue_stream<kEpiGeluSaveGrad, false>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
    return epilogue_stream<kEpiMulAux, false>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
  }
  if (p.out_fp32) {
    if (p.epi == kEpiAtomicAdd)
      return epilogue_stream<kEpiAtomicAdd, true>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
    if (p.epi == kEpiAccumulate)
      return epilogue_stream<kEpiAccumulate, true>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
    if (p.epi == kEpiNone)
      return epilogue_stream<kEpiNone, true>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
  } else {
    if (p.epi == kEpiNone)
      return epilogue_stream<kEpiNone, false>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
    if (p.epi == kEpiResidual)
      return epilogue_stream<kEpiResidual, false>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
    if (p.epi == kEpiGelu)
      return epilogue_stream<kEpiGelu, false>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
    if (p.epi == kEpiGeluGrad)
      return epilogue_stream<kEpiGeluGrad, false>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
  }
  return epilogue_stream<kEpiGeneric, false>(p, taddr, grow, gcol0, sbias, lane, stage, active, 0, release);
}

// Called before the wait for the accumulator: asks L2 for this lane's 128 columns (256 bytes) of the
// epilogue's second operand, so that the loads after the wait find them there instead of in DRAM.
__device__ __forceinline__ void prefetch_second_operand(const KernelParams& p, long long grow, int gcol0) {
  const __nv_bfloat16* src = nullptr;
  if (p.epi == kEpiResidual) src = p.residual + grow * p.ldr + gcol0;
  else if (p.epi == kEpiGeluGrad || p.epi == kEpiMulAux) src = p.aux_in + grow * p.ldaux + gcol0;
  if (src == nullptr || grow >= p.M) return;
  if (gcol0 < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
  if (gcol0 + 64 < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + 64));
}

// Each epilogue warp copies the bias of the 128 columns it will drain into its own slice of
// shared memory (lane l takes columns 4l..4l+3, zero past N), so that the row epilogue reads it
// with broadcast loads. Only warp-level synchronisation is needed. Returns the slice, or null
// when the GEMM has no bias.
__device__ __forceinline__ const float* stage_bias(const KernelParams& p, float* my_sbias, int gcol0,
                                                   int lane) {
  if (p.bias == nullptr) return nullptr;
  __syncwarp();  // the previous tile's reads are done
  const int c = gcol0 + lane * 4;
  float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c + 4 <= p.N) {
    b = load_bf16x4(p.bias + c);
  } else {
    if (c + 0 < p.N) b.x = __bfloat162float(p.bias[c + 0]);
    if (c + 1 < p.N) b.y = __bfloat162float(p.bias[c + 1]);
    if (c + 2 < p.N) b.z = __bfloat162float(p.bias[c + 2]);
  }
  *reinterpret_cast<float4*>(my_sbias + lane * 4) = b;
  __syncwarp();
  return my_sbias;
}

inline KernelParams make_kernel_params(const GemmArgs& g) {
  KernelParams p;
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.split_k = g.split_k < 1 ? 1 : g.split_k;
  p.stream_k = (g.split_k <= 0 && g.epi == kEpiAtomicAdd) ? 1 : 0;
  p.sk_ws = nullptr;
  p.sk_flags = nullptr;
  p.raster_n = 0;  // the launchers decide (they know their tile shape)
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
  p.colsum = reinterpret_cast<float*>(g.colsum);
  p.slice_stride = g.slice_stride;
  {
    // 32-byte vectors need 32-byte aligned bases and pitches (bf16: 16 elements, fp32: 8)
    auto a32 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0; };
    const long long cmul = g.out_fp32 ? 8 : 16;
    p.wide = a32(g.C) && (g.ldc % cmul) == 0 && a32(g.residual) && (g.ldr % 16) == 0 && a32(g.aux_out) &&
             a32(g.aux_in) && (g.ldaux % 16) == 0;
  }
  return p;
}

// N-fastest tile order when the output is narrower (in tiles) than it is tall and either A is too
// big to live in L2 across the waves or there are enough N tiles to fill a wave's width: the
// workers of a wave then cover every N tile of a few row panels, and A is streamed from DRAM once.
// Measured on B200 (CTA-pair kernel, M = 16384): N768 K3072 71.7 -> 61.4 us, N768 K2304 55.3 -> 49.2,
// N3072 K768 63.5 -> 61.4, N2304 K768 51.2 -> 50.2; the other way round for N768 K768 (26.7 -> 28.7,
// A is 25 MB and stays in L2) and for the lm_head (N50304: 942 -> 1057), which keep M fastest.
// Split-K and stream-K launches keep M fastest as well. Z2H_GEMM_RASTER=m|n forces one order.
inline int pick_raster_n(const GemmArgs& g, int tm, int tn) {
  static const int forced = [] {
    const char* e = std::getenv("Z2H_GEMM_RASTER");
    return e == nullptr ? -1 : (e[0] == 'n' ? 1 : 0);
  }();
  if (forced >= 0) return forced;
  if (g.split_k != 1) return 0;
  const int tiles_m = (g.M + tm - 1) / tm, tiles_n = (g.N + tn - 1) / tn;
  const long long a_bytes = (long long)g.M * g.K * 2;
  return (tiles_n < tiles_m && (a_bytes >= (48LL << 20) || tiles_n >= 8)) ? 1 : 0;
}

}  // namespace gemm_detail
}  // namespace z2h
