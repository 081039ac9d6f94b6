// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T with fp32
// accumulation in tensor memory and a fused epilogue.
//
// One persistent CTA per SM walks a static tile schedule (M fastest, so the CTAs that run at
// the same time share one B panel out of L2). Inside the CTA the work is split by warp role:
//
//   warp 0      TMA producer   cp.async.bulk.tensor 2-D tiles, 128-byte swizzle, 4-stage ring
//   warp 1      MMA issuer     one elected lane issues tcgen05.mma (128x256x16) and commits
//                              stage releases / accumulator completions to mbarriers
//   warps 2-9   epilogue       tcgen05.ld the 128x256 fp32 accumulator (one row per thread, two
//                              warps per TMEM lane quarter, each taking half of the columns),
//                              apply bias / GELU / residual / GELU' and store
//
// Two accumulators of 256 TMEM columns each are used in turn, so the epilogue of tile i runs
// while the tensor cores already work on tile i+1.
//
// Either operand may be K-major (the contraction index is contiguous in global memory) or
// MN-major (the M / N index is contiguous); the second form is what the weight-gradient and
// data-gradient GEMMs of a linear layer need, so no transposed copies are ever made.
//
// Replaces the nn.Linear calls of the reference model (nn/gpt2/modules.py:21-22,49-51,82) and
// their autograd; the reference's own tensor-core kernel is gpu-mojo/problems/p33/p33.mojo:130-245.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "gemm.h"

#include "../common/trace.cuh"

#include "gemm_epilogue.cuh"

namespace z2h {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int NUM_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES =
    1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256 + EPI_WARPS * gemm_detail::kEpiWarpBytes;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB a CTA may use");

using gemm_detail::KernelParams;


// EXTRA: the instantiation that carries the newer epilogue kinds (see epilogue_tile_streamed).
template <int A_MN, int B_MN, bool EXTRA>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB, const KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + STAGES * B_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* epi_bias = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(full_bar) + 256);  // 4 KiB per epilogue warp: bias slice or transposition buffer

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_launch_dependents();

  // every role walks the same sequence of work segments
  gemm_detail::TileScheduler sched(p, BM, BN, BK, blockIdx.x, gridDim.x);
  gemm_detail::Segment sg;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // everything above overlaps the previous kernel's tail; global memory from here on

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Z2H_TRACE_DECL(0)
      Z2H_TRACE();
      while (ok && sched.next(sg)) {
        const int mt = sg.mt, nt = sg.nt, kb0 = sg.kb0, kb1 = sg.kb1;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.status,
                                 kTimeoutEmpty)) {
            ok = false;
            break;
          }
          Z2H_TRACE();
          mbar_arrive_expect_tx(&full_bar[stage], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
          if (A_MN == 0) {
            tma_load_2d(a_dst, &tmA, &full_bar[stage], kb * BK, mt * BM);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(a_dst + c * (64 * BK * 2), &tmA, &full_bar[stage], mt * BM + c * 64,
                          kb * BK);
          }
          if (B_MN == 0) {
            tma_load_2d(b_dst, &tmB, &full_bar[stage], kb * BK, nt * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + c * (64 * BK * 2), &tmB, &full_bar[stage], nt * BN + c * 64,
                          kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight a bounded time to land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      constexpr uint32_t a_lbo = A_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t b_lbo = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t a_kstep = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      constexpr uint32_t b_kstep = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      Z2H_TRACE_DECL(1)
      Z2H_TRACE();
      for (; ok && sched.next(sg); ++it) {
        const int kb0 = sg.kb0, kb1 = sg.kb1;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, p.status,
                               kTimeoutTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status, kTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          Z2H_TRACE();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
            tc_mma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          Z2H_TRACE();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue (8 warps) ------------------------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    int it = 0;
    bool ok = true;
    Z2H_TRACE_DECL(2)
    for (; ok && sched.next(sg); ++it) {
      const int mt = sg.mt, nt = sg.nt;
      const bool empty_split = sg.kb0 >= sg.kb1;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      // bias of this warp's 128 columns, staged before the wait for the accumulator
      const int gcol0 = nt * BN + half * 128;
      const float* sbias = gemm_detail::stage_bias(p, epi_bias + (warp - 2) * gemm_detail::kEpiBiasFloats, gcol0, lane);
      if (!empty_split) gemm_detail::prefetch_second_operand(p, (long long)mt * BM + quarter * 32 + lane, gcol0);
      if (!mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (warp == 2 && lane == 0) Z2H_TRACE();
      const long long row_base = (long long)mt * BM + quarter * 32;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      // this warp drains 4 of the 8 column blocks of its 32 rows
      const int c0 = half * 4;
      uint64_t* const tempty = &tempty_bar[acc];
      gemm_detail::epilogue_tile_streamed<EXTRA>(p, taddr + c0 * 32, row_base + lane, gcol0, sbias, lane,
                                          smem_u32(epi_bias + (warp - 2) * gemm_detail::kEpiBiasFloats),
                                          !empty_split, (EXTRA && p.split_k > 1) ? sg.kb0 / sched.kb_per_split : 0,
                                          [tempty] { mbar_arrive(tempty); });
      if (warp == 2 && lane == 0) Z2H_TRACE();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int A_MN, int B_MN>
int launch(const GemmArgs& g, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  bool ok;
  if (A_MN == 0)
    ok = make_tma_2d_bf16(&tmA, g.A, g.M, g.K, g.lda, BM, BK, kSwizzle128);
  else
    ok = make_tma_2d_bf16(&tmA, g.A, g.K, g.M, g.lda, BK, 64, kSwizzle128);
  if (!ok) return 2;
  if (B_MN == 0)
    ok = make_tma_2d_bf16(&tmB, g.B, g.N, g.K, g.ldb, BN, BK, kSwizzle128);
  else
    ok = make_tma_2d_bf16(&tmB, g.B, g.K, g.N, g.ldb, BK, 64, kSwizzle128);
  if (!ok) return 2;

  KernelParams p = gemm_detail::make_kernel_params(g);
  p.raster_n = gemm_detail::pick_raster_n(g, BM, BN);

  auto kern = g.epi >= kEpiGeluSaveGrad ? gemm_bf16_tcgen05_kernel<A_MN, B_MN, true>
                                        : gemm_bf16_tcgen05_kernel<A_MN, B_MN, false>;
  static std::atomic<unsigned long long> attr_seen{0};
  if (first_use_on_current_device(attr_seen)) {
    cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<A_MN, B_MN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<A_MN, B_MN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  }
  const int num_sms = sm_count_current_device();
  const long long tiles = (long long)((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN) *
                          (p.stream_k ? (g.K + BK - 1) / BK : p.split_k);
  int grid = tiles < num_sms ? (int)tiles : num_sms;
  if (g.max_ctas > 0 && grid > g.max_ctas) grid = g.max_ctas;
  if (grid < 1) return 0;
  return launch_kernel(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, true, tmA, tmB, p) == cudaSuccess
             ? 0
             : 3;
}

}  // namespace

static int g_algo = 2;
void gemm_set_algo(int algo) { g_algo = algo; }
int gemm_get_algo() { return g_algo; }

int gemm_bf16(const GemmArgs& g, cudaStream_t stream) {
  // argument checks: everything the TMA descriptors and the vector epilogue rely on
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.B) & 15) ||
      (reinterpret_cast<uintptr_t>(g.C) & 15))
    return 1;
  if ((g.lda % 8) || (g.ldb % 8) || (g.ldc % 8)) return 1;
  if ((g.epi == kEpiAtomicAdd || g.epi == kEpiAccumulate) && !g.out_fp32) return 1;
  if (g.split_k > 1 && g.epi != kEpiAtomicAdd && g.epi != kEpiSliceStore) return 1;
  if (g.epi == kEpiSliceStore && (!g.out_fp32 || g.split_k < 1 || g.bias != nullptr ||
                                  g.slice_stride < (long long)(g.M - 1) * g.ldc + g.N || (g.slice_stride % 4)))
    return 1;
  if (g.epi == kEpiResidual && (g.residual == nullptr || (g.ldr % 8))) return 1;
  if (g.epi == kEpiGelu && (g.aux_out == nullptr || (g.ldaux % 8))) return 1;
  if (g.epi == kEpiGeluGrad && (g.aux_in == nullptr || (g.ldaux % 8))) return 1;
  if (g.epi == kEpiGeluSaveGrad && (g.aux_out == nullptr || (g.ldaux % 8) || g.out_fp32)) return 1;
  if (g.epi == kEpiMulAux && (g.aux_in == nullptr || (g.ldaux % 8) || g.out_fp32)) return 1;
  if (g.epi < kEpiNone || g.epi > kEpiSliceStore) return 1;
  if (reinterpret_cast<uintptr_t>(g.bias) & 7) return 1;
  if (g.colsum != nullptr && (g.out_fp32 || g.split_k != 1 || (g.M % 32) || (g.N % 32) ||
                              (reinterpret_cast<uintptr_t>(g.colsum) & 3)))
    return 1;
  if ((reinterpret_cast<uintptr_t>(g.residual) & 15) || (reinterpret_cast<uintptr_t>(g.aux_out) & 15) ||
      (reinterpret_cast<uintptr_t>(g.aux_in) & 15))
    return 1;
  {
    const bool stream_k = g.split_k <= 0 && g.epi == kEpiAtomicAdd;  // fills every SM whatever the tile count
    const long long tiles256 = (long long)((g.M + 255) / 256) * ((g.N + 255) / 256) * (g.split_k < 1 ? 1 : g.split_k);
    // split-K and stream-K launches always take the pair kernel: it measured faster at every factor
    const bool pair = g_algo == 1 ? g.M >= 256
                                  : (g_algo == 2 && g.M >= 256 && (stream_k || g.split_k > 1 || tiles256 >= sm_count_current_device() / 2));
    if (pair) return gemm_bf16_pair(g, stream);
  }
  if (g.a_mn == 0 && g.b_mn == 0) return launch<0, 0>(g, stream);
  if (g.a_mn == 0 && g.b_mn == 1) return launch<0, 1>(g, stream);
  if (g.a_mn == 1 && g.b_mn == 0) return launch<1, 0>(g, stream);
  return launch<1, 1>(g, stream);
}

}  // namespace z2h

#ifdef Z2H_KERNEL_TRACE
extern "C" int z2h_gemm_trace_read(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_kernel_trace, sizeof(g_kernel_trace));
}
#endif
extern "C" void z2h_gemm_set_algo(int algo) { z2h::gemm_set_algo(algo); }
extern "C" void z2h_gemm_set_fixup(int on) { z2h::gemm_set_fixup(on); }
extern "C" int z2h_gemm_get_algo() { return z2h::gemm_get_algo(); }
namespace z2h {
namespace {
__global__ void fold_slices_kernel(const float* __restrict__ slices, int num_slices, long long n4,
                                   float* __restrict__ dst) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(dst)[i];
    for (int s = 0; s < num_slices; ++s) {  // slice order: the sum is the same bits every time
      const float4 v = reinterpret_cast<const float4*>(slices)[(long long)s * n4 + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(dst)[i] = acc;
  }
}
}  // namespace
int gemm_fold_slices(const float* slices, int num_slices, long long n, float* dst, cudaStream_t stream) {
  if (n % 4 != 0 || num_slices < 1 || (reinterpret_cast<uintptr_t>(slices) & 15) ||
      (reinterpret_cast<uintptr_t>(dst) & 15))
    return 1;
  const long long n4 = n / 4;
  const int grid = (int)((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
  fold_slices_kernel<<<grid < 1 ? 1 : grid, 256, 0, stream>>>(slices, num_slices, n4, dst);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
}  // namespace z2h

extern "C" int z2h_gemm_fold_slices(const float* slices, int num_slices, long long n, float* dst, void* stream) {
  return z2h::gemm_fold_slices(slices, num_slices, n, dst, reinterpret_cast<cudaStream_t>(stream));
}

// z2h_gemm_bf16 plus the column-sum by-product (GemmArgs::colsum) and the K-slice stride of
// kEpiSliceStore (GemmArgs::slice_stride).
extern "C" int z2h_gemm_bf16_ex(const void* A, int a_mn, long long lda, const void* B, int b_mn,
                                long long ldb, void* C, long long ldc, int out_fp32, int M, int N, int K,
                                int epi, int split_k, const void* bias, const void* residual,
                                long long ldr, void* aux_out, const void* aux_in, long long ldaux,
                                int* status, int max_ctas, void* colsum, long long slice_stride, void* stream) {
  z2h::GemmArgs g;
  g.A = A; g.a_mn = a_mn; g.lda = lda;
  g.B = B; g.b_mn = b_mn; g.ldb = ldb;
  g.C = C; g.ldc = ldc; g.out_fp32 = out_fp32;
  g.M = M; g.N = N; g.K = K;
  g.epi = epi; g.split_k = split_k;
  g.bias = bias; g.residual = residual; g.ldr = ldr;
  g.aux_out = aux_out; g.aux_in = aux_in; g.ldaux = ldaux;
  g.status = status; g.max_ctas = max_ctas;
  g.colsum = colsum;
  g.slice_stride = slice_stride;
  return z2h::gemm_bf16(g, reinterpret_cast<cudaStream_t>(stream));
}
extern "C" int z2h_gemm_bf16_colsum(const void* A, int a_mn, long long lda, const void* B, int b_mn,
                                    long long ldb, void* C, long long ldc, int out_fp32, int M, int N, int K,
                                    int epi, int split_k, const void* bias, const void* residual,
                                    long long ldr, void* aux_out, const void* aux_in, long long ldaux,
                                    int* status, int max_ctas, void* colsum, void* stream) {
  return z2h_gemm_bf16_ex(A, a_mn, lda, B, b_mn, ldb, C, ldc, out_fp32, M, N, K, epi, split_k, bias, residual,
                          ldr, aux_out, aux_in, ldaux, status, max_ctas, colsum, 0, stream);
}
extern "C" int z2h_gemm_bf16(const void* A, int a_mn, long long lda, const void* B, int b_mn,
                             long long ldb, void* C, long long ldc, int out_fp32, int M, int N, int K,
                             int epi, int split_k, const void* bias, const void* residual,
                             long long ldr, void* aux_out, const void* aux_in, long long ldaux,
                             int* status, int max_ctas, void* stream) {
  return z2h_gemm_bf16_colsum(A, a_mn, lda, B, b_mn, ldb, C, ldc, out_fp32, M, N, K, epi, split_k, bias,
                              residual, ldr, aux_out, aux_in, ldaux, status, max_ctas, nullptr, stream);
}
