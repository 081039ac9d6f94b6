// bf16 GEMM on CTA pairs: C[M,N] = A[M,K] * B[N,K]^T with tcgen05.mma.cta_group::2.
//
// Two CTAs of a cluster (two neighbouring SMs) work on one 256 x 256 output tile. Each CTA
// loads 128 rows of A and 128 of the 256 rows of B per K-block (32 KiB instead of the 48 KiB a
// lone CTA needs for a 128 x 256 tile), the even CTA issues one MMA of shape 256 x 256 x 16 for
// both, and each CTA keeps its 128 x 256 half of the fp32 accumulator in its own tensor
// memory. Per SM this halves the B traffic through shared memory, which is what bounds the
// one-CTA kernel (128 B/clk per SM against 192 B/clk wanted); a 6-stage ring fits instead of 4.
//
// Synchronisation: the "full" barrier of a stage lives in the even CTA and counts the bytes of
// both CTAs' TMA loads (the odd CTA's loads name that barrier; there is no multicast load,
// every CTA fetches its own tiles). Stage release and accumulator completion are
// tcgen05.commit arrivals multicast to the same barrier offset in both CTAs. The epilogue
// warps of both CTAs arrive on the even CTA's "accumulator drained" barrier.
// Warp roles, epilogues, split-K and operand layouts are those of gemm_tcgen05.cu.
#include <cstdlib>
#include <mutex>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "gemm.h"
#include "../common/trace.cuh"
#include "gemm_epilogue.cuh"

namespace z2h {
namespace {

using gemm_detail::KernelParams;

constexpr int TM = 256;        // tile rows per CTA pair
constexpr int HM = 128;        // tile rows per CTA
constexpr int BN = 256;        // tile columns
constexpr int HN = 128;        // B rows loaded per CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = HM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = HN * BK * 2;  // 16 KiB
constexpr int NUM_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES =
    STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256 + EPI_WARPS * gemm_detail::kEpiWarpBytes;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB a CTA may use");

// FIXUP: the instantiation that can run stream-K with fix-up (KernelParams::stream_k == 2). Its
// epilogue needs a warp's whole piece of a tile in registers at once, which costs register spills;
// the kernels every other launch uses are compiled without that path.
// EXTRA: the instantiation that carries the newer epilogue kinds (see epilogue_tile_streamed).
template <int A_MN, int B_MN, bool FIXUP, bool EXTRA>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const KernelParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sA = smem_raw;
  uint8_t* sB = smem_raw + STAGES * A_STAGE_BYTES;
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
  const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs), 1 = peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const bool aligned = (smem_u32(smem_raw) & 1023u) == 0;

  // every role of both CTAs walks the same sequence of work segments (none if misaligned)
  gemm_detail::TileScheduler sched(p, TM, BN, BK, aligned ? pair : 0, aligned ? num_pairs : 1);
  if (!aligned) sched.total_items = 0, sched.u_end = sched.u;
  gemm_detail::Segment sg;
  if (!aligned && threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, (int)kBadArgument);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * EPI_WARPS);  // the epilogue warps of both CTAs of the pair
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers must exist before any remote arrival or load completion targets them
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // everything above overlaps the previous kernel's tail; global memory from here on

  if (warp == 0) {
    // ------------------------------ TMA producer (one per CTA) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Z2H_TRACE_DECL(0)
      Z2H_TRACE();
      while (ok && sched.next(sg)) {
        const int mt = sg.mt, nt = sg.nt, kb0 = sg.kb0, kb1 = sg.kb1;
        const int m0 = mt * TM + (int)rank * HM;
        const int n0 = nt * BN + (int)rank * HN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, kTimeoutEmpty)) {
            ok = false;
            break;
          }
          Z2H_TRACE();
          // the leader's barrier counts the bytes of both CTAs
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
          if (A_MN == 0) {
            tma_load_2d_pair(a_dst, &tmA, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < HM / 64; ++c)
              tma_load_2d_pair(a_dst + c * (64 * BK * 2), &tmA, &full_bar[stage], m0 + c * 64, kb * BK);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(b_dst, &tmB, &full_bar[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < HN / 64; ++c)
              tma_load_2d_pair(b_dst + c * (64 * BK * 2), &tmB, &full_bar[stage], n0 + c * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TM, BN, A_MN, B_MN);
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
        if (!mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, kTimeoutTmemEmpty)) {
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
          const uint64_t adesc0 = make_smem_desc_sw128(smem_u32(sA + stage * A_STAGE_BYTES), a_lbo, 1024);
          const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(sB + stage * B_STAGE_BYTES), b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16_ss_2cta(d_tmem, desc_advance(adesc0, k * a_kstep), desc_advance(bdesc0, k * b_kstep),
                               idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          tc_commit_2cta(&empty_bar[stage], 3);  // frees the stage in both CTAs
          Z2H_TRACE();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit_2cta(&tfull_bar[acc], 3);
      }
    }
  } else {
    // ------------------------------ epilogue (8 warps per CTA) ------------------------------
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
      if (!empty_split) gemm_detail::prefetch_second_operand(p, (long long)mt * TM + (long long)rank * HM + quarter * 32 + lane, gcol0);
      if (!mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (warp == 2 && lane == 0) Z2H_TRACE();
      const long long row_base = (long long)mt * TM + (long long)rank * HM + quarter * 32;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      // this warp drains 4 of the 8 column blocks of its 32 rows
      const int c0 = half * 4;
      uint64_t* const tempty = &tempty_bar[acc];
      if (!FIXUP || p.stream_k != 2) {
        gemm_detail::epilogue_tile_streamed<EXTRA>(p, taddr + c0 * 32, row_base + lane, gcol0, sbias, lane,
                                            smem_u32(epi_bias + (warp - 2) * gemm_detail::kEpiBiasFloats),
                                            !empty_split, (EXTRA && p.split_k > 1) ? sg.kb0 / sched.kb_per_split : 0,
                                            [tempty] { mbar_arrive_leader_relaxed(tempty); });
        if (warp == 2 && lane == 0) Z2H_TRACE();
        continue;
      }
      // Stream-K with fix-up needs the warp's whole 32 x 128 piece at once (it is parked in, or
      // completed from, the workspace): all four tensor-memory loads issued back to back and
      // awaited once, the accumulator handed back as soon as it is in registers.
      uint32_t r[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(taddr + (c0 + c) * 32, r[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty_bar[acc]);
      if (warp == 2 && lane == 0) Z2H_TRACE();
      if (p.stream_k == 2 && !empty_split) {
        // Stream-K with fix-up. A run of k-blocks may start inside a tile (this worker then has
        // the tile's tail, the previous worker its head) and may end inside one (this worker has
        // the head, the next worker the tail). The tail comes first in a run, so it is parked in the
        // workspace early; the head comes last, so by the time its owner wants the other piece it
        // has long been there. Both workers map the tile to warps and lanes identically, so a
        // warp exchanges with the same warp of the neighbouring pair, 128 bytes per instruction.
        const int slot = ((int)rank * EPI_WARPS + (warp - 2));
        if (sg.kb0 > 0) {  // tail piece: park it, no epilogue
          float* ws = p.sk_ws + ((long long)pair * 2 * EPI_WARPS + slot) * gemm_detail::kSkWarpFloats + lane;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(ws + (c * 32 + j) * 32, __uint_as_float(r[c][j]));
          __threadfence();
          __syncwarp();
          if (lane == 0)
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.sk_flags + pair * 2 * EPI_WARPS + slot), "r"(1)
                         : "memory");
          continue;
        }
        if (sg.kb1 < sched.num_kb) {  // head piece: fetch the neighbour's tail, then the epilogue
          int* flag = p.sk_flags + (pair + 1) * 2 * EPI_WARPS + slot;
          int got = 0;
          if (lane == 0) {
            const uint64_t t0 = globaltimer_ns();
            while (true) {
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(got) : "l"(flag) : "memory");
              if (got != 0) break;
              if (*abort_flag != 0 || globaltimer_ns() - t0 > Z2H_WAIT_BUDGET_NS) {
                *abort_flag = 1;
                if (p.status != nullptr) atomicCAS(p.status, 0, (int)kTimeoutLocal);
                break;
              }
            }
          }
          got = __shfl_sync(0xffffffffu, got, 0);
          if (got == 0) {
            ok = false;
            break;
          }
          const float* ws =
              p.sk_ws + ((long long)(pair + 1) * 2 * EPI_WARPS + slot) * gemm_detail::kSkWarpFloats + lane;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int j = 0; j < 32; ++j)
              r[c][j] = __float_as_uint(__uint_as_float(r[c][j]) + __ldcg(ws + (c * 32 + j) * 32));
          __syncwarp();
          if (lane == 0) *flag = 0;  // consumed: the next launch starts from a clear flag
        }
      }
      if (!empty_split)
        gemm_detail::epilogue_tile(p, r, row_base + lane, gcol0, sbias, lane,
                                   smem_u32(epi_bias + (warp - 2) * gemm_detail::kEpiBiasFloats));
      if (warp == 2 && lane == 0) Z2H_TRACE();
    }
  }

  // nobody leaves while the other CTA may still signal or read this CTA's barriers / memory
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

// Workspace of the stream-K fix-up mode: one 256 KiB slot and 16 flags per CTA pair of the current
// device, allocated on first use (never while the stream is being captured: the first use then
// simply keeps the whole-tile schedule) and kept until the process ends. The mode is off by default
// (see the measurements where it is chosen); Z2H_GEMM_FIXUP=1 or gemm_set_fixup(1) turn it on.
int g_fixup = -1;  // -1: not decided yet (environment), 0 off, 1 on
bool fixup_enabled() {
  if (g_fixup < 0) {
    const char* e = std::getenv("Z2H_GEMM_FIXUP");
    g_fixup = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return g_fixup == 1;
}

bool fixup_workspace(cudaStream_t stream, float** ws, int** flags) {
  static std::mutex mu;
  static float* ws_dev[64] = {};
  static int* flags_dev[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (ws_dev[dev] == nullptr) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return false;
    const int pairs = sm_count_current_device() / 2 + 1;
    float* w = nullptr;
    int* f = nullptr;
    if (cudaMalloc(&w, (size_t)pairs * gemm_detail::kSkPairFloats * sizeof(float)) != cudaSuccess) return false;
    if (cudaMalloc(&f, (size_t)pairs * 2 * EPI_WARPS * sizeof(int)) != cudaSuccess) {
      cudaFree(w);
      return false;
    }
    cudaMemset(f, 0, (size_t)pairs * 2 * EPI_WARPS * sizeof(int));
    cudaDeviceSynchronize();
    ws_dev[dev] = w;
    flags_dev[dev] = f;
  }
  *ws = ws_dev[dev];
  *flags = flags_dev[dev];
  return true;
}

template <int A_MN, int B_MN>
int launch_pair(const GemmArgs& g, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  bool ok;
  if (A_MN == 0)
    ok = make_tma_2d_bf16(&tmA, g.A, g.M, g.K, g.lda, HM, BK, kSwizzle128);
  else
    ok = make_tma_2d_bf16(&tmA, g.A, g.K, g.M, g.lda, BK, 64, kSwizzle128);
  if (!ok) return 2;
  if (B_MN == 0)
    ok = make_tma_2d_bf16(&tmB, g.B, g.N, g.K, g.ldb, HN, BK, kSwizzle128);
  else
    ok = make_tma_2d_bf16(&tmB, g.B, g.K, g.N, g.ldb, BK, 64, kSwizzle128);
  if (!ok) return 2;
  KernelParams p = gemm_detail::make_kernel_params(g);
  p.raster_n = gemm_detail::pick_raster_n(g, TM, BN);
  const int num_sms_all = sm_count_current_device();
  {
    // Stream-K with fix-up for tile counts that leave a ragged last wave (192 tiles on 74 pairs =
    // 2.6 waves): OFF unless switched on (Z2H_GEMM_FIXUP=1 / gemm_set_fixup). Measured on B200 it
    // loses everywhere it was tried: M16384 N768 K3072 76.8 us against 72.7 us, N768 K768 35.8 against
    // 28.7, N3072 K768 79.9 against 67.6, and even the long-K data gradient of the lm_head (K = 50304)
    // 1133 us against 969 us. Two reasons: every pair parks and fetches one fp32 tile (19 MB each way
    // per launch), and pairs that walk contiguous runs sit at different k offsets of different tiles, so
    // the B panel that the whole-tile schedule shares out of L2 (all pairs stream the same k-blocks in
    // step) is re-read from DRAM. The mode stays as a tested option for shapes with few, very long tiles.
    int pairs_avail = num_sms_all / 2;
    if (g.max_ctas > 0 && pairs_avail > g.max_ctas / 2) pairs_avail = g.max_ctas / 2 > 0 ? g.max_ctas / 2 : 1;
    const long long tiles_sk = (long long)((g.M + TM - 1) / TM) * ((g.N + BN - 1) / BN);
    const int num_kb = (g.K + BK - 1) / BK;
    const bool plain = p.stream_k == 0 && p.split_k == 1 && g.epi != kEpiAtomicAdd && g.epi != kEpiAccumulate &&
                       g.epi < kEpiGeluSaveGrad && !g.out_fp32;  // (the newer kinds have no fix-up instantiation)
    if (plain && fixup_enabled() && tiles_sk >= pairs_avail && num_kb >= 8) {
      const double waves = (double)tiles_sk / pairs_avail;
      const double whole = (double)((tiles_sk + pairs_avail - 1) / pairs_avail);
      if (waves + 0.1 < 0.96 * whole) {  // the balanced schedule is shorter on paper
        float* ws = nullptr;
        int* flags = nullptr;
        if (fixup_workspace(stream, &ws, &flags)) {
          p.stream_k = 2;
          p.sk_ws = ws;
          p.sk_flags = flags;
        }
      }
    }
  }

  const bool extra = g.epi >= kEpiGeluSaveGrad;
  auto kern = extra ? gemm_bf16_2cta_kernel<A_MN, B_MN, false, true>
                    : (p.stream_k == 2 ? gemm_bf16_2cta_kernel<A_MN, B_MN, true, false>
                                       : gemm_bf16_2cta_kernel<A_MN, B_MN, false, false>);
  static std::atomic<unsigned long long> attr_seen{0};
  if (first_use_on_current_device(attr_seen)) {
    cudaFuncSetAttribute(gemm_bf16_2cta_kernel<A_MN, B_MN, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_2cta_kernel<A_MN, B_MN, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_2cta_kernel<A_MN, B_MN, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  }
  const int num_sms = num_sms_all;
  const long long tiles = (long long)((g.M + TM - 1) / TM) * ((g.N + BN - 1) / BN) *
                          (p.stream_k ? (g.K + BK - 1) / BK : p.split_k);
  int pairs = num_sms / 2;
  if (g.max_ctas > 0 && pairs > g.max_ctas / 2) pairs = g.max_ctas / 2 > 0 ? g.max_ctas / 2 : 1;
  if (tiles < pairs) pairs = (int)tiles;
  if (pairs < 1) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p) == cudaSuccess ? 0 : 3;
}

}  // namespace

void gemm_set_fixup(int on) { g_fixup = on ? 1 : 0; }

int gemm_bf16_pair(const GemmArgs& g, cudaStream_t stream) {
  if (g.a_mn == 0 && g.b_mn == 0) return launch_pair<0, 0>(g, stream);
  if (g.a_mn == 0 && g.b_mn == 1) return launch_pair<0, 1>(g, stream);
  if (g.a_mn == 1 && g.b_mn == 0) return launch_pair<1, 0>(g, stream);
  return launch_pair<1, 1>(g, stream);
}

}  // namespace z2h

#ifdef Z2H_KERNEL_TRACE
extern "C" int z2h_gemm_trace_read_pair(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_kernel_trace, sizeof(g_kernel_trace));
}
#endif
