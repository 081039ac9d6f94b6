// Causal flash attention backward, head_dim 64, bf16, on tcgen05 tensor cores.
//
// One CTA owns one KV tile (128 keys of one batch/head) and walks the query tiles from the
// diagonal to the end of the sequence. All five products of the backward run on the tensor
// cores, with the "transposed" formulation so that a thread owns one key row:
//
//   S^T  = K  Q^T          (128 x 128 x 64)    TMEM cols   0..127
//   dP^T = V  dO^T         (128 x 128 x 64)    TMEM cols 128..255
//   P^T  = exp(S^T * scale - lse),  dS^T = P^T o (dP^T - delta)        (threads, fp32)
//   dV  += P^T  dO         (128 x 64 x 128)    TMEM cols 256..319, accumulated over q tiles
//   dK  += dS^T Q          (128 x 64 x 128)    TMEM cols 320..383, accumulated over q tiles
//   dQ_i = dS K            (128 x 64 x 128)    TMEM cols 384..447, added to an fp32 buffer
//   P^T as packed bf16 pairs                   TMEM cols 448..511
//
// P^T goes back to tensor memory (tcgen05.st) and is the A operand of the dV product from there;
// dS^T is written once to swizzled shared memory as bf16 and is consumed as the K-major A operand
// of the dK product and as the MN-major A operand of the dQ product; Q, dO and K tiles serve as
// K-major or MN-major B operands straight from their TMA tiles, so nothing is transposed in
// memory. dQ contributions of different KV tiles meet in an fp32 accumulation buffer (vector
// red.global.add into a blocked layout in which a warp's 32 rows are contiguous), which a small
// kernel scales, converts and writes row-major.
//
// Pipeline: the scores of query tile i+1 are issued as soon as the compute warps hold tile i's
// scores in registers, three Q / dO stages keep two tiles of operands in flight, the dQ of tile
// i-1 is read out while the products of tile i run.
//
// Roles (20 warps): warp 0 issues the TMA copies; warps 1, 2 and 3 each have one thread that issues
// MMAs (S^T / dP^T and dV; dK; dQ), so that the three products of a tile are issued from three
// schedulers at once; warps 4-19 do the arithmetic, four per tensor-memory lane quarter with 32
// query columns each.
//
// By-product: the column sums of dK and dV (this kernel's epilogue) and of dQ (the conversion kernel)
// can be added to an fp32 vector, which is the gradient of the QKV projection's bias.
// Reproducible form (flash_bwd_ex, ordered): one launch per KV tile, so the additions to the fp32 dQ
// buffer happen in KV-tile order.
//
// This is the hand-written counterpart of what autograd runs for
// F.scaled_dot_product_attention in the reference (nn/gpt2/modules.py:37, train_ddp.py:141).
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "attn.h"
#include "../common/trace.cuh"
#include "../common/dropout.cuh"
#include "../common/warp_colsum.cuh"
#include <cstdlib>

namespace z2h {
namespace {

constexpr int TS = 128;  // tile size (queries and keys)
constexpr int HD = 64;
constexpr int TILE_BYTES = TS * HD * 2;  // 16 KiB
constexpr int PT_BYTES = TS * TS * 2;    // 32 KiB
constexpr int Q_STAGES = 3;
// Warp 0 loads (TMA), warps 1-3 issue MMAs (one thread each), warps 4-19 compute: four per
// tensor-memory lane quarter, each taking 32 of the 128 query columns of its 32 key rows.
//
// Why three issuing threads. A tcgen05.mma of this kernel's shapes occupies the tensor pipe for
// 43 cycles (A from tensor memory, N 64), 76 (A from shared memory, N 64) or 107 (N 128): measured
// with one CTA issuing back to back. Those figures hold only while the issuing warp gets issue
// slots: with the compute warps of the same scheduler busy, one thread needed 106 cycles per MMA for
// the dV / dK products instead of 60, and the issuing thread, not the tensor pipe, set the tile
// period. dV, dK and dQ of a tile are independent, so each has its own issuing thread on its own
// scheduler and the three streams interleave in the pipe.
constexpr int NUM_SPECIAL_WARPS = 4;
constexpr int NUM_COMPUTE = 512;
constexpr int NUM_THREADS = NUM_SPECIAL_WARPS * 32 + NUM_COMPUTE;
constexpr int WCOLS = 32;  // query columns per compute warp
constexpr int TMEM_COLS = 512;
// S^T and dP^T (fp32, 128 columns each), the dV / dK / dQ accumulators (64 each) and P^T as packed
// bf16 pairs (64 columns): all 512 columns
constexpr int ST_COL = 0, DPT_COL = 128, DV_COL = 256, DK_COL = 320, DQ_COL = 384, PT_COL = 448;
constexpr int P_BUFS = 2;  // dS^T is double-buffered in shared memory; P^T lives in tensor memory
constexpr int SMEM_BYTES =
    2 * TILE_BYTES + 2 * Q_STAGES * TILE_BYTES + P_BUFS * PT_BYTES + Q_STAGES * 2 * TS * 4 + 256;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB a CTA may use");

struct BwdParams {
  const float* stats;  // [2][B*H][Tpad]: lse * log2(e), then delta; zero beyond T
  int Tpad;
  __nv_bfloat16* dqkv;
  float* dq_accum;
  int B, T, H, C;
  float scale, scale_log2;
  int* status;
  // fp32 [3C] or null: the column sums of dqkv (as stored) are added here, i.e. the gradient of the
  // QKV projection's bias; the dK / dV thirds by this kernel's epilogue, the dQ third by the
  // conversion kernel
  float* dbias;
  // >= 0: this launch covers only KV tile j_fixed of every (batch, head) (grid = B * H). The host then
  // launches the tiles one after the other, so the additions to the fp32 dQ buffer happen in KV-tile
  // order whatever the CTA scheduling: the bitwise reproducible form, about 1.5 x slower.
  int j_fixed;
  // attention-probability dropout (DROP instantiation only), same stream as the forward kernel
  float drop_p;
  const unsigned long long* seed_ptr;
  uint32_t site;
};

// DROP: with M the keep mask and s = 1/(1-p), the forward used P~ = P o M * s in P V. Then
// dV = P~^T dO, dP = (dO V^T) o M * s, and dS = P o (dP - delta) with delta = rowsum(dO o O)
// unchanged, so the mask enters in two places of the per-element code and nowhere else.
template <bool DROP>
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                 const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  pdl_launch_dependents();
  if (smem_u32(smem_raw) & 1023u) {  // the swizzled tiles need a 1 KiB aligned base
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, (int)kBadArgument);
    return;
  }
  uint8_t* sK = smem_raw;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;
  uint8_t* sdO = sQ + Q_STAGES * TILE_BYTES;
  uint8_t* sdSt = sdO + Q_STAGES * TILE_BYTES;
  float* sLse = reinterpret_cast<float*>(sdSt + P_BUFS * PT_BYTES);  // [Q_STAGES][TS], already * log2(e)
  float* sDelta = sLse + Q_STAGES * TS;                      // [Q_STAGES][TS]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDelta + Q_STAGES * TS);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = qdo_full + Q_STAGES;
  uint64_t* st_full = qdo_empty + Q_STAGES;
  uint64_t* pds_full = st_full + 1;
  uint64_t* dq_full = pds_full + 1;   // the three products of a tile are complete
  uint64_t* s_read = dq_full + 1;     // the compute warps hold S^T / dP^T of the tile in registers
  uint64_t* dv_done = s_read + 1;     // dV of the tile is complete: P^T may be overwritten
  uint64_t* dq_empty = dv_done + 1;   // the compute warps have read the dQ accumulator
  uint64_t* dk_done = dq_empty + 1;   // dK of the tile is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dk_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = (p.T + TS - 1) / TS;
  // KV tile 0 has the most query tiles to visit: schedule it first
  const int j = p.j_fixed >= 0 ? p.j_fixed : (int)(blockIdx.x % n_t);
  const int bh = p.j_fixed >= 0 ? (int)blockIdx.x : (int)(blockIdx.x / n_t);
  const int h = bh % p.H, b = bh / p.H;
  const int row0 = b * p.T;
  const int n_iter = n_t - j;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 2);  // the dV thread (after S^T, dP^T, dV) and the dK thread
    }
    mbar_init(st_full, 1);
    mbar_init(pds_full, NUM_COMPUTE / 32);
    mbar_init(dq_full, 1);
    mbar_init(s_read, NUM_COMPUTE / 32);
    mbar_init(dv_done, 1);
    mbar_init(dq_empty, NUM_COMPUTE / 32);
    mbar_init(dk_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_qkv);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // the set-up above overlaps the previous kernel's tail; global memory from here on

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_2d(sK, &tm_qkv, kv_full, p.C + h * HD, row0 + j * TS);
      tma_load_2d(sV, &tm_qkv, kv_full, 2 * p.C + h * HD, row0 + j * TS);
      Z2H_TRACE_DECL(0)
      Z2H_TRACE();
      for (int it = 0; it < n_iter; ++it) {
        const int i = j + it;
        const int s = it % Q_STAGES;
        const uint32_t ph = (it / Q_STAGES) & 1;
        if (!mbar_wait_bounded(&qdo_empty[s], ph ^ 1u, abort_flag, p.status, kTimeoutEmpty)) break;
        Z2H_TRACE();
        mbar_arrive_expect_tx(&qdo_full[s], 2 * TILE_BYTES + 2 * TS * 4);
        tma_load_2d(sQ + s * TILE_BYTES, &tm_qkv, &qdo_full[s], h * HD, row0 + i * TS);
        tma_load_2d(sdO + s * TILE_BYTES, &tm_do, &qdo_full[s], h * HD, row0 + i * TS);
        const float* st_row = p.stats + (long long)bh * p.Tpad + i * TS;
        bulk_load_1d(sLse + s * TS, st_row, TS * 4, &qdo_full[s]);
        bulk_load_1d(sDelta + s * TS, st_row + (long long)p.B * p.H * p.Tpad, TS * 4, &qdo_full[s]);
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(TS, TS, 0, 0);
      constexpr uint32_t idesc_dvk = make_idesc_bf16(TS, HD, 0, 1);
      // descriptors are built once; inside the loop an MMA costs one 64-bit add per operand
      const uint64_t k_desc = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t v_desc = make_smem_desc_sw128(smem_u32(sV), 16, 1024);
      uint64_t q_desc[Q_STAGES], do_desc[Q_STAGES];
#pragma unroll
      for (int s = 0; s < Q_STAGES; ++s) {
        q_desc[s] = make_smem_desc_sw128(smem_u32(sQ + s * TILE_BYTES), 16, 1024);
        do_desc[s] = make_smem_desc_sw128(smem_u32(sdO + s * TILE_BYTES), 16, 1024);
      }
      auto issue_st = [&](int s) {
        const uint64_t qd = s == 0 ? q_desc[0] : (s == 1 ? q_desc[1] : q_desc[2]);
        const uint64_t dod = s == 0 ? do_desc[0] : (s == 1 ? do_desc[1] : do_desc[2]);
        // the two products accumulate into different tensor-memory columns: issued alternately,
        // neither waits for the other's previous step
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          tc_mma_f16_ss(tmem_base + ST_COL, desc_advance(k_desc, k * 32), desc_advance(qd, k * 32),
                        idesc_st, k > 0);
          tc_mma_f16_ss(tmem_base + DPT_COL, desc_advance(v_desc, k * 32), desc_advance(dod, k * 32),
                        idesc_st, k > 0);
        }
        tc_commit(st_full);
      };
      Z2H_TRACE_DECL(1)
      Z2H_TRACE();
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag, p.status, kTimeoutFull);
      if (ok) ok = mbar_wait_bounded(&qdo_full[0], 0, abort_flag, p.status, kTimeoutFull);
      Z2H_TRACE();
      if (ok) {
        tc_fence_after();
        issue_st(0);
      }
      Z2H_TRACE();
      // Per tile `it`:
      //   S^T, dP^T of it+1   as soon as the compute warps hold the scores of tile `it` in
      //                       registers (s_read), i.e. while they still work on tile `it`; three
      //                       Q / dO stages keep the operands of tiles it+1 and it+2 in flight
      //   dV += P^T dO        once P^T (tensor memory) is written; the A operand comes straight
      //                       from tensor memory
      // (dK += dS^T Q and dQ = dS K are issued by warps 2 and 3)
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % Q_STAGES;
        if (it + 1 < n_iter) {
          const int s2 = (it + 1) % Q_STAGES;
          const uint32_t ph2 = ((it + 1) / Q_STAGES) & 1;
          if (!mbar_wait_bounded(s_read, it & 1, abort_flag, p.status, kTimeoutLocal)) break;
          if (!mbar_wait_bounded(&qdo_full[s2], ph2, abort_flag, p.status, kTimeoutFull)) break;
          tc_fence_after();
          issue_st(s2);
        }
        Z2H_TRACE();
        if (!mbar_wait_bounded(pds_full, it & 1, abort_flag, p.status, kTimeoutLocal)) break;
        Z2H_TRACE();
        tc_fence_after();
        const uint64_t dod = s == 0 ? do_desc[0] : (s == 1 ? do_desc[1] : do_desc[2]);
#pragma unroll
        for (int k = 0; k < TS / 16; ++k) {  // queries 16k..16k+15 of P^T are 8 packed columns
          tc_mma_f16_ts(tmem_base + DV_COL, tmem_base + PT_COL + k * 8, desc_advance(dod, k * 2048),
                        idesc_dvk, (it > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(dv_done);
        tc_commit(&qdo_empty[s]);  // covers this thread's earlier reads of the stage (S^T, dP^T) too
        Z2H_TRACE();
      }
    }
  } else if (warp == 2) {
    // dK += dS^T Q: A is dS^T of the tile (shared memory, K-major), B the Q tile (MN-major)
    if (lane == 0) {
      constexpr uint32_t idesc_dvk = make_idesc_bf16(TS, HD, 0, 1);
      const uint64_t dst_desc = make_smem_desc_sw128(smem_u32(sdSt), 16, 1024);
      uint64_t q_desc[Q_STAGES];
#pragma unroll
      for (int s = 0; s < Q_STAGES; ++s) q_desc[s] = make_smem_desc_sw128(smem_u32(sQ + s * TILE_BYTES), 16, 1024);
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % Q_STAGES;
        const uint32_t pb = (it & 1) * PT_BYTES;
        if (!mbar_wait_bounded(&qdo_full[s], (it / Q_STAGES) & 1, abort_flag, p.status, kTimeoutFull)) break;
        if (!mbar_wait_bounded(pds_full, it & 1, abort_flag, p.status, kTimeoutLocal)) break;
        tc_fence_after();
        const uint64_t qd = s == 0 ? q_desc[0] : (s == 1 ? q_desc[1] : q_desc[2]);
#pragma unroll
        for (int k = 0; k < TS / 16; ++k) {
          const uint32_t a_off = pb + (k >> 2) * (TS * 128) + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + DK_COL, desc_advance(dst_desc, a_off), desc_advance(qd, k * 2048),
                        idesc_dvk, (it > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(dk_done);
        tc_commit(&qdo_empty[s]);
      }
    }
  } else if (warp == 3) {
    // dQ = dS K: A is dS read MN-major from the dS^T tile, B the K tile (MN-major); the compute warps
    // must have read the previous tile's dQ out of the accumulator first
    if (lane == 0) {
      constexpr uint32_t idesc_dq = make_idesc_bf16(TS, HD, 1, 1);
      const uint64_t k_desc = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t dst_mn_desc = make_smem_desc_sw128(smem_u32(sdSt), TS * 128, 1024);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag, p.status, kTimeoutFull);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t pb = (it & 1) * PT_BYTES;
        if (!mbar_wait_bounded(pds_full, it & 1, abort_flag, p.status, kTimeoutLocal)) break;
        if (it > 0 && !mbar_wait_bounded(dq_empty, (it - 1) & 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < TS / 16; ++k) {
          tc_mma_f16_ss(tmem_base + DQ_COL, desc_advance(dst_mn_desc, pb + k * 2048),
                        desc_advance(k_desc, k * 2048), idesc_dq, k > 0);
        }
        tc_commit(dq_full);
      }
    }
  } else {
    // Four warps share each TMEM lane quarter: warp (4 + q + 4 * part) takes query columns
    // part*32 .. part*32+31 of a key row, so every SM sub-partition has four compute warps.
    const int quarter = warp & 3;
    const int part = (warp - NUM_SPECIAL_WARPS) >> 2;   // 0..3: which 32 query columns
    const int half = part >> 1;         // which 64-column swizzle atom of dS^T
    const int sub = part & 1;           // which 32-column half of that atom
    const int r = quarter * 32 + lane;  // key row (S^T, dV, dK) or query row (dQ) == TMEM lane
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    const uint32_t dst_row = smem_u32(sdSt) + half * (TS * 128) + r * 128;
    // dQ of tile `t` (TMEM lane == query row; this warp takes 32 of the 64 columns) is added to
    // the fp32 accumulation buffer; the accumulator is handed back as soon as it is in registers
    auto drain_dq = [&](int t) {
      tc_fence_after();
      const int tq = (j + t) * TS + r;
      // blocked layout [row / 32][head][16-byte column group][row % 32]: the 32 lanes of a warp
      // (32 consecutive rows) hit 512 contiguous bytes per instruction instead of 32 rows
      const long long g = (long long)row0 + tq;
      float* dq_row = p.dq_accum + ((((g >> 5) * p.H + h) * 16 + part * 4) * 32 + (g & 31)) * 4;
      uint32_t v[16];
      tmem_ld_32x32b_x16(t_lane + DQ_COL + part * 16, v);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
      if (tq < p.T) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq_row + q * 128),
                       "f"(__uint_as_float(v[q * 4 + 0])), "f"(__uint_as_float(v[q * 4 + 1])),
                       "f"(__uint_as_float(v[q * 4 + 2])), "f"(__uint_as_float(v[q * 4 + 3]))
                       : "memory");
        }
      }
      tc_fence_before();
    };
    DropoutSpec drop = {};
    if (DROP) drop = make_dropout_spec(p.seed_ptr, p.site, p.drop_p);
    const unsigned long long drop_wpr = (unsigned long long)((p.T + 3) / 4);  // mask words per query row
    const int drop_byte = (j * TS + r) & 3;
    bool ok = true;
    Z2H_TRACE_DECL(2)
#define Z2H_CTRACE()                      \
  do {                                    \
    if (warp == NUM_SPECIAL_WARPS && lane == 0) Z2H_TRACE(); \
  } while (0)
    Z2H_CTRACE();
    for (int it = 0; it < n_iter; ++it) {
      const int i = j + it;
      const int s = it % Q_STAGES;
      // the per-query statistics of this q tile arrive with the Q / dO tiles (bulk copies)
      if (!mbar_wait_bounded(&qdo_full[s], (it / Q_STAGES) & 1, abort_flag, p.status, kTimeoutFull)) {
        ok = false;
        break;
      }
      Z2H_CTRACE();  // Q / dO tile and statistics are there
      if (!mbar_wait_bounded(st_full, it & 1, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      Z2H_CTRACE();  // scores are there
      const uint32_t pb = (it & 1) * PT_BYTES;  // which P^T / dS^T buffer this tile uses
      // mask word of (first query of tile i, this thread's key); one row of words per query
      const unsigned long long drop_q0 =
          DROP ? ((unsigned long long)bh * p.T + (unsigned long long)i * TS) * drop_wpr + (unsigned long long)((j * TS + r) >> 2)
               : 0ull;
      const bool diag = (i == j);
      const int q_valid = p.T - i * TS;  // columns >= q_valid are past the end of the sequence
      const bool fast = !diag && q_valid >= TS;  // no masking anywhere in this tile
      const float4* lse4 = reinterpret_cast<const float4*>(sLse + s * TS + part * WCOLS);
      const float4* dlt4 = reinterpret_cast<const float4*>(sDelta + s * TS + part * WCOLS);
      uint32_t sv[1][32], dv[1][32];
      tmem_ld_32x32b_x32(t_lane + ST_COL + part * WCOLS, sv[0]);
      tmem_ld_32x32b_x32(t_lane + DPT_COL + part * WCOLS, dv[0]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_read);  // S^T / dP^T columns may be overwritten from here on
      Z2H_CTRACE();  // scores in registers
#pragma unroll
      for (int ch = 0; ch < 1; ++ch) {
        uint32_t pt[16];  // P^T of these 32 queries, packed bf16 pairs
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t dk[4];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int e4 = q * 2 + e;
            const float4 L = lse4[ch * 8 + e4];
            const float4 D = dlt4[ch * 8 + e4];
            // packed fp32 pairs: one instruction scales and shifts two scores
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            const float2 x01 = fma2(make_float2(__uint_as_float(sv[ch][e4 * 4 + 0]), __uint_as_float(sv[ch][e4 * 4 + 1])),
                                    sc2, make_float2(-L.x, -L.y));
            const float2 x23 = fma2(make_float2(__uint_as_float(sv[ch][e4 * 4 + 2]), __uint_as_float(sv[ch][e4 * 4 + 3])),
                                    sc2, make_float2(-L.z, -L.w));
            float p0 = ex2_fast(x01.x), p1 = ex2_fast(x01.y), p2 = ex2_fast(x23.x), p3 = ex2_fast(x23.y);
            if (!fast) {
              const int c0 = part * WCOLS + e4 * 4;
              if ((diag && c0 + 0 < r) || c0 + 0 >= q_valid) p0 = 0.f;
              if ((diag && c0 + 1 < r) || c0 + 1 >= q_valid) p1 = 0.f;
              if ((diag && c0 + 2 < r) || c0 + 2 >= q_valid) p2 = 0.f;
              if ((diag && c0 + 3 < r) || c0 + 3 >= q_valid) p3 = 0.f;
            }
            float g0 = __uint_as_float(dv[ch][e4 * 4 + 0]), g1 = __uint_as_float(dv[ch][e4 * 4 + 1]);
            float g2 = __uint_as_float(dv[ch][e4 * 4 + 2]), g3 = __uint_as_float(dv[ch][e4 * 4 + 3]);
            float pd0 = p0, pd1 = p1, pd2 = p2, pd3 = p3;  // what multiplied V in the forward pass
            if (DROP) {
              // this thread's key is fixed; the four queries of this step are consecutive rows
              const unsigned long long w0 = drop_q0 + (unsigned long long)(part * WCOLS + e4 * 4) * drop_wpr;
              const bool k0 = dropout_keep(dropout_word(drop.seed_lo, drop.seed_hi, w0), drop_byte, drop.threshold);
              const bool k1 = dropout_keep(dropout_word(drop.seed_lo, drop.seed_hi, w0 + drop_wpr), drop_byte, drop.threshold);
              const bool k2 = dropout_keep(dropout_word(drop.seed_lo, drop.seed_hi, w0 + 2 * drop_wpr), drop_byte, drop.threshold);
              const bool k3 = dropout_keep(dropout_word(drop.seed_lo, drop.seed_hi, w0 + 3 * drop_wpr), drop_byte, drop.threshold);
              pd0 = k0 ? p0 * drop.scale : 0.f; g0 = k0 ? g0 * drop.scale : 0.f;
              pd1 = k1 ? p1 * drop.scale : 0.f; g1 = k1 ? g1 * drop.scale : 0.f;
              pd2 = k2 ? p2 * drop.scale : 0.f; g2 = k2 ? g2 * drop.scale : 0.f;
              pd3 = k3 ? p3 * drop.scale : 0.f; g3 = k3 ? g3 * drop.scale : 0.f;
            }
            const float2 d01 = mul2(make_float2(p0, p1), add2(make_float2(g0, g1), make_float2(-D.x, -D.y)));
            const float2 d23 = mul2(make_float2(p2, p3), add2(make_float2(g2, g3), make_float2(-D.z, -D.w)));
            const float d0 = d01.x, d1 = d01.y, d2 = d23.x, d3 = d23.y;
            pt[q * 4 + e * 2 + 0] = pack_bf16x2(pd0, pd1);
            pt[q * 4 + e * 2 + 1] = pack_bf16x2(pd2, pd3);
            dk[e * 2 + 0] = pack_bf16x2(d0, d1);
            dk[e * 2 + 1] = pack_bf16x2(d2, d3);
          }
          // 8 columns = one 16-byte chunk of this row inside swizzle atom `half`
          const uint32_t chunk = ((uint32_t)(sub * 4 + q) ^ (uint32_t)(r & 7)) * 16;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst_row + pb + chunk), "r"(dk[0]),
                       "r"(dk[1]), "r"(dk[2]), "r"(dk[3])
                       : "memory");
        }
        // P^T goes to its tensor-memory columns (the dV product reads its A operand there); the
        // previous tile's dV must have finished reading them
        if (it > 0 && !mbar_wait_bounded(dv_done, (it - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tmem_st_32x32b_x16(t_lane + PT_COL + part * 16, pt);
      }
      if (!ok) break;
      tmem_st_wait();
      Z2H_CTRACE();  // P^T / dS^T written
      // The products of tile it-1 must have completed before this warp signals tile `it`: a later
      // wait could otherwise see the barrier two phases ahead and mistake the parity.
      if (it > 0 && !(mbar_wait_bounded(dq_full, (it - 1) & 1, abort_flag, p.status, kTimeoutTmemFull) &&
                      mbar_wait_bounded(dk_done, (it - 1) & 1, abort_flag, p.status, kTimeoutTmemFull))) {
        ok = false;
        break;
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);  // one arrival per compute warp
      Z2H_CTRACE();  // arrived
      // while the tensor cores work on this tile, fold dQ of the previous one into global memory
      if (it > 0) drain_dq(it - 1);
      Z2H_CTRACE();  // dQ of the previous tile drained
    }
    if (ok && n_iter > 0) {
      ok = mbar_wait_bounded(dq_full, (n_iter - 1) & 1, abort_flag, p.status, kTimeoutTmemFull);
      if (ok) drain_dq(n_iter - 1);
      // dV and dK of this KV tile are complete once their last commits have fired
      if (ok) ok = mbar_wait_bounded(dv_done, (n_iter - 1) & 1, abort_flag, p.status, kTimeoutTmemFull);
      if (ok) ok = mbar_wait_bounded(dk_done, (n_iter - 1) & 1, abort_flag, p.status, kTimeoutTmemFull);
      if (ok) tc_fence_after();
    }
    const int tk = j * TS + r;
    ok = __all_sync(0xffffffffu, ok);  // the column sums below shuffle across the whole warp
    if (ok) {
      __nv_bfloat16* dk_row = p.dqkv + (long long)(row0 + tk) * (3 * p.C) + p.C + h * HD + part * 16;
      __nv_bfloat16* dv_row = dk_row + p.C;
      uint32_t v[16];
      tmem_ld_32x32b_x16(t_lane + DV_COL + part * 16, v);
      tmem_ld_wait();
      if (tk < p.T) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
          u.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
          u.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
          u.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
          *reinterpret_cast<uint4*>(dv_row + q * 8) = u;
        }
      }
      auto add_column_sums = [&](float* dst) {  // of v as rounded to bf16, rows past T left out
        float f[16];
#pragma unroll
        for (int e = 0; e < 16; ++e)
          f[e] = tk < p.T ? __bfloat162float(__float2bfloat16(__uint_as_float(v[e]))) : 0.f;
        const float sum = warp_column_sums<16>(f, lane);  // column lane / 2, in both lanes of the pair
        if ((lane & 1) == 0) atomicAdd(dst + h * HD + part * 16 + (lane >> 1), sum);
      };
      if (p.dbias != nullptr) add_column_sums(p.dbias + 2 * p.C);
      tmem_ld_32x32b_x16(t_lane + DK_COL + part * 16, v);
      tmem_ld_wait();
      if (tk < p.T) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]) * p.scale, __uint_as_float(v[q * 8 + 1]) * p.scale);
          u.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]) * p.scale, __uint_as_float(v[q * 8 + 3]) * p.scale);
          u.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]) * p.scale, __uint_as_float(v[q * 8 + 5]) * p.scale);
          u.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]) * p.scale, __uint_as_float(v[q * 8 + 7]) * p.scale);
          *reinterpret_cast<uint4*>(dk_row + q * 8) = u;
        }
      }
      if (p.dbias != nullptr) {
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * p.scale);
        add_column_sums(p.dbias + p.C);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// stats[0][bh][t] = lse[bh][t] * log2(e); stats[1][bh][t] = sum_d dO[b,t,h,d] * O[b,t,h,d];
// both zero for T <= t < Tpad. Also clears the fp32 dQ rows.
// Eight threads share one (row, head): each takes 16 bytes of O and dO, so a warp reads four
// contiguous 128-byte segments per instruction.
__global__ void flash_bwd_prep_kernel(const __nv_bfloat16* __restrict__ out,
                                      const __nv_bfloat16* __restrict__ dout,
                                      const float* __restrict__ lse, float* __restrict__ stats,
                                      float* __restrict__ dq_accum, int B, int T, int H, int Tpad) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)B * T * H * 8;
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool valid = idx < total;  // every lane stays until after the shuffles
  const int q = (int)(idx & 7);
  const long long mh = idx >> 3;  // == m * H + hh, and O / dO / dQ rows are contiguous in it
  float s = 0.f;
  if (valid) {
    const uint4 a = *reinterpret_cast<const uint4*>(out + mh * HD + q * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dout + mh * HD + q * 8);
    const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(&c);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 x = unpack_bf16x2(aw[e]), y = unpack_bf16x2(cw[e]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  // clear the fp32 dQ buffer (ceil(B*T / 32) * 32 rows in its blocked layout): 8 floats per thread
  {
    const long long rows32 = ((long long)B * T + 31) / 32 * 32;
    if (idx < rows32 * H * 8) {
      float* dq = dq_accum + idx * 8;
      reinterpret_cast<float4*>(dq)[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      reinterpret_cast<float4*>(dq)[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (valid && q == 0) {
    const int hh = (int)(mh % H);
    const long long m = mh / H;
    const int bb = (int)(m / T), t = (int)(m % T);
    const long long bhh = (long long)bb * H + hh;
    stats[bhh * Tpad + t] = lse[bhh * T + t] * 1.4426950408889634f;
    stats[((long long)B * H + bhh) * Tpad + t] = s;
  }
  // the padding of every stats row must read as zero
  if (Tpad > T) {
    const int pad = Tpad - T;
    const long long npad = 2LL * B * H * pad;
    if (idx < npad) {
      const long long row = idx / pad;
      stats[row * Tpad + T + (int)(idx % pad)] = 0.f;
    }
  }
}

// dqkv[m, 0:C] = bf16(dQ[m, :] * scale), dQ read from its blocked layout
// [row / 32][head][16-byte column group][row % 32]: a thread converts 16 columns of one row (four
// coalesced 16-byte loads across the warp, one 32-byte store).
// dbias (fp32 [C] or null): the column sums of what is stored are added to it; a warp holds 32 rows
// of the same 16 columns.
__global__ void flash_bwd_dq_convert_kernel(const float* __restrict__ dq_accum,
                                            __nv_bfloat16* __restrict__ dqkv, long long M, int H,
                                            float scale, float* __restrict__ dbias) {
  pdl_launch_dependents();
  pdl_wait();
  const int C = H * HD;
  const long long blocks = (M + 31) / 32;
  const long long total = blocks * H * 4 * 32;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int lane = (int)(idx & 31);
    const int c16 = (int)((idx >> 5) & 3);
    const long long bh = idx >> 7;  // == blk * H + h
    const int h = (int)(bh % H);
    const long long g = (bh / H) * 32 + lane;
    const bool valid = g < M;  // whole warps stay for the shuffles
    const float4* src = reinterpret_cast<const float4*>(dq_accum) + (bh * 16 + c16 * 4) * 32 + lane;
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4 a = valid ? src[k * 32] : make_float4(0.f, 0.f, 0.f, 0.f);
      w[2 * k] = pack_bf16x2(a.x * scale, a.y * scale);
      w[2 * k + 1] = pack_bf16x2(a.z * scale, a.w * scale);
    }
    if (valid) {
      uint4* dst = reinterpret_cast<uint4*>(dqkv + g * 3 * C + h * HD + c16 * 16);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
    if (dbias != nullptr) {
      float f[16];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float2 x = unpack_bf16x2(w[k]);
        f[2 * k] = x.x; f[2 * k + 1] = x.y;
      }
      const float sum = warp_column_sums<16>(f, lane);
      if ((lane & 1) == 0) atomicAdd(dbias + h * HD + c16 * 16 + (lane >> 1), sum);
    }
  }
}

}  // namespace

int flash_bwd_dropout(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                      float* dq_accum, float* stats, int B, int T, int H, float drop_p,
                      const unsigned long long* seed_ptr, unsigned int site, int* status,
                      cudaStream_t stream) {
  return flash_bwd_dbias(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, drop_p, seed_ptr, site, nullptr,
                         status, stream);
}

int flash_bwd_dbias(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                    float* dq_accum, float* stats, int B, int T, int H, float drop_p,
                    const unsigned long long* seed_ptr, unsigned int site, float* dbias, int* status,
                    cudaStream_t stream) {
  return flash_bwd_ex(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, drop_p, seed_ptr, site, dbias, 0,
                      status, stream);
}

int flash_bwd_ex(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                 float* dq_accum, float* stats, int B, int T, int H, float drop_p,
                 const unsigned long long* seed_ptr, unsigned int site, float* dbias, int ordered, int* status,
                 cudaStream_t stream) {
  const int C = H * HD;
  if (ordered && dbias != nullptr) return 1;  // the bias by-product is accumulated with atomics
  if (!(drop_p >= 0.f) || drop_p >= 1.f) return 1;
  if (B <= 0 || T <= 0) return 0;
  const int Tpad = (T + TS - 1) / TS * TS;
  CUtensorMap tm_qkv, tm_do;
  if (!make_tma_2d_bf16(&tm_qkv, qkv, (uint64_t)B * T, 3 * C, 3 * C, 128, HD, kSwizzle128)) return 2;
  if (!make_tma_2d_bf16(&tm_do, dout, (uint64_t)B * T, C, C, 128, HD, kSwizzle128)) return 2;
  {
    long long total = (long long)B * T * H * 8;
    const long long npad = 2LL * B * H * (Tpad - T);
    if (npad > total) total = npad;
    const long long nzero = (((long long)B * T + 31) / 32 * 32) * H * 8;
    if (nzero > total) total = nzero;
    const int grid = (int)((total + 255) / 256);
    launch_kernel(flash_bwd_prep_kernel, dim3(grid), dim3(256), 0, stream, true, (const __nv_bfloat16*)out,
                  (const __nv_bfloat16*)dout, lse, stats, dq_accum, B, T, H, Tpad);
  }
  BwdParams p;
  p.stats = stats; p.Tpad = Tpad;
  p.dqkv = (__nv_bfloat16*)dqkv;
  p.dq_accum = dq_accum;
  p.B = B; p.T = T; p.H = H; p.C = C;
  p.scale = 0.125f;
  p.scale_log2 = 0.125f * 1.4426950408889634f;
  p.status = status;
  p.dbias = dbias;
  p.drop_p = drop_p;
  p.seed_ptr = seed_ptr;
  p.site = site;
  static std::atomic<unsigned long long> attr_seen{0};
  if (first_use_on_current_device(attr_seen)) {
    cudaFuncSetAttribute(flash_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(flash_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  }
  const int n_t = (T + TS - 1) / TS;
  if (ordered) {
    for (int jt = 0; jt < n_t; ++jt) {
      p.j_fixed = jt;
      launch_kernel(drop_p > 0.f ? flash_bwd_kernel<true> : flash_bwd_kernel<false>, dim3(B * H),
                    dim3(NUM_THREADS), SMEM_BYTES, stream, true, tm_qkv, tm_do, p);
    }
  } else {
    p.j_fixed = -1;
    launch_kernel(drop_p > 0.f ? flash_bwd_kernel<true> : flash_bwd_kernel<false>, dim3(B * H * n_t),
                  dim3(NUM_THREADS), SMEM_BYTES, stream, true, tm_qkv, tm_do, p);
  }
  {
    const long long total = (((long long)B * T + 31) / 32) * H * 4 * 32;
    const int grid = (int)((total + 255) / 256);
    launch_kernel(flash_bwd_dq_convert_kernel, dim3(grid), dim3(256), 0, stream, true, (const float*)dq_accum,
                  (__nv_bfloat16*)dqkv, (long long)B * T, H, 0.125f, dbias);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int flash_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
              float* dq_accum, float* stats, int B, int T, int H, int* status, cudaStream_t stream) {
  return flash_bwd_dropout(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, 0.f, nullptr, 0, status,
                           stream);
}

}  // namespace z2h

extern "C" int z2h_flash_bwd_dropout(const void* qkv, const void* out, const void* dout, const float* lse,
                                     void* dqkv, float* dq_accum, float* stats, int B, int T, int H,
                                     float drop_p, const unsigned long long* seed_ptr, unsigned int site,
                                     int* status, void* stream) {
  return z2h::flash_bwd_dropout(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, drop_p, seed_ptr, site,
                                status, (cudaStream_t)stream);
}
extern "C" int z2h_flash_bwd_dbias(const void* qkv, const void* out, const void* dout, const float* lse,
                                   void* dqkv, float* dq_accum, float* stats, int B, int T, int H,
                                   float drop_p, const unsigned long long* seed_ptr, unsigned int site,
                                   float* dbias, int* status, void* stream) {
  return z2h::flash_bwd_dbias(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, drop_p, seed_ptr, site,
                              dbias, status, (cudaStream_t)stream);
}
extern "C" int z2h_flash_bwd_ex(const void* qkv, const void* out, const void* dout, const float* lse,
                                void* dqkv, float* dq_accum, float* stats, int B, int T, int H,
                                float drop_p, const unsigned long long* seed_ptr, unsigned int site,
                                float* dbias, int ordered, int* status, void* stream) {
  return z2h::flash_bwd_ex(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, drop_p, seed_ptr, site, dbias,
                           ordered, status, (cudaStream_t)stream);
}
extern "C" long long z2h_flash_bwd_dq_elems(int B, int T, int H) {
  return (((long long)B * T + 31) / 32 * 32) * H * 64;
}
extern "C" int z2h_flash_bwd_stats_elems(int B, int T, int H) {
  return 2 * B * H * ((T + 127) / 128 * 128);
}
extern "C" int z2h_flash_bwd(const void* qkv, const void* out, const void* dout, const float* lse,
                             void* dqkv, float* dq_accum, float* stats, int B, int T, int H,
                             int* status, void* stream) {
  return z2h::flash_bwd(qkv, out, dout, lse, dqkv, dq_accum, stats, B, T, H, status,
                        (cudaStream_t)stream);
}

#ifdef Z2H_KERNEL_TRACE
extern "C" int z2h_flash_bwd_trace_read(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_kernel_trace, sizeof(g_kernel_trace));
}
#endif
