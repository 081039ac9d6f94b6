// Causal flash attention forward, head_dim 64, bf16, on tcgen05 tensor cores.
//
// Input is the fused projection output qkv[B*T, 3*C] (q | k | v, head h in columns h*64..),
// exactly what the QKV GEMM writes; output is out[B*T, C] with heads already merged, so the
// split / transpose / contiguous copies of the reference (nn/gpt2/modules.py:31-39) never
// happen. The softmax scale is 1/sqrt(64), masking is causal, as in
// F.scaled_dot_product_attention(q, k, v, is_causal=True) (nn/gpt2/modules.py:37).
//
// Work items are (batch, head, 128-row query tile); an item walks the KV tiles 0..diagonal. The
// kernel is persistent: two CTAs per SM, each taking items from a static schedule that sorts the
// items by length (longest first) and deals them out in a snake over the CTAs, so every CTA gets
// the same amount of work to within one tile, pays the set-up (barriers, tensor memory) once,
// and loads the next item's Q and K while the current item drains. Roles inside a CTA:
//   warp 0     TMA: Q per item, K/V tiles through a 3-stage ring (128-byte swizzle)
//   warp 1     tcgen05.mma: S = Q K^T (128x128x64) into TMEM, then O += P V (128x64x128); the
//              scores of tile t+1 (also across an item boundary) are issued as soon as the
//              softmax warps hold tile t in registers
//   warps 2-5  one query row per thread: read S from TMEM, online softmax in fp32 (no
//              shuffles: a thread owns its row), write P as packed bf16 back into TMEM, where
//              the second MMA reads its A operand (P never touches shared memory, whose
//              bandwidth the operand reads of the MMAs and the TMA writes already use up).
//              O accumulates in TMEM across KV tiles and is rescaled
//              there only when a row maximum grows by more than 2^8. On the diagonal tile a
//              warp (32 consecutive rows) skips the 32-column chunks that are masked for all of
//              its rows: no TMEM load, no exponentials, zeros into P.
// TMEM use is 256 columns and shared memory ~113 KiB, so two CTAs share an
// SM and one CTA's tensor-core work overlaps the other's exponentials.
#include "../common/checked.cuh"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "attn.h"
#include "../common/trace.cuh"
#include "../common/dropout.cuh"

namespace z2h {
namespace {

constexpr int QT = 128;   // query rows per item
constexpr int KT = 128;   // kv rows per tile
constexpr int HD = 64;
constexpr int TILE_BYTES = 128 * HD * 2;  // 16 KiB
constexpr int KV_STAGES = 3;
// Of every 8 pairs of exponentials, this many are computed with a polynomial on the FMA pipe
// instead of the special-function unit (which two CTAs per SM keep saturated otherwise).
#ifndef Z2H_FWD_POLY_OF_8
#define Z2H_FWD_POLY_OF_8 0
#endif
constexpr int kPolyOf8 = Z2H_FWD_POLY_OF_8;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 256;
// scores (fp32, 128 columns), output accumulator (fp32, 64), probabilities as packed bf16 pairs (64)
constexpr int S_COL = 0, PV_COL = 128, P_COL = 192;
// two CTAs per SM need (dynamic + 1 KiB reserved) * 2 <= 228 KiB, i.e. at most 115,712 bytes each
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * KV_STAGES) + 256;
static_assert(SMEM_BYTES <= 115712, "two CTAs per SM no longer fit");

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  int B, T, H, C;
  float scale_log2;  // softmax_scale * log2(e)
  float scale;
  int* status;
  // attention-probability dropout (DROP instantiation only)
  float drop_p;
  const unsigned long long* seed_ptr;
  uint32_t site;
};

// The flat sequence of (item, kv tile) pairs one CTA works through. Items are numbered longest
// first (index i -> query tile n_qt-1 - i / BH, batch*head i % BH); CTA c of G takes, in round k,
// item k*G + c (k even) or k*G + G-1-c (k odd). Every role of the CTA runs its own copy of the
// iterator (the MMA warp two: current tile and look-ahead), so no schedule is communicated.
struct TileIter {
  int k, j, qi, bh;  // round of the schedule, kv tile within the item, the item itself
  bool valid;
  // grid size, CTA index and the problem's shape are re-read where needed rather than kept here:
  // the softmax warps, which hold a whole score row in registers, run one of these too
  __device__ __forceinline__ void init(int T, int BH) {
    k = 0;
    valid = next_item(T, BH);
  }
  __device__ __forceinline__ bool next_item(int T, int BH) {
    const int G = gridDim.x, c = blockIdx.x, n_qt = (T + QT - 1) / QT;
    const int i = k * G + ((k & 1) ? G - 1 - c : c);
    if (i >= n_qt * BH) return false;
    ++k;
    qi = n_qt - 1 - i / BH;
    bh = i - (i / BH) * BH;
    j = 0;
    return true;
  }
  __device__ __forceinline__ void next_tile(int T, int BH) {
    if (++j > qi) valid = next_item(T, BH);
  }
  __device__ __forceinline__ bool first() const { return j == 0; }
  __device__ __forceinline__ bool last() const { return j == qi; }
};


// Row maximum of one score tile (one thread = one query row, 128 scores in registers).
// DIAG: the tile on the diagonal; a warp's rows (quarter*32 .. +31) see the 32-column chunks
// 0..quarter only, the last of them triangular (column i visible iff i <= lane). The common
// (off-diagonal) instantiation carries no masking instructions at all.
template <bool DIAG>
__device__ __forceinline__ float tile_row_max(const uint32_t (&sv)[KT / 32][32], float m_in, int quarter,
                                              int lane) {
  // eight independent chains (two per chunk), so the maxima do not wait on one another
  float mx[KT / 16] = {m_in, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int ch = 0; ch < KT / 32; ++ch) {
    if (DIAG && ch > quarter) continue;
    if (DIAG && ch == quarter) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i <= lane) mx[2 * ch + (i & 1)] = fmaxf(mx[2 * ch + (i & 1)], __uint_as_float(sv[ch][i]));
    } else {
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        mx[2 * ch] = max3(mx[2 * ch], __uint_as_float(sv[ch][i]), __uint_as_float(sv[ch][i + 1]));
        mx[2 * ch + 1] = max3(mx[2 * ch + 1], __uint_as_float(sv[ch][16 + i]), __uint_as_float(sv[ch][17 + i]));
      }
    }
  }
  mx[0] = max3(mx[0], mx[1], mx[2]);
  mx[3] = max3(mx[3], mx[4], mx[5]);
  mx[6] = fmaxf(mx[6], mx[7]);
  return max3(mx[0], mx[3], mx[6]);
}

// p = 2^(s * c - m * c) for the whole row, packed bf16 pairs into pk, returns the row sum.
// Dropout (DROP) masks what enters P V, not the sum.
template <bool DIAG, bool DROP>
__device__ __forceinline__ float tile_exponentials(const uint32_t (&sv)[KT / 32][32], uint32_t (&pk)[KT / 32][16],
                                                   float scale_log2, float mc, int quarter, int lane,
                                                   const DropoutSpec& drop, unsigned long long drop_word0) {
  float2 rs = make_float2(0.f, 0.f), rs_b = make_float2(0.f, 0.f);
  const float2 sc2 = make_float2(scale_log2, scale_log2), nmc2 = make_float2(-mc, -mc);
#pragma unroll
  for (int ch = 0; ch < KT / 32; ++ch) {
    if (DIAG && ch > quarter) {  // masked for every row of this warp: zeros, no exponentials
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[ch][i] = 0u;
      continue;
    }
    const bool tri = DIAG && ch == quarter;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t mw[2] = {0, 0};
      if (DROP) {
        const unsigned long long w0 = drop_word0 + (unsigned long long)(ch * 8 + q * 2);
        mw[0] = dropout_word(drop.seed_lo, drop.seed_hi, w0);
        mw[1] = dropout_word(drop.seed_lo, drop.seed_hi, w0 + 1);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = q * 8 + e * 2;
        // one packed multiply-add for the pair, two exponentials, one packed add for the sums
        const float2 x = fma2(make_float2(__uint_as_float(sv[ch][i]), __uint_as_float(sv[ch][i + 1])), sc2, nmc2);
        float p0, p1;
        if (((q * 4 + e) & 7) < kPolyOf8) {
          const float2 pp = ex2_poly2(x);
          p0 = pp.x;
          p1 = pp.y;
        } else {
          p0 = ex2_fast(x.x);
          p1 = ex2_fast(x.y);
        }
        if (tri) {
          if (i > lane) p0 = 0.f;
          if (i + 1 > lane) p1 = 0.f;
        }
        if (e & 1) rs_b = add2(rs_b, make_float2(p0, p1));
        else rs = add2(rs, make_float2(p0, p1));
        if (DROP) {
          if (!dropout_keep(mw[e >> 1], (e & 1) * 2, drop.threshold)) p0 = 0.f;
          if (!dropout_keep(mw[e >> 1], (e & 1) * 2 + 1, drop.threshold)) p1 = 0.f;
        }
        pk[ch][q * 4 + e] = pack_bf16x2(p0, p1);
      }
    }
  }
  return (rs.x + rs.y) + (rs_b.x + rs_b.y);
}

// DROP: the probabilities that enter P V are masked (mask of element (b, h, q, k): word
// ((b*H + h)*T + q) * ceil(T/4) + k/4 of the site's stream); the softmax normaliser is not, and the
// 1/(1-p) scale is applied once to the output row.
template <bool DROP>
__global__ void __launch_bounds__(NUM_THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  pdl_launch_dependents();
  if (smem_u32(smem_raw) & 1023u) {  // the swizzled tiles need a 1 KiB aligned base
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, (int)kBadArgument);
    return;
  }
  uint8_t* sQ = smem_raw;
  uint8_t* sK = sQ + TILE_BYTES;
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KV_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;             // every score MMA of the item has read Q
  uint64_t* k_full = bars + 2;
  uint64_t* v_full = k_full + KV_STAGES;
  uint64_t* k_empty = v_full + KV_STAGES;   // K stage free: the score MMAs that read it are done
  uint64_t* v_empty = k_empty + KV_STAGES;  // V stage free: the P V MMAs that read it are done
  uint64_t* s_full = v_empty + KV_STAGES;
  uint64_t* p_full = s_full + 1;
  uint64_t* pv_full = p_full + 1;   // completes once per KV tile, when P V of that tile is done
  uint64_t* s_read = pv_full + 1;   // the softmax warps have the score tile in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_read + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(pv_full, 1);
    mbar_init(s_read, 4);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_qkv);
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
  const int BH = p.B * p.H;

  if (warp == 0) {
    if (lane == 0) {
      // K tiles run one tile ahead of V tiles: a K stage is free as soon as its scores are
      // computed, a V stage only after P V, and the scores of tile t+1 are wanted early
      TileIter kt, vt;
      kt.init(p.T, BH);
      vt.init(p.T, BH);
      uint32_t tk = 0, tv = 0, items = 0;
      bool ok = true;
      auto load_v = [&]() -> bool {
        const int h = vt.bh % p.H, row0 = (vt.bh / p.H) * p.T;
        const int s = tv % KV_STAGES;
        if (!mbar_wait_bounded(&v_empty[s], ((tv / KV_STAGES) & 1) ^ 1u, abort_flag, p.status, kTimeoutEmpty))
          return false;
        mbar_arrive_expect_tx(&v_full[s], TILE_BYTES);
        tma_load_2d(sV + s * TILE_BYTES, &tm_qkv, &v_full[s], 2 * p.C + h * HD, row0 + vt.j * KT);
        vt.next_tile(p.T, BH);
        ++tv;
        return true;
      };
      while (ok && kt.valid) {
        const int h = kt.bh % p.H, row0 = (kt.bh / p.H) * p.T;
        if (kt.first()) {
          if (!mbar_wait_bounded(q_empty, (items & 1u) ^ 1u, abort_flag, p.status, kTimeoutEmpty)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(q_full, TILE_BYTES);
          tma_load_2d(sQ, &tm_qkv, q_full, h * HD, row0 + kt.qi * QT);
          ++items;
        }
        const int s = tk % KV_STAGES;
        if (!mbar_wait_bounded(&k_empty[s], ((tk / KV_STAGES) & 1) ^ 1u, abort_flag, p.status, kTimeoutEmpty)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&k_full[s], TILE_BYTES);
        tma_load_2d(sK + s * TILE_BYTES, &tm_qkv, &k_full[s], p.C + h * HD, row0 + kt.j * KT);
        kt.next_tile(p.T, BH);
        ++tk;
        if (tk >= 2) ok = load_v();  // V(t-1) follows K(t)
      }
      while (ok && vt.valid) ok = load_v();
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(QT, KT, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(QT, HD, 0, 1);
      // descriptors are built once; inside the loop an MMA costs one 64-bit add per operand
      const uint64_t q_desc = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
      uint64_t k_desc[KV_STAGES], v_desc[KV_STAGES];
#pragma unroll
      for (int s = 0; s < KV_STAGES; ++s) {
        k_desc[s] = make_smem_desc_sw128(smem_u32(sK + s * TILE_BYTES), 16, 1024);
        v_desc[s] = make_smem_desc_sw128(smem_u32(sV + s * TILE_BYTES), 16, 1024);
      }
      TileIter cur, nxt;
      cur.init(p.T, BH);
      nxt.init(p.T, BH);
      uint32_t q_items = 0;  // items whose Q this warp has started to use
      Z2H_TRACE_DECL(1)
      Z2H_TRACE();
      // S of flat tile `tn` (the tile `nxt` points at): wait for its operands, issue, commit
      auto issue_scores = [&](uint32_t tn) -> bool {
        if (nxt.first()) {
          if (!mbar_wait_bounded(q_full, q_items & 1u, abort_flag, p.status, kTimeoutFull)) return false;
          ++q_items;
        }
        const int s2 = tn % KV_STAGES;
        if (!mbar_wait_bounded(&k_full[s2], (tn / KV_STAGES) & 1, abort_flag, p.status, kTimeoutFull))
          return false;
        tc_fence_after();
        const uint64_t kd = s2 == 0 ? k_desc[0] : (s2 == 1 ? k_desc[1] : k_desc[2]);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc_mma_f16_ss(tmem_base + S_COL, desc_advance(q_desc, k * 32), desc_advance(kd, k * 32),
                        idesc_s, k > 0);
        tc_commit(s_full);
        tc_commit(&k_empty[s2]);
        if (nxt.last()) tc_commit(q_empty);
        nxt.next_tile(p.T, BH);
        return true;
      };
      bool ok = cur.valid;
      if (ok) ok = issue_scores(0);
      // Per flat tile t: the scores of tile t+1 are issued as soon as the softmax warps hold tile t
      // in registers, i.e. while they still work on it, and only then P V of tile t. The softmax
      // chain therefore never waits for an MMA of its own tile: S is ready a tile ahead and P V
      // runs behind it.
      for (uint32_t t = 0; ok && cur.valid; ++t) {
        const int s = t % KV_STAGES;
        const uint32_t ph = (t / KV_STAGES) & 1;
        if (nxt.valid) {
          if (!mbar_wait_bounded(s_read, t & 1, abort_flag, p.status, kTimeoutLocal)) break;
          Z2H_TRACE();  // the softmax warps hold tile t
          if (!issue_scores(t + 1)) break;
        }
        Z2H_TRACE();  // scores of the next tile issued
        if (!mbar_wait_bounded(p_full, t & 1, abort_flag, p.status, kTimeoutLocal)) break;
        Z2H_TRACE();  // P of this tile is there
        if (!mbar_wait_bounded(&v_full[s], ph, abort_flag, p.status, kTimeoutFull)) break;
        tc_fence_after();
        const uint64_t vd = s == 0 ? v_desc[0] : (s == 1 ? v_desc[1] : v_desc[2]);
        const bool fresh = cur.first();
#pragma unroll
        for (int k = 0; k < KT / 16; ++k) {  // keys 16k..16k+15 of P are 8 packed columns
          tc_mma_f16_ts(tmem_base + PV_COL, tmem_base + P_COL + k * 8, desc_advance(vd, k * 2048),
                        idesc_pv, (!fresh || k > 0) ? 1u : 0u);
        }
        tc_commit(pv_full);
        tc_commit(&v_empty[s]);
        cur.next_tile(p.T, BH);
        Z2H_TRACE();  // P V issued
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // query row within the tile == TMEM lane
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    // m_run is the maximum the stored O / l are expressed against. It only moves when the row
    // maximum grows by more than 2^8 (in the exp2 domain), so O, which accumulates in TMEM
    // across KV tiles, rarely needs rescaling; P stays <= 2^8, well inside bf16 / fp32 range.
    float m_run = -INFINITY, l_run = 0.f;
    DropoutSpec drop = {};
    unsigned long long drop_row = 0;  // first mask word of this query row
    if (DROP) drop = make_dropout_spec(p.seed_ptr, p.site, p.drop_p);
    bool ok = true;
    TileIter it;
    it.init(p.T, BH);
    Z2H_TRACE_DECL(2)
#define Z2H_CTRACE()                         \
  do {                                       \
    if (warp == 2 && lane == 0) Z2H_TRACE(); \
  } while (0)
    Z2H_CTRACE();
    for (uint32_t t = 0; ok && it.valid; ++t) {
      const int qi = it.qi, j = it.j;
      if (it.first()) {
        m_run = -INFINITY;
        l_run = 0.f;
        if (DROP)
          drop_row = ((unsigned long long)it.bh * p.T + (unsigned long long)(qi * QT + r)) *
                     (unsigned long long)((p.T + 3) / 4);
      }
      Z2H_CTRACE();  // about to wait for the scores
      if (!mbar_wait_bounded(s_full, t & 1, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      Z2H_CTRACE();  // scores are there
      const bool diag = (j == qi);
      // the whole score row (128 fp32) comes into registers with one wait (loading only the
      // visible chunks would make the register array conditionally defined, which spills)
      uint32_t sv[KT / 32][32];
#pragma unroll
      for (int ch = 0; ch < KT / 32; ++ch)
        tmem_ld_32x32b_x32(t_lane + S_COL + ch * 32, sv[ch]);
      tmem_ld_wait();
      // the score columns may be overwritten with the next tile from here on
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_read);
      Z2H_CTRACE();  // scores in registers
      const float m_new = diag ? tile_row_max<true>(sv, m_run, quarter, lane)
                               : tile_row_max<false>(sv, m_run, quarter, lane);
      Z2H_CTRACE();  // row maximum of this tile known
      // P V of tile t-1 must be complete before O is rescaled and before P (one buffer in TMEM) is
      // overwritten. Rescaling is rare (the maximum must grow by 2^8), so the wait normally comes
      // only after this tile's exponentials, which therefore overlap the previous tile's P V.
      bool pv_waited = it.first();  // the previous item's epilogue awaited its last P V
      if (it.first()) {
        m_run = m_new;  // nothing accumulated yet
      } else {
        const bool grow = (m_new - m_run) * p.scale_log2 > 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          if (!mbar_wait_bounded(pv_full, (t - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
            ok = false;
            break;
          }
          pv_waited = true;
          tc_fence_after();
          const float alpha = grow ? ex2_fast((m_run - m_new) * p.scale_log2) : 1.f;
#pragma unroll
          for (int q = 0; q < HD / 16; ++q) {
            uint32_t ov[16];
            tmem_ld_32x32b_x16(t_lane + PV_COL + q * 16, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_32x32b_x16(t_lane + PV_COL + q * 16, ov);
          }
          tmem_st_wait();
          if (grow) {
            l_run *= alpha;
            m_run = m_new;
          }
        }
      }
      Z2H_CTRACE();  // maximum known (and O rescaled if it had to be)
      const float mc = m_run * p.scale_log2;
      // p = 2^(s * c - m * c), row sum, P as packed bf16 pairs into its tensor-memory columns (the
      // second MMA takes its A operand from there: no shared-memory round trip for P)
      uint32_t pk[KT / 32][16];
      const unsigned long long dw0 = DROP ? drop_row + (unsigned long long)(j * (KT / 4)) : 0ull;
      l_run += diag ? tile_exponentials<true, DROP>(sv, pk, p.scale_log2, mc, quarter, lane, drop, dw0)
                    : tile_exponentials<false, DROP>(sv, pk, p.scale_log2, mc, quarter, lane, drop, dw0);
      Z2H_CTRACE();  // exponentials done (in registers)
      if (!pv_waited) {
        if (!mbar_wait_bounded(pv_full, (t - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
      }
#pragma unroll
      for (int ch = 0; ch < KT / 32; ++ch) tmem_st_32x32b_x16(t_lane + P_COL + ch * 16, pk[ch]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);  // one arrival per softmax warp
      Z2H_CTRACE();  // P written
      if (it.last()) {
        // the item is complete once P V of its last tile is: normalise and write the output rows
        if (!mbar_wait_bounded(pv_full, t & 1, abort_flag, p.status, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t ov[HD / 32][32];
#pragma unroll
        for (int q = 0; q < HD / 32; ++q) tmem_ld_32x32b_x32(t_lane + PV_COL + q * 32, ov[q]);
        tmem_ld_wait();
        tc_fence_before();
        const int tq = qi * QT + r;
        if (tq < p.T &&
            in_bounds((long long)(it.bh / p.H) * p.T + tq, (long long)p.B * p.T, p.status, kSiteFlashFwdOut)) {
          const int h = it.bh % p.H, b = it.bh / p.H;
          const float inv = DROP ? drop.scale / l_run : 1.f / l_run;
          __nv_bfloat16* op = p.out + (long long)(b * p.T + tq) * p.C + h * HD;
#pragma unroll
          for (int q = 0; q < HD / 8; ++q) {
            const uint32_t* o8 = &ov[q >> 2][(q & 3) * 8];
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o8[0]) * inv, __uint_as_float(o8[1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(o8[2]) * inv, __uint_as_float(o8[3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(o8[4]) * inv, __uint_as_float(o8[5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(o8[6]) * inv, __uint_as_float(o8[7]) * inv);
            *reinterpret_cast<uint4*>(op + q * 8) = u;
          }
          if (p.lse != nullptr)
            p.lse[((long long)b * p.H + h) * p.T + tq] = m_run * p.scale + __logf(l_run);
        }
        Z2H_CTRACE();  // output written
      }
      it.next_tile(p.T, BH);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

int flash_fwd_dropout(const void* qkv, void* out, float* lse, int B, int T, int H, float drop_p,
                      const unsigned long long* seed_ptr, unsigned int site, int* status,
                      cudaStream_t stream) {
  const int C = H * HD;
  if (B <= 0 || T <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(qkv) & 15 || reinterpret_cast<uintptr_t>(out) & 15) return 1;
  CUtensorMap tm;
  if (!make_tma_2d_bf16(&tm, qkv, (uint64_t)B * T, 3 * C, 3 * C, 128, HD, kSwizzle128)) return 2;
  FwdParams p;
  p.out = (__nv_bfloat16*)out;
  p.lse = lse;
  p.B = B; p.T = T; p.H = H; p.C = C;
  p.scale = 0.125f;
  p.scale_log2 = 0.125f * 1.4426950408889634f;
  p.status = status;
  if (!(drop_p >= 0.f) || drop_p >= 1.f) return 1;
  p.drop_p = drop_p;
  p.seed_ptr = seed_ptr;
  p.site = site;
  static std::atomic<unsigned long long> attr_seen{0};
  if (first_use_on_current_device(attr_seen)) {
    cudaFuncSetAttribute(flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  }
  const int n_qt = (T + QT - 1) / QT;
  const int items = B * H * n_qt;
  const int slots = 2 * sm_count_current_device();  // two CTAs per SM
  const cudaError_t err = launch_kernel(drop_p > 0.f ? flash_fwd_kernel<true> : flash_fwd_kernel<false>,
                                        dim3(items < slots ? items : slots), dim3(NUM_THREADS), SMEM_BYTES,
                                        stream, true, tm, p);
  return err == cudaSuccess ? 0 : 3;
}

int flash_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int* status,
              cudaStream_t stream) {
  return flash_fwd_dropout(qkv, out, lse, B, T, H, 0.f, nullptr, 0, status, stream);
}

}  // namespace z2h

extern "C" int z2h_flash_fwd_dropout(const void* qkv, void* out, float* lse, int B, int T, int H,
                                     float drop_p, const unsigned long long* seed_ptr, unsigned int site,
                                     int* status, void* stream) {
  return z2h::flash_fwd_dropout(qkv, out, lse, B, T, H, drop_p, seed_ptr, site, status,
                                (cudaStream_t)stream);
}
extern "C" int z2h_flash_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int* status,
                             void* stream) {
  return z2h::flash_fwd(qkv, out, lse, B, T, H, status, (cudaStream_t)stream);
}

#ifdef Z2H_KERNEL_TRACE
extern "C" int z2h_flash_fwd_trace_read(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_kernel_trace, sizeof(g_kernel_trace));
}
#endif
