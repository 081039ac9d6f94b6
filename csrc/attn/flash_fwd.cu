// Causal flash attention forward, head_dim 64, bf16, on tcgen05 tensor cores.
//
// Input is the fused projection output qkv[B*T, 3*C] (q | k | v, head h in columns h*64..),
// exactly what the QKV GEMM writes; output is out[B*T, C] with heads already merged, so the
// split / transpose / contiguous copies of the reference (nn/gpt2/modules.py:31-39) never
// happen. The softmax scale is 1/sqrt(64), masking is causal, as in
// F.scaled_dot_product_attention(q, k, v, is_causal=True) (nn/gpt2/modules.py:37).
//
// One CTA handles 128 query rows of one (batch, head) and walks the KV tiles 0..diagonal:
//   warp 0     TMA: Q once, K/V tiles through a 2-stage ring (128-byte swizzle)
//   warp 1     tcgen05.mma: S = Q K^T (128x128x64) into TMEM, then O += P V (128x64x128)
//   warps 2-5  one query row per thread: read S from TMEM, online softmax in fp32 (no
//              shuffles: a thread owns its row), write P as bf16 into swizzled shared memory
//              for the second MMA. O accumulates in TMEM across KV tiles and is rescaled
//              there only when a row maximum grows by more than 2^8.
// TMEM use is 192 columns (allocated as 256) and shared memory ~113 KiB, so two CTAs share an
// SM and one CTA's tensor-core work overlaps the other's exponentials.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "attn.h"
#include "../common/trace.cuh"
#include "../common/dropout.cuh"

namespace z2h {
namespace {

constexpr int QT = 128;   // query rows per CTA
constexpr int KT = 128;   // kv rows per tile
constexpr int HD = 64;
constexpr int TILE_BYTES = 128 * HD * 2;  // 16 KiB
constexpr int P_BYTES = QT * KT * 2;      // 32 KiB
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr int S_COL = 0, PV_COL = 128;
// two CTAs per SM need (dynamic + 1 KiB reserved) * 2 <= 228 KiB, i.e. at most 115,712 bytes each
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * KV_STAGES) + P_BYTES + 256;
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
  uint8_t* sP = sV + KV_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
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
  const int n_qt = (p.T + QT - 1) / QT;
  // heavy (late) query tiles first
  const int qi = n_qt - 1 - (int)(blockIdx.x % n_qt);
  const int bh = blockIdx.x / n_qt;
  const int h = bh % p.H, b = bh / p.H;
  const int n_kv = qi + 1;
  const int row0 = b * p.T;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, TILE_BYTES);
      tma_load_2d(sQ, &tm_qkv, q_full, h * HD, row0 + qi * QT);
      // K tiles run one tile ahead of V tiles: a K stage is free as soon as its scores are
      // computed, a V stage only after P V, and the scores of tile j+1 are wanted early
      for (int j = 0; j <= n_kv; ++j) {
        if (j < n_kv) {
          const int s = j % KV_STAGES;
          const uint32_t ph = (j / KV_STAGES) & 1;
          if (!mbar_wait_bounded(&k_empty[s], ph ^ 1u, abort_flag, p.status, kTimeoutEmpty)) break;
          mbar_arrive_expect_tx(&k_full[s], TILE_BYTES);
          tma_load_2d(sK + s * TILE_BYTES, &tm_qkv, &k_full[s], p.C + h * HD, row0 + j * KT);
        }
        if (j > 0) {
          const int jv = j - 1, s = jv % KV_STAGES;
          const uint32_t ph = (jv / KV_STAGES) & 1;
          if (!mbar_wait_bounded(&v_empty[s], ph ^ 1u, abort_flag, p.status, kTimeoutEmpty)) break;
          mbar_arrive_expect_tx(&v_full[s], TILE_BYTES);
          tma_load_2d(sV + s * TILE_BYTES, &tm_qkv, &v_full[s], 2 * p.C + h * HD, row0 + jv * KT);
        }
      }
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
      const uint64_t p_desc = make_smem_desc_sw128(smem_u32(sP), 16, 1024);
      uint64_t k_desc[KV_STAGES], v_desc[KV_STAGES];
#pragma unroll
      for (int s = 0; s < KV_STAGES; ++s) {
        k_desc[s] = make_smem_desc_sw128(smem_u32(sK + s * TILE_BYTES), 16, 1024);
        v_desc[s] = make_smem_desc_sw128(smem_u32(sV + s * TILE_BYTES), 16, 1024);
      }
      Z2H_TRACE_DECL(1)
      Z2H_TRACE();
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, kTimeoutFull);
      if (ok) ok = mbar_wait_bounded(&k_full[0], 0, abort_flag, p.status, kTimeoutFull);
      Z2H_TRACE();
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc_mma_f16_ss(tmem_base + S_COL, desc_advance(q_desc, k * 32), desc_advance(k_desc[0], k * 32),
                        idesc_s, k > 0);
        tc_commit(s_full);
        tc_commit(&k_empty[0]);
      }
      // Per KV tile j: the scores of tile j+1 are issued as soon as the softmax warps hold tile j
      // in registers, i.e. while they still work on it, and only then P V of tile j. The softmax
      // chain therefore never waits for an MMA of its own tile: S is ready a tile ahead and P V
      // runs behind it.
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (j + 1 < n_kv) {
          const int s2 = (j + 1) % KV_STAGES;
          const uint32_t ph2 = ((j + 1) / KV_STAGES) & 1;
          if (!mbar_wait_bounded(s_read, j & 1, abort_flag, p.status, kTimeoutLocal)) break;
          if (!mbar_wait_bounded(&k_full[s2], ph2, abort_flag, p.status, kTimeoutFull)) break;
          tc_fence_after();
          const uint64_t kd = s2 == 0 ? k_desc[0] : k_desc[1];
#pragma unroll
          for (int k = 0; k < HD / 16; ++k)
            tc_mma_f16_ss(tmem_base + S_COL, desc_advance(q_desc, k * 32), desc_advance(kd, k * 32),
                          idesc_s, k > 0);
          tc_commit(s_full);
          tc_commit(&k_empty[s2]);
        }
        Z2H_TRACE();  // scores of the next tile issued
        if (!mbar_wait_bounded(p_full, j & 1, abort_flag, p.status, kTimeoutLocal)) break;
        Z2H_TRACE();  // P of this tile is there
        if (!mbar_wait_bounded(&v_full[s], ph, abort_flag, p.status, kTimeoutFull)) break;
        tc_fence_after();
        const uint64_t vd = s == 0 ? v_desc[0] : v_desc[1];
#pragma unroll
        for (int k = 0; k < KT / 16; ++k) {
          tc_mma_f16_ss(tmem_base + PV_COL,
                        desc_advance(p_desc, (k >> 2) * (QT * 128) + (k & 3) * 32),
                        desc_advance(vd, k * 2048), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(pv_full);
        tc_commit(&v_empty[s]);
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
    const uint32_t p_row = smem_u32(sP) + r * 128;
    DropoutSpec drop = {};
    unsigned long long drop_row = 0;  // first mask word of this query row
    if (DROP) {
      drop = make_dropout_spec(p.seed_ptr, p.site, p.drop_p);
      drop_row = ((unsigned long long)bh * p.T + (unsigned long long)(qi * QT + r)) *
                 (unsigned long long)((p.T + 3) / 4);
    }
    bool ok = true;
    Z2H_TRACE_DECL(2)
#define Z2H_CTRACE()                         \
  do {                                       \
    if (warp == 2 && lane == 0) Z2H_TRACE(); \
  } while (0)
    Z2H_CTRACE();
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait_bounded(s_full, j & 1, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      Z2H_CTRACE();  // scores are there
      const bool diag = (j == qi);
      // the whole score row (128 fp32) comes into registers with one wait
      uint32_t sv[KT / 32][32];
#pragma unroll
      for (int ch = 0; ch < KT / 32; ++ch) tmem_ld_32x32b_x32(t_lane + S_COL + ch * 32, sv[ch]);
      tmem_ld_wait();
      // the score columns may be overwritten with the next tile from here on
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_read);
      Z2H_CTRACE();  // scores in registers
      float m_new = m_run;
      if (!diag) {
        float m0 = m_new, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          m0 = max3(m0, __uint_as_float(sv[0][i]), __uint_as_float(sv[0][i + 1]));
          m1 = max3(m1, __uint_as_float(sv[1][i]), __uint_as_float(sv[1][i + 1]));
          m2 = max3(m2, __uint_as_float(sv[2][i]), __uint_as_float(sv[2][i + 1]));
          m3 = max3(m3, __uint_as_float(sv[3][i]), __uint_as_float(sv[3][i + 1]));
        }
        m_new = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      } else {
#pragma unroll
        for (int ch = 0; ch < KT / 32; ++ch)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (ch * 32 + i <= r) m_new = fmaxf(m_new, __uint_as_float(sv[ch][i]));
      }
      if (j == 0) {
        m_run = m_new;  // nothing accumulated yet
      } else {
        // P V of tile j-1 must be complete before O is rescaled and before P is overwritten
        if (!mbar_wait_bounded(pv_full, (j - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const bool grow = (m_new - m_run) * p.scale_log2 > 8.f;
        if (__any_sync(0xffffffffu, grow)) {
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
      Z2H_CTRACE();  // maximum known, previous P V complete
      const float mc = m_run * p.scale_log2;
      // p = 2^(s * c - m * c), row sum, bf16 P into swizzled shared memory
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int ch = 0; ch < KT / 32; ++ch) {
        // 32 columns = four 16-byte chunks of this row inside swizzle atom (ch >> 1)
        const uint32_t atom = p_row + (ch >> 1) * (QT * 128);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t pk[4];
          uint32_t mw[2] = {0, 0};
          if (DROP) {
            const unsigned long long w0 = drop_row + (unsigned long long)(j * (KT / 4) + ch * 8 + q * 2);
            mw[0] = dropout_word(drop.seed_lo, drop.seed_hi, w0);
            mw[1] = dropout_word(drop.seed_lo, drop.seed_hi, w0 + 1);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = q * 8 + e * 2;
            float p0 = ex2_fast(fmaf(__uint_as_float(sv[ch][i]), p.scale_log2, -mc));
            float p1 = ex2_fast(fmaf(__uint_as_float(sv[ch][i + 1]), p.scale_log2, -mc));
            if (diag) {
              if (ch * 32 + i > r) p0 = 0.f;
              if (ch * 32 + i + 1 > r) p1 = 0.f;
            }
            rs0 += p0;
            rs1 += p1;
            if (DROP) {
              if (!dropout_keep(mw[e >> 1], (e & 1) * 2, drop.threshold)) p0 = 0.f;
              if (!dropout_keep(mw[e >> 1], (e & 1) * 2 + 1, drop.threshold)) p1 = 0.f;
            }
            pk[e] = pack_bf16x2(p0, p1);
          }
          const uint32_t chunk = (uint32_t)((ch & 1) * 4 + q) ^ (uint32_t)(r & 7);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(atom + chunk * 16),
                       "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                       : "memory");
        }
      }
      l_run += rs0 + rs1;
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);  // one arrival per softmax warp
      Z2H_CTRACE();  // P written
    }
    if (ok && !mbar_wait_bounded(pv_full, (n_kv - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) ok = false;
    tc_fence_after();
    float o[HD];
    if (ok) {
#pragma unroll
      for (int q = 0; q < HD / 32; ++q) {
        uint32_t ov[32];
        tmem_ld_32x32b_x32(t_lane + PV_COL + q * 32, ov);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[q * 32 + i] = __uint_as_float(ov[i]);
      }
    }
    const int t = qi * QT + r;
    if (ok && t < p.T) {
      const float inv = DROP ? drop.scale / l_run : 1.f / l_run;
      __nv_bfloat16* op = p.out + (long long)(row0 + t) * p.C + h * HD;
#pragma unroll
      for (int q = 0; q < HD / 8; ++q) {
        uint4 u;
        u.x = pack_bf16x2(o[q * 8 + 0] * inv, o[q * 8 + 1] * inv);
        u.y = pack_bf16x2(o[q * 8 + 2] * inv, o[q * 8 + 3] * inv);
        u.z = pack_bf16x2(o[q * 8 + 4] * inv, o[q * 8 + 5] * inv);
        u.w = pack_bf16x2(o[q * 8 + 6] * inv, o[q * 8 + 7] * inv);
        *reinterpret_cast<uint4*>(op + q * 8) = u;
      }
      if (p.lse != nullptr)
        p.lse[((long long)b * p.H + h) * p.T + t] = m_run * p.scale + __logf(l_run);
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
  const cudaError_t err = launch_kernel(drop_p > 0.f ? flash_fwd_kernel<true> : flash_fwd_kernel<false>,
                                        dim3(B * H * n_qt), dim3(NUM_THREADS), SMEM_BYTES, stream, true, tm, p);
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
