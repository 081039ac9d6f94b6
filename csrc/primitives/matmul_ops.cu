// fp32 teaching kernels around matrix products and small fused ops: naive / shared / tiled
// cp.async matmul, tiled transpose, 1-D softmax, single-query attention, a TF32 mma.sync
// tensor-core matmul (the legacy tensor path; the tcgen05 twin is csrc/gemm), embedding
// gathers, and LayerNorm+Linear forward / backward in unfused, fused-with-atomics and
// deterministic forms. CUDA C++ counterparts of gpu-mojo/problems/p16, p18, p19, p21, p22 and
// p33 of the reference, including the GPU orchestration of the attention op and the
// LayerNorm kernel that the reference leaves unfilled (p19/op/attention.mojo:372-394,
// p22/op/layernorm_linear.mojo:141).
#include <cuda_runtime.h>
#include <cstdint>

#include "../common/ptx.cuh"

namespace z2h {
namespace prim {

// ---------------------------------------------------------------- p16: three matmuls, C = A B
__global__ void matmul_naive_kernel(float* c, const float* a, const float* b, int M, int N, int K) {
  const int row = blockIdx.y * blockDim.y + threadIdx.y, col = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < M && col < N) {
    float s = 0.f;
    for (int k = 0; k < K; ++k) s += a[row * K + k] * b[k * N + col];
    c[row * N + col] = s;
  }
}
// whole (small) problem in one block's shared memory
__global__ void matmul_single_block_kernel(float* c, const float* a, const float* b, int M, int N, int K) {
  extern __shared__ float sh[];
  float* sa = sh;
  float* sb = sh + M * K;
  for (int i = threadIdx.y * blockDim.x + threadIdx.x; i < M * K; i += blockDim.x * blockDim.y) sa[i] = a[i];
  for (int i = threadIdx.y * blockDim.x + threadIdx.x; i < K * N; i += blockDim.x * blockDim.y) sb[i] = b[i];
  __syncthreads();
  for (int row = threadIdx.y; row < M; row += blockDim.y)
    for (int col = threadIdx.x; col < N; col += blockDim.x) {
      float s = 0.f;
      for (int k = 0; k < K; ++k) s += sa[row * K + k] * sb[k * N + col];
      c[row * N + col] = s;
    }
}
// TILE x TILE tiles staged with cp.async (4-byte copies, zero fill outside the matrices)
template <int TILE>
__global__ void matmul_tiled_kernel(float* c, const float* a, const float* b, int M, int N, int K) {
  __shared__ float sa[TILE][TILE], sb[TILE][TILE];
  const int ty = threadIdx.y, tx = threadIdx.x;
  const int row = blockIdx.y * TILE + ty, col = blockIdx.x * TILE + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += TILE) {
    if (row < M && k0 + tx < K) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(&sa[ty][tx])),
                   "l"(a + row * K + k0 + tx)
                   : "memory");
    } else {
      sa[ty][tx] = 0.f;
    }
    if (k0 + ty < K && col < N) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(&sb[ty][tx])),
                   "l"(b + (k0 + ty) * N + col)
                   : "memory");
    } else {
      sb[ty][tx] = 0.f;
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TILE; ++k) acc += sa[ty][k] * sb[k][tx];
    __syncthreads();
  }
  if (row < M && col < N) c[row * N + col] = acc;
}

// ---------------------------------------------------------------- transpose, softmax, attention
__global__ void transpose_kernel(float* out, const float* in, int rows, int cols) {
  __shared__ float tile[16][17];
  int r = blockIdx.y * 16 + threadIdx.y, c = blockIdx.x * 16 + threadIdx.x;
  if (r < rows && c < cols) tile[threadIdx.y][threadIdx.x] = in[r * cols + c];
  __syncthreads();
  r = blockIdx.x * 16 + threadIdx.y;
  c = blockIdx.y * 16 + threadIdx.x;
  if (r < cols && c < rows) out[r * rows + c] = tile[threadIdx.x][threadIdx.y];
}
// numerically stable softmax of one vector per block (blockDim.x a power of two)
__global__ void softmax_kernel(float* out, const float* in, int n) {
  extern __shared__ float sh[];
  const float* x = in + (long long)blockIdx.x * n;
  float* y = out + (long long)blockIdx.x * n;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, x[i]);
  sh[threadIdx.x] = m;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) sh[threadIdx.x] = fmaxf(sh[threadIdx.x], sh[threadIdx.x + s]);
    __syncthreads();
  }
  m = sh[0];
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sum += expf(x[i] - m);
  sh[threadIdx.x] = sum;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
    __syncthreads();
  }
  sum = sh[0];
  for (int i = threadIdx.x; i < n; i += blockDim.x) y[i] = expf(x[i] - m) / sum;
}
// single-query attention in one kernel: out = softmax(q K^T) V, K and V are [seq, d]
// (no scaling and no mask, as in the reference op)
__global__ void attention_vec_kernel(float* out, const float* q, const float* k, const float* v, int seq,
                                     int d) {
  extern __shared__ float sh[];  // seq scores + blockDim.x reduction slots
  float* score = sh;
  float* red = sh + seq;
  for (int s = threadIdx.x; s < seq; s += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < d; ++j) acc += q[j] * k[s * d + j];
    score[s] = acc;
  }
  __syncthreads();
  float m = -INFINITY;
  for (int s = threadIdx.x; s < seq; s += blockDim.x) m = fmaxf(m, score[s]);
  red[threadIdx.x] = m;
  __syncthreads();
  for (int st = blockDim.x / 2; st > 0; st >>= 1) {
    if (threadIdx.x < st) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + st]);
    __syncthreads();
  }
  m = red[0];
  __syncthreads();
  float sum = 0.f;
  for (int s = threadIdx.x; s < seq; s += blockDim.x) {
    const float e = expf(score[s] - m);
    score[s] = e;
    sum += e;
  }
  red[threadIdx.x] = sum;
  __syncthreads();
  for (int st = blockDim.x / 2; st > 0; st >>= 1) {
    if (threadIdx.x < st) red[threadIdx.x] += red[threadIdx.x + st];
    __syncthreads();
  }
  sum = red[0];
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < seq; ++s) acc += score[s] * v[s * d + j];
    out[j] = acc / sum;
  }
}

// ---------------------------------------------------------------- p33: TF32 mma.sync matmul
// C[M,N] = A[M,K] B[K,N], fp32 in memory, TF32 m16n8k8 tensor-core MMAs, fp32 accumulate.
// Block tile 128 x 64 x 32, 8 warps as 4 x 2, each warp a 32 x 32 tile (2 x 4 MMA tiles).
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__global__ void __launch_bounds__(256)
matmul_tf32_mma_kernel(float* c, const float* a, const float* b, int M, int N, int K) {
  constexpr int BM = 128, BN = 64, BK = 32;
  __shared__ float sa[BM][BK + 4], sb[BK][BN + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp >> 1, wn = warp & 1;
  const int gid = lane >> 2, tig = lane & 3;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[2][4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int i = threadIdx.x; i < BM * BK; i += 256) {
      const int r = i / BK, cc = i % BK;
      sa[r][cc] = (m0 + r < M && k0 + cc < K) ? a[(long long)(m0 + r) * K + k0 + cc] : 0.f;
    }
    for (int i = threadIdx.x; i < BK * BN; i += 256) {
      const int r = i / BN, cc = i % BN;
      sb[r][cc] = (k0 + r < K && n0 + cc < N) ? b[(long long)(k0 + r) * N + n0 + cc] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk += 8) {
      uint32_t af[2][4], bf[4][2];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        const int r = wm * 32 + mi * 16;
        af[mi][0] = to_tf32(sa[r + gid][kk + tig]);
        af[mi][1] = to_tf32(sa[r + gid + 8][kk + tig]);
        af[mi][2] = to_tf32(sa[r + gid][kk + tig + 4]);
        af[mi][3] = to_tf32(sa[r + gid + 8][kk + tig + 4]);
      }
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int cc = wn * 32 + ni * 8;
        bf[ni][0] = to_tf32(sb[kk + tig][cc + gid]);
        bf[ni][1] = to_tf32(sb[kk + tig + 4][cc + gid]);
      }
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
          asm volatile(
              "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
              "{%0,%1,%2,%3};"
              : "+f"(acc[mi][ni][0]), "+f"(acc[mi][ni][1]), "+f"(acc[mi][ni][2]), "+f"(acc[mi][ni][3])
              : "r"(af[mi][0]), "r"(af[mi][1]), "r"(af[mi][2]), "r"(af[mi][3]), "r"(bf[ni][0]),
                "r"(bf[ni][1]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      const int r = m0 + wm * 32 + mi * 16 + gid, cc = n0 + wn * 32 + ni * 8 + tig * 2;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int rr = r + h * 8;
        if (rr < M) {
          if (cc < N) c[(long long)rr * N + cc] = acc[mi][ni][h * 2];
          if (cc + 1 < N) c[(long long)rr * N + cc + 1] = acc[mi][ni][h * 2 + 1];
        }
      }
    }
}

// ---------------------------------------------------------------- p21: embedding gathers (int32 ids)
// 1-D: one thread per output element, consecutive threads walk the embedding dimension
__global__ void embedding_coalesced_kernel(float* out, const int* idx, const float* w, int n_idx, int dim,
                                           int vocab) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)n_idx * dim) return;
  const int t = (int)(i / dim), e = (int)(i % dim);
  const int id = idx[t];
  out[i] = (id >= 0 && id < vocab) ? w[(long long)id * dim + e] : 0.f;
}
// 2-D: x over tokens, y over the embedding dimension (the uncoalesced variant of the study)
__global__ void embedding_2d_kernel(float* out, const int* idx, const float* w, int n_idx, int dim,
                                    int vocab) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x, e = blockIdx.y * blockDim.y + threadIdx.y;
  if (t >= n_idx || e >= dim) return;
  const int id = idx[t];
  out[(long long)t * dim + e] = (id >= 0 && id < vocab) ? w[(long long)id * dim + e] : 0.f;
}

// ---------------------------------------------------------------- p22: LayerNorm + Linear
// LayerNorm of each row (biased variance, eps inside the square root), one block per row
__global__ void ln_rows_kernel(float* out, const float* x, const float* gamma, const float* beta, int H,
                               float eps) {
  extern __shared__ float sh[];
  const float* xr = x + (long long)blockIdx.x * H;
  float s = 0.f, q = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    s += xr[i];
    q += xr[i] * xr[i];
  }
  sh[threadIdx.x] = s;
  sh[blockDim.x + threadIdx.x] = q;
  __syncthreads();
  for (int st = blockDim.x / 2; st > 0; st >>= 1) {
    if (threadIdx.x < st) {
      sh[threadIdx.x] += sh[threadIdx.x + st];
      sh[blockDim.x + threadIdx.x] += sh[blockDim.x + threadIdx.x + st];
    }
    __syncthreads();
  }
  const float mean = sh[0] / H;
  const float var = sh[blockDim.x] / H - mean * mean;
  const float inv = rsqrtf(var + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(long long)blockIdx.x * H + i] = (xr[i] - mean) * inv * gamma[i] + beta[i];
}
__global__ void add_bias_kernel(float* y, const float* bias, int rows, int cols) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < (long long)rows * cols) y[i] += bias[i % cols];
}
// fused forward: one thread per token recomputes the statistics and produces all outputs
// y[t, o] = sum_h LN(x)[t, h] * W[o, h] + b[o]
__global__ void ln_linear_fused_fwd_kernel(float* y, const float* x, const float* gamma, const float* beta,
                                           const float* w, const float* bias, int T, int H, int O, float eps) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* xr = x + (long long)t * H;
  float s = 0.f, q = 0.f;
  for (int h = 0; h < H; ++h) {
    s += xr[h];
    q += xr[h] * xr[h];
  }
  const float mean = s / H, inv = rsqrtf(q / H - mean * mean + eps);
  for (int o = 0; o < O; ++o) {
    float acc = bias[o];
    for (int h = 0; h < H; ++h) acc += ((xr[h] - mean) * inv * gamma[h] + beta[h]) * w[(long long)o * H + h];
    y[(long long)t * O + o] = acc;
  }
}
// fused backward with atomics (the reference's scheme, layernorm_linear.mojo:290-459): one
// thread per token; dW, db, dgamma, dbeta via atomicAdd (order-dependent rounding), dX closed form
__global__ void ln_linear_bwd_atomic_kernel(const float* dy, const float* x, const float* gamma,
                                            const float* beta, const float* w, float* dx, float* dgamma,
                                            float* dbeta, float* dw, float* dbias, int T, int H, int O,
                                            float eps) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* xr = x + (long long)t * H;
  const float* dyr = dy + (long long)t * O;
  float s = 0.f, q = 0.f;
  for (int h = 0; h < H; ++h) {
    s += xr[h];
    q += xr[h] * xr[h];
  }
  const float mean = s / H, inv = rsqrtf(q / H - mean * mean + eps);
  for (int o = 0; o < O; ++o) atomicAdd(&dbias[o], dyr[o]);
  float sum_g = 0.f, sum_gx = 0.f;
  for (int h = 0; h < H; ++h) {
    const float xh = (xr[h] - mean) * inv;
    const float ln = xh * gamma[h] + beta[h];
    float dln = 0.f;
    for (int o = 0; o < O; ++o) {
      dln += dyr[o] * w[(long long)o * H + h];
      atomicAdd(&dw[(long long)o * H + h], dyr[o] * ln);
    }
    atomicAdd(&dgamma[h], dln * xh);
    atomicAdd(&dbeta[h], dln);
    const float g = dln * gamma[h];
    sum_g += g;
    sum_gx += g * xh;
  }
  for (int h = 0; h < H; ++h) {
    const float xh = (xr[h] - mean) * inv;
    float dln = 0.f;
    for (int o = 0; o < O; ++o) dln += dyr[o] * w[(long long)o * H + h];
    const float g = dln * gamma[h];
    dx[(long long)t * H + h] = inv * (g - sum_g / H - xh * sum_gx / H);
  }
}
// deterministic backward: dX per token as above without the atomics; the parameter gradients
// are computed by a second kernel in which one thread owns one output element and walks the
// tokens in order, so the result does not depend on scheduling
__global__ void ln_linear_bwd_dx_kernel(const float* dy, const float* x, const float* gamma,
                                        const float* w, float* dx, int T, int H, int O, float eps) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* xr = x + (long long)t * H;
  const float* dyr = dy + (long long)t * O;
  float s = 0.f, q = 0.f;
  for (int h = 0; h < H; ++h) {
    s += xr[h];
    q += xr[h] * xr[h];
  }
  const float mean = s / H, inv = rsqrtf(q / H - mean * mean + eps);
  float sum_g = 0.f, sum_gx = 0.f;
  for (int h = 0; h < H; ++h) {
    float dln = 0.f;
    for (int o = 0; o < O; ++o) dln += dyr[o] * w[(long long)o * H + h];
    const float g = dln * gamma[h], xh = (xr[h] - mean) * inv;
    sum_g += g;
    sum_gx += g * xh;
  }
  for (int h = 0; h < H; ++h) {
    float dln = 0.f;
    for (int o = 0; o < O; ++o) dln += dyr[o] * w[(long long)o * H + h];
    const float xh = (xr[h] - mean) * inv;
    dx[(long long)t * H + h] = inv * (dln * gamma[h] - sum_g / H - xh * sum_gx / H);
  }
}
__global__ void ln_linear_bwd_params_kernel(const float* dy, const float* x, const float* gamma,
                                            const float* beta, const float* w, float* dgamma, float* dbeta,
                                            float* dw, float* dbias, int T, int H, int O, float eps) {
  // element ids: [0, O*H) -> dW, then O -> dbias, then H -> dgamma, then H -> dbeta
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int total = O * H + O + 2 * H;
  if (e >= total) return;
  float acc = 0.f;
  for (int t = 0; t < T; ++t) {
    const float* xr = x + (long long)t * H;
    const float* dyr = dy + (long long)t * O;
    if (e >= O * H && e < O * H + O) {
      acc += dyr[e - O * H];
      continue;
    }
    float s = 0.f, q = 0.f;
    for (int h = 0; h < H; ++h) {
      s += xr[h];
      q += xr[h] * xr[h];
    }
    const float mean = s / H, inv = rsqrtf(q / H - mean * mean + eps);
    if (e < O * H) {
      const int o = e / H, h = e % H;
      acc += dyr[o] * ((xr[h] - mean) * inv * gamma[h] + beta[h]);
    } else {
      const int h = (e - O * H - O) % H;
      float dln = 0.f;
      for (int o = 0; o < O; ++o) dln += dyr[o] * w[(long long)o * H + h];
      acc += (e < O * H + O + H) ? dln * (xr[h] - mean) * inv : dln;
    }
  }
  if (e < O * H) dw[e] = acc;
  else if (e < O * H + O) dbias[e - O * H] = acc;
  else if (e < O * H + O + H) dgamma[e - O * H - O] = acc;
  else dbeta[e - O * H - O - H] = acc;
}

inline int ok() { return cudaGetLastError() == cudaSuccess ? 0 : 3; }
inline int cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }
inline int pow2_at_least(int x) { int p = 1; while (p < x) p <<= 1; return p; }

}  // namespace prim
}  // namespace z2h

using namespace z2h::prim;
#define ST(s) ((cudaStream_t)(s))

extern "C" {
// variant: 0 naive, 1 single block in shared memory (small problems), 2 tiled with cp.async,
//          3 TF32 mma.sync tensor cores
int z2h_p_matmul(float* c, const float* a, const float* b, int M, int N, int K, int variant, void* s) {
  if (variant == 0) {
    dim3 block(16, 16), grid(cdiv(N, 16), cdiv(M, 16));
    matmul_naive_kernel<<<grid, block, 0, ST(s)>>>(c, a, b, M, N, K);
  } else if (variant == 1) {
    const size_t smem = (size_t)(M * K + K * N) * sizeof(float);
    if (smem > 48 * 1024) return 1;
    matmul_single_block_kernel<<<1, dim3(16, 16), smem, ST(s)>>>(c, a, b, M, N, K);
  } else if (variant == 2) {
    dim3 block(16, 16), grid(cdiv(N, 16), cdiv(M, 16));
    matmul_tiled_kernel<16><<<grid, block, 0, ST(s)>>>(c, a, b, M, N, K);
  } else if (variant == 3) {
    dim3 grid(cdiv(N, 64), cdiv(M, 128));
    matmul_tf32_mma_kernel<<<grid, 256, 0, ST(s)>>>(c, a, b, M, N, K);
  } else {
    return 1;
  }
  return ok();
}
int z2h_p_transpose(float* out, const float* in, int rows, int cols, void* s) {
  dim3 block(16, 16), grid(cdiv(cols, 16), cdiv(rows, 16));
  transpose_kernel<<<grid, block, 0, ST(s)>>>(out, in, rows, cols);
  return ok();
}
int z2h_p_softmax(float* out, const float* in, int rows, int n, void* s) {
  const int block = n >= 128 ? 128 : pow2_at_least(n < 32 ? 32 : n);
  softmax_kernel<<<rows, block, block * sizeof(float), ST(s)>>>(out, in, n);
  return ok();
}
int z2h_p_attention_vec(float* out, const float* q, const float* k, const float* v, int seq, int d, void* s) {
  const int block = 128;
  const size_t smem = (size_t)(seq + block) * sizeof(float);
  if (smem > 48 * 1024) return 1;
  attention_vec_kernel<<<1, block, smem, ST(s)>>>(out, q, k, v, seq, d);
  return ok();
}
int z2h_p_embedding(float* out, const int* idx, const float* w, int n_idx, int dim, int vocab, int variant,
                    void* s) {
  if (variant == 0) {
    embedding_coalesced_kernel<<<cdiv((long long)n_idx * dim, 256), 256, 0, ST(s)>>>(out, idx, w, n_idx, dim,
                                                                                   vocab);
  } else {
    dim3 block(16, 16), grid(cdiv(n_idx, 16), cdiv(dim, 16));
    embedding_2d_kernel<<<grid, block, 0, ST(s)>>>(out, idx, w, n_idx, dim, vocab);
  }
  return ok();
}
// fused == 0: LayerNorm -> transpose W -> tiled matmul -> add bias (tmp: T*H + H*O floats)
// fused == 1: one kernel
int z2h_p_ln_linear_fwd(float* y, const float* x, const float* gamma, const float* beta, const float* w,
                        const float* bias, int T, int H, int O, float eps, int fused, float* tmp, void* s) {
  if (fused) {
    ln_linear_fused_fwd_kernel<<<cdiv(T, 64), 64, 0, ST(s)>>>(y, x, gamma, beta, w, bias, T, H, O, eps);
    return ok();
  }
  float* ln = tmp;
  float* wt = tmp + (long long)T * H;
  const int block = H >= 128 ? 128 : pow2_at_least(H < 32 ? 32 : H);
  ln_rows_kernel<<<T, block, 2 * block * sizeof(float), ST(s)>>>(ln, x, gamma, beta, H, eps);
  dim3 tb(16, 16), tg(cdiv(H, 16), cdiv(O, 16));
  transpose_kernel<<<tg, tb, 0, ST(s)>>>(wt, w, O, H);  // W[O,H] -> Wt[H,O]
  dim3 mg(cdiv(O, 16), cdiv(T, 16));
  matmul_tiled_kernel<16><<<mg, tb, 0, ST(s)>>>(y, ln, wt, T, O, H);
  add_bias_kernel<<<cdiv((long long)T * O, 256), 256, 0, ST(s)>>>(y, bias, T, O);
  return ok();
}
// deterministic == 0: atomics (gradient buffers must be zero on entry); 1: two-kernel ordered sums
int z2h_p_ln_linear_bwd(const float* dy, const float* x, const float* gamma, const float* beta,
                        const float* w, float* dx, float* dgamma, float* dbeta, float* dw, float* dbias,
                        int T, int H, int O, float eps, int deterministic, void* s) {
  if (!deterministic) {
    ln_linear_bwd_atomic_kernel<<<cdiv(T, 64), 64, 0, ST(s)>>>(dy, x, gamma, beta, w, dx, dgamma, dbeta, dw,
                                                              dbias, T, H, O, eps);
  } else {
    ln_linear_bwd_dx_kernel<<<cdiv(T, 64), 64, 0, ST(s)>>>(dy, x, gamma, w, dx, T, H, O, eps);
    const int total = O * H + O + 2 * H;
    ln_linear_bwd_params_kernel<<<cdiv(total, 128), 128, 0, ST(s)>>>(dy, x, gamma, beta, w, dgamma, dbeta, dw,
                                                                    dbias, T, H, O, eps);
  }
  return ok();
}
}
