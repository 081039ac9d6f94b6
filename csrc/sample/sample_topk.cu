// Next-token sampling in one kernel per batch: temperature, top-k filter, softmax, multinomial.
//
// One CTA per row of fp32 logits [B, V]:
//   1. (top-k) the k-th largest logit is found exactly by a 4-pass, 8-bit radix select over
//      order-preserving integer keys; every logit >= that value is kept, ties included, which is
//      what masking with `logits < topk(logits, k).values[-1]` keeps
//      (nn/gpt2/modules.py:131-133 of the reference);
//   2. row maximum and sum of exp((x - max) / T) over the kept logits;
//   3. a uniform number from a counter-based generator (Philox 4x32-10 keyed by seed, counter
//      = offset + row) picks the token by inverse CDF: per-thread segment sums, a block scan of
//      those, and a serial walk inside the one segment that contains the target.
// The result depends only on (logits, temperature, k, seed, offset): no atomics, no
// scheduling-dependent order. Replaces softmax + torch.multinomial (modules.py:134-135).
#include <cuda_runtime.h>
#include <cstdint>

namespace z2h {
namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float <-> larger key
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ uint32_t mulhilo(uint32_t a, uint32_t b, uint32_t* hi) {
  const uint64_t p = (uint64_t)a * b;
  *hi = (uint32_t)(p >> 32);
  return (uint32_t)p;
}
// Philox 4x32 with 10 rounds; returns the first output word as a float in [0, 1).
__device__ float philox_uniform(uint64_t seed, uint64_t counter) {
  uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, hi1;
    const uint32_t lo0 = mulhilo(0xD2511F53u, c0, &hi0);
    const uint32_t lo1 = mulhilo(0xCD9E8D57u, c2, &hi1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (c0 >> 8) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int w = 0; w < kThreads / 32; ++w) r = is_max ? fmaxf(r, sh[w]) : r + sh[w];
  return r;
}

__global__ void __launch_bounds__(kThreads)
sample_topk_kernel(const float* __restrict__ logits, long long* __restrict__ out, int V, long long ld,
                   float inv_temperature, int top_k, uint64_t seed, uint64_t offset) {
  __shared__ unsigned int hist[256];
  __shared__ float sh[kThreads / 32];
  __shared__ float seg_prefix[kThreads];
  __shared__ uint32_t s_prefix_key;
  __shared__ int s_remaining;
  const int row = blockIdx.x;
  const float* x = logits + (long long)row * ld;

  // ---- 1. threshold = k-th largest logit (or -inf when no top-k filter applies)
  float threshold = -INFINITY;
  if (top_k > 0 && top_k < V) {
    uint32_t prefix = 0, mask = 0;
    int remaining = top_k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = threadIdx.x; i < 256; i += kThreads) hist[i] = 0;
      __syncthreads();
      for (int i = threadIdx.x; i < V; i += kThreads) {
        const uint32_t k = order_key(x[i]);
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int rem = remaining, b = 255;
        for (; b > 0; --b) {  // walk from the largest digit down
          if ((int)hist[b] >= rem) break;
          rem -= (int)hist[b];
        }
        s_prefix_key = prefix | ((uint32_t)b << shift);
        s_remaining = rem;
      }
      __syncthreads();
      prefix = s_prefix_key;
      remaining = s_remaining;
      mask |= 255u << shift;
      __syncthreads();
    }
    threshold = key_to_float(prefix);
  }

  // ---- 2. max and normaliser over the kept logits
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float v = x[i];
    if (v >= threshold) m = fmaxf(m, v);
  }
  m = block_reduce(m, sh, true);

  // ---- 3. inverse-CDF draw over contiguous per-thread segments
  const int seg = (V + kThreads - 1) / kThreads;
  const int i0 = threadIdx.x * seg, i1 = min(V, i0 + seg);
  float local = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float v = x[i];
    if (v >= threshold) local += __expf((v - m) * inv_temperature);
  }
  seg_prefix[threadIdx.x] = local;
  __syncthreads();
  // inclusive Hillis-Steele scan over the 1024 segment sums
  for (int off = 1; off < kThreads; off <<= 1) {
    float t = 0.f;
    if (threadIdx.x >= off) t = seg_prefix[threadIdx.x - off];
    __syncthreads();
    seg_prefix[threadIdx.x] += t;
    __syncthreads();
  }
  const float total = seg_prefix[kThreads - 1];
  const float target = philox_uniform(seed, offset + row) * total;
  const float before = threadIdx.x == 0 ? 0.f : seg_prefix[threadIdx.x - 1];
  const float upto = seg_prefix[threadIdx.x];
  // exactly one non-empty segment satisfies before <= target < upto (the last one also takes
  // target == total, which rounding can produce)
  const bool last_nonempty = (upto == total) && (before < total);
  if (local > 0.f && target >= before && (target < upto || last_nonempty)) {
    float acc = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float v = x[i];
      if (v >= threshold) {
        acc += __expf((v - m) * inv_temperature);
        pick = i;  // the last kept index so far: the fallback when rounding leaves acc < target
        if (acc > target) break;
      }
    }
    if (pick >= 0) out[row] = pick;
  }
}

}  // namespace

int sample_topk(const float* logits, long long* out, int B, int V, long long ld, float temperature,
                int top_k, unsigned long long seed, unsigned long long offset, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (V <= 0 || !(temperature > 0.f)) return 1;
  sample_topk_kernel<<<B, kThreads, 0, stream>>>(logits, out, V, ld, 1.0f / temperature, top_k, seed, offset);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace z2h

extern "C" int z2h_sample_topk(const float* logits, long long* out, int B, int V, long long ld,
                               float temperature, int top_k, unsigned long long seed,
                               unsigned long long offset, void* stream) {
  return z2h::sample_topk(logits, out, B, V, ld, temperature, top_k, seed, offset, (cudaStream_t)stream);
}
