// out = dropout(x) (+ residual): the elementwise dropout sites of the GPT-2 block (embedding sum,
// attention projection output, MLP projection output; nn/gpt2/modules.py:23,52,79 of the
// reference) and their backward, which is the same kernel applied to the gradient.
// bf16 in and out, 8 elements (two mask words) per thread, in place allowed.
#include "../common/dropout.cuh"
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "dropout.h"

namespace z2h {
namespace {

__global__ void __launch_bounds__(256)
dropout_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                     __nv_bfloat16* __restrict__ out, long long n_vec, float p,
                     const unsigned long long* __restrict__ seed_ptr, uint32_t site) {
  pdl_launch_dependents();
  pdl_wait();
  const DropoutSpec d = make_dropout_spec(seed_ptr, site, p);
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < n_vec;
       v += (long long)gridDim.x * blockDim.x) {
    const uint4 u = *reinterpret_cast<const uint4*>(x + v * 8);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
    const uint32_t m0 = dropout_word(d.seed_lo, d.seed_hi, (unsigned long long)v * 2);
    const uint32_t m1 = dropout_word(d.seed_lo, d.seed_hi, (unsigned long long)v * 2 + 1);
    uint4 r = make_uint4(0, 0, 0, 0);
    if (residual != nullptr) r = *reinterpret_cast<const uint4*>(residual + v * 8);
    const uint32_t* rw = reinterpret_cast<const uint32_t*>(&r);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      const float2 g = unpack_bf16x2(rw[j]);
      const uint32_t m = j < 2 ? m0 : m1;
      const int e = (2 * j) & 3;
      const float a = dropout_keep(m, e, d.threshold) ? f.x * d.scale : 0.f;
      const float b = dropout_keep(m, e + 1, d.threshold) ? f.y * d.scale : 0.f;
      ow[j] = pack_bf16x2(a + g.x, b + g.y);
    }
    *reinterpret_cast<uint4*>(out + v * 8) = o;
  }
}

}  // namespace

int dropout_apply(const void* x, const void* residual, void* out, long long n, float p,
                  const unsigned long long* seed_ptr, unsigned int site, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0) return 1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(residual) & 15))
    return 1;
  if (!(p >= 0.f) || p >= 1.f) return 1;
  const long long n_vec = n / 8;
  long long blocks = (n_vec + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_kernel(dropout_apply_kernel, dim3((int)blocks), dim3(256), 0, stream, true, (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual,
                                                       (__nv_bfloat16*)out, n_vec, p, seed_ptr, site);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace z2h

extern "C" int z2h_dropout_apply(const void* x, const void* residual, void* out, long long n, float p,
                                 const unsigned long long* seed_ptr, unsigned int site, void* stream) {
  return z2h::dropout_apply(x, residual, out, n, p, seed_ptr, site, (cudaStream_t)stream);
}
