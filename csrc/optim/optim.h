// Optimizer-side host API: global grad-norm, fused clip + AdamW over flat fp32 buffers,
// bias-gradient column sums and small utilities.
#pragma once
#include <cuda_runtime.h>

namespace z2h {

// Device-resident hyper-parameters (16 floats), rewritten by the host before every step so
// that a captured CUDA graph picks up the new learning rate without being re-captured.
enum HyperSlot : int {
  kHyLr = 0, kHyBeta1 = 1, kHyBeta2 = 2, kHyEps = 3, kHyWeightDecay = 4,
  kHyBiasCorr1 = 5,   // 1 - beta1^t
  kHyBiasCorr2 = 6,   // 1 - beta2^t
  kHyMaxNorm = 7,     // <= 0 disables clipping
  kHyGradScale = 8,   // multiplied into every gradient before use (1/accumulation etc.)
  kHyNumSlots = 16,
};

constexpr int kGradNormMaxPartials = 1024;

// partials[0 .. num_blocks) = per-CTA sums of g^2; returns the number of CTAs it used
// (<= kGradNormMaxPartials) or a negative error.
int gradnorm_partials(const float* g, long long n, float* partials, cudaStream_t stream);

// One pass over the flat buffers: total norm from the partials, clip coefficient, AdamW
// (decoupled weight decay on elements [0, n_decay)), bf16 working copy, optional grad zeroing.
// norm_out (may be null) receives the pre-clip global L2 norm.
int adamw_step(float* p32, float* g, float* m, float* v, void* p16, long long n, long long n_decay,
               const float* hyper, const float* partials, int num_partials, float* norm_out,
               int zero_grad, cudaStream_t stream);

// db[n] (+)= sum_m dy[m, n]; dy is bf16 [M, ld].
int colsum_bf16_ordered(const void* dy, int M, int N, long long ld, float* db, int accumulate, int ordered,
                        float* scratch, cudaStream_t stream);
long long colsum_scratch_elems(int M, int N);
int colsum_bf16(const void* dy, int M, int N, long long ld, float* db, int accumulate,
                cudaStream_t stream);

int cast_f32_to_bf16(const float* src, void* dst, long long n, cudaStream_t stream);

}  // namespace z2h
