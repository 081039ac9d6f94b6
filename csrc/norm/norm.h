// LayerNorm host API (bf16 activations / weights, fp32 statistics and gradients).
#pragma once
#include <cuda_runtime.h>

namespace z2h {

// Upper bound on the number of CTAs (= partial rows in the scratch buffer) of the backward.
constexpr int kLayerNormBwdMaxCtas = 296;  // 2 per SM on a 148-SM part

// Number of partial rows the backward writes for M rows; scratch must hold
// num_partials * 2 * C floats.
int layernorm_bwd_num_partials(int M);

int layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                  int M, int C, float eps, cudaStream_t stream);

// dx = dresid + d(LN)/dx; dw/db are fp32 and are overwritten or accumulated into.
// dresid and db may be null; dx may alias dresid or dy.
int layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                  const void* dresid, void* dx, float* dw, float* db, float* scratch, int M, int C,
                  int accumulate, cudaStream_t stream);

// The same, and in addition dxsum[C] += column sums of dx (always accumulated). dx is the gradient
// of whatever was added into the residual stream before this LayerNorm, so its column sums are the
// bias gradient of that projection. scratch must hold num_partials * 3 * C floats here.
int layernorm_bwd_dxsum(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                        const void* dresid, void* dx, float* dw, float* db, float* dxsum, float* scratch,
                        int M, int C, int accumulate, cudaStream_t stream);

}  // namespace z2h
