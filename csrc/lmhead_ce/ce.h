// Cross-entropy host API.
#pragma once
#include <cuda_runtime.h>
namespace z2h {
// logits: bf16 [M, ld] (ld >= V_pad, multiple of 8); overwritten with dlogits when write_grad.
// losses: fp32 [M] per-row loss (may be null). Rows whose target equals ignore_index (or is out
// of range) contribute zero loss and zero gradient.
int ce_fwd_bwd(void* logits, const void* targets, int idx_is_64, float* losses, int M, int V_real,
               int V_pad, long long ld, float grad_scale, int write_grad, int ignore_index,
               cudaStream_t stream);
int reduce_sum(const float* x, int n, float scale, float* out, int accumulate, cudaStream_t stream);
}  // namespace z2h
