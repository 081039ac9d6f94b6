// Checked accesses for debug builds (-DZ2H_BOUNDS).
//
// compute-sanitizer's memcheck is what the reference runs its sanitizer puzzle under
// (gpu-mojo/README.md:17-18); where that tool is not at hand, a build with -DZ2H_BOUNDS makes
// the kernels check themselves: every guarded access first tests its index (or its row and
// column) against the extent it must stay inside, records the FIRST violation in the status
// word as kBoundsViolation | site << 8 (site: a small number naming the access), and skips the
// access. Nothing traps and nothing is read or written out of range, so the context stays
// usable and the host sees the failure with its next status read. In the product build the
// functions below are constant true and cost nothing.
//
//   python -m zero_to_hero_b200.build --bounds      builds zero_to_hero_b200/lib/libz2h_bounds.so
//   Z2H_NATIVE_LIB=bounds python -m pytest tests -m gpu   runs the GPU tests against it
#pragma once
#include <cuda_runtime.h>

namespace z2h {

constexpr int kBoundsViolation = 8;  // low byte of the status word; bits 8.. name the site

enum BoundsSite : int {
  kSiteGemmRow = 1,        // GEMM epilogue, full 32-column block of an output row
  kSiteGemmEdge = 2,       // GEMM epilogue, element-wise edge block
  kSiteGemmAtomic = 3,     // GEMM epilogue, coalesced atomic accumulation
  kSiteEmbedTable = 4,     // embedding: row of the token table
  kSiteEmbedOut = 5,       // embedding: output row
  kSiteFlashFwdOut = 6,    // attention forward: output row / log-sum-exp slot
  kSiteFlashBwdOut = 7,    // attention backward: dK / dV rows
};

#ifdef Z2H_BOUNDS
__device__ __forceinline__ bool in_bounds(long long idx, long long extent, int* status, int site) {
  if (idx >= 0 && idx < extent) return true;
  if (status != nullptr) atomicCAS(status, 0, kBoundsViolation | (site << 8));
  return false;
}
// [row, row + nrows) x [col, col + ncols) inside an M x N matrix
__device__ __forceinline__ bool in_bounds_2d(long long row, long long nrows, long long M, long long col,
                                             long long ncols, long long N, int* status, int site) {
  if (row >= 0 && row + nrows <= M && col >= 0 && col + ncols <= N) return true;
  if (status != nullptr) atomicCAS(status, 0, kBoundsViolation | (site << 8));
  return false;
}
#else
__device__ __forceinline__ bool in_bounds(long long, long long, int*, int) { return true; }
__device__ __forceinline__ bool in_bounds_2d(long long, long long, long long, long long, long long, long long,
                                             int*, int) {
  return true;
}
#endif

}  // namespace z2h
