// Column sums of a block held one row per lane.
#pragma once
#include <cuda_runtime.h>

namespace z2h {

// v[j] = column j of this lane's row, N in {1, 2, 4, 8, 16, 32}. A butterfly in which every step
// halves the columns a lane keeps and doubles the rows they cover; once a lane is down to one column
// the remaining steps add whole partners. Afterwards every lane holds, as the return value, the sum
// over the warp's 32 rows of column (lane >> (5 - log2 N)), so 32 / N neighbouring lanes share a
// column. N - 1 + (5 - log2 N) shuffles instead of 5 N. All 32 lanes must call it.
template <int N>
__device__ __forceinline__ float warp_column_sums(float (&v)[N], int lane) {
  static_assert(N >= 1 && N <= 32 && (N & (N - 1)) == 0, "N must be a power of two up to 32");
  int n = N;  // a compile-time quantity once the loop is unrolled
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    if (n > 1) {
      n >>= 1;
      const bool upper = (lane & s) != 0;
#pragma unroll
      for (int j = 0; j < N / 2; ++j) {
        if (j < n) {
          const float send = upper ? v[j] : v[j + n];
          const float keep = upper ? v[j + n] : v[j];
          v[j] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
      }
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], s);
    }
  }
  return v[0];
}

}  // namespace z2h
