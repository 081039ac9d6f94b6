// Debugging / sanitizer exercises as *fixed* kernels, plus a checked accessor that turns an
// out-of-range index into a recorded violation instead of a fault.
//
// The reference's p09 and p10 ship kernels with planted bugs (a window loop to inspect with a
// debugger, a neighbour filter whose barriers sit in divergent code, an accumulation into
// uninitialised shared memory, gpu-mojo/problems/p09/p09.mojo:35-99, p10/p10.mojo:20-42) meant
// to be run under cuda-gdb and compute-sanitizer. Here the kernels are the corrected versions,
// and the memory-error lesson is carried by `checked_gather_kernel`: every index goes through
// an accessor that records {first bad index, count} in a status block and skips the access, so
// the context stays healthy.
#include <cuda_runtime.h>

namespace z2h {
namespace prim {

// p09 second case: out[i] = a[i-1] + a[i] + a[i+1], terms outside [0, n) dropped
__global__ void sliding_window3_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int off = -1; off <= 1; ++off) {
    const int j = i + off;
    if (j >= 0 && j < n) s += a[j];
  }
  out[i] = s;
}
// p09 third case: the first n-1 elements get half of their left neighbour added (using the
// neighbour's original value), the last element passes through; one block, all threads reach
// both barriers
__global__ void collaborative_filter_kernel(float* out, const float* a, int n) {
  extern __shared__ float ws[];
  const int t = threadIdx.x;
  if (t < n - 1) ws[t] = a[t];
  __syncthreads();
  float v = 0.f;
  if (t < n - 1) v = ws[t] + (t > 0 ? ws[t - 1] * 0.5f : 0.f);
  __syncthreads();
  if (t < n - 1) out[t] = v;
  else if (t < n) out[t] = a[t];
}
// p10: every element of the size x size output receives the sum of the input; the shared
// accumulator is initialised before use and written by a single thread
__global__ void shared_sum_broadcast_kernel(float* out, const float* a, int size) {
  __shared__ float total;
  if (threadIdx.x == 0 && threadIdx.y == 0) {
    float s = 0.f;
    for (int r = 0; r < size; ++r)
      for (int c = 0; c < size; ++c) s += a[r * size + c];
    total = s;
  }
  __syncthreads();
  const int r = threadIdx.y, c = threadIdx.x;
  if (r < size && c < size) out[r * size + c] = total;
}

// status block: [0] number of violations, [1] first offending thread, [2] its index
struct Checked {
  const float* base;
  int n;
  int* status;
  __device__ float load(int i, int who) const {
    if (i < 0 || i >= n) {
      if (atomicAdd(&status[0], 1) == 0) {
        status[1] = who;
        status[2] = i;
      }
      return 0.f;
    }
    return base[i];
  }
};
// out[t] = src[idx[t]] through the checked accessor
__global__ void checked_gather_kernel(float* out, const float* src, const int* idx, int n_out, int n_src,
                                      int* status) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_out) return;
  Checked acc{src, n_src, status};
  out[t] = acc.load(idx[t], t);
}

}  // namespace prim
}  // namespace z2h

using namespace z2h::prim;

extern "C" {
int z2h_p_sliding_window3(float* out, const float* a, int n, void* s) {
  sliding_window3_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)s>>>(out, a, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
int z2h_p_collaborative_filter(float* out, const float* a, int n, void* s) {
  if (n < 1 || n > 1024) return 1;
  collaborative_filter_kernel<<<1, n, n * sizeof(float), (cudaStream_t)s>>>(out, a, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
int z2h_p_shared_sum_broadcast(float* out, const float* a, int size, void* s) {
  if (size < 1 || size > 32) return 1;
  shared_sum_broadcast_kernel<<<1, dim3(size, size), 0, (cudaStream_t)s>>>(out, a, size);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
// status: 3 ints, zeroed by the caller
int z2h_p_checked_gather(float* out, const float* src, const int* idx, int n_out, int n_src, int* status,
                         void* s) {
  checked_gather_kernel<<<(n_out + 127) / 128, 128, 0, (cudaStream_t)s>>>(out, src, idx, n_out, n_src,
                                                                        status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
}
