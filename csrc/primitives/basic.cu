// Elementary GPU primitives: maps, guards, 2-D indexing, broadcast, shared-memory staging,
// pooling, tree reductions, 1-D convolution with halo, block and multi-block prefix sums, row
// sums. CUDA C++ counterparts of the reference's first puzzles (gpu-mojo/problems/p01 .. p08,
// p11 .. p15), generic in size, plus 16-byte vectorised variants for large inputs.
//
// All kernels take fp32 data; every global access is guarded, so any launch geometry that
// covers the problem is valid.
#include <cuda_runtime.h>
#include <cstdint>

namespace z2h {
namespace prim {

// p01 / p03 / p06: out[i] = a[i] + 10, guarded, any number of blocks
__global__ void add10_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + 10.f;
}
// 16-byte vectorised variant for large n
__global__ void add10_vec4_kernel(float* out, const float* a, long long n) {
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(a)[i];
    v.x += 10.f; v.y += 10.f; v.z += 10.f; v.w += 10.f;
    reinterpret_cast<float4*>(out)[i] = v;
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) out[i] = a[i] + 10.f;
}
// p02: out = a + b
__global__ void zip_add_kernel(float* out, const float* a, const float* b, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i];
}
// p04 / p07: 2-D map over a rows x cols matrix, any 2-D grid
__global__ void add10_2d_kernel(float* out, const float* a, int rows, int cols) {
  const int r = blockIdx.y * blockDim.y + threadIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows && c < cols) out[r * cols + c] = a[r * cols + c] + 10.f;
}
// p05: out[r, c] = a[0, c] + b[r, 0]
__global__ void broadcast_add_kernel(float* out, const float* a, const float* b, int rows, int cols) {
  const int r = blockIdx.y * blockDim.y + threadIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows && c < cols) out[r * cols + c] = a[c] + b[r];
}
// p08: stage through shared memory, barrier, then map
__global__ void add10_shared_kernel(float* out, const float* a, int n) {
  extern __shared__ float sh[];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) sh[threadIdx.x] = a[i];
  __syncthreads();
  if (i < n) out[i] = sh[threadIdx.x] + 10.f;
}
// p11: out[i] = a[i] + a[i-1] + a[i-2] (missing terms dropped), via shared memory
__global__ void pool3_kernel(float* out, const float* a, int n) {
  extern __shared__ float sh[];  // blockDim.x + 2: two elements of left halo
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int l = threadIdx.x + 2;
  sh[l] = i < n ? a[i] : 0.f;
  if (threadIdx.x < 2) {
    const int h = (int)(blockIdx.x * blockDim.x) - 2 + threadIdx.x;
    sh[threadIdx.x] = h >= 0 ? a[h] : 0.f;
  }
  __syncthreads();
  if (i < n) out[i] = sh[l] + sh[l - 1] + sh[l - 2];
}
// p12: dot product with a shared-memory tree; one partial per block, folded with a second pass
__global__ void dot_tree_kernel(float* partial, const float* a, const float* b, int n) {
  extern __shared__ float sh[];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  sh[threadIdx.x] = i < n ? a[i] * b[i] : 0.f;
  __syncthreads();
  for (int stride = blockDim.x / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) sh[threadIdx.x] += sh[threadIdx.x + stride];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
__global__ void fold_partials_kernel(float* out, const float* partial, int n) {
  // single block, fixed order
  __shared__ float sh[256];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int stride = blockDim.x / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) sh[threadIdx.x] += sh[threadIdx.x + stride];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = sh[0];
}
// p13 / p17 / p20: out[i] = sum_k a[i + k] * w[k] (correlation, zero beyond the end); the block
// loads its tile plus a right halo of (k - 1) elements
__global__ void conv1d_kernel(float* out, const float* a, const float* w, int n, int k) {
  extern __shared__ float sh[];  // blockDim.x + k - 1 inputs, then k weights
  float* sw = sh + blockDim.x + k - 1;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  sh[threadIdx.x] = i < n ? a[i] : 0.f;
  for (int h = threadIdx.x; h < k - 1; h += blockDim.x) {
    const int g = (blockIdx.x + 1) * blockDim.x + h;
    sh[blockDim.x + h] = g < n ? a[g] : 0.f;
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) sw[j] = w[j];
  __syncthreads();
  if (i < n) {
    float s = 0.f;
    for (int j = 0; j < k; ++j) s += sh[threadIdx.x + j] * sw[j];
    out[i] = s;
  }
}
// p14: Hillis-Steele inclusive scan inside a block; optionally writes the block total
__global__ void scan_block_kernel(float* out, const float* a, float* block_sums, int n) {
  extern __shared__ float sh[];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  sh[threadIdx.x] = i < n ? a[i] : 0.f;
  __syncthreads();
  for (int off = 1; off < blockDim.x; off <<= 1) {
    float v = 0.f;
    if (threadIdx.x >= off) v = sh[threadIdx.x - off];
    __syncthreads();
    if (threadIdx.x >= off) sh[threadIdx.x] += v;
    __syncthreads();
  }
  if (i < n) out[i] = sh[threadIdx.x];
  if (block_sums != nullptr && threadIdx.x == blockDim.x - 1) block_sums[blockIdx.x] = sh[threadIdx.x];
}
// second phase of the multi-block scan: add the totals of all earlier blocks
__global__ void scan_add_block_sums_kernel(float* out, const float* block_sums, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (blockIdx.x == 0 || i >= n) return;
  float s = 0.f;
  for (int b = 0; b < blockIdx.x; ++b) s += block_sums[b];
  out[i] += s;
}
// p15: out[r] = sum_c a[r, c]; one block per row
__global__ void axis_sum_kernel(float* out, const float* a, int rows, int cols) {
  extern __shared__ float sh[];
  const int r = blockIdx.y;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s += a[r * cols + c];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int stride = blockDim.x / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) sh[threadIdx.x] += sh[threadIdx.x + stride];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[r] = sh[0];
}

inline int ok() { return cudaGetLastError() == cudaSuccess ? 0 : 3; }
inline int cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }
inline int pow2_at_least(int x) { int p = 1; while (p < x) p <<= 1; return p; }

}  // namespace prim
}  // namespace z2h

using namespace z2h::prim;

extern "C" {
int z2h_p_add10(float* out, const float* a, int n, int block, void* s) {
  add10_kernel<<<cdiv(n, block), block, 0, (cudaStream_t)s>>>(out, a, n);
  return ok();
}
int z2h_p_add10_vec4(float* out, const float* a, long long n, void* s) {
  if (((uintptr_t)out | (uintptr_t)a) & 15) return 1;
  int grid = cdiv(n / 4 + 1, 256);
  if (grid > 148 * 8) grid = 148 * 8;
  add10_vec4_kernel<<<grid, 256, 0, (cudaStream_t)s>>>(out, a, n);
  return ok();
}
int z2h_p_zip_add(float* out, const float* a, const float* b, int n, int block, void* s) {
  zip_add_kernel<<<cdiv(n, block), block, 0, (cudaStream_t)s>>>(out, a, b, n);
  return ok();
}
int z2h_p_add10_2d(float* out, const float* a, int rows, int cols, int bx, int by, void* s) {
  dim3 block(bx, by), grid(cdiv(cols, bx), cdiv(rows, by));
  add10_2d_kernel<<<grid, block, 0, (cudaStream_t)s>>>(out, a, rows, cols);
  return ok();
}
int z2h_p_broadcast_add(float* out, const float* a, const float* b, int rows, int cols, int bx, int by,
                        void* s) {
  dim3 block(bx, by), grid(cdiv(cols, bx), cdiv(rows, by));
  broadcast_add_kernel<<<grid, block, 0, (cudaStream_t)s>>>(out, a, b, rows, cols);
  return ok();
}
int z2h_p_add10_shared(float* out, const float* a, int n, int block, void* s) {
  add10_shared_kernel<<<cdiv(n, block), block, block * sizeof(float), (cudaStream_t)s>>>(out, a, n);
  return ok();
}
int z2h_p_pool3(float* out, const float* a, int n, int block, void* s) {
  pool3_kernel<<<cdiv(n, block), block, (block + 2) * sizeof(float), (cudaStream_t)s>>>(out, a, n);
  return ok();
}
// scratch: at least ceil(n / block) floats
int z2h_p_dot(float* out, const float* a, const float* b, int n, int block, float* scratch, void* s) {
  block = pow2_at_least(block);
  const int grid = cdiv(n, block);
  dot_tree_kernel<<<grid, block, block * sizeof(float), (cudaStream_t)s>>>(scratch, a, b, n);
  fold_partials_kernel<<<1, 256, 0, (cudaStream_t)s>>>(out, scratch, grid);
  return ok();
}
int z2h_p_conv1d(float* out, const float* a, const float* w, int n, int k, int block, void* s) {
  if (k < 1) return 1;
  const size_t smem = (block + k - 1 + k) * sizeof(float);
  conv1d_kernel<<<cdiv(n, block), block, smem, (cudaStream_t)s>>>(out, a, w, n, k);
  return ok();
}
// scratch: at least ceil(n / block) floats; block is rounded up to a power of two
int z2h_p_prefix_sum(float* out, const float* a, int n, int block, float* scratch, void* s) {
  block = pow2_at_least(block);
  const int grid = cdiv(n, block);
  scan_block_kernel<<<grid, block, block * sizeof(float), (cudaStream_t)s>>>(out, a,
                                                                            grid > 1 ? scratch : nullptr, n);
  if (grid > 1) scan_add_block_sums_kernel<<<grid, block, 0, (cudaStream_t)s>>>(out, scratch, n);
  return ok();
}
int z2h_p_axis_sum(float* out, const float* a, int rows, int cols, int block, void* s) {
  block = pow2_at_least(block);
  dim3 grid(1, rows);
  axis_sum_kernel<<<grid, block, block * sizeof(float), (cudaStream_t)s>>>(out, a, rows, cols);
  return ok();
}
}
