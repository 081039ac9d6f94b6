// Warp-, block- and cluster-level primitives: shuffles, butterflies, warp scans and
// partition, block collectives, asynchronous copies, mbarrier-coordinated pipelines, access
// pattern / occupancy / bank-conflict study kernels, thread-block-cluster reductions.
// CUDA C++ counterparts of gpu-mojo/problems/p23 .. p32 and p34 of the reference.
//
// Two deliberate differences from the reference kernels: every mbarrier wait is bounded (the
// reference spins without limit, p29.mojo:183-184,219-220,241-242) and the cluster reduction
// also comes in a distributed-shared-memory form that needs no global scratch.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "../common/ptx.cuh"

namespace cg = cooperative_groups;

namespace z2h {
namespace prim {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}
__device__ __forceinline__ float warp_inclusive_scan(float v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(FULL, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// ---------------------------------------------------------------- p23: elementwise add variants
__global__ void ew_add_scalar_kernel(float* out, const float* a, const float* b, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i];
}
// each block owns a tile of `tile` elements, threads stride through it
__global__ void ew_add_tiled_kernel(float* out, const float* a, const float* b, int n, int tile) {
  const int base = blockIdx.x * tile;
  for (int j = threadIdx.x; j < tile && base + j < n; j += blockDim.x) out[base + j] = a[base + j] + b[base + j];
}
// 16-byte vector loads/stores
__global__ void ew_add_vec4_kernel(float* out, const float* a, const float* b, long long n) {
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 x = reinterpret_cast<const float4*>(a)[i], y = reinterpret_cast<const float4*>(b)[i];
    reinterpret_cast<float4*>(out)[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) out[i] = a[i] + b[i];
}

// ---------------------------------------------------------------- p24: per-warp dot products
// out[w] = sum over the w-th group of 32 elements of a * b
__global__ void warp_dot_kernel(float* out, const float* a, const float* b, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const float v = i < n ? a[i] * b[i] : 0.f;
  const float s = warp_sum(v);
  if ((threadIdx.x & 31) == 0 && i < n) out[i >> 5] = s;
}
// redux.sync flavour for integer data (single instruction warp reduction)
__global__ void warp_sum_int_kernel(int* out, const int* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int v = i < n ? a[i] : 0;
  const int s = __reduce_add_sync(FULL, v);
  if ((threadIdx.x & 31) == 0 && i < n) out[i >> 5] = s;
}

// ---------------------------------------------------------------- p25: shuffle_down / broadcast
__global__ void neighbor_difference_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const float cur = i < n ? a[i] : 0.f;
  const float nxt = __shfl_down_sync(FULL, cur, 1);
  if (i < n) out[i] = lane < 31 ? nxt - cur : 0.f;
}
__global__ void moving_average3_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const float cur = i < n ? a[i] : 0.f;
  const float n1 = __shfl_down_sync(FULL, cur, 1), n2 = __shfl_down_sync(FULL, cur, 2);
  if (i < n) {
    if (lane < 30) out[i] = (cur + n1 + n2) / 3.f;
    else if (lane < 31 && i < n - 1) out[i] = (cur + n1) / 2.f;
    else out[i] = cur;
  }
}
__global__ void broadcast_shuffle_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const float cur = i < n ? a[i] : 0.f;
  const float n1 = __shfl_down_sync(FULL, cur, 1), n2 = __shfl_down_sync(FULL, cur, 2),
              n3 = __shfl_down_sync(FULL, cur, 3);
  float scale = lane == 0 ? (cur + n1 + n2 + n3) / 4.f : 0.f;
  scale = __shfl_sync(FULL, scale, 0);
  if (i < n) out[i] = lane < 31 ? (cur + n1) * scale : cur * scale;
}
__global__ void basic_broadcast_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const float cur = i < n ? a[i] : 0.f;
  const float n1 = __shfl_down_sync(FULL, cur, 1), n2 = __shfl_down_sync(FULL, cur, 2),
              n3 = __shfl_down_sync(FULL, cur, 3);
  float v = lane == 0 ? cur + n1 + n2 + n3 : 0.f;
  v = __shfl_sync(FULL, v, 0);
  if (i < n) out[i] = cur + v;
}
__global__ void conditional_broadcast_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const float cur = i < n ? a[i] : 0.f;
  float decision = lane == 0 ? cur : 0.f;
#pragma unroll
  for (int off = 1; off < 8; ++off) {
    const float nx = __shfl_down_sync(FULL, cur, off);
    if (lane == 0) decision = fmaxf(decision, nx);
  }
  decision = __shfl_sync(FULL, decision, 0);
  if (i < n) out[i] = cur >= decision / 2.f ? cur * 2.f : cur / 2.f;
}

// ---------------------------------------------------------------- p26: butterflies, scan, partition
__global__ void butterfly_pair_swap_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const float cur = i < n ? a[i] : 0.f;
  const float other = __shfl_xor_sync(FULL, cur, 1);
  if (i < n) out[i] = other;
}
__global__ void butterfly_max_kernel(float* out, const float* a, int n, int conditional) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const float cur = i < n ? a[i] : -INFINITY;
  float mx = cur, mn = i < n ? a[i] : INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
    mn = fminf(mn, __shfl_xor_sync(FULL, mn, o));
  }
  if (i < n) out[i] = (conditional && (lane & 1)) ? mn : mx;
}
__global__ void warp_prefix_sum_kernel(float* out, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const float cur = i < n ? a[i] : 0.f;
  const float s = warp_inclusive_scan(cur, threadIdx.x & 31);
  if (i < n) out[i] = s;
}
// one warp: elements < pivot to the left (in order), the others to the right (in order)
__global__ void warp_partition_kernel(float* out, const float* a, int n, float pivot) {
  const int lane = threadIdx.x & 31;
  const bool valid = lane < n;
  const float cur = valid ? a[lane] : 0.f;
  const bool is_less = valid && cur < pivot;
  const unsigned less_mask = __ballot_sync(FULL, is_less);
  const unsigned more_mask = __ballot_sync(FULL, valid && !is_less);
  const unsigned below = (1u << lane) - 1u;
  const int left = __popc(less_mask & below), right = __popc(more_mask & below);
  const int less_total = __popc(less_mask);
  if (valid) out[is_less ? left : less_total + right] = cur;
}

// ---------------------------------------------------------------- p27: block collectives
template <int TPB>
__device__ __forceinline__ float block_sum_f(float v, float* sh) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < TPB / 32; ++w) t += sh[w];
  __syncthreads();
  return t;
}
__global__ void block_dot_kernel(float* out, const float* a, const float* b, int n) {
  __shared__ float sh[8];
  const int i = threadIdx.x;
  const float s = block_sum_f<256>(i < n ? a[i] * b[i] : 0.f, sh);
  if (i == 0) out[0] = s;
}
// pack the elements of one histogram bin (values in [0,1)) to the front of bin_out, in order
__global__ void block_histogram_bin_extract_kernel(const float* a, float* bin_out, int* count_out, int n,
                                                   int target_bin, int num_bins) {
  __shared__ int warp_tot[8];
  const int i = threadIdx.x, lane = i & 31, warp = i >> 5;
  float val = 0.f;
  int bin = -1;
  if (i < n) {
    val = a[i];
    bin = (int)floorf(val * num_bins);
    bin = bin >= num_bins ? num_bins - 1 : (bin < 0 ? 0 : bin);
  }
  const int match = (i < n && bin == target_bin) ? 1 : 0;
  const unsigned m = __ballot_sync(FULL, match);
  const int in_warp = __popc(m & ((1u << lane) - 1u));
  if (lane == 0) warp_tot[warp] = __popc(m);
  __syncthreads();
  int before = 0, total = 0;
  for (int w = 0; w < 8; ++w) {
    if (w < warp) before += warp_tot[w];
    total += warp_tot[w];
  }
  if (match) bin_out[before + in_warp] = val;
  if (i == 0) count_out[0] = total;
}
__global__ void block_normalize_kernel(const float* a, float* out, int n) {
  __shared__ float sh[8];
  __shared__ float mean_sh;
  const int i = threadIdx.x;
  const float val = i < n ? a[i] : 0.f;
  const float s = block_sum_f<256>(val, sh);
  if (i == 0) mean_sh = s / n;  // one thread computes, everyone reads: a block broadcast
  __syncthreads();
  if (i < n) out[i] = val / mean_sh;
}

// ---------------------------------------------------------------- p28: async copy + convolution
// tile-local 5-tap convolution; the two elements at each tile edge pass through unchanged
template <bool USE_BULK>
__global__ void async_copy_conv_kernel(float* out, const float* a, const float* w, int n, int* status) {
  constexpr int TILE = 256, K = 5, HALO = 2;
  __shared__ __align__(128) float tile[TILE];
  __shared__ float ws[K];
  __shared__ uint64_t bar;
  const int l = threadIdx.x, g = blockIdx.x * TILE + l;
  const int valid = min(TILE, n - blockIdx.x * TILE);
  bool ok_wait = true;
  if (USE_BULK && valid == TILE) {
    // one elected thread starts a 1 KiB bulk copy and everyone waits on its mbarrier (bounded)
    __shared__ int abort_flag;
    if (l == 0) {
      mbar_init(&bar, 1);
      abort_flag = 0;
      fence_mbar_init();
    }
    __syncthreads();
    if (l == 0) {
      mbar_arrive_expect_tx(&bar, TILE * sizeof(float));
      bulk_load_1d(tile, a + blockIdx.x * TILE, TILE * sizeof(float), &bar);
    }
    if (l < K) ws[l] = w[l];
    ok_wait = mbar_wait_bounded(&bar, 0, &abort_flag, status, kTimeoutFull);
  } else {
    if (g < n) {
      const uint32_t dst = smem_u32(&tile[l]);
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(a + g) : "memory");
    } else {
      tile[l] = 0.f;
    }
    if (l < K) ws[l] = w[l];
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
  }
  __syncthreads();
  if (g < n && ok_wait) {
    float r;
    if (l >= HALO && l < TILE - HALO) {
      r = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k) r += tile[l + k - HALO] * ws[k];
    } else {
      r = tile[l];
    }
    out[g] = r;
  }
}

// ---------------------------------------------------------------- p29: barrier-coordinated pipelines
// three stages inside one 256-thread block: scale by 1.1 (threads 0-127 load two elements each),
// 5-point blur (threads 128-255, two outputs each), neighbour smoothing by everyone
__global__ void pipeline_blur_kernel(float* out, const float* a, int n) {
  constexpr int TPB = 256, S1 = 128, R = 2;
  __shared__ float in_sh[TPB], blur_sh[TPB];
  const int l = threadIdx.x, g = blockIdx.x * TPB + l;
  if (l < S1) {
    in_sh[l] = g < n ? a[g] * 1.1f : 0.f;
    in_sh[l + S1] = g + S1 < n ? a[g + S1] * 1.1f : 0.f;
  }
  __syncthreads();
  if (l >= S1) {
    for (int rep = 0; rep < 2; ++rep) {
      const int bi = l - S1 + rep * S1;
      float s = 0.f;
      int cnt = 0;
      for (int off = -R; off <= R; ++off) {
        const int j = bi + off;
        if (j >= 0 && j < TPB) {
          s += in_sh[j];
          ++cnt;
        }
      }
      blur_sh[bi] = s / cnt;
    }
  }
  __syncthreads();
  if (g < n) {
    float v = blur_sh[l];
    if (l > 0) v = (v + blur_sh[l - 1]) * 0.6f;
    if (l < TPB - 1) v = (v + blur_sh[l + 1]) * 0.6f;
    out[g] = v;
  }
}
// ping-pong 3-point stencil; buffer hand-over is coordinated with an mbarrier whose phases are
// waited on with a time budget (status word on expiry, never an endless spin)
__global__ void double_buffer_stencil_kernel(float* out, const float* a, int n, int iterations,
                                             int* status) {
  constexpr int TPB = 256;
  __shared__ float buf[2][TPB];
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const int l = threadIdx.x, g = blockIdx.x * TPB + l;
  if (l == 0) {
    mbar_init(&bar, TPB);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  buf[0][l] = g < n ? a[g] : 0.f;
  uint32_t phase = 0;
  mbar_arrive(&bar);
  bool ok = mbar_wait_bounded(&bar, phase, &abort_flag, status, kTimeoutLocal);
  phase ^= 1u;
  int cur = 0;
  for (int it = 0; it < iterations && ok; ++it) {
    float s = 0.f;
    int cnt = 0;
    for (int off = -1; off <= 1; ++off) {
      const int j = l + off;
      if (j >= 0 && j < TPB) {
        s += buf[cur][j];
        ++cnt;
      }
    }
    buf[cur ^ 1][l] = s / cnt;
    mbar_arrive(&bar);
    ok = mbar_wait_bounded(&bar, phase, &abort_flag, status, kTimeoutLocal);
    phase ^= 1u;
    cur ^= 1;
  }
  if (ok && g < n) out[g] = buf[cur][l];
}

// ---------------------------------------------------------------- p30-p32: study kernels
// mode 0: coalesced, 1: stride-512 grid-stride remap, 2: reversed
__global__ void access_pattern_add_kernel(float* out, const float* a, const float* b, int n, int mode) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int j = i;
  if (mode == 1) j = (int)(((long long)i * 512) % n + ((long long)i * 512) / n) % n;
  if (mode == 2) j = n - 1 - i;
  out[j] = a[j] + b[j];
}
// SAXPY with a chosen amount of dynamic shared memory (occupancy study): smem is touched so the
// allocation is real, the arithmetic result is identical for every setting
__global__ void occupancy_saxpy_kernel(float* y, const float* x, float alpha, int n) {
  extern __shared__ float pad[];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  pad[threadIdx.x] = i < n ? x[i] : 0.f;
  __syncthreads();
  if (i < n) y[i] = alpha * pad[threadIdx.x] + y[i];
}
// (x + 10) * 2 through shared memory read back with a configurable stride (1 = conflict free,
// 2 = two-way bank conflicts, ...)
__global__ void bank_conflict_kernel(float* out, const float* a, int n, int stride) {
  extern __shared__ float sh[];  // blockDim.x * stride floats
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  sh[threadIdx.x * stride] = i < n ? a[i] : 0.f;
  __syncthreads();
  if (i < n) out[i] = (sh[threadIdx.x * stride] + 10.f) * 2.f;
}

// ---------------------------------------------------------------- p34: thread-block clusters
// per-block partial sums of in * (block + 1), with arrive / wait around the independent work
__global__ void cluster_block_sums_kernel(float* out, const float* a, int n, int warp_elected) {
  extern __shared__ float sh[];
  cg::cluster_group cluster = cg::this_cluster();
  const int l = threadIdx.x, g = blockIdx.x * blockDim.x + l;
  sh[l] = g < n ? a[g] * (float)(blockIdx.x + 1) : 0.f;
  __syncthreads();
  if (warp_elected) {
    // one elected lane per warp folds its warp's 32 values first
    if (elect_one()) {
      const int w0 = (l / 32) * 32;
      float s = 0.f;
      for (int i = 0; i < 32 && w0 + i < blockDim.x; ++i) s += sh[w0 + i];
      sh[w0] = s;
    }
    __syncthreads();
  }
  cluster.barrier_arrive();
  if (l == 0) {
    float s = 0.f;
    for (int i = 0; i < blockDim.x; i += (warp_elected ? 32 : 1)) s += sh[i];
    out[blockIdx.x] = s;
  }
  cluster.barrier_wait();
}
// cluster-wide sum: block tree reduction, then rank 0 gathers the partials of the other blocks.
// use_dsmem = 0: through a global scratch array (the reference's scheme, p34.mojo:84-127)
// use_dsmem = 1: rank 0 reads the other blocks' shared memory directly (ld.shared::cluster)
__global__ void cluster_reduce_kernel(float* out, const float* a, float* temp, int n, int use_dsmem) {
  extern __shared__ float sh[];
  cg::cluster_group cluster = cg::this_cluster();
  const int l = threadIdx.x, g = blockIdx.x * blockDim.x + l;
  sh[l] = g < n ? a[g] : 0.f;
  __syncthreads();
  for (int stride = blockDim.x / 2; stride > 0; stride >>= 1) {
    if (l < stride) sh[l] += sh[l + stride];
    __syncthreads();
  }
  if (!use_dsmem && l == 0) temp[blockIdx.x] = sh[0];
  cluster.sync();
  if (cluster.block_rank() == 0 && l == 0) {
    float s = 0.f;
    const unsigned nb = cluster.num_blocks();
    const unsigned first = blockIdx.x;  // rank 0 of this cluster
    for (unsigned r = 0; r < nb; ++r) {
      if (use_dsmem) s += *cluster.map_shared_rank(&sh[0], r);
      else s += temp[first + r];
    }
    out[blockIdx.x / nb] = s;
  }
  cluster.sync();  // keep every block's shared memory alive until rank 0 has read it
}

inline int ok() { return cudaGetLastError() == cudaSuccess ? 0 : 3; }
inline int cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }

template <typename K, typename... Args>
int launch_cluster(K kern, int grid, int block, size_t smem, int cluster, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? 0 : 3;
}

}  // namespace prim
}  // namespace z2h

using namespace z2h::prim;
#define ST(s) ((cudaStream_t)(s))

extern "C" {
int z2h_p_ew_add(float* out, const float* a, const float* b, long long n, int variant, int tile, void* s) {
  if (variant == 0) ew_add_scalar_kernel<<<cdiv(n, 256), 256, 0, ST(s)>>>(out, a, b, (int)n);
  else if (variant == 1) ew_add_tiled_kernel<<<cdiv(n, tile), 32, 0, ST(s)>>>(out, a, b, (int)n, tile);
  else {
    if (((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) & 15) return 1;
    int grid = cdiv(n / 4 + 1, 256);
    ew_add_vec4_kernel<<<grid > 1184 ? 1184 : grid, 256, 0, ST(s)>>>(out, a, b, n);
  }
  return ok();
}
int z2h_p_warp_dot(float* out, const float* a, const float* b, int n, void* s) {
  warp_dot_kernel<<<cdiv(n, 32), 32, 0, ST(s)>>>(out, a, b, n);
  return ok();
}
int z2h_p_warp_sum_int(int* out, const int* a, int n, void* s) {
  warp_sum_int_kernel<<<cdiv(n, 128), 128, 0, ST(s)>>>(out, a, n);
  return ok();
}
// op: 0 neighbor_difference, 1 moving_average_3, 2 broadcast_shuffle, 3 basic_broadcast,
//     4 conditional_broadcast, 5 butterfly_pair_swap, 6 butterfly_max, 7 butterfly_conditional_max,
//     8 warp_inclusive_prefix_sum
int z2h_p_warp_op(float* out, const float* a, int n, int op, void* s) {
  const int grid = cdiv(n, 32);
  switch (op) {
    case 0: neighbor_difference_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n); break;
    case 1: moving_average3_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n); break;
    case 2: broadcast_shuffle_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n); break;
    case 3: basic_broadcast_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n); break;
    case 4: conditional_broadcast_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n); break;
    case 5: butterfly_pair_swap_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n); break;
    case 6: butterfly_max_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n, 0); break;
    case 7: butterfly_max_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n, 1); break;
    case 8: warp_prefix_sum_kernel<<<grid, 32, 0, ST(s)>>>(out, a, n); break;
    default: return 1;
  }
  return ok();
}
int z2h_p_warp_partition(float* out, const float* a, int n, float pivot, void* s) {
  if (n > 32) return 1;
  warp_partition_kernel<<<1, 32, 0, ST(s)>>>(out, a, n, pivot);
  return ok();
}
int z2h_p_block_dot(float* out, const float* a, const float* b, int n, void* s) {
  if (n > 256) return 1;
  block_dot_kernel<<<1, 256, 0, ST(s)>>>(out, a, b, n);
  return ok();
}
int z2h_p_block_histogram_bin_extract(const float* a, float* bin_out, int* count_out, int n, int target_bin,
                                      int num_bins, void* s) {
  if (n > 256) return 1;
  block_histogram_bin_extract_kernel<<<1, 256, 0, ST(s)>>>(a, bin_out, count_out, n, target_bin, num_bins);
  return ok();
}
int z2h_p_block_normalize(const float* a, float* out, int n, void* s) {
  if (n > 256) return 1;
  block_normalize_kernel<<<1, 256, 0, ST(s)>>>(a, out, n);
  return ok();
}
int z2h_p_async_copy_conv(float* out, const float* a, const float* w5, int n, int use_bulk, int* status,
                          void* s) {
  if (use_bulk) {
    if ((uintptr_t)a & 15) return 1;
    async_copy_conv_kernel<true><<<cdiv(n, 256), 256, 0, ST(s)>>>(out, a, w5, n, status);
  } else {
    async_copy_conv_kernel<false><<<cdiv(n, 256), 256, 0, ST(s)>>>(out, a, w5, n, status);
  }
  return ok();
}
int z2h_p_pipeline_blur(float* out, const float* a, int n, void* s) {
  pipeline_blur_kernel<<<cdiv(n, 256), 256, 0, ST(s)>>>(out, a, n);
  return ok();
}
int z2h_p_double_buffer_stencil(float* out, const float* a, int n, int iterations, int* status, void* s) {
  double_buffer_stencil_kernel<<<cdiv(n, 256), 256, 0, ST(s)>>>(out, a, n, iterations, status);
  return ok();
}
int z2h_p_access_pattern_add(float* out, const float* a, const float* b, int n, int mode, void* s) {
  access_pattern_add_kernel<<<cdiv(n, 1024), 1024, 0, ST(s)>>>(out, a, b, n, mode);
  return ok();
}
int z2h_p_occupancy_saxpy(float* y, const float* x, float alpha, int n, int smem_bytes, void* s) {
  if (smem_bytes < 1024 * 4) smem_bytes = 1024 * 4;
  static int configured = 0;
  if (smem_bytes > configured) {
    cudaFuncSetAttribute(occupancy_saxpy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    configured = smem_bytes;
  }
  occupancy_saxpy_kernel<<<cdiv(n, 1024), 1024, smem_bytes, ST(s)>>>(y, x, alpha, n);
  return ok();
}
int z2h_p_bank_conflict(float* out, const float* a, int n, int stride, void* s) {
  if (stride < 1 || stride > 32) return 1;
  bank_conflict_kernel<<<cdiv(n, 256), 256, 256 * stride * sizeof(float), ST(s)>>>(out, a, n, stride);
  return ok();
}
// grid blocks of `block` threads in clusters of `cluster` blocks; out has one value per block
int z2h_p_cluster_block_sums(float* out, const float* a, int n, int block, int cluster, int warp_elected,
                             void* s) {
  const int grid = cdiv(n, block);
  if (grid % cluster) return 1;
  return launch_cluster(cluster_block_sums_kernel, grid, block, block * sizeof(float), cluster, ST(s), out,
                        a, n, warp_elected);
}
// out has one value per cluster; temp needs one float per block when use_dsmem == 0
int z2h_p_cluster_reduce(float* out, const float* a, float* temp, int n, int block, int cluster,
                         int use_dsmem, void* s) {
  const int grid = cdiv(n, block);
  if (grid % cluster || (block & (block - 1))) return 1;
  return launch_cluster(cluster_reduce_kernel, grid, block, block * sizeof(float), cluster, ST(s), out, a,
                        temp, n, use_dsmem);
}
}
