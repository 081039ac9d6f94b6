// Gradient all-reduce fused with grad-norm clipping and AdamW, over NVLink peer memory.
//
// Every rank maps every peer's gradient buffer, bf16 parameter buffer and signal pad
// (symmetric memory). One optimizer step is three launches per rank and no NCCL call:
//
//   reduce_scatter_sumsq   wait until every peer's gradients are final, then read this rank's
//                          shard from all peers with 16-byte P2P loads, sum in fp32, keep the
//                          reduced shard locally and produce per-CTA sums of squares
//   norm_adamw_allgather   exchange the per-rank sums of squares through the signal pads
//                          (epoch | payload in one 64-bit word), form the global norm in rank
//                          order on every rank, clip, run AdamW on the owned shard (fp32
//                          master weights and moments exist only there), and write the updated
//                          bf16 parameters into every peer's parameter buffer with P2P stores;
//                          also clears the local gradient buffer for the next step
//   finish                 wait until every peer has finished writing, bump the epoch
//
// NVLS flavour (FusedStepArgs::grads_mc / p16_mc set): the same three launches and signalling,
// but the reduce-scatter reads each 16 bytes of the shard once through the multicast address with
// multimem.ld_reduce (the NVSwitch adds the ranks' copies in fp32) and the all-gather is one
// multimem.st per 16 bytes (the switch replicates the store), so every byte crosses this GPU's
// links once instead of once per peer.
//
// This replaces DistributedDataParallel's bucketed NCCL all-reduce + clip_grad_norm_ + fused
// AdamW of the reference trainer (nn/gpt2/train_ddp.py:89,141-143). A one-shot variant for
// small models (every rank reduces everything and updates a replicated state) and standalone
// one-/two-shot all-reduce kernels (for eval scalars and for bandwidth sweeps against NCCL)
// use the same signalling code.
//
// Signalling: slot (kind, src) of a rank's pad is written only by rank src with
// st.release.sys and polled by the owner with ld.acquire.sys; epochs only grow, so pads are
// never cleared. Every poll loop has a time budget; on expiry the kernel records
// kTimeoutPeer in the status word and returns, leaving the context usable.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../optim/adamw_update.cuh"
#include "comm.h"

namespace z2h {
namespace {

constexpr int kThreads = 512;

struct Peers {
  void* ptr[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t* slot(void* pad, int kind, int src) {
  return reinterpret_cast<uint64_t*>(pad) + kind * kMaxRanks + src;
}

// Poll one slot of the local pad until its epoch reaches `epoch`; bounded.
__device__ __forceinline__ bool wait_slot(uint64_t* s, uint32_t epoch, uint64_t budget_ns,
                                          uint64_t* value, int* status) {
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    const uint64_t v = ld_acquire_sys(s);
    if ((int32_t)((uint32_t)(v >> 32) - epoch) >= 0) {
      *value = v;
      return true;
    }
    if (globaltimer_ns() - t0 > budget_ns) {
      if (status != nullptr) atomicCAS(status, 0, (int)kTimeoutPeer);
      return false;
    }
    __nanosleep(64);
  }
}

// Cross-rank barrier at the start of a kernel: CTA 0 announces (kind, epoch, payload) to every
// peer, every CTA waits for all peers. Returns false (for the whole CTA) when a wait ran out.
// `payloads` (shared memory, kMaxRanks words) receives each peer's 32-bit payload.
__device__ __forceinline__ bool announce_and_wait(const Peers& pads, int rank, int world, int kind,
                                                  uint32_t epoch, uint32_t payload, bool announce,
                                                  uint64_t budget_ns, uint32_t* payloads,
                                                  int* failed, int* status) {
  if (threadIdx.x == 0) *failed = 0;
  __syncthreads();
  if (announce && blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(slot(pads.ptr[threadIdx.x], kind, rank), ((uint64_t)epoch << 32) | payload);
  }
  if (threadIdx.x < world) {
    uint64_t v = 0;
    if (!wait_slot(slot(pads.ptr[rank], kind, threadIdx.x), epoch, budget_ns, &v, status))
      atomicExch(failed, 1);
    if (payloads != nullptr) payloads[threadIdx.x] = (uint32_t)v;
  }
  __syncthreads();
  return *failed == 0;
}

enum SlotKind : int {
  kSlotReady = 0,     // "my gradients / input are final"
  kSlotNorm = 1,      // payload: this rank's sum of squares (float bits)
  kSlotDone = 2,      // "I have finished writing into / reading from peers"
  kSlotPhase = 3,     // generic second barrier of the standalone all-reduce
};

// -------------------------------------------------------------------------------------------
// two-shot fused step
// -------------------------------------------------------------------------------------------
// in-switch reduction: the sum over all ranks of the 16 bytes at a multicast address
__device__ __forceinline__ float4 multimem_ld_reduce_add_f32x4(const void* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
// in-switch broadcast: 16 bytes stored to every rank's copy behind a multicast address
__device__ __forceinline__ void multimem_st_b128(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

template <bool NVLS>
__global__ void __launch_bounds__(kThreads)
reduce_scatter_sumsq_kernel(Peers grads, const float* grads_mc, Peers pads, int rank, int world,
                            long long shard_off, long long shard_n, float* partials,
                            const uint32_t* epoch_ptr, uint64_t budget_ns, int* status) {
  __shared__ int failed;
  __shared__ float sh[kThreads / 32];
  const uint32_t epoch = *epoch_ptr + 1;
  if (!announce_and_wait(pads, rank, world, kSlotReady, epoch, 0, true, budget_ns, nullptr, &failed,
                         status)) {
    if (threadIdx.x == 0) partials[blockIdx.x] = 0.f;
    return;
  }
  float sumsq = 0.f;
  float* mine = reinterpret_cast<float*>(grads.ptr[rank]) + shard_off;
  const long long nvec = shard_n / 4;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * kThreads) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (NVLS) {
      acc = multimem_ld_reduce_add_f32x4(reinterpret_cast<const float4*>(grads_mc + shard_off) + i);
    } else {
      // start at the next rank so that the ranks do not all pull from the same peer at once
      for (int k = 1; k <= world; ++k) {
        const int r = (rank + k) % world;
        const float4 x = reinterpret_cast<const float4*>(
            reinterpret_cast<const float*>(grads.ptr[r]) + shard_off)[i];
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      }
    }
    reinterpret_cast<float4*>(mine)[i] = acc;
    sumsq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  sumsq = block_sum<kThreads>(sumsq, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = sumsq;
}

template <bool NVLS>
__global__ void __launch_bounds__(kThreads)
norm_adamw_allgather_kernel(Peers p16, __nv_bfloat16* p16_mc, Peers pads, float* g_local, float* p32, float* m, float* v,
                            int rank, int world, long long shard_off, long long shard_n,
                            long long total_n, long long n_decay, const float* hyper,
                            const float* partials, int num_partials, float* norm_out,
                            const uint32_t* epoch_ptr, unsigned int* done_counter,
                            uint64_t budget_ns, int* status) {
  __shared__ int failed;
  __shared__ float sh[kThreads / 32];
  __shared__ uint32_t payloads[kMaxRanks];
  __shared__ float s_scale;
  const uint32_t epoch = *epoch_ptr + 1;
  float t = 0.f;
  for (int i = threadIdx.x; i < num_partials; i += kThreads) t += partials[i];
  t = block_sum<kThreads>(t, sh);
  if (!announce_and_wait(pads, rank, world, kSlotNorm, epoch, __float_as_uint(t), true, budget_ns,
                         payloads, &failed, status))
    return;
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int r = 0; r < world; ++r) total += __uint_as_float(payloads[r]);  // same order everywhere
    const float gs = hyper[kHyGradScale];
    const float norm = sqrtf(total) * gs;
    const float max_norm = hyper[kHyMaxNorm];
    float clip = 1.f;
    if (max_norm > 0.f) clip = fminf(1.f, max_norm / (norm + 1e-6f));
    s_scale = clip * gs;
    if (blockIdx.x == 0 && norm_out != nullptr) *norm_out = norm;
  }
  __syncthreads();
  const AdamConsts k = load_adam_consts(hyper, s_scale);
  // every peer has left the reduce-scatter (it has sent its norm), so nobody reads the local
  // gradient buffer any more: clear the parts that are not this rank's shard ...
  {
    const long long nvec = total_n / 4;
    const long long s0 = shard_off / 4, s1 = (shard_off + shard_n) / 4;
    for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * kThreads) {
      if (i < s0 || i >= s1) reinterpret_cast<float4*>(g_local)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // ... and update the shard (8 elements per thread per trip: one 16-byte bf16 store per peer)
  const long long nvec8 = shard_n / 8;
  float* gs = g_local + shard_off;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec8;
       i += (long long)gridDim.x * kThreads) {
    float pv[8], mv[8], vv[8], gv[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 a = reinterpret_cast<const float4*>(p32)[i * 2 + h];
      const float4 b = reinterpret_cast<const float4*>(m)[i * 2 + h];
      const float4 c = reinterpret_cast<const float4*>(v)[i * 2 + h];
      const float4 d = reinterpret_cast<const float4*>(gs)[i * 2 + h];
      pv[h * 4 + 0] = a.x; pv[h * 4 + 1] = a.y; pv[h * 4 + 2] = a.z; pv[h * 4 + 3] = a.w;
      mv[h * 4 + 0] = b.x; mv[h * 4 + 1] = b.y; mv[h * 4 + 2] = b.z; mv[h * 4 + 3] = b.w;
      vv[h * 4 + 0] = c.x; vv[h * 4 + 1] = c.y; vv[h * 4 + 2] = c.z; vv[h * 4 + 3] = c.w;
      gv[h * 4 + 0] = d.x; gv[h * 4 + 1] = d.y; gv[h * 4 + 2] = d.z; gv[h * 4 + 3] = d.w;
    }
    const long long e0 = shard_off + i * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) adamw_update(pv[j], mv[j], vv[j], gv[j], k, e0 + j < n_decay);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(p32)[i * 2 + h] =
          make_float4(pv[h * 4 + 0], pv[h * 4 + 1], pv[h * 4 + 2], pv[h * 4 + 3]);
      reinterpret_cast<float4*>(m)[i * 2 + h] =
          make_float4(mv[h * 4 + 0], mv[h * 4 + 1], mv[h * 4 + 2], mv[h * 4 + 3]);
      reinterpret_cast<float4*>(v)[i * 2 + h] =
          make_float4(vv[h * 4 + 0], vv[h * 4 + 1], vv[h * 4 + 2], vv[h * 4 + 3]);
      reinterpret_cast<float4*>(gs)[i * 2 + h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    uint4 o;
    o.x = pack_bf16x2(pv[0], pv[1]); o.y = pack_bf16x2(pv[2], pv[3]);
    o.z = pack_bf16x2(pv[4], pv[5]); o.w = pack_bf16x2(pv[6], pv[7]);
    if (NVLS) {
      multimem_st_b128(reinterpret_cast<uint4*>(p16_mc + shard_off) + i, o);
    } else {
      for (int kk = 0; kk < world; ++kk) {
        const int r = (rank + kk) % world;
        reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p16.ptr[r]) + shard_off)[i] = o;
      }
    }
  }
  // last CTA out tells every peer that this rank's writes are complete
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    failed = (prev == gridDim.x - 1) ? 1 : 0;  // reuse as "I am last"
  }
  __syncthreads();
  if (failed && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(slot(pads.ptr[threadIdx.x], kSlotDone, rank), (uint64_t)epoch << 32);
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

__global__ void finish_kernel(Peers pads, int rank, int world, uint32_t* epoch_ptr, int kind,
                              uint64_t budget_ns, int* status) {
  __shared__ int failed;
  const uint32_t epoch = *epoch_ptr + 1;
  const bool ok = announce_and_wait(pads, rank, world, kind, epoch, 0, false, budget_ns, nullptr,
                                    &failed, status);
  (void)ok;
  // the epoch advances even after a timeout, so a later step does not match stale signals
  if (threadIdx.x == 0) *epoch_ptr = epoch;
}

// -------------------------------------------------------------------------------------------
// standalone all-reduce (sum), fp32 or bf16 storage, fp32 accumulation
// -------------------------------------------------------------------------------------------
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    f[0] = x.x; f[1] = x.y; f[2] = x.z; f[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

// One-shot: every rank reads all peers' buffers and writes the full sum to `out` (local).
template <typename T>
__global__ void __launch_bounds__(kThreads)
allreduce_oneshot_kernel(Peers bufs, Peers pads, T* out, int rank, int world, long long n,
                         const uint32_t* epoch_ptr, unsigned int* done_counter, uint64_t budget_ns,
                         int* status) {
  __shared__ int failed;
  const uint32_t epoch = *epoch_ptr + 1;
  if (!announce_and_wait(pads, rank, world, kSlotReady, epoch, 0, true, budget_ns, nullptr, &failed,
                         status))
    return;
  constexpr int E = Vec16<T>::kElems;
  const long long nvec = n / E;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * kThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {  // rank order: every rank gets bit-identical sums
      float f[8];
      Vec16<T>::load(reinterpret_cast<const T*>(bufs.ptr[r]) + i * E, f);
#pragma unroll
      for (int j = 0; j < E; ++j) acc[j] += f[j];
    }
    Vec16<T>::store(out + i * E, acc);
  }
  if (blockIdx.x == 0) {
    for (long long e = nvec * E + threadIdx.x; e < n; e += kThreads) {
      float acc = 0.f;
      for (int r = 0; r < world; ++r) acc += (float)reinterpret_cast<const T*>(bufs.ptr[r])[e];
      out[e] = (T)acc;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    failed = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (failed && threadIdx.x < world) {
    st_release_sys(slot(pads.ptr[threadIdx.x], kSlotDone, rank), (uint64_t)epoch << 32);
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// Two-shot, phase 1: reduce this rank's shard of every peer's buffer in place (local buffer).
template <typename T>
__global__ void __launch_bounds__(kThreads)
allreduce_rs_kernel(Peers bufs, Peers pads, int rank, int world, long long shard_off,
                    long long shard_n, const uint32_t* epoch_ptr, uint64_t budget_ns, int* status) {
  __shared__ int failed;
  const uint32_t epoch = *epoch_ptr + 1;
  if (!announce_and_wait(pads, rank, world, kSlotReady, epoch, 0, true, budget_ns, nullptr, &failed,
                         status))
    return;
  constexpr int E = Vec16<T>::kElems;
  const long long nvec = shard_n / E;
  T* mine = reinterpret_cast<T*>(bufs.ptr[rank]) + shard_off;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * kThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 1; k <= world; ++k) {
      const int r = (rank + k) % world;
      float f[8];
      Vec16<T>::load(reinterpret_cast<const T*>(bufs.ptr[r]) + shard_off + i * E, f);
#pragma unroll
      for (int j = 0; j < E; ++j) acc[j] += f[j];
    }
    Vec16<T>::store(mine + i * E, acc);
  }
}

// Two-shot, phase 2: after every rank has reduced its shard, pull the other shards.
template <typename T>
__global__ void __launch_bounds__(kThreads)
allreduce_ag_kernel(Peers bufs, Peers pads, int rank, int world, long long shard_len, long long n,
                    const uint32_t* epoch_ptr, unsigned int* done_counter, uint64_t budget_ns,
                    int* status) {
  __shared__ int failed;
  const uint32_t epoch = *epoch_ptr + 1;
  if (!announce_and_wait(pads, rank, world, kSlotPhase, epoch, 0, true, budget_ns, nullptr, &failed,
                         status))
    return;
  constexpr int E = Vec16<T>::kElems;
  T* mine = reinterpret_cast<T*>(bufs.ptr[rank]);
  for (int k = 1; k < world; ++k) {
    const int r = (rank + k) % world;
    const long long off = (long long)r * shard_len;
    const long long len = (off + shard_len <= n ? shard_len : (n > off ? n - off : 0));
    const long long nvec = len / E;
    const T* src = reinterpret_cast<const T*>(bufs.ptr[r]) + off;
    for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * kThreads) {
      *reinterpret_cast<uint4*>(mine + off + i * E) = *reinterpret_cast<const uint4*>(src + i * E);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    failed = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (failed && threadIdx.x < world) {
    st_release_sys(slot(pads.ptr[threadIdx.x], kSlotDone, rank), (uint64_t)epoch << 32);
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// Waits on one slot of a pad for a given epoch; used to exercise the bounded wait on one GPU.
__global__ void wait_probe_kernel(uint64_t* pad, int kind, int src, uint32_t epoch,
                                  uint64_t budget_ns, int* status, int* result) {
  uint64_t v = 0;
  const bool ok = wait_slot(slot(pad, kind, src), epoch, budget_ns, &v, status);
  *result = ok ? 1 : 0;
}

Peers to_peers(void* const* p, int world) {
  Peers t;
  for (int i = 0; i < kMaxRanks; ++i) t.ptr[i] = i < world ? p[i] : nullptr;
  return t;
}

int grid_for(long long nvec, int cap) {
  long long b = (nvec + kThreads - 1) / kThreads;
  if (b < 1) b = 1;
  return (int)(b < cap ? b : cap);
}

}  // namespace

int fused_step_twoshot(const FusedStepArgs& a, cudaStream_t stream) {
  if (a.world < 1 || a.world > kMaxRanks || a.rank < 0 || a.rank >= a.world) return 1;
  if ((a.shard_off % 8) || (a.shard_n % 8) || (a.total_n % 4)) return 1;
  const Peers grads = to_peers(a.grads, a.world);
  const Peers p16 = to_peers(a.p16, a.world);
  const Peers pads = to_peers(a.pads, a.world);
  const int grid_a = grid_for(a.shard_n / 4, a.max_ctas > 0 ? a.max_ctas : 2 * sm_count_current_device());
  const bool nvls = a.grads_mc != nullptr && a.p16_mc != nullptr;
  if (nvls)
    reduce_scatter_sumsq_kernel<true><<<grid_a, kThreads, 0, stream>>>(
        grads, reinterpret_cast<const float*>(a.grads_mc), pads, a.rank, a.world, a.shard_off, a.shard_n,
        a.partials, a.epoch, a.budget_ns, a.status);
  else
    reduce_scatter_sumsq_kernel<false><<<grid_a, kThreads, 0, stream>>>(
        grads, nullptr, pads, a.rank, a.world, a.shard_off, a.shard_n, a.partials, a.epoch, a.budget_ns,
        a.status);
  const int grid_b = grid_for(a.total_n / 4, a.max_ctas > 0 ? a.max_ctas : 2 * sm_count_current_device());
  if (nvls)
    norm_adamw_allgather_kernel<true><<<grid_b, kThreads, 0, stream>>>(
        p16, reinterpret_cast<__nv_bfloat16*>(a.p16_mc), pads, reinterpret_cast<float*>(a.grads[a.rank]),
        a.p32, a.m, a.v, a.rank, a.world, a.shard_off, a.shard_n, a.total_n, a.n_decay, a.hyper,
        a.partials, grid_a, a.norm_out, a.epoch, a.done_counter, a.budget_ns, a.status);
  else
    norm_adamw_allgather_kernel<false><<<grid_b, kThreads, 0, stream>>>(
        p16, nullptr, pads, reinterpret_cast<float*>(a.grads[a.rank]), a.p32, a.m, a.v, a.rank, a.world,
        a.shard_off, a.shard_n, a.total_n, a.n_decay, a.hyper, a.partials, grid_a, a.norm_out, a.epoch,
        a.done_counter, a.budget_ns, a.status);
  finish_kernel<<<1, 32, 0, stream>>>(pads, a.rank, a.world, a.epoch, kSlotDone, a.budget_ns,
                                      a.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

template <typename T>
static int allreduce_impl(void* const* bufs, void* const* pads, void* out, int rank, int world,
                          long long n, int algo, uint32_t* epoch, unsigned int* done_counter,
                          uint64_t budget_ns, int* status, int max_ctas, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks) return 1;
  const Peers b = to_peers(bufs, world), p = to_peers(pads, world);
  constexpr int E = Vec16<T>::kElems;
  const int cap = max_ctas > 0 ? max_ctas : 2 * sm_count_current_device();
  if (algo == kAllReduceOneShot) {
    allreduce_oneshot_kernel<T><<<grid_for(n / E, cap), kThreads, 0, stream>>>(
        b, p, reinterpret_cast<T*>(out), rank, world, n, epoch, done_counter, budget_ns, status);
  } else {
    // shards are multiples of 16 bytes; the last shard takes what is left
    long long shard_len = ((n + world - 1) / world + E - 1) / E * E;
    if (n % E) return 1;
    const long long off = (long long)rank * shard_len;
    const long long len = off + shard_len <= n ? shard_len : (n > off ? n - off : 0);
    allreduce_rs_kernel<T><<<grid_for(len / E, cap), kThreads, 0, stream>>>(
        b, p, rank, world, off, len, epoch, budget_ns, status);
    allreduce_ag_kernel<T><<<grid_for(shard_len / E, cap), kThreads, 0, stream>>>(
        b, p, rank, world, shard_len, n, epoch, done_counter, budget_ns, status);
  }
  finish_kernel<<<1, 32, 0, stream>>>(p, rank, world, epoch, kSlotDone, budget_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int allreduce(void* const* bufs, void* const* pads, void* out, int rank, int world, long long n,
              int dtype, int algo, uint32_t* epoch, unsigned int* done_counter, uint64_t budget_ns,
              int* status, int max_ctas, cudaStream_t stream) {
  if (dtype == kCommF32)
    return allreduce_impl<float>(bufs, pads, out, rank, world, n, algo, epoch, done_counter,
                                 budget_ns, status, max_ctas, stream);
  return allreduce_impl<__nv_bfloat16>(bufs, pads, out, rank, world, n, algo, epoch, done_counter,
                                       budget_ns, status, max_ctas, stream);
}

int wait_probe(void* pad, int kind, int src, uint32_t epoch, uint64_t budget_ns, int* status,
               int* result, cudaStream_t stream) {
  if (kind < 0 || kind >= 8 || src < 0 || src >= kMaxRanks) return 1;
  wait_probe_kernel<<<1, 1, 0, stream>>>(reinterpret_cast<uint64_t*>(pad), kind, src, epoch, budget_ns,
                                         status, result);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace z2h

extern "C" {
int z2h_wait_probe(void* pad, int kind, int src, unsigned int epoch, unsigned long long budget_ns,
                   int* status, int* result, void* stream) {
  return z2h::wait_probe(pad, kind, src, epoch, budget_ns, status, result, (cudaStream_t)stream);
}
int z2h_fused_step_twoshot(void* const* grads, void* const* p16, void* const* pads, float* p32,
                           float* m, float* v, int rank, int world, long long shard_off,
                           long long shard_n, long long total_n, long long n_decay,
                           const float* hyper, float* partials, float* norm_out, unsigned int* epoch,
                           unsigned int* done_counter, unsigned long long budget_ns, int* status,
                           int max_ctas, void* stream) {
  z2h::FusedStepArgs a;
  a.grads = grads; a.p16 = p16; a.pads = pads;
  a.p32 = p32; a.m = m; a.v = v;
  a.rank = rank; a.world = world;
  a.shard_off = shard_off; a.shard_n = shard_n; a.total_n = total_n; a.n_decay = n_decay;
  a.hyper = hyper; a.partials = partials; a.norm_out = norm_out;
  a.epoch = epoch; a.done_counter = done_counter; a.budget_ns = budget_ns; a.status = status;
  a.max_ctas = max_ctas;
  a.grads_mc = nullptr;
  a.p16_mc = nullptr;
  return z2h::fused_step_twoshot(a, (cudaStream_t)stream);
}
int z2h_fused_step_twoshot_nvls(void* const* grads, void* const* p16, void* const* pads, void* grads_mc,
                                void* p16_mc, float* p32, float* m, float* v, int rank, int world,
                                long long shard_off, long long shard_n, long long total_n,
                                long long n_decay, const float* hyper, float* partials, float* norm_out,
                                unsigned int* epoch, unsigned int* done_counter,
                                unsigned long long budget_ns, int* status, int max_ctas, void* stream) {
  z2h::FusedStepArgs a;
  a.grads = grads; a.p16 = p16; a.pads = pads;
  a.p32 = p32; a.m = m; a.v = v;
  a.rank = rank; a.world = world;
  a.shard_off = shard_off; a.shard_n = shard_n; a.total_n = total_n; a.n_decay = n_decay;
  a.hyper = hyper; a.partials = partials; a.norm_out = norm_out;
  a.epoch = epoch; a.done_counter = done_counter; a.budget_ns = budget_ns; a.status = status;
  a.max_ctas = max_ctas;
  a.grads_mc = grads_mc;
  a.p16_mc = p16_mc;
  return z2h::fused_step_twoshot(a, (cudaStream_t)stream);
}
int z2h_allreduce(void* const* bufs, void* const* pads, void* out, int rank, int world, long long n,
                  int dtype, int algo, unsigned int* epoch, unsigned int* done_counter,
                  unsigned long long budget_ns, int* status, int max_ctas, void* stream) {
  return z2h::allreduce(bufs, pads, out, rank, world, n, dtype, algo, epoch, done_counter, budget_ns,
                        status, max_ctas, (cudaStream_t)stream);
}
}
