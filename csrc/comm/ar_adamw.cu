// Gradient all-reduce fused with grad-norm clipping and AdamW, over NVLink peer memory.
//
// Every rank maps every peer's gradient buffer, bf16 parameter buffer and signal pad
// (symmetric memory). The flat gradient buffer is cut into buckets in the order in which the
// backward pass completes them; one optimizer step is, per rank, with no NCCL call:
//
//   reduce_bucket (one launch per bucket, on a communication stream, while the backward pass of
//                  the last micro-step still runs for the buckets that are complete early)
//       two-shot bucket: wait until every peer's bucket is final, read this rank's slice of it
//                  from all peers with 16-byte P2P loads, sum in fp32, keep the reduced slice in
//                  place and produce per-CTA sums of squares
//       one-shot bucket (small buckets, below the measured crossover): every rank reduces the
//                  WHOLE bucket, in rank order so that all ranks get bit-identical sums, into a
//                  local buffer; its optimizer state is replicated and no all-gather is needed
//   norm_adamw_allgather (one launch, after the last bucket)
//                  exchange the per-rank sums of squares through the signal pads (epoch |
//                  payload in one 64-bit word), form the global norm in rank order on every
//                  rank, clip, run AdamW on the slices this rank owns (fp32 master weights and
//                  moments exist only there), write the updated bf16 parameters of two-shot
//                  slices into every peer's parameter buffer with P2P stores, and clear the local
//                  gradient buffer for the next step
//   finish         wait until every peer has finished writing, bump the epoch
//
// NVLS flavour (multicast addresses given): two-shot slices are read once through the multicast
// address with multimem.ld_reduce (the NVSwitch adds the ranks' copies in fp32) and written with
// one multimem.st per 16 bytes (the switch replicates the store). One-shot buckets always use
// plain peer loads in rank order: replicas must be bit-identical.
//
// This replaces DistributedDataParallel's bucketed NCCL all-reduce overlapped with backward +
// clip_grad_norm_ + fused AdamW of the reference trainer (nn/gpt2/train_ddp.py:89,141-143).
// Standalone one-/two-shot all-reduce kernels (for bandwidth sweeps against NCCL) follow below.
//
// Signalling (signal_protocol.h): word (kind, src) of a rank's pad is written only by rank src
// with st.release.sys and polled by the owner with ld.acquire.sys; epochs only grow, so pads are
// never cleared. Every poll loop has a time budget; on expiry the kernel records kTimeoutPeer in
// the status word and returns, leaving the context usable. The status word is sticky: every
// kernel of this file returns at once, without signalling and without touching parameters, when
// it finds the word non-zero, so a step in which any wait gave up on any rank applies no update
// anywhere (the peers' own waits for this rank then run out as well) until the host has read the
// word and raised.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../optim/adamw_update.cuh"
#include "comm.h"
#include "signal_protocol.h"

namespace z2h {
namespace {

constexpr int kThreads = 512;        // standalone all-reduce kernels and the optimizer phase
constexpr int kBucketThreads = 256;  // bucket reduce: small enough to share an SM with a GEMM CTA

struct Peers {
  void* ptr[kMaxRanks];
};

// Device instantiation of the signalling backend (see signal_protocol.h).
struct DeviceBackend {
  static __device__ __forceinline__ uint64_t load_acquire(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void store_release(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
  }
  static __device__ __forceinline__ uint64_t now_ns() { return globaltimer_ns(); }
  static __device__ __forceinline__ void pause() { __nanosleep(64); }
  static __device__ __forceinline__ void report_timeout(int* status) {
    if (status != nullptr) atomicCAS(status, 0, (int)kTimeoutPeer);
  }
  static __device__ __forceinline__ unsigned fetch_add(unsigned* p, unsigned v) { return atomicAdd(p, v); }
};

using proto::kSlotBucket0;
using proto::kSlotDone;
using proto::kSlotNorm;
using proto::kSlotPhase;
using proto::kSlotReady;

__device__ __forceinline__ bool status_is_set(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0;
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
    proto::signal<DeviceBackend>(reinterpret_cast<uint64_t*>(pads.ptr[threadIdx.x]), kind, rank, epoch,
                                 payload);
  }
  if (threadIdx.x < world) {
    uint64_t w = 0;
    if (!proto::wait_signal<DeviceBackend>(reinterpret_cast<const uint64_t*>(pads.ptr[rank]), kind,
                                           threadIdx.x, epoch, budget_ns, &w, status))
      atomicExch(failed, 1);
    if (payloads != nullptr) payloads[threadIdx.x] = proto::word_payload(w);
  }
  __syncthreads();
  return *failed == 0;
}

// "Last CTA out" tells every peer that this rank's part of the phase is complete.
__device__ __forceinline__ void last_cta_signals_done(const Peers& pads, int rank, int world,
                                                      uint32_t epoch, unsigned int* done_counter,
                                                      int* last_flag) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0)
    *last_flag = proto::last_one_out<DeviceBackend>(done_counter, gridDim.x) ? 1 : 0;
  __syncthreads();
  if (*last_flag && threadIdx.x < world) {
    __threadfence_system();
    proto::signal<DeviceBackend>(reinterpret_cast<uint64_t*>(pads.ptr[threadIdx.x]), kSlotDone, rank,
                                 epoch, 0);
  }
}

// -------------------------------------------------------------------------------------------
// fused step
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
__device__ __forceinline__ void add4(float4& a, const float4& x) {
  a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
}

// Reduce elements [goff, goff + n) of the gradient buffers of all ranks into `dst` (n floats)
// and write this CTA's sum of squares of the result to partials[blockIdx.x].
//   ONESHOT = false: [goff, goff+n) is this rank's slice of the bucket, dst = own buffer + goff
//                    (in place: peers never read this rank's slice of this rank's buffer... they
//                    read their own slices of it), summation starts at the next rank so that
//                    the ranks do not all pull from the same peer at once;
//   ONESHOT = true:  [goff, goff+n) is the whole bucket, dst is a local buffer, summation in rank
//                    order (every rank computes the same bits).
// count_sumsq = 0 makes the partial zero (a one-shot bucket is counted by one rank only).
template <bool NVLS, bool ONESHOT>
__global__ void __launch_bounds__(kBucketThreads, 6)
reduce_bucket_kernel(Peers grads, const float* grads_mc, Peers pads, int rank, int world, int bucket,
                     long long goff, long long n, float* dst, float* partials, int count_sumsq,
                     const uint32_t* epoch_ptr, uint64_t budget_ns, int* status) {
  __shared__ int failed;
  __shared__ float sh[kBucketThreads / 32];
  if (status_is_set(status)) {
    if (threadIdx.x == 0) partials[blockIdx.x] = 0.f;
    return;
  }
  const uint32_t epoch = *epoch_ptr + 1;
  if (!announce_and_wait(pads, rank, world, kSlotBucket0 + bucket, epoch, 0, true, budget_ns, nullptr,
                         &failed, status)) {
    if (threadIdx.x == 0) partials[blockIdx.x] = 0.f;
    return;
  }
  float sumsq = 0.f;
  const long long nvec = n / 4;
  const long long stride = (long long)gridDim.x * kBucketThreads;
  for (long long i = blockIdx.x * (long long)kBucketThreads + threadIdx.x; i < nvec; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (NVLS && !ONESHOT) {
      acc = multimem_ld_reduce_add_f32x4(reinterpret_cast<const float4*>(grads_mc + goff) + i);
    } else {
      // four peers' loads in flight at a time (16 registers)
      for (int k0 = 0; k0 < world; k0 += 4) {
        float4 x[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = k0 + j;
          if (k < world) {
            const int r = ONESHOT ? k : (rank + 1 + k) % world;
            x[j] = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.ptr[r]) + goff)[i];
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (k0 + j < world) add4(acc, x[j]);
      }
    }
    reinterpret_cast<float4*>(dst)[i] = acc;
    sumsq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  sumsq = block_sum<kBucketThreads>(sumsq, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = count_sumsq ? sumsq : 0.f;
}

constexpr int kMaxRanges = 3 * proto::kMaxBuckets + 8;

template <bool NVLS>
__global__ void __launch_bounds__(kThreads)
norm_adamw_allgather_kernel(Peers p16, __nv_bfloat16* p16_mc, Peers pads, float* g_local, const float* red,
                            float* p32, float* m, float* v, int rank, int world,
                            const StepRange* ranges, int num_ranges, long long n_decay,
                            const float* hyper, const float* partials, int num_partials,
                            float* norm_out, const uint32_t* epoch_ptr, unsigned int* done_counter,
                            uint64_t budget_ns, int* status) {
  __shared__ int failed;
  __shared__ float sh[kThreads / 32];
  __shared__ uint32_t payloads[kMaxRanks];
  __shared__ float s_scale;
  __shared__ StepRange s_rng[kMaxRanges];
  __shared__ long long s_pref[kMaxRanges + 1];  // in units of 8 floats
  if (status_is_set(status)) return;  // an earlier wait of this step gave up: apply nothing
  const uint32_t epoch = *epoch_ptr + 1;
  for (int i = threadIdx.x; i < num_ranges; i += kThreads) s_rng[i] = ranges[i];
  float t = 0.f;
  for (int i = threadIdx.x; i < num_partials; i += kThreads) t += partials[i];
  t = block_sum<kThreads>(t, sh);
  if (threadIdx.x == 0) {
    long long acc = 0;
    for (int i = 0; i < num_ranges; ++i) {
      s_pref[i] = acc;
      acc += s_rng[i].n / 8;
    }
    s_pref[num_ranges] = acc;
  }
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
  // Every peer has sent its norm, so every peer has finished all its bucket reductions and nobody
  // reads the local gradient buffer any more. One pass over the ranges: update what this rank
  // owns (8 elements per thread per trip: one 16-byte bf16 store per peer) and clear the rest.
  const long long units = s_pref[num_ranges];
  int d = 0;
  for (long long u = blockIdx.x * (long long)kThreads + threadIdx.x; u < units;
       u += (long long)gridDim.x * kThreads) {
    while (u >= s_pref[d + 1]) ++d;
    const StepRange rg = s_rng[d];
    const long long e = (u - s_pref[d]) * 8;
    float* gp = g_local + rg.goff + e;
    if (rg.kind == kRangeZero) {
      reinterpret_cast<float4*>(gp)[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      reinterpret_cast<float4*>(gp)[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      continue;
    }
    const float* src = rg.kind == kRangeOneShot ? red + rg.roff + e : gp;
    const long long lo = rg.loff + e;
    float pv[8], mv[8], vv[8], gv[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 a = reinterpret_cast<const float4*>(p32 + lo)[h];
      const float4 b = reinterpret_cast<const float4*>(m + lo)[h];
      const float4 c = reinterpret_cast<const float4*>(v + lo)[h];
      const float4 dd = reinterpret_cast<const float4*>(src)[h];
      pv[h * 4 + 0] = a.x; pv[h * 4 + 1] = a.y; pv[h * 4 + 2] = a.z; pv[h * 4 + 3] = a.w;
      mv[h * 4 + 0] = b.x; mv[h * 4 + 1] = b.y; mv[h * 4 + 2] = b.z; mv[h * 4 + 3] = b.w;
      vv[h * 4 + 0] = c.x; vv[h * 4 + 1] = c.y; vv[h * 4 + 2] = c.z; vv[h * 4 + 3] = c.w;
      gv[h * 4 + 0] = dd.x; gv[h * 4 + 1] = dd.y; gv[h * 4 + 2] = dd.z; gv[h * 4 + 3] = dd.w;
    }
    const long long e0 = rg.goff + e;
#pragma unroll
    for (int j = 0; j < 8; ++j) adamw_update(pv[j], mv[j], vv[j], gv[j], k, e0 + j < n_decay);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(p32 + lo)[h] =
          make_float4(pv[h * 4 + 0], pv[h * 4 + 1], pv[h * 4 + 2], pv[h * 4 + 3]);
      reinterpret_cast<float4*>(m + lo)[h] =
          make_float4(mv[h * 4 + 0], mv[h * 4 + 1], mv[h * 4 + 2], mv[h * 4 + 3]);
      reinterpret_cast<float4*>(v + lo)[h] =
          make_float4(vv[h * 4 + 0], vv[h * 4 + 1], vv[h * 4 + 2], vv[h * 4 + 3]);
      reinterpret_cast<float4*>(gp)[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    uint4 o;
    o.x = pack_bf16x2(pv[0], pv[1]); o.y = pack_bf16x2(pv[2], pv[3]);
    o.z = pack_bf16x2(pv[4], pv[5]); o.w = pack_bf16x2(pv[6], pv[7]);
    if (rg.kind == kRangeOneShot) {
      // replicated state: every rank computed the same bits, the local copy is all there is to write
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p16.ptr[rank]) + e0) = o;
    } else if (NVLS) {
      multimem_st_b128(reinterpret_cast<uint4*>(p16_mc + e0), o);
    } else {
      for (int kk = 0; kk < world; ++kk) {
        const int r = (rank + kk) % world;
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p16.ptr[r]) + e0) = o;
      }
    }
  }
  last_cta_signals_done(pads, rank, world, epoch, done_counter, &failed);
}

__global__ void finish_kernel(Peers pads, int rank, int world, uint32_t* epoch_ptr, int kind,
                              uint64_t budget_ns, int* status) {
  __shared__ int failed;
  const uint32_t epoch = *epoch_ptr + 1;
  if (!status_is_set(status))
    (void)announce_and_wait(pads, rank, world, kind, epoch, 0, false, budget_ns, nullptr, &failed, status);
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
  // 16 bytes summed over all ranks by the switch
  static __device__ __forceinline__ uint4 mc_reduce(const float* mc) {
    const float4 r = multimem_ld_reduce_add_f32x4(mc);
    return make_uint4(__float_as_uint(r.x), __float_as_uint(r.y), __float_as_uint(r.z), __float_as_uint(r.w));
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
  // eight bf16 summed over all ranks by the switch, accumulated in fp32 there
  static __device__ __forceinline__ uint4 mc_reduce(const __nv_bfloat16* mc) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc)
                 : "memory");
    return r;
  }
};

// One-shot: every rank reads all peers' buffers and writes the full sum to `out` (local).
template <typename T>
__global__ void __launch_bounds__(kThreads)
allreduce_oneshot_kernel(Peers bufs, Peers pads, T* out, int rank, int world, long long n,
                         const uint32_t* epoch_ptr, unsigned int* done_counter, uint64_t budget_ns,
                         int* status) {
  __shared__ int failed;
  if (status_is_set(status)) return;
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
  last_cta_signals_done(pads, rank, world, epoch, done_counter, &failed);
}

// Two-shot, phase 1: reduce this rank's shard of every peer's buffer in place (local buffer).
template <typename T>
__global__ void __launch_bounds__(kThreads)
allreduce_rs_kernel(Peers bufs, Peers pads, int rank, int world, long long shard_off,
                    long long shard_n, const uint32_t* epoch_ptr, uint64_t budget_ns, int* status) {
  __shared__ int failed;
  if (status_is_set(status)) return;
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
  if (status_is_set(status)) return;
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
  last_cta_signals_done(pads, rank, world, epoch, done_counter, &failed);
}

// NVLS all-reduce in one kernel: each rank takes its shard, reads 16 bytes summed by the switch
// (multimem.ld_reduce) and stores the sum to every rank's copy at once (multimem.st). The
// reduce traffic leaves this GPU (its copy of the other shards is read by the switch) while the
// broadcast traffic arrives, so both link directions are busy at the same time, which the
// two-phase forms above cannot do. In place on the symmetric buffer.
template <typename T>
__global__ void __launch_bounds__(kThreads)
allreduce_nvls_kernel(T* buf_mc, Peers pads, int rank, int world, long long shard_off, long long shard_n,
                      const uint32_t* epoch_ptr, unsigned int* done_counter, uint64_t budget_ns,
                      int* status) {
  __shared__ int failed;
  if (status_is_set(status)) return;
  const uint32_t epoch = *epoch_ptr + 1;
  if (!announce_and_wait(pads, rank, world, kSlotReady, epoch, 0, true, budget_ns, nullptr, &failed,
                         status))
    return;
  constexpr int E = Vec16<T>::kElems;
  const long long nvec = shard_n / E;
  T* mc = buf_mc + shard_off;
  const long long stride = (long long)gridDim.x * kThreads;
  long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
  for (; i + stride < nvec; i += 2 * stride) {  // two independent round trips in flight
    const uint4 a = Vec16<T>::mc_reduce(mc + i * E);
    const uint4 b = Vec16<T>::mc_reduce(mc + (i + stride) * E);
    multimem_st_b128(mc + i * E, a);
    multimem_st_b128(mc + (i + stride) * E, b);
  }
  if (i < nvec) multimem_st_b128(mc + i * E, Vec16<T>::mc_reduce(mc + i * E));
  last_cta_signals_done(pads, rank, world, epoch, done_counter, &failed);
}

// Waits on one slot of a pad for a given epoch; used to exercise the bounded wait on one GPU.
__global__ void wait_probe_kernel(uint64_t* pad, int kind, int src, uint32_t epoch,
                                  uint64_t budget_ns, int* status, int* result) {
  uint64_t w = 0;
  const bool ok = proto::wait_signal<DeviceBackend>(pad, kind, src, epoch, budget_ns, &w, status);
  *result = ok ? 1 : 0;
}

Peers to_peers(void* const* p, int world) {
  Peers t;
  for (int i = 0; i < kMaxRanks; ++i) t.ptr[i] = i < world ? p[i] : nullptr;
  return t;
}

int grid_for(long long nvec, int threads, int cap) {
  long long b = (nvec + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b < cap ? b : cap);
}

bool world_ok(int rank, int world) { return world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world; }

}  // namespace

int reduce_bucket_grid(long long n, int max_ctas) {
  return grid_for(n / 4, kBucketThreads, max_ctas > 0 ? max_ctas : 2 * sm_count_current_device());
}

int reduce_bucket(const BucketArgs& a, cudaStream_t stream) {
  if (!world_ok(a.rank, a.world) || a.bucket < 0 || a.bucket >= proto::kMaxBuckets) return -1;
  if ((a.goff % 8) || (a.n % 8) || a.n < 0 || a.dst == nullptr || a.partials == nullptr) return -1;
  if (reinterpret_cast<uintptr_t>(a.dst) & 15) return -1;
  const Peers grads = to_peers(a.grads, a.world);
  const Peers pads = to_peers(a.pads, a.world);
  const int grid = reduce_bucket_grid(a.n, a.max_ctas);
  const float* mc = reinterpret_cast<const float*>(a.grads_mc);
#define Z2H_RB(NVLS, ONE)                                                                             \
  reduce_bucket_kernel<NVLS, ONE><<<grid, kBucketThreads, 0, stream>>>(                               \
      grads, mc, pads, a.rank, a.world, a.bucket, a.goff, a.n, a.dst, a.partials, a.count_sumsq, a.epoch, \
      a.budget_ns, a.status)
  if (a.one_shot) Z2H_RB(false, true);
  else if (mc != nullptr) Z2H_RB(true, false);
  else Z2H_RB(false, false);
#undef Z2H_RB
  return cudaGetLastError() == cudaSuccess ? grid : -3;
}

int optimizer_phase(const PhaseArgs& a, cudaStream_t stream) {
  if (!world_ok(a.rank, a.world) || a.num_ranges < 1 || a.num_ranges > kMaxRanges) return 1;
  const Peers p16 = to_peers(a.p16, a.world);
  const Peers pads = to_peers(a.pads, a.world);
  const int cap = a.max_ctas > 0 ? a.max_ctas : 2 * sm_count_current_device();
  const int grid = grid_for(a.total_units, kThreads, cap);
  float* g_local = reinterpret_cast<float*>(a.grads[a.rank]);
  if (a.p16_mc != nullptr)
    norm_adamw_allgather_kernel<true><<<grid, kThreads, 0, stream>>>(
        p16, reinterpret_cast<__nv_bfloat16*>(a.p16_mc), pads, g_local, a.red, a.p32, a.m, a.v, a.rank,
        a.world, a.ranges, a.num_ranges, a.n_decay, a.hyper, a.partials, a.num_partials, a.norm_out,
        a.epoch, a.done_counter, a.budget_ns, a.status);
  else
    norm_adamw_allgather_kernel<false><<<grid, kThreads, 0, stream>>>(
        p16, nullptr, pads, g_local, a.red, a.p32, a.m, a.v, a.rank, a.world, a.ranges, a.num_ranges,
        a.n_decay, a.hyper, a.partials, a.num_partials, a.norm_out, a.epoch, a.done_counter,
        a.budget_ns, a.status);
  finish_kernel<<<1, 32, 0, stream>>>(pads, a.rank, a.world, a.epoch, kSlotDone, a.budget_ns, a.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Forces the fused-step kernels to be loaded on the current device, so that their first launch
// can happen inside a stream capture.
int comm_preload() {
  cudaFuncAttributes fa;
  cudaError_t e = cudaFuncGetAttributes(&fa, reduce_bucket_kernel<false, false>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, reduce_bucket_kernel<false, true>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, reduce_bucket_kernel<true, false>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, norm_adamw_allgather_kernel<false>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, norm_adamw_allgather_kernel<true>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, finish_kernel);
  return e == cudaSuccess ? 0 : 3;
}

template <typename T>
static int allreduce_impl(void* const* bufs, void* const* pads, void* out, void* buf_mc, int rank,
                          int world, long long n, int algo, uint32_t* epoch, unsigned int* done_counter,
                          uint64_t budget_ns, int* status, int max_ctas, cudaStream_t stream) {
  if (!world_ok(rank, world)) return 1;
  const Peers b = to_peers(bufs, world), p = to_peers(pads, world);
  constexpr int E = Vec16<T>::kElems;
  const int cap = max_ctas > 0 ? max_ctas : 2 * sm_count_current_device();
  if (algo == kAllReduceOneShot) {
    allreduce_oneshot_kernel<T><<<grid_for(n / E, kThreads, cap), kThreads, 0, stream>>>(
        b, p, reinterpret_cast<T*>(out), rank, world, n, epoch, done_counter, budget_ns, status);
  } else {
    // shards are multiples of 16 bytes; the last shard takes what is left
    long long shard_len = ((n + world - 1) / world + E - 1) / E * E;
    if (n % E) return 1;
    const long long off = (long long)rank * shard_len;
    const long long len = off + shard_len <= n ? shard_len : (n > off ? n - off : 0);
    if (algo == kAllReduceNvls) {
      if (buf_mc == nullptr) return 1;
      allreduce_nvls_kernel<T><<<grid_for(len / E, kThreads, cap), kThreads, 0, stream>>>(
          reinterpret_cast<T*>(buf_mc), p, rank, world, off < n ? off : 0, len, epoch, done_counter,
          budget_ns, status);
    } else {
      allreduce_rs_kernel<T><<<grid_for(len / E, kThreads, cap), kThreads, 0, stream>>>(
          b, p, rank, world, off, len, epoch, budget_ns, status);
      allreduce_ag_kernel<T><<<grid_for(shard_len / E, kThreads, cap), kThreads, 0, stream>>>(
          b, p, rank, world, shard_len, n, epoch, done_counter, budget_ns, status);
    }
  }
  finish_kernel<<<1, 32, 0, stream>>>(p, rank, world, epoch, kSlotDone, budget_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int allreduce(void* const* bufs, void* const* pads, void* out, void* buf_mc, int rank, int world,
              long long n, int dtype, int algo, uint32_t* epoch, unsigned int* done_counter,
              uint64_t budget_ns, int* status, int max_ctas, cudaStream_t stream) {
  if (dtype == kCommF32)
    return allreduce_impl<float>(bufs, pads, out, buf_mc, rank, world, n, algo, epoch, done_counter,
                                 budget_ns, status, max_ctas, stream);
  return allreduce_impl<__nv_bfloat16>(bufs, pads, out, buf_mc, rank, world, n, algo, epoch, done_counter,
                                       budget_ns, status, max_ctas, stream);
}

int wait_probe(void* pad, int kind, int src, uint32_t epoch, uint64_t budget_ns, int* status,
               int* result, cudaStream_t stream) {
  if (kind < 0 || kind >= proto::kPadKinds || src < 0 || src >= kMaxRanks) return 1;
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
int z2h_comm_pad_slots(void) { return z2h::proto::kPadSlots; }
int z2h_comm_max_buckets(void) { return z2h::proto::kMaxBuckets; }
int z2h_comm_preload(void) { return z2h::comm_preload(); }
int z2h_reduce_bucket_grid(long long n, int max_ctas) { return z2h::reduce_bucket_grid(n, max_ctas); }
// Returns the number of CTAs launched (= partial sums written), or a negative error code.
int z2h_reduce_bucket(void* const* grads, void* const* pads, void* grads_mc, int rank, int world,
                      int bucket, long long goff, long long n, float* dst, int one_shot,
                      float* partials, int count_sumsq, unsigned int* epoch,
                      unsigned long long budget_ns, int* status, int max_ctas, void* stream) {
  z2h::BucketArgs a;
  a.grads = grads; a.pads = pads; a.grads_mc = grads_mc;
  a.rank = rank; a.world = world; a.bucket = bucket;
  a.goff = goff; a.n = n; a.dst = dst; a.one_shot = one_shot;
  a.partials = partials; a.count_sumsq = count_sumsq;
  a.epoch = epoch; a.budget_ns = budget_ns; a.status = status; a.max_ctas = max_ctas;
  return z2h::reduce_bucket(a, (cudaStream_t)stream);
}
int z2h_optimizer_phase(void* const* grads, void* const* p16, void* const* pads, void* p16_mc,
                        const float* red, float* p32, float* m, float* v, int rank, int world,
                        const void* ranges, int num_ranges, long long total_units, long long n_decay,
                        const float* hyper, const float* partials, int num_partials, float* norm_out,
                        unsigned int* epoch, unsigned int* done_counter, unsigned long long budget_ns,
                        int* status, int max_ctas, void* stream) {
  z2h::PhaseArgs a;
  a.grads = grads; a.p16 = p16; a.pads = pads; a.p16_mc = p16_mc;
  a.red = red; a.p32 = p32; a.m = m; a.v = v;
  a.rank = rank; a.world = world;
  a.ranges = reinterpret_cast<const z2h::StepRange*>(ranges);
  a.num_ranges = num_ranges; a.total_units = total_units; a.n_decay = n_decay;
  a.hyper = hyper; a.partials = partials; a.num_partials = num_partials; a.norm_out = norm_out;
  a.epoch = epoch; a.done_counter = done_counter; a.budget_ns = budget_ns; a.status = status;
  a.max_ctas = max_ctas;
  return z2h::optimizer_phase(a, (cudaStream_t)stream);
}
int z2h_allreduce(void* const* bufs, void* const* pads, void* out, void* buf_mc, int rank, int world,
                  long long n, int dtype, int algo, unsigned int* epoch, unsigned int* done_counter,
                  unsigned long long budget_ns, int* status, int max_ctas, void* stream) {
  return z2h::allreduce(bufs, pads, out, buf_mc, rank, world, n, dtype, algo, epoch, done_counter,
                        budget_ns, status, max_ctas, (cudaStream_t)stream);
}
}
