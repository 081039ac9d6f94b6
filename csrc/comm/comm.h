// Host API of the peer-memory collectives (P2P loads/stores over NVLink, no NCCL).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace z2h {

constexpr int kMaxRanks = 8;
// A signal pad holds kPadSlots 64-bit words per rank: slot = kind * kMaxRanks + source rank.
constexpr int kPadSlots = 8 * kMaxRanks;

enum CommDtype : int { kCommF32 = 0, kCommBF16 = 1 };
enum AllReduceAlgo : int { kAllReduceOneShot = 0, kAllReduceTwoShot = 1 };

struct FusedStepArgs {
  void* const* grads;   // [world] fp32 gradient buffers (total_n each), peer-mapped
  void* const* p16;     // [world] bf16 parameter buffers (total_n each), peer-mapped
  void* const* pads;    // [world] signal pads (kPadSlots uint64 each), peer-mapped, zero-initialised
  float* p32;           // this rank's shard: fp32 master weights  [shard_n]
  float* m;             //                    first moment          [shard_n]
  float* v;             //                    second moment         [shard_n]
  int rank, world;
  long long shard_off, shard_n;  // this rank's shard of the flat buffer (multiples of 8)
  long long total_n;             // flat buffer length (multiple of 4)
  long long n_decay;             // elements [0, n_decay) get weight decay
  const float* hyper;            // device, see HyperSlot
  float* partials;               // device scratch, >= 1024 floats
  float* norm_out;               // device, receives the global pre-clip gradient norm
  uint32_t* epoch;               // device counter owned by this communicator
  unsigned int* done_counter;    // device, zero-initialised
  uint64_t budget_ns;            // time budget of every cross-rank wait
  int* status;                   // device status word
  int max_ctas;                  // 0 = default
  // NVLS flavour: multicast addresses of the gradient and bf16 parameter buffers (the same
  // symmetric allocations seen through the NVSwitch multicast object), or null for plain peer
  // loads / stores. With them the reduce-scatter is one multimem.ld_reduce per 16 bytes (the
  // switch adds the ranks' copies) and the all-gather one multimem.st (the switch replicates it).
  void* grads_mc;
  void* p16_mc;
};

// Reduce-scatter + global-norm clip + AdamW on the shard + all-gather of bf16 parameters.
int fused_step_twoshot(const FusedStepArgs& a, cudaStream_t stream);

// Sum all-reduce over peer memory. One-shot writes the result to `out` (must not alias the
// local input); two-shot works in place on bufs[rank] (`out` ignored, n a multiple of 16 bytes).
int allreduce(void* const* bufs, void* const* pads, void* out, int rank, int world, long long n,
              int dtype, int algo, uint32_t* epoch, unsigned int* done_counter, uint64_t budget_ns,
              int* status, int max_ctas, cudaStream_t stream);

// Single-thread kernel that waits (bounded) for pad slot (kind, src) to reach `epoch`; writes 1 to
// *result on success, 0 after the budget ran out (and kTimeoutPeer to *status).
int wait_probe(void* pad, int kind, int src, uint32_t epoch, uint64_t budget_ns, int* status,
               int* result, cudaStream_t stream);

}  // namespace z2h
