// Host API of the peer-memory collectives (P2P loads/stores or multimem over NVLink, no NCCL).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "signal_protocol.h"

namespace z2h {

constexpr int kMaxRanks = proto::kMaxRanks;
// A signal pad holds kPadSlots 64-bit words per rank: slot = kind * kMaxRanks + source rank.
constexpr int kPadSlots = proto::kPadSlots;

enum CommDtype : int { kCommF32 = 0, kCommBF16 = 1 };
enum AllReduceAlgo : int { kAllReduceOneShot = 0, kAllReduceTwoShot = 1, kAllReduceNvls = 2 };

// One gradient bucket's reduction (see ar_adamw.cu). Launches one kernel.
struct BucketArgs {
  void* const* grads;   // [world] fp32 gradient buffers, peer-mapped
  void* const* pads;    // [world] signal pads (kPadSlots uint64 each), peer-mapped, zero-initialised
  void* grads_mc;       // multicast address of the gradient buffer (NVLS flavour) or null
  int rank, world;
  int bucket;           // index of the bucket: selects the signal slot, < proto::kMaxBuckets
  long long goff, n;    // two-shot: this rank's slice of the bucket; one-shot: the whole bucket
  float* dst;           // two-shot: own gradient buffer + goff; one-shot: a local buffer of n floats
  int one_shot;
  float* partials;      // receives one sum of squares per CTA launched
  int count_sumsq;      // 0: write zeros instead (a one-shot bucket is counted by one rank only)
  uint32_t* epoch;      // device counter owned by this communicator
  uint64_t budget_ns;   // time budget of every cross-rank wait
  int* status;          // device status word (sticky)
  int max_ctas;         // 0 = fill the device
};
// Returns the grid size (>= 1), -1 for a bad argument or -3 if the launch failed.
int reduce_bucket(const BucketArgs& a, cudaStream_t stream);
int reduce_bucket_grid(long long n, int max_ctas);

// What the optimizer phase does with a range of the flat buffers.
enum RangeKind : int {
  kRangeTwoShot = 0,  // reduced slice in own gradient buffer at goff: AdamW, bf16 to every peer, clear
  kRangeOneShot = 1,  // reduced bucket in `red` at roff: AdamW on the replicated state, local bf16
  kRangeZero = 2,     // not owned: clear the local gradient buffer only
};
struct StepRange {
  long long goff;  // offset in the flat parameter / gradient buffers
  long long n;     // elements (multiple of 8)
  long long loff;  // offset in this rank's p32 / m / v (update kinds)
  long long roff;  // offset in `red` (kRangeOneShot)
  int kind;
  int pad_;
};

struct PhaseArgs {
  void* const* grads;
  void* const* p16;     // [world] bf16 parameter buffers, peer-mapped
  void* const* pads;
  void* p16_mc;         // multicast address of the bf16 parameter buffer (NVLS flavour) or null
  const float* red;     // reduced one-shot buckets (local)
  float* p32; float* m; float* v;  // this rank's optimizer state, indexed by StepRange::loff
  int rank, world;
  const StepRange* ranges;  // device array
  int num_ranges;
  long long total_units;    // sum of n / 8 over the ranges
  long long n_decay;        // elements [0, n_decay) of the flat buffer get weight decay
  const float* hyper;       // device, see HyperSlot
  const float* partials; int num_partials;
  float* norm_out;          // device, receives the global pre-clip gradient norm
  uint32_t* epoch;
  unsigned int* done_counter;  // device, zero-initialised
  uint64_t budget_ns;
  int* status;
  int max_ctas;
};
// Global-norm clip + AdamW on the owned ranges + all-gather of bf16 parameters + finish.
int optimizer_phase(const PhaseArgs& a, cudaStream_t stream);

int comm_preload();

// Sum all-reduce over peer memory. One-shot writes the result to `out` (must not alias the
// local input); two-shot and NVLS work in place on bufs[rank] (`out` ignored, n a multiple of
// 16 bytes). NVLS needs `buf_mc`, the multicast address of the same symmetric buffer.
int allreduce(void* const* bufs, void* const* pads, void* out, void* buf_mc, int rank, int world,
              long long n, int dtype, int algo, uint32_t* epoch, unsigned int* done_counter,
              uint64_t budget_ns, int* status, int max_ctas, cudaStream_t stream);

// Single-thread kernel that waits (bounded) for pad slot (kind, src) to reach `epoch`; writes 1 to
// *result on success, 0 after the budget ran out (and kTimeoutPeer to *status).
int wait_probe(void* pad, int kind, int src, uint32_t epoch, uint64_t budget_ns, int* status,
               int* result, cudaStream_t stream);

}  // namespace z2h
