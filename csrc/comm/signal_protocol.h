// Cross-rank signalling protocol of the peer-memory collectives, written once for two worlds.
//
// Every rank owns a "signal pad": kPadKinds x kMaxRanks 64-bit words in memory that every peer can
// write. Word (kind, src) of rank r's pad is written only by rank src and read only by rank r.
// A word is (epoch << 32) | payload. Epochs only grow (one per collective step), so a pad is
// never cleared: a waiter asks "has this word reached epoch E yet", with a wrap-safe signed
// comparison, and a signal left over from an earlier step can never satisfy a later wait.
// Every wait has a time budget; when it runs out the waiter records a status code and gives up,
// it never spins for ever.
//
// The functions are templates over a Backend that supplies the memory operations and the clock:
//   static uint64_t load_acquire(const uint64_t* p);      system-scope acquire load
//   static void     store_release(uint64_t* p, uint64_t v);  system-scope release store
//   static uint64_t now_ns();                               monotonic clock
//   static void     pause();                                back-off between polls
//   static void     report_timeout(int* status);            first failure wins
//   static unsigned fetch_add(unsigned* p, unsigned v);     device-/process-scope atomic add
// The CUDA kernels (ar_adamw.cu) instantiate them with PTX ld.acquire.sys / st.release.sys and
// %globaltimer; the host test (csrc/cpu/protocol_sim.cpp) instantiates the same code with
// std::atomic and std::chrono and drives it with one thread per rank, which is how epoch wrap,
// a peer that never signals, stale epochs after a timeout and the last-one-out counter are
// tested without a GPU.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define Z2H_HD __host__ __device__ __forceinline__
#else
#define Z2H_HD inline
#endif

namespace z2h {
namespace proto {

constexpr int kMaxRanks = 8;
constexpr int kMaxBuckets = 64;

enum SlotKind : int {
  kSlotReady = 0,   // "my input is final" (standalone all-reduce)
  kSlotNorm = 1,    // payload: this rank's sum of squares (float bits)
  kSlotDone = 2,    // "I have finished writing into / reading from peers"
  kSlotPhase = 3,   // second barrier of the standalone two-shot all-reduce
  kSlotBucket0 = 8, // kSlotBucket0 + b: "gradient bucket b is final on my side"
};
constexpr int kPadKinds = kSlotBucket0 + kMaxBuckets;
constexpr int kPadSlots = kPadKinds * kMaxRanks;  // 64-bit words per pad

Z2H_HD int slot_index(int kind, int src) { return kind * kMaxRanks + src; }
Z2H_HD uint64_t make_word(uint32_t epoch, uint32_t payload) { return ((uint64_t)epoch << 32) | payload; }
Z2H_HD uint32_t word_epoch(uint64_t w) { return (uint32_t)(w >> 32); }
Z2H_HD uint32_t word_payload(uint64_t w) { return (uint32_t)w; }
// true once `seen` is at or past `wanted`, also across the 2^32 wrap
Z2H_HD bool epoch_reached(uint32_t seen, uint32_t wanted) { return (int32_t)(seen - wanted) >= 0; }

// Tell peer `dst` (whose pad is `dst_pad`) that rank `src` reached `epoch` for `kind`.
template <class B>
Z2H_HD void signal(uint64_t* dst_pad, int kind, int src, uint32_t epoch, uint32_t payload) {
  B::store_release(dst_pad + slot_index(kind, src), make_word(epoch, payload));
}

// Wait on this rank's own pad until word (kind, src) reaches `epoch`. Returns false, after
// recording the failure in *status, when `budget_ns` runs out first.
template <class B>
Z2H_HD bool wait_signal(const uint64_t* my_pad, int kind, int src, uint32_t epoch, uint64_t budget_ns,
                        uint64_t* word_out, int* status) {
  const uint64_t* s = my_pad + slot_index(kind, src);
  const uint64_t t0 = B::now_ns();
  while (true) {
    const uint64_t w = B::load_acquire(s);
    if (epoch_reached(word_epoch(w), epoch)) {
      if (word_out != nullptr) *word_out = w;
      return true;
    }
    if (B::now_ns() - t0 > budget_ns) {
      B::report_timeout(status);
      return false;
    }
    B::pause();
  }
}

// "Last one out": each of `n` participants calls this once after its work is complete; exactly
// one of them (the last to arrive) gets true and resets the counter for the next use.
template <class B>
Z2H_HD bool last_one_out(unsigned* counter, unsigned n) {
  const unsigned prev = B::fetch_add(counter, 1u);
  if (prev == n - 1) {
    B::fetch_add(counter, 0u - n);  // back to zero, atomically
    return true;
  }
  return false;
}

}  // namespace proto
}  // namespace z2h
