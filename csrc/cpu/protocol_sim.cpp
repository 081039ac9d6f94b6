// Host-side drive of the cross-rank signalling protocol (csrc/comm/signal_protocol.h): the very
// functions the CUDA kernels use, instantiated with std::atomic and a steady clock, and run with
// one thread per simulated rank on pads that live in ordinary memory. This is how the protocol's
// corner cases are tested without a GPU and without ever making a GPU wait for something that
// does not come: epochs that wrap around 2^32, a peer that never signals (the others must give
// up inside their budget and report it), a signal from a step that has already timed out arriving
// late (it must not be taken for the current step's), and the last-one-out counter.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../comm/signal_protocol.h"

namespace {

using namespace z2h::proto;

struct HostBackend {
  static uint64_t load_acquire(const uint64_t* p) {
    return reinterpret_cast<const std::atomic<uint64_t>*>(p)->load(std::memory_order_acquire);
  }
  static void store_release(uint64_t* p, uint64_t v) {
    reinterpret_cast<std::atomic<uint64_t>*>(p)->store(v, std::memory_order_release);
  }
  static uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
  }
  static void pause() { std::this_thread::yield(); }
  static void report_timeout(int* status) {
    if (status == nullptr) return;
    int expected = 0;
    reinterpret_cast<std::atomic<int>*>(status)->compare_exchange_strong(expected, 5 /* kTimeoutPeer */);
  }
  static unsigned fetch_add(unsigned* p, unsigned v) {
    return reinterpret_cast<std::atomic<unsigned>*>(p)->fetch_add(v, std::memory_order_acq_rel);
  }
};

struct Sim {
  int world;
  std::vector<std::vector<uint64_t>> pads;  // one pad per rank
  std::vector<int> status;                  // one status word per rank
  explicit Sim(int w) : world(w), pads(w, std::vector<uint64_t>(kPadSlots, 0)), status(w, 0) {}

  // rank tells every peer (and itself) "I reached `epoch` for `kind`", with a payload
  void announce(int rank, int kind, uint32_t epoch, uint32_t payload) {
    for (int dst = 0; dst < world; ++dst) signal<HostBackend>(pads[dst].data(), kind, rank, epoch, payload);
  }
  // rank waits for all peers; returns false when any wait ran out. payload_sum: sum of payloads.
  bool wait_all(int rank, int kind, uint32_t epoch, uint64_t budget_ns, uint64_t* payload_sum) {
    bool ok = true;
    uint64_t sum = 0;
    for (int src = 0; src < world; ++src) {
      uint64_t w = 0;
      if (!wait_signal<HostBackend>(pads[rank].data(), kind, src, epoch, budget_ns, &w, &status[rank]))
        ok = false;
      else
        sum += word_payload(w);
    }
    if (payload_sum != nullptr) *payload_sum = sum;
    return ok;
  }
};

}  // namespace

extern "C" {

// Scenario 0: `steps` clean steps of `buckets` bucket barriers + a norm exchange, starting at
// `first_epoch` (choose it near 2^32 to cross the wrap). Returns 0 when every rank saw every
// barrier complete and the same payload sum in every step, else a negative code.
int z2h_protocol_sim_steps(int world, int steps, int buckets, unsigned int first_epoch) {
  if (world < 1 || world > kMaxRanks || buckets < 0 || buckets > kMaxBuckets) return -100;
  Sim sim(world);
  // the pads of a communicator that has already run `first_epoch` steps: every word carries that
  // epoch (a zero-filled pad is the special case first_epoch = 0)
  for (auto& pad : sim.pads)
    for (auto& w : pad) w = make_word(first_epoch, 0);
  std::vector<int> result(world, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) {
    th.emplace_back([&, r] {
      uint32_t epoch = first_epoch;
      for (int s = 0; s < steps; ++s) {
        const uint32_t e = epoch + 1;
        for (int b = 0; b < buckets; ++b) {
          sim.announce(r, kSlotBucket0 + b, e, 0);
          if (!sim.wait_all(r, kSlotBucket0 + b, e, 2000000000ull, nullptr)) result[r] = -1;
        }
        uint64_t sum = 0;
        sim.announce(r, kSlotNorm, e, (uint32_t)(r + 1 + s));
        if (!sim.wait_all(r, kSlotNorm, e, 2000000000ull, &sum)) result[r] = -2;
        uint64_t want = 0;
        for (int q = 0; q < world; ++q) want += (uint64_t)(q + 1 + s);
        if (sum != want) result[r] = -3;
        sim.announce(r, kSlotDone, e, 0);
        if (!sim.wait_all(r, kSlotDone, e, 2000000000ull, nullptr)) result[r] = -4;
        epoch = e;
      }
    });
  }
  for (auto& t : th) t.join();
  for (int r = 0; r < world; ++r)
    if (result[r] != 0 || sim.status[r] != 0) return result[r] != 0 ? result[r] : -5;
  return 0;
}

// Scenario 1: rank world-1 stays silent in step 1 of 3. The other ranks must give up within
// `budget_ms` (status 5), move their epoch on, and complete step 2 (in which the silent rank takes
// part again, after first delivering its step-1 signal LATE, which must not satisfy step 2).
// out[r] = { step-1 wait result (0 = timed out as it must), status word after step 1,
//            step-2 wait result (1 = completed), waited ms in step 1 }.
int z2h_protocol_sim_silent_peer(int world, int budget_ms, int* out /* [world][4] */) {
  if (world < 2 || world > kMaxRanks) return -100;
  Sim sim(world);
  const uint64_t budget = (uint64_t)budget_ms * 1000000ull;
  std::atomic<int> others_done_step1{0};
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) {
    th.emplace_back([&, r] {
      const bool silent = r == world - 1;
      int* o = out + 4 * r;
      // step 0: everyone takes part
      sim.announce(r, kSlotNorm, 1, 0);
      sim.wait_all(r, kSlotNorm, 1, 5000000000ull, nullptr);
      // step 1: the last rank says nothing
      if (!silent) {
        sim.announce(r, kSlotNorm, 2, 0);
        const uint64_t t0 = HostBackend::now_ns();
        o[0] = sim.wait_all(r, kSlotNorm, 2, budget, nullptr) ? 1 : 0;
        o[3] = (int)((HostBackend::now_ns() - t0) / 1000000ull);
        o[1] = sim.status[r];
        sim.status[r] = 0;  // the host read it and carries on
        others_done_step1.fetch_add(1);
      } else {
        while (others_done_step1.load() < world - 1) std::this_thread::yield();
        o[0] = 0;
        o[1] = 5;
        o[3] = 0;
        // the late signal of the abandoned step arrives while the others already wait for step 2
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
        sim.announce(r, kSlotNorm, 2, 0);
        std::this_thread::sleep_for(std::chrono::milliseconds(40));
      }
      // step 2: epoch 3 for everybody (a timed-out step still advances the epoch)
      const uint64_t t1 = HostBackend::now_ns();
      sim.announce(r, kSlotNorm, 3, 0);
      o[2] = sim.wait_all(r, kSlotNorm, 3, 5000000000ull, nullptr) ? 1 : 0;
      // the non-silent ranks can only have completed step 2 after the silent rank's real signal,
      // i.e. at least ~40 ms after its late one
      if (!silent && (HostBackend::now_ns() - t1) < 30000000ull) o[2] = -1;
    });
  }
  for (auto& t : th) t.join();
  return 0;
}

// Scenario 2: `groups` rounds in which `n` threads call last_one_out once each; returns the number
// of rounds in which exactly one caller was told it is the last (must equal `groups`) or -1 if the
// counter is not back at zero at the end.
int z2h_protocol_sim_last_one_out(int n, int groups) {
  unsigned counter = 0;
  int good = 0;
  for (int g = 0; g < groups; ++g) {
    std::atomic<int> winners{0};
    std::vector<std::thread> th;
    for (int i = 0; i < n; ++i)
      th.emplace_back([&] {
        if (last_one_out<HostBackend>(&counter, (unsigned)n)) winners.fetch_add(1);
      });
    for (auto& t : th) t.join();
    if (winners.load() == 1) ++good;
  }
  return counter == 0 ? good : -1;
}

// epoch_reached across the wrap, for a direct unit check from Python.
int z2h_protocol_epoch_reached(unsigned int seen, unsigned int wanted) { return epoch_reached(seen, wanted) ? 1 : 0; }
int z2h_protocol_pad_slots(void) { return kPadSlots; }
}
