// Counter-based dropout masks shared by every kernel that drops activations.
//
// A mask is a pure function of (seed, element index): one 32-bit word per 4 consecutive elements
// of a logical stream, one byte per element, an element is kept when its byte is >= the
// threshold round(p * 256). The forward and backward kernels of a site therefore agree on the
// mask without storing it, in whatever order they walk the elements, and a host program can
// restate the same arithmetic to check them (zero_to_hero_b200/ops/dropout.py).
// The drop probability is quantised to 1/256; kept values are scaled by 256 / (256 - threshold).
//
// Replaces torch's Philox-based nn.Dropout / SDPA dropout_p of the reference model
// (nn/gpt2/modules.py:23,36,52,79): same semantics, different random stream.
#pragma once
#include <cstdint>

namespace z2h {

struct DropoutSpec {
  uint32_t seed_lo, seed_hi;  // already combined with the site identifier
  uint32_t threshold;         // 0 (keep everything) .. 255
  float scale;                // 256 / (256 - threshold)
};

__host__ __device__ __forceinline__ uint32_t dropout_word(uint32_t seed_lo, uint32_t seed_hi,
                                                          unsigned long long word_index) {
  uint32_t x = (uint32_t)word_index * 0x9E3779B1u + seed_lo;
  uint32_t y = (uint32_t)(word_index >> 32) * 0x85EBCA77u + seed_hi;
  x ^= y;
  x ^= x >> 16;
  x *= 0x85EBCA6Bu;
  x ^= x >> 13;
  x *= 0xC2B2AE35u;
  x ^= x >> 16;
  x += y * 0x27D4EB2Fu;
  x ^= x >> 15;
  x *= 0x2C1B3C6Du;
  x ^= x >> 12;
  return x;
}

// keep flag of element (word_index * 4 + j), j in 0..3, given its word
__host__ __device__ __forceinline__ bool dropout_keep(uint32_t word, int j, uint32_t threshold) {
  return ((word >> (8 * j)) & 0xffu) >= threshold;
}

// Combines the run's seed (read from device memory, so that a captured graph can be replayed
// with a new seed) with a site identifier (layer and position in the layer).
__device__ __forceinline__ DropoutSpec make_dropout_spec(const unsigned long long* seed_ptr,
                                                         uint32_t site, float p) {
  DropoutSpec d;
  unsigned long long s = (seed_ptr != nullptr ? *seed_ptr : 0ull) + (unsigned long long)site * 0x9E3779B97F4A7C15ull;
  s ^= s >> 31;
  s *= 0xBF58476D1CE4E5B9ull;
  s ^= s >> 29;
  d.seed_lo = (uint32_t)s;
  d.seed_hi = (uint32_t)(s >> 32);
  int t = (int)(p * 256.0f + 0.5f);
  t = t < 0 ? 0 : (t > 255 ? 255 : t);
  d.threshold = (uint32_t)t;
  d.scale = 256.0f / (256.0f - (float)t);
  return d;
}

}  // namespace z2h
