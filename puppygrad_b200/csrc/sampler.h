// Host-side token selection: the reference's LogitsSampler (src/models/generation.rs:209-362).
#pragma once
#include <cstdint>
#include <vector>

#include "common.h"

namespace pg {

// SplitMix64 seeded with seed ^ 0x9e3779b97f4a7c15 (generation.rs:243-267).
struct SmallRng {
  uint64_t state;
  explicit SmallRng(uint64_t seed) : state(seed ^ 0x9e3779b97f4a7c15ULL) {}
  uint64_t next_u64();
  double next_unit_f64();
};

uint64_t argmax_logits(const float* v, size_t n);
int validate_generation_config(const pg_generation_config& g);

}  // namespace pg

struct pg_sampler {
  pg::SmallRng rng;
  std::vector<float> adjusted;                       // scratch: logits after repeat penalty
  std::vector<std::pair<uint32_t, float>> candidates; // scratch: finite logits
  explicit pg_sampler(uint64_t seed) : rng(seed) {}
  int select_next_token(const float* logits, size_t n, const uint64_t* history, size_t n_hist,
                        const pg_generation_config& g, uint64_t* out);
  int select_from_sorted(const float* vals, const int32_t* idx, size_t k, const pg_generation_config& g,
                         uint64_t* out);
};
