// Host-side token selection (see sampler.h). Everything here is O(vocab) per token at most and
// runs on the caller's thread between decode steps, like the reference's sampler does.
#include "sampler.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace pg {

uint64_t SmallRng::next_u64() {
  state += 0x9e3779b97f4a7c15ULL;
  uint64_t v = state;
  v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ULL;
  v = (v ^ (v >> 27)) * 0x94d049bb133111ebULL;
  return v ^ (v >> 31);
}

double SmallRng::next_unit_f64() {
  return (double)(next_u64() >> 11) * (1.0 / 9007199254740992.0);  // 2^-53
}

// generation.rs:269-279: first strict maximum starting from -inf; NaN never compares greater.
uint64_t argmax_logits(const float* v, size_t n) {
  uint64_t best_idx = 0;
  float best = -INFINITY;
  for (size_t i = 0; i < n; ++i)
    if (v[i] > best) {
      best = v[i];
      best_idx = i;
    }
  return best_idx;
}

int validate_generation_config(const pg_generation_config& g) {
  if (!std::isfinite(g.temperature) || g.temperature < 0.0f)
    return set_error(PG_INVALID_CONFIG, "generation temperature must be finite and >= 0");
  if (!(g.top_p < 0.0f)) {
    if (!std::isfinite(g.top_p) || g.top_p <= 0.0f || g.top_p > 1.0f)
      return set_error(PG_INVALID_CONFIG, "generation top_p must be finite and in (0, 1]");
  }
  if (g.top_k == 0) return set_error(PG_INVALID_CONFIG, "generation top_k must be > 0");
  if (!std::isfinite(g.repeat_penalty) || g.repeat_penalty <= 0.0f)
    return set_error(PG_INVALID_CONFIG, "generation repeat_penalty must be finite and > 0");
  return PG_OK;
}

// Order of f32::total_cmp as a signed integer key.
static inline int32_t total_key(float f) {
  int32_t b;
  memcpy(&b, &f, 4);
  return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

// Steps after the sort/truncate of sample_logits (generation.rs:320-361) on a descending list.
static uint64_t draw_from_sorted(SmallRng& rng, const std::vector<std::pair<uint32_t, float>>& cand,
                                 const pg_generation_config& g) {
  double temp = (double)g.temperature;
  double max_logit = (double)cand[0].second / temp;
  std::vector<std::pair<uint32_t, double>> weighted;
  weighted.reserve(cand.size());
  for (auto& c : cand) weighted.emplace_back(c.first, std::exp((double)c.second / temp - max_logit));
  if (!(g.top_p < 0.0f)) {
    double full = 0.0;
    for (auto& w : weighted) full += w.second;
    if (full > 0.0) {
      double cum = 0.0;
      size_t keep = 0;
      for (auto& w : weighted) {
        cum += w.second;
        ++keep;
        if (cum / full >= (double)g.top_p) break;
      }
      weighted.resize(std::max<size_t>(keep, 1));
    }
  }
  double total = 0.0;
  for (auto& w : weighted) total += w.second;
  if (total <= 0.0 || !std::isfinite(total)) return weighted[0].first;
  uint64_t fallback = weighted.back().first;
  double target = rng.next_unit_f64() * total;
  for (auto& w : weighted) {
    target -= w.second;
    if (target <= 0.0) return w.first;
  }
  return fallback;
}

}  // namespace pg

int pg_sampler::select_next_token(const float* logits, size_t n, const uint64_t* history, size_t n_hist,
                                  const pg_generation_config& g, uint64_t* out) {
  using namespace pg;
  const float* src = logits;
  // apply_repeat_penalty, generation.rs:281-298
  if (!(g.repeat_penalty == 1.0f || g.repeat_last_n == 0)) {
    adjusted.assign(logits, logits + n);
    std::vector<uint64_t> seen;
    size_t take = std::min<size_t>(g.repeat_last_n, n_hist);
    for (size_t i = 0; i < take; ++i) {
      uint64_t tok = history[n_hist - 1 - i];
      if (tok >= n || std::find(seen.begin(), seen.end(), tok) != seen.end()) continue;
      seen.push_back(tok);
      if (adjusted[tok] < 0.0f) adjusted[tok] *= g.repeat_penalty;
      else adjusted[tok] /= g.repeat_penalty;
    }
    src = adjusted.data();
  }
  if (g.temperature <= 0.0f) {
    *out = argmax_logits(src, n);
    return PG_OK;
  }
  candidates.clear();
  candidates.reserve(n);
  for (size_t i = 0; i < n; ++i)
    if (std::isfinite(src[i])) candidates.emplace_back((uint32_t)i, src[i]);
  if (candidates.empty())
    return set_error(PG_INVALID_INPUT, "token sampling failed: cannot sample from empty or non-finite logits");
  auto desc = [](const std::pair<uint32_t, float>& l, const std::pair<uint32_t, float>& r) {
    int32_t a = total_key(l.second), b = total_key(r.second);
    return a != b ? a > b : l.first < r.first;  // stable descending == ties by lower index
  };
  if (g.top_k > 0 && (size_t)g.top_k < candidates.size()) {
    // the first top_k of the stable descending sort, without sorting the whole vocabulary
    std::partial_sort(candidates.begin(), candidates.begin() + g.top_k, candidates.end(), desc);
    candidates.resize((size_t)g.top_k);
  } else {
    std::sort(candidates.begin(), candidates.end(), desc);
  }
  *out = draw_from_sorted(rng, candidates, g);
  return PG_OK;
}

int pg_sampler::select_from_sorted(const float* vals, const int32_t* idx, size_t k,
                                   const pg_generation_config& g, uint64_t* out) {
  using namespace pg;
  if (!(g.repeat_penalty == 1.0f || g.repeat_last_n == 0))
    return set_error(PG_INVALID_INPUT, "top-k shortcut needs repeat_penalty == 1");
  if (g.temperature <= 0.0f) {
    if (k == 0) return set_error(PG_INVALID_INPUT, "empty top-k list");
    *out = (uint64_t)idx[0];
    return PG_OK;
  }
  if (g.top_k <= 0 || (size_t)g.top_k > k)
    return set_error(PG_INVALID_INPUT, "top-k shortcut needs 0 < top_k <= k");
  candidates.clear();
  for (size_t i = 0; i < (size_t)g.top_k; ++i)
    if (std::isfinite(vals[i])) candidates.emplace_back((uint32_t)idx[i], vals[i]);
  if (candidates.empty())
    return set_error(PG_INVALID_INPUT, "token sampling failed: cannot sample from empty or non-finite logits");
  *out = draw_from_sorted(rng, candidates, g);
  return PG_OK;
}

// ------------------------------------------------------------------ C ABI (host-only entry points)
extern "C" {

void pg_generation_config_default(uint64_t max_new_tokens, pg_generation_config* out) {
  if (!out) return;
  // TextGenerationConfig::new, src/models/generation.rs:73-85
  *out = pg_generation_config{max_new_tokens, -1, 0.0f, -1.0f, -1, 299792458ULL, 1.0f, 128};
}

int pg_generation_config_validate(const pg_generation_config* cfg) {
  if (!cfg) return pg::set_error(PG_INVALID_CONFIG, "null generation config");
  return pg::validate_generation_config(*cfg);
}

uint64_t pg_argmax_logits(const float* logits, size_t n) { return pg::argmax_logits(logits, n); }

int pg_sampler_new(uint64_t seed, pg_sampler** out) {
  if (!out) return pg::set_error(PG_INVALID_INPUT, "null output");
  *out = new pg_sampler(seed);
  return PG_OK;
}

void pg_sampler_free(pg_sampler* sampler) { delete sampler; }

int pg_sampler_select_next_token(pg_sampler* sampler, const float* logits, size_t n, const uint64_t* history,
                                 size_t n_history, const pg_generation_config* cfg, uint64_t* out_token) {
  if (!sampler || !logits || !cfg || !out_token) return pg::set_error(PG_INVALID_INPUT, "null argument");
  return sampler->select_next_token(logits, n, history, n_history, *cfg, out_token);
}

int pg_sampler_select_from_topk(pg_sampler* sampler, const float* topk_vals, const int32_t* topk_idx, size_t k,
                                const pg_generation_config* cfg, uint64_t* out_token) {
  if (!sampler || !topk_vals || !topk_idx || !cfg || !out_token) return pg::set_error(PG_INVALID_INPUT, "null argument");
  return sampler->select_from_sorted(topk_vals, topk_idx, k, *cfg, out_token);
}

int pg_sampler_select_from_topk_batch(pg_sampler* const* samplers, const float* topk_vals, const int32_t* topk_idx,
                                      size_t batch, size_t k, const pg_generation_config* cfg, uint64_t* out_tokens) {
  if (!samplers || !topk_vals || !topk_idx || !cfg || !out_tokens) return pg::set_error(PG_INVALID_INPUT, "null argument");
  for (size_t i = 0; i < batch; ++i) {
    if (!samplers[i]) return pg::set_error(PG_INVALID_INPUT, "null sampler at index " + std::to_string(i));
    if (int r = samplers[i]->select_from_sorted(topk_vals + i * k, topk_idx + i * k, k, *cfg, out_tokens + i)) return r;
  }
  return PG_OK;
}

}  // extern "C"
