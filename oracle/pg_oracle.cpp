// CPU oracle for the GPT-2 inference path. TEST INFRASTRUCTURE ONLY (see pg_oracle.h).
//
// A restatement of the reference's CPU algorithm, element for element and in the same
// floating-point evaluation order on an x86-64 host with AVX:
//   - dot: 8 independent lanes, multiply then add (not fused), lanes summed 0..7, scalar tail
//     (src/models/cpu.rs:231-254)
//   - every other reduction is a sequential f32 sum in index order
//   - expf / tanhf / sqrtf from the platform libm, as Rust's f32::exp/tanh/sqrt resolve to
// Build with: g++ -O2 -mavx -ffp-contract=off (never -ffast-math, never -mfma).
#include "pg_oracle.h"

#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_err;
int fail(int code, const std::string& msg) {
  g_err = msg;
  return code;
}

// ---------------------------------------------------------------- cpu.rs kernels
// cpu.rs:231-254 dot_avx
inline float dot_avx(const float* a, const float* b, size_t n) {
  size_t i = 0;
  __m256 acc = _mm256_setzero_ps();
  while (i + 8 <= n) {
    __m256 av = _mm256_loadu_ps(a + i);
    __m256 bv = _mm256_loadu_ps(b + i);
    acc = _mm256_add_ps(acc, _mm256_mul_ps(av, bv));
    i += 8;
  }
  float lanes[8];
  _mm256_storeu_ps(lanes, acc);
  float sum = 0.0f;  // iter().sum(): only the sign of an all-zero sum can depend on the start value
  for (int j = 0; j < 8; ++j) sum += lanes[j];
  while (i < n) {
    sum += a[i] * b[i];
    i += 1;
  }
  return sum;
}

// cpu.rs:206-208
inline float dot_scalar(const float* a, const float* b, size_t n) {
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) sum += a[i] * b[i];
  return sum;
}

// cpu.rs:119-143
void layer_norm_in_place(float* x, size_t rows, size_t cols, const float* gamma, const float* beta,
                         float eps) {
  for (size_t r = 0; r < rows; ++r) {
    float* row = x + r * cols;
    float s = 0.0f;
    for (size_t c = 0; c < cols; ++c) s += row[c];
    float mean = s / (float)cols;
    float v = 0.0f;
    for (size_t c = 0; c < cols; ++c) {
      float d = row[c] - mean;
      v += d * d;
    }
    float variance = v / (float)cols;
    float inv_std = 1.0f / sqrtf(variance + eps);
    for (size_t c = 0; c < cols; ++c) row[c] = (row[c] - mean) * inv_std * gamma[c] + beta[c];
  }
}

// cpu.rs:145-150
void gelu_in_place(float* v, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    float x = v[i];
    v[i] = 0.5f * x * (1.0f + tanhf(0.7978846f * (x + 0.044715f * x * x * x)));
  }
}

// cpu.rs:152-165
void softmax_in_place(float* v, size_t n) {
  float mx = -INFINITY;
  for (size_t i = 0; i < n; ++i) mx = fmaxf(mx, v[i]);
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) {
    v[i] = expf(v[i] - mx);
    sum += v[i];
  }
  for (size_t i = 0; i < n; ++i) v[i] /= sum;
}

// cpu.rs:167-171
void add_in_place(float* dst, const float* src, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] += src[i];
}

// cpu.rs:281-289
void transpose_in_out(const float* w, size_t in_f, size_t out_f, float* out) {
  for (size_t i = 0; i < in_f; ++i)
    for (size_t o = 0; o < out_f; ++o) out[o * in_f + i] = w[i * out_f + o];
}

// ---------------------------------------------------------------- thread pool
// thread_pool.rs: fixed workers behind one queue; scoped_parallel_chunks gives worker w the
// chunks w, w+workers, ... and returns the per-chunk results in chunk order (107-170).
class Pool {
 public:
  explicit Pool(size_t threads) : threads_(std::max<size_t>(threads, 1)) {
    if (threads_ > 1)
      for (size_t i = 0; i < threads_; ++i) workers_.emplace_back([this] { loop(); });
  }
  ~Pool() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  size_t threads() const { return threads_; }

  // f(start, end) appends its values to the vector it is given; returns per-chunk vectors.
  std::vector<std::vector<float>> scoped_parallel_chunks(
      size_t len, size_t chunk_size,
      const std::function<void(size_t, size_t, std::vector<float>&)>& f) {
    std::vector<std::vector<float>> results;
    if (len == 0) return results;
    chunk_size = std::max<size_t>(chunk_size, 1);
    size_t chunks = (len + chunk_size - 1) / chunk_size;
    results.resize(chunks);
    if (threads_ == 1 || chunks == 1) {
      for (size_t c = 0; c < chunks; ++c) {
        size_t s = c * chunk_size, e = std::min(s + chunk_size, len);
        f(s, e, results[c]);
      }
      return results;
    }
    size_t workers = std::min(threads_, chunks);
    std::mutex done_mu;
    std::condition_variable done_cv;
    size_t remaining = workers;
    for (size_t w = 0; w < workers; ++w) {
      submit([&, w] {
        for (size_t c = w; c < chunks; c += workers) {
          size_t s = c * chunk_size, e = std::min(s + chunk_size, len);
          f(s, e, results[c]);
        }
        std::lock_guard<std::mutex> g(done_mu);
        if (--remaining == 0) done_cv.notify_one();
      });
    }
    std::unique_lock<std::mutex> lk(done_mu);
    done_cv.wait(lk, [&] { return remaining == 0; });
    return results;
  }

 private:
  void submit(std::function<void()> job) {
    {
      std::lock_guard<std::mutex> g(mu_);
      jobs_.push_back(std::move(job));
    }
    cv_.notify_one();
  }
  void loop() {
    for (;;) {
      std::function<void()> job;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stop_ || !jobs_.empty(); });
        if (jobs_.empty()) return;
        job = std::move(jobs_.front());
        jobs_.erase(jobs_.begin());
      }
      job();
    }
  }
  size_t threads_;
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<std::function<void()>> jobs_;
  bool stop_ = false;
};

// ---------------------------------------------------------------- model types
struct Block {  // rust.rs:111-125; dense matrices stored [out,in] after rust.rs:1345-1352
  std::vector<float> ln_1_g, ln_1_b, c_attn_w, c_attn_b, c_proj_w, c_proj_b, ln_2_g, ln_2_b, c_fc_w,
      c_fc_b, c_proj_mlp_w, c_proj_mlp_b;
};

}  // namespace

struct QRows {  // QuantizedRows, cpu.rs:26-31
  std::vector<int8_t> q;
  std::vector<float> scales;
  size_t cols = 0;
};
struct QBlock {  // Gpt2QuantizedBlockWeights
  QRows c_attn_w, c_proj_w, c_fc_w, c_proj_mlp_w;
};

struct po_model {
  po_config cfg;
  po_rust_config rc;
  std::vector<float> wte, wpe, ln_f_g, ln_f_b;
  std::vector<Block> blocks;
  // Gpt2RustConfig::quantized_weights (options.rs:62-104): Some(Gpt2QuantizedWeights) when set (rust.rs:812-822)
  bool quantized = false;
  QRows qwte;
  std::vector<QBlock> qblocks;
  std::unique_ptr<Pool> pool;
  size_t head_dim() const { return cfg.n_embd / cfg.n_head; }
};

struct po_cache {  // rust.rs:178-267
  std::vector<std::vector<float>> keys, values;
  size_t seq_len = 0, max_seq_len = 0, n_head = 0, head_dim = 0;
};

namespace {

// rust.rs:1851-1855
inline size_t kv_index(size_t pos, size_t head, size_t dim, size_t max_seq_len, size_t head_dim) {
  return (head * max_seq_len + pos) * head_dim + dim;
}

enum Which { CAttn, AttnProj, MlpFc, MlpProj };

size_t chunk_size_of(const po_rust_config& rc, Which w) {  // rust.rs:1386-1395
  switch (w) {
    case CAttn: return rc.qkv_chunk_size;
    case AttnProj: return rc.attention_projection_chunk_size;
    case MlpFc: return rc.mlp_fc_chunk_size;
    default: return rc.mlp_projection_chunk_size;
  }
}

void block_linear(const po_model& m, size_t layer, Which w, const float** weight, const float** bias) {
  const Block& b = m.blocks[layer];  // rust.rs:1422-1436
  switch (w) {
    case CAttn: *weight = b.c_attn_w.data(); *bias = b.c_attn_b.data(); break;
    case AttnProj: *weight = b.c_proj_w.data(); *bias = b.c_proj_b.data(); break;
    case MlpFc: *weight = b.c_fc_w.data(); *bias = b.c_fc_b.data(); break;
    default: *weight = b.c_proj_mlp_w.data(); *bias = b.c_proj_mlp_b.data(); break;
  }
}

// quantized_dot, cpu.rs:173-184: every weight dequantised on the fly, one sequential f32 sum
inline float quantized_dot(const float* a, const QRows& rows, size_t row_index) {
  const int8_t* values = rows.q.data() + row_index * rows.cols;
  const float scale = rows.scales[row_index];
  float sum = 0.0f;
  for (size_t i = 0; i < rows.cols; ++i) sum += a[i] * ((float)values[i] * scale);
  return sum;
}

const QRows& quantized_block_linear(const po_model& m, size_t layer, Which w) {  // rust.rs:1438-1452
  const QBlock& b = m.qblocks[layer];
  switch (w) {
    case CAttn: return b.c_attn_w;
    case AttnProj: return b.c_proj_w;
    case MlpFc: return b.c_fc_w;
    default: return b.c_proj_mlp_w;
  }
}

// rust.rs:1481-1532 + cpu.rs:58-75; with quantised weights quantized_linear_into, rust.rs:1535-1578
void linear_block_into(const po_model& m, const float* x, size_t rows, size_t in_f, size_t out_f,
                       size_t layer, Which which, std::vector<float>& out) {
  const float *weight, *bias;
  block_linear(m, layer, which, &weight, &bias);
  Pool& pool = *m.pool;
  if (m.quantized) {
    const QRows& qw = quantized_block_linear(m, layer, which);
    if (pool.threads() == 1 || rows * in_f * out_f < m.rc.dense_parallel_threshold) {
      out.assign(rows * out_f, 0.0f);
      for (size_t r = 0; r < rows; ++r)
        for (size_t o = 0; o < out_f; ++o) out[r * out_f + o] = bias[o] + quantized_dot(x + r * in_f, qw, o);
      return;
    }
    auto chunks = pool.scoped_parallel_chunks(
        rows * out_f, chunk_size_of(m.rc, which), [&](size_t s, size_t e, std::vector<float>& v) {
          v.reserve(e - s);
          for (size_t idx = s; idx < e; ++idx) {
            size_t r = idx / out_f, o = idx % out_f;
            v.push_back(bias[o] + quantized_dot(x + r * in_f, qw, o));
          }
        });
    out.clear();
    out.reserve(rows * out_f);
    for (auto& c : chunks) out.insert(out.end(), c.begin(), c.end());
    return;
  }
  if (pool.threads() == 1 || rows * in_f * out_f < m.rc.dense_parallel_threshold) {
    out.assign(rows * out_f, 0.0f);
    for (size_t r = 0; r < rows; ++r)
      for (size_t o = 0; o < out_f; ++o)
        out[r * out_f + o] = bias[o] + dot_avx(x + r * in_f, weight + o * in_f, in_f);
    return;
  }
  auto chunks = pool.scoped_parallel_chunks(
      rows * out_f, chunk_size_of(m.rc, which), [&](size_t s, size_t e, std::vector<float>& v) {
        v.reserve(e - s);
        for (size_t idx = s; idx < e; ++idx) {
          size_t r = idx / out_f, o = idx % out_f;
          v.push_back(bias[o] + dot_avx(x + r * in_f, weight + o * in_f, in_f));
        }
      });
  out.clear();
  out.reserve(rows * out_f);
  for (auto& c : chunks) out.insert(out.end(), c.begin(), c.end());
}

// rust.rs:1580-1659: one (head, query) pair of the full-sequence attention
void causal_head_query(const float* qkv, size_t n_embd, size_t head_dim, size_t h, size_t q_pos,
                       float scale, float* dst /* head_dim, pre-zeroed */, std::vector<float>& scores) {
  scores.assign(q_pos + 1, 0.0f);
  for (size_t k_pos = 0; k_pos <= q_pos; ++k_pos) {
    float score = 0.0f;
    for (size_t d = 0; d < head_dim; ++d) {
      float q = qkv[q_pos * 3 * n_embd + h * head_dim + d];
      float k = qkv[k_pos * 3 * n_embd + n_embd + h * head_dim + d];
      score += q * k;
    }
    scores[k_pos] = score * scale;
  }
  softmax_in_place(scores.data(), scores.size());
  for (size_t k_pos = 0; k_pos <= q_pos; ++k_pos) {
    float prob = scores[k_pos];
    for (size_t d = 0; d < head_dim; ++d) {
      float v = qkv[k_pos * 3 * n_embd + 2 * n_embd + h * head_dim + d];
      dst[d] += prob * v;
    }
  }
}

std::vector<float> causal_self_attention(const po_model& m, const float* qkv, size_t seq_len) {
  size_t n_head = m.cfg.n_head, head_dim = m.head_dim(), n_embd = n_head * head_dim;
  std::vector<float> out(seq_len * n_embd, 0.0f);
  float scale = 1.0f / sqrtf((float)head_dim);
  size_t work = seq_len * seq_len * n_head * head_dim;
  Pool& pool = *m.pool;
  if (pool.threads() > 1 && work >= m.rc.attention_head_parallel_threshold) {
    pool.scoped_parallel_chunks(n_head, 1, [&](size_t s, size_t e, std::vector<float>&) {
      std::vector<float> scores;
      for (size_t h = s; h < e; ++h)
        for (size_t q = 0; q < seq_len; ++q)
          causal_head_query(qkv, n_embd, head_dim, h, q, scale, &out[q * n_embd + h * head_dim], scores);
    });
    return out;
  }
  std::vector<float> scores;
  for (size_t h = 0; h < n_head; ++h)
    for (size_t q = 0; q < seq_len; ++q)
      causal_head_query(qkv, n_embd, head_dim, h, q, scale, &out[q * n_embd + h * head_dim], scores);
  return out;
}

// rust.rs:1662-1741: one head of the cached attention
void cached_head(const float* qkv, size_t pos, const po_cache& c, size_t layer, size_t h,
                 float scale, float* dst /* head_dim, pre-zeroed */, std::vector<float>& scores) {
  size_t head_dim = c.head_dim;
  const float* keys = c.keys[layer].data();
  const float* values = c.values[layer].data();
  scores.assign(pos + 1, 0.0f);
  for (size_t k_pos = 0; k_pos <= pos; ++k_pos) {
    float sum = 0.0f;
    for (size_t d = 0; d < head_dim; ++d) {
      float q = qkv[h * head_dim + d];
      float k = keys[kv_index(k_pos, h, d, c.max_seq_len, head_dim)];
      sum += q * k;
    }
    scores[k_pos] = sum * scale;
  }
  softmax_in_place(scores.data(), scores.size());
  for (size_t k_pos = 0; k_pos <= pos; ++k_pos) {
    float prob = scores[k_pos];
    for (size_t d = 0; d < head_dim; ++d)
      dst[d] += prob * values[kv_index(k_pos, h, d, c.max_seq_len, head_dim)];
  }
}

void cached_self_attention_into(const po_model& m, const float* qkv, size_t pos, po_cache& c,
                                size_t layer, std::vector<float>& out, bool allow_threads = true) {
  size_t n_head = m.cfg.n_head, head_dim = m.head_dim(), n_embd = n_head * head_dim;
  out.assign(n_embd, 0.0f);
  float scale = 1.0f / sqrtf((float)head_dim);
  for (size_t h = 0; h < n_head; ++h)
    for (size_t d = 0; d < head_dim; ++d) {
      size_t idx = kv_index(pos, h, d, c.max_seq_len, head_dim);
      c.keys[layer][idx] = qkv[n_embd + h * head_dim + d];
      c.values[layer][idx] = qkv[2 * n_embd + h * head_dim + d];
    }
  size_t work = (pos + 1) * n_head * head_dim;
  Pool& pool = *m.pool;
  if (allow_threads && pool.threads() > 1 && work >= m.rc.attention_head_parallel_threshold) {
    pool.scoped_parallel_chunks(n_head, 1, [&](size_t s, size_t e, std::vector<float>&) {
      std::vector<float> scores;
      for (size_t h = s; h < e; ++h) cached_head(qkv, pos, c, layer, h, scale, &out[h * head_dim], scores);
    });
    return;
  }
  std::vector<float> scores;
  for (size_t h = 0; h < n_head; ++h) cached_head(qkv, pos, c, layer, h, scale, &out[h * head_dim], scores);
}

// rust.rs:1767-1813; with quantised weights quantized_logits_from_hidden_into, rust.rs:1815-1849
void logits_from_hidden_into(const po_model& m, const float* hidden, std::vector<float>& logits) {
  size_t v = m.cfg.vocab_size, c = m.cfg.n_embd;
  Pool& pool = *m.pool;
  if (m.quantized) {
    if (pool.threads() == 1) {
      logits.assign(v, 0.0f);
      for (size_t t = 0; t < v; ++t) logits[t] = quantized_dot(hidden, m.qwte, t);
      return;
    }
    auto chunks = pool.scoped_parallel_chunks(v, m.rc.logits_chunk_size,
                                              [&](size_t s, size_t e, std::vector<float>& out) {
                                                out.reserve(e - s);
                                                for (size_t t = s; t < e; ++t) out.push_back(quantized_dot(hidden, m.qwte, t));
                                              });
    logits.clear();
    logits.reserve(v);
    for (auto& ch : chunks) logits.insert(logits.end(), ch.begin(), ch.end());
    return;
  }
  if (pool.threads() == 1) {
    logits.assign(v, 0.0f);
    for (size_t t = 0; t < v; ++t) logits[t] = dot_avx(hidden, m.wte.data() + t * c, c);
    return;
  }
  auto chunks = pool.scoped_parallel_chunks(v, m.rc.logits_chunk_size,
                                            [&](size_t s, size_t e, std::vector<float>& out) {
                                              out.reserve(e - s);
                                              for (size_t t = s; t < e; ++t)
                                                out.push_back(dot_avx(hidden, m.wte.data() + t * c, c));
                                            });
  logits.clear();
  logits.reserve(v);
  for (auto& ch : chunks) logits.insert(logits.end(), ch.begin(), ch.end());
}

struct Scratch {  // rust.rs:656-682
  std::vector<float> x, norm, qkv, attn, attn_proj, residual, mlp, mlp_proj, logits;
};

// rust.rs:1136-1250
void block_forward_one(const po_model& m, size_t layer, po_cache& cache, Scratch& s) {
  size_t c = m.cfg.n_embd;
  const Block& b = m.blocks[layer];
  s.norm = s.x;
  layer_norm_in_place(s.norm.data(), 1, c, b.ln_1_g.data(), b.ln_1_b.data(), m.cfg.layer_norm_epsilon);
  linear_block_into(m, s.norm.data(), 1, c, 3 * c, layer, CAttn, s.qkv);
  cached_self_attention_into(m, s.qkv.data(), cache.seq_len, cache, layer, s.attn);
  linear_block_into(m, s.attn.data(), 1, c, c, layer, AttnProj, s.attn_proj);
  s.residual = s.x;
  add_in_place(s.residual.data(), s.attn_proj.data(), c);
  s.norm = s.residual;
  layer_norm_in_place(s.norm.data(), 1, c, b.ln_2_g.data(), b.ln_2_b.data(), m.cfg.layer_norm_epsilon);
  linear_block_into(m, s.norm.data(), 1, c, m.cfg.n_inner, layer, MlpFc, s.mlp);
  gelu_in_place(s.mlp.data(), s.mlp.size());
  linear_block_into(m, s.mlp.data(), 1, m.cfg.n_inner, c, layer, MlpProj, s.mlp_proj);
  add_in_place(s.residual.data(), s.mlp_proj.data(), c);
}

// rust.rs:206-234
int check_compatible(const po_model& m, const po_cache& c) {
  if (c.keys.size() != m.cfg.n_layer)
    return fail(PO_INVALID_INPUT, "cache layer count " + std::to_string(c.keys.size()) +
                                      " does not match n_layer " + std::to_string(m.cfg.n_layer));
  if (c.max_seq_len != m.cfg.n_positions)
    return fail(PO_INVALID_INPUT, "cache max_seq_len " + std::to_string(c.max_seq_len) +
                                      " does not match n_positions " + std::to_string(m.cfg.n_positions));
  if (c.n_head != m.cfg.n_head)
    return fail(PO_INVALID_INPUT, "cache n_head " + std::to_string(c.n_head) +
                                      " does not match n_head " + std::to_string(m.cfg.n_head));
  if (c.head_dim != m.head_dim())
    return fail(PO_INVALID_INPUT, "cache head_dim " + std::to_string(c.head_dim) +
                                      " does not match head_dim " + std::to_string(m.head_dim()));
  return PO_OK;
}

// rust.rs:943-1006
int forward_one_with_scratch(const po_model& m, size_t token, po_cache& cache, Scratch& s) {
  if (int rc = check_compatible(m, cache)) return rc;
  if (token >= m.cfg.vocab_size)
    return fail(PO_INVALID_INPUT, "token id " + std::to_string(token) + " exceeds vocab_size " +
                                      std::to_string(m.cfg.vocab_size));
  if (cache.seq_len >= cache.max_seq_len)
    return fail(PO_INVALID_INPUT, "cache is full at seq_len " + std::to_string(cache.seq_len));
  size_t c = m.cfg.n_embd, pos = cache.seq_len;
  s.x.assign(c, 0.0f);
  const float* tok = m.wte.data() + token * c;
  const float* pe = m.wpe.data() + pos * c;
  for (size_t i = 0; i < c; ++i) s.x[i] = tok[i] + pe[i];
  for (size_t layer = 0; layer < m.blocks.size(); ++layer) {
    block_forward_one(m, layer, cache, s);
    std::swap(s.x, s.residual);
  }
  layer_norm_in_place(s.x.data(), 1, c, m.ln_f_g.data(), m.ln_f_b.data(), m.cfg.layer_norm_epsilon);
  logits_from_hidden_into(m, s.x.data(), s.logits);
  cache.seq_len += 1;
  return PO_OK;
}

// rust.rs:1029-1051
int validate_input(const po_model& m, const uint64_t* ids, size_t t) {
  if (t == 0) return fail(PO_INVALID_INPUT, "input_ids must not be empty");
  if (t > m.cfg.n_positions)
    return fail(PO_INVALID_INPUT, "sequence length " + std::to_string(t) + " exceeds n_positions " +
                                      std::to_string(m.cfg.n_positions));
  for (size_t i = 0; i < t; ++i)
    if (ids[i] >= m.cfg.vocab_size)
      return fail(PO_INVALID_INPUT, "token id " + std::to_string(ids[i]) + " at index " +
                                        std::to_string(i) + " exceeds vocab_size " +
                                        std::to_string(m.cfg.vocab_size));
  return PO_OK;
}

// rust.rs:1053-1134
std::vector<float> block_forward(const po_model& m, const std::vector<float>& x, size_t t, size_t layer) {
  size_t c = m.cfg.n_embd;
  const Block& b = m.blocks[layer];
  std::vector<float> norm = x, qkv, attn_proj, mlp, mlp_proj;
  layer_norm_in_place(norm.data(), t, c, b.ln_1_g.data(), b.ln_1_b.data(), m.cfg.layer_norm_epsilon);
  linear_block_into(m, norm.data(), t, c, 3 * c, layer, CAttn, qkv);
  std::vector<float> attn = causal_self_attention(m, qkv.data(), t);
  linear_block_into(m, attn.data(), t, c, c, layer, AttnProj, attn_proj);
  std::vector<float> residual = x;
  add_in_place(residual.data(), attn_proj.data(), residual.size());
  norm = residual;
  layer_norm_in_place(norm.data(), t, c, b.ln_2_g.data(), b.ln_2_b.data(), m.cfg.layer_norm_epsilon);
  linear_block_into(m, norm.data(), t, c, m.cfg.n_inner, layer, MlpFc, mlp);
  gelu_in_place(mlp.data(), mlp.size());
  linear_block_into(m, mlp.data(), t, m.cfg.n_inner, c, layer, MlpProj, mlp_proj);
  add_in_place(residual.data(), mlp_proj.data(), residual.size());
  return residual;
}

int expect_len(const std::string& name, uint64_t actual, uint64_t expected) {  // rust.rs:1335-1343
  if (actual != expected)
    return fail(PO_INVALID_WEIGHTS, name + " len " + std::to_string(actual) +
                                        " does not match expected " + std::to_string(expected));
  return PO_OK;
}

// generation.rs:243-267 SplitMix64
struct SmallRng {
  uint64_t state;
  explicit SmallRng(uint64_t seed) : state(seed ^ 0x9e3779b97f4a7c15ULL) {}
  uint64_t next_u64() {
    state += 0x9e3779b97f4a7c15ULL;
    uint64_t v = state;
    v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ULL;
    v = (v ^ (v >> 27)) * 0x94d049bb133111ebULL;
    return v ^ (v >> 31);
  }
  double next_unit_f64() {
    uint64_t v = next_u64() >> 11;
    return (double)v * (1.0 / (double)(1ULL << 53));
  }
};

// f32::total_cmp key: sign-magnitude bits mapped to a signed integer order
inline int32_t total_order_key(float f) {
  int32_t b;
  std::memcpy(&b, &f, 4);
  b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
  return b;
}

}  // namespace

struct po_sampler {
  SmallRng rng;
  explicit po_sampler(uint64_t seed) : rng(seed) {}
};

extern "C" {

const char* po_last_error(void) { return g_err.c_str(); }

void po_default_rust_config(po_rust_config* o) {
  *o = po_rust_config{1, 262144, 48, 64, 128, 64, 256, 4096};
}

float po_dot(const float* a, const float* b, size_t n) { return dot_avx(a, b, n); }
float po_dot_scalar(const float* a, const float* b, size_t n) { return dot_scalar(a, b, n); }

void po_transposed_dense_projection(const float* x, size_t rows, size_t in_f, size_t out_f,
                                    const float* w, const float* bias, float* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t o = 0; o < out_f; ++o)
      out[r * out_f + o] = bias[o] + dot_avx(x + r * in_f, w + o * in_f, in_f);
}

// QuantizedRows::from_f32 (cpu.rs:33-57): per row scale = max|w| / 127 (1 for an all-zero row; f32::max
// ignores NaN), q = clamp(round-half-away(w / scale), -127, 127) as i8 (NaN casts to 0).
void po_quantize_rows(const float* w, size_t rows, size_t cols, int8_t* q, float* scales) {
  for (size_t r = 0; r < rows; ++r) {
    const float* src = w + r * cols;
    float max_abs = 0.0f;
    for (size_t i = 0; i < cols; ++i) {
      const float v = std::fabs(src[i]);
      if (!(v != v)) max_abs = v > max_abs ? v : max_abs;
    }
    const float scale = max_abs == 0.0f ? 1.0f : max_abs / 127.0f;
    scales[r] = scale;
    for (size_t i = 0; i < cols; ++i) {
      float t = std::round(src[i] / scale);
      t = t < -127.0f ? -127.0f : (t > 127.0f ? 127.0f : t);
      q[r * cols + i] = (t != t) ? (int8_t)0 : (int8_t)t;
    }
  }
}

// quantized_transposed_dense_projection_into + quantized_dot (cpu.rs:99-117, 173-184): every weight is
// dequantised on the fly as (q as f32) * scale; one sequential f32 sum per output, bias added last.
void po_quantized_projection(const float* x, size_t rows, size_t in_f, size_t out_f, const int8_t* q,
                             const float* scales, const float* bias, float* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t o = 0; o < out_f; ++o) {
      const float scale = scales[o];
      float sum = 0.0f;
      for (size_t i = 0; i < in_f; ++i) sum += x[r * in_f + i] * ((float)q[o * in_f + i] * scale);
      out[r * out_f + o] = bias[o] + sum;
    }
}

void po_dense_projection(const float* x, size_t rows, size_t in_f, size_t out_f, const float* w,
                         const float* bias, float* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t o = 0; o < out_f; ++o) {
      float sum = bias[o];
      for (size_t i = 0; i < in_f; ++i) sum += x[r * in_f + i] * w[i * out_f + o];
      out[r * out_f + o] = sum;
    }
}

void po_layer_norm_in_place(float* x, size_t rows, size_t cols, const float* g, const float* b, float eps) {
  layer_norm_in_place(x, rows, cols, g, b, eps);
}
void po_gelu_in_place(float* v, size_t n) { gelu_in_place(v, n); }
void po_softmax_in_place(float* v, size_t n) { softmax_in_place(v, n); }
void po_add_in_place(float* d, const float* s, size_t n) { add_in_place(d, s, n); }
void po_transpose_in_out(const float* w, size_t in_f, size_t out_f, float* out) {
  transpose_in_out(w, in_f, out_f, out);
}

// rust.rs:59-94
int po_config_validate(const po_config* c) {
  if (c->vocab_size == 0) return fail(PO_INVALID_CONFIG, "vocab_size must be > 0");
  if (c->n_positions == 0) return fail(PO_INVALID_CONFIG, "n_positions must be > 0");
  if (c->n_embd == 0) return fail(PO_INVALID_CONFIG, "n_embd must be > 0");
  if (c->n_layer == 0) return fail(PO_INVALID_CONFIG, "n_layer must be > 0");
  if (c->n_head == 0) return fail(PO_INVALID_CONFIG, "n_head must be > 0");
  if (c->n_inner == 0) return fail(PO_INVALID_CONFIG, "n_inner must be > 0");
  if (c->n_embd % c->n_head != 0)
    return fail(PO_INVALID_CONFIG, "n_embd " + std::to_string(c->n_embd) +
                                       " must be divisible by n_head " + std::to_string(c->n_head));
  if (!(c->layer_norm_epsilon > 0.0f)) return fail(PO_INVALID_CONFIG, "layer_norm_epsilon must be > 0");
  return PO_OK;
}

// rust.rs:803-829, 1279-1352
int po_model_new(const po_config* cfg, const float* const* t, const uint64_t* lens, uint64_t n_tensors,
                 const po_rust_config* rc, po_model** out) {
  if (int r = po_config_validate(cfg)) return r;
  po_rust_config rcfg;
  if (rc) rcfg = *rc; else po_default_rust_config(&rcfg);
  if (rcfg.threads == 0) return fail(PO_INVALID_CONFIG, "rust backend threads must be > 0");
  if (rcfg.dense_parallel_threshold == 0)
    return fail(PO_INVALID_CONFIG, "rust dense_parallel_threshold must be > 0");
  uint64_t c = cfg->n_embd, f = cfg->n_inner, L = cfg->n_layer;
  if (n_tensors < 4) return fail(PO_INVALID_WEIGHTS, "blocks len 0 does not match n_layer " + std::to_string(L));
  if (int r = expect_len("wte", lens[0], cfg->vocab_size * c)) return r;
  if (int r = expect_len("wpe", lens[1], cfg->n_positions * c)) return r;
  if (int r = expect_len("ln_f_g", lens[2], c)) return r;
  if (int r = expect_len("ln_f_b", lens[3], c)) return r;
  if ((n_tensors - 4) / 12 != L || (n_tensors - 4) % 12 != 0)
    return fail(PO_INVALID_WEIGHTS, "blocks len " + std::to_string((n_tensors - 4) / 12) +
                                        " does not match n_layer " + std::to_string(L));
  static const char* names[12] = {"ln_1_g", "ln_1_b", "c_attn_w", "c_attn_b", "c_proj_w", "c_proj_b",
                                  "ln_2_g", "ln_2_b", "c_fc_w", "c_fc_b", "c_proj_mlp_w", "c_proj_mlp_b"};
  for (uint64_t i = 0; i < L; ++i) {
    uint64_t expect[12] = {c, c, c * 3 * c, 3 * c, c * c, c, c, c, c * f, f, f * c, c};
    for (int k = 0; k < 12; ++k)
      if (int r = expect_len("blocks[" + std::to_string(i) + "]." + names[k], lens[4 + 12 * i + k], expect[k]))
        return r;
  }
  auto m = std::make_unique<po_model>();
  m->cfg = *cfg;
  m->rc = rcfg;
  auto vec = [&](uint64_t idx) { return std::vector<float>(t[idx], t[idx] + lens[idx]); };
  m->wte = vec(0); m->wpe = vec(1); m->ln_f_g = vec(2); m->ln_f_b = vec(3);
  m->blocks.resize(L);
  for (uint64_t i = 0; i < L; ++i) {
    uint64_t o = 4 + 12 * i;
    Block& b = m->blocks[i];
    b.ln_1_g = vec(o); b.ln_1_b = vec(o + 1);
    b.c_attn_w.resize(lens[o + 2]); transpose_in_out(t[o + 2], c, 3 * c, b.c_attn_w.data());
    b.c_attn_b = vec(o + 3);
    b.c_proj_w.resize(lens[o + 4]); transpose_in_out(t[o + 4], c, c, b.c_proj_w.data());
    b.c_proj_b = vec(o + 5);
    b.ln_2_g = vec(o + 6); b.ln_2_b = vec(o + 7);
    b.c_fc_w.resize(lens[o + 8]); transpose_in_out(t[o + 8], c, f, b.c_fc_w.data());
    b.c_fc_b = vec(o + 9);
    b.c_proj_mlp_w.resize(lens[o + 10]); transpose_in_out(t[o + 10], f, c, b.c_proj_mlp_w.data());
    b.c_proj_mlp_b = vec(o + 11);
  }
  m->pool = std::make_unique<Pool>(rcfg.threads);
  *out = m.release();
  return PO_OK;
}
void po_model_free(po_model* m) { delete m; }

// quantize_weights, rust.rs:1354-1376: the (already transposed) dense matrices and the tied embedding
// as QuantizedRows; from then on every linear and the lm_head use them (the embedding lookup does not).
void po_model_quantize_weights(po_model* m) {
  auto rows_of = [](const std::vector<float>& w, size_t rows, size_t cols) {
    QRows r;
    r.cols = cols;
    r.q.resize(rows * cols);
    r.scales.resize(rows);
    po_quantize_rows(w.data(), rows, cols, r.q.data(), r.scales.data());
    return r;
  };
  const size_t c = m->cfg.n_embd, f = m->cfg.n_inner;
  m->qwte = rows_of(m->wte, m->cfg.vocab_size, c);
  m->qblocks.clear();
  for (const Block& b : m->blocks)
    m->qblocks.push_back(QBlock{rows_of(b.c_attn_w, 3 * c, c), rows_of(b.c_proj_w, c, c), rows_of(b.c_fc_w, f, c),
                                rows_of(b.c_proj_mlp_w, c, f)});
  m->quantized = true;
}

int po_cache_new(const po_model* m, po_cache** out) {
  auto c = std::make_unique<po_cache>();
  size_t len = m->cfg.n_positions * m->cfg.n_head * m->head_dim();
  c->keys.assign(m->cfg.n_layer, std::vector<float>(len, 0.0f));
  c->values.assign(m->cfg.n_layer, std::vector<float>(len, 0.0f));
  c->max_seq_len = m->cfg.n_positions;
  c->n_head = m->cfg.n_head;
  c->head_dim = m->head_dim();
  *out = c.release();
  return PO_OK;
}
void po_cache_free(po_cache* c) { delete c; }
uint64_t po_cache_seq_len(const po_cache* c) { return c->seq_len; }
uint64_t po_cache_max_seq_len(const po_cache* c) { return c->max_seq_len; }
void po_cache_clear(po_cache* c) { c->seq_len = 0; }
void po_cache_set_seq_len(po_cache* c, uint64_t n) { c->seq_len = n; }
int po_cache_read_layer(const po_cache* c, uint64_t layer, float* keys, float* values) {
  if (layer >= c->keys.size()) return fail(PO_INVALID_INPUT, "layer out of range");
  std::memcpy(keys, c->keys[layer].data(), c->keys[layer].size() * 4);
  std::memcpy(values, c->values[layer].data(), c->values[layer].size() * 4);
  return PO_OK;
}

int po_forward(const po_model* m, const uint64_t* ids, uint64_t t, float* logits) {
  if (int r = validate_input(*m, ids, t)) return r;
  size_t c = m->cfg.n_embd, v = m->cfg.vocab_size;
  std::vector<float> x(t * c);
  for (size_t pos = 0; pos < t; ++pos)
    for (size_t i = 0; i < c; ++i) x[pos * c + i] = m->wte[ids[pos] * c + i] + m->wpe[pos * c + i];
  for (size_t layer = 0; layer < m->blocks.size(); ++layer) x = block_forward(*m, x, t, layer);
  layer_norm_in_place(x.data(), t, c, m->ln_f_g.data(), m->ln_f_b.data(), m->cfg.layer_norm_epsilon);
  std::vector<float> row;
  for (size_t pos = 0; pos < t; ++pos) {
    logits_from_hidden_into(*m, x.data() + pos * c, row);
    std::memcpy(logits + pos * v, row.data(), v * 4);
  }
  return PO_OK;
}

int po_prefill(const po_model* m, const uint64_t* ids, uint64_t t, po_cache* cache, float* logits) {
  if (int r = validate_input(*m, ids, t)) return r;
  if (int r = check_compatible(*m, *cache)) return r;
  cache->seq_len = 0;
  Scratch s;
  for (size_t i = 0; i < t; ++i)
    if (int r = forward_one_with_scratch(*m, ids[i], *cache, s)) return r;
  if (logits) std::memcpy(logits, s.logits.data(), s.logits.size() * 4);
  return PO_OK;
}

int po_forward_one(const po_model* m, uint64_t token, po_cache* cache, float* logits) {
  Scratch s;
  if (int r = forward_one_with_scratch(*m, token, *cache, s)) return r;
  if (logits) std::memcpy(logits, s.logits.data(), s.logits.size() * 4);
  return PO_OK;
}

uint64_t po_argmax_logits(const float* v, size_t n) {
  uint64_t best_idx = 0;
  float best = -INFINITY;
  for (size_t i = 0; i < n; ++i)
    if (v[i] > best) {
      best = v[i];
      best_idx = i;
    }
  return best_idx;
}

int po_generate_greedy(const po_model* m, const uint64_t* ids, uint64_t t, uint64_t max_new,
                       uint64_t* out_tokens, uint64_t* out_len) {
  if (int r = validate_input(*m, ids, t)) return r;
  std::vector<uint64_t> tokens(ids, ids + t);
  size_t v = m->cfg.vocab_size;
  std::vector<float> logits;
  for (uint64_t i = 0; i < max_new; ++i) {
    if (tokens.size() >= m->cfg.n_positions) break;
    logits.resize(tokens.size() * v);
    if (int r = po_forward(m, tokens.data(), tokens.size(), logits.data())) return r;
    tokens.push_back(po_argmax_logits(logits.data() + (tokens.size() - 1) * v, v));
  }
  std::memcpy(out_tokens, tokens.data(), tokens.size() * 8);
  *out_len = tokens.size();
  return PO_OK;
}

// autoregressive.rs:61-87
int po_generate_greedy_cached(const po_model* m, const uint64_t* ids, uint64_t t, uint64_t max_new,
                              po_token_cb cb, void* user, uint64_t* out_tokens, uint64_t* out_len) {
  po_cache* cache = nullptr;
  if (int r = po_cache_new(m, &cache)) return r;
  std::unique_ptr<po_cache> guard(cache);
  std::vector<float> logits(m->cfg.vocab_size);
  if (int r = po_prefill(m, ids, t, cache, logits.data())) return r;
  std::vector<uint64_t> tokens(ids, ids + t);
  for (uint64_t i = 0; i < max_new; ++i) {
    if (tokens.size() >= m->cfg.n_positions) break;
    uint64_t next = po_argmax_logits(logits.data(), logits.size());
    tokens.push_back(next);
    if (cb && cb(next, user)) return fail(PO_INVALID_INPUT, "token callback aborted generation");
    if (int r = po_forward_one(m, next, cache, logits.data())) return r;
  }
  std::memcpy(out_tokens, tokens.data(), tokens.size() * 8);
  *out_len = tokens.size();
  return PO_OK;
}

int po_forward_one_batch(const po_model* mp, const uint64_t* tokens, po_cache* const* caches, uint64_t nb,
                         float* logits, uint64_t* argmax) {
  const po_model& m = *mp;
  size_t c = m.cfg.n_embd, f = m.cfg.n_inner, v = m.cfg.vocab_size;
  for (uint64_t b = 0; b < nb; ++b) {
    if (int r = check_compatible(m, *caches[b])) return r;
    if (tokens[b] >= v)
      return fail(PO_INVALID_INPUT, "token id " + std::to_string(tokens[b]) + " exceeds vocab_size " + std::to_string(v));
    if (caches[b]->seq_len >= caches[b]->max_seq_len)
      return fail(PO_INVALID_INPUT, "cache is full at seq_len " + std::to_string(caches[b]->seq_len));
  }
  Pool& pool = *m.pool;
  std::vector<float> x(nb * c), norm(nb * c), qkv(nb * 3 * c), attn(nb * c), ap(nb * c), mlp(nb * f), mp2(nb * c);
  for (uint64_t b = 0; b < nb; ++b)
    for (size_t i = 0; i < c; ++i)
      x[b * c + i] = m.wte[tokens[b] * c + i] + m.wpe[caches[b]->seq_len * c + i];
  // out[b][o] = bias[o] + dot(x[b], W[o]): the same expression as linear_block_into, weight row outermost
  auto linear = [&](const float* in, size_t in_f, size_t out_f, const float* w, const float* bias, float* out,
                    const QRows* qw = nullptr) {
    pool.scoped_parallel_chunks(out_f, 64, [&](size_t s, size_t e, std::vector<float>&) {
      for (size_t o = s; o < e; ++o)
        for (uint64_t b = 0; b < nb; ++b)
          out[b * out_f + o] = (bias ? bias[o] : 0.0f) +
                               (qw ? quantized_dot(in + b * in_f, *qw, o) : dot_avx(in + b * in_f, w + o * in_f, in_f));
    });
  };
  for (size_t layer = 0; layer < m.blocks.size(); ++layer) {
    const Block& bl = m.blocks[layer];
    norm = x;
    layer_norm_in_place(norm.data(), nb, c, bl.ln_1_g.data(), bl.ln_1_b.data(), m.cfg.layer_norm_epsilon);
    const QBlock* qb = m.quantized ? &m.qblocks[layer] : nullptr;
    linear(norm.data(), c, 3 * c, bl.c_attn_w.data(), bl.c_attn_b.data(), qkv.data(), qb ? &qb->c_attn_w : nullptr);
    pool.scoped_parallel_chunks(nb, 1, [&](size_t s, size_t e, std::vector<float>&) {
      std::vector<float> o;
      for (size_t b = s; b < e; ++b) {
        cached_self_attention_into(m, qkv.data() + b * 3 * c, caches[b]->seq_len, *caches[b], layer, o, false);
        std::memcpy(attn.data() + b * c, o.data(), c * 4);
      }
    });
    linear(attn.data(), c, c, bl.c_proj_w.data(), bl.c_proj_b.data(), ap.data(), qb ? &qb->c_proj_w : nullptr);
    add_in_place(x.data(), ap.data(), nb * c);  // residual = x + attn_proj
    norm = x;
    layer_norm_in_place(norm.data(), nb, c, bl.ln_2_g.data(), bl.ln_2_b.data(), m.cfg.layer_norm_epsilon);
    linear(norm.data(), c, f, bl.c_fc_w.data(), bl.c_fc_b.data(), mlp.data(), qb ? &qb->c_fc_w : nullptr);
    gelu_in_place(mlp.data(), mlp.size());
    linear(mlp.data(), f, c, bl.c_proj_mlp_w.data(), bl.c_proj_mlp_b.data(), mp2.data(), qb ? &qb->c_proj_mlp_w : nullptr);
    add_in_place(x.data(), mp2.data(), nb * c);
  }
  if (!logits && !argmax) {  // prompt positions whose logits nobody reads: the cache is all that is kept
    for (uint64_t b = 0; b < nb; ++b) caches[b]->seq_len += 1;
    return PO_OK;
  }
  layer_norm_in_place(x.data(), nb, c, m.ln_f_g.data(), m.ln_f_b.data(), m.cfg.layer_norm_epsilon);
  std::vector<float> local;
  float* lg = logits;
  if (!lg) {
    local.resize(nb * v);
    lg = local.data();
  }
  // logits[v] = dot(hidden, wte[v]) with no bias term at all (rust.rs:1787-1790)
  pool.scoped_parallel_chunks(v, 256, [&](size_t s, size_t e, std::vector<float>&) {
    for (size_t o = s; o < e; ++o)
      for (uint64_t b = 0; b < nb; ++b)
        lg[b * v + o] = m.quantized ? quantized_dot(x.data() + b * c, m.qwte, o) : dot_avx(x.data() + b * c, m.wte.data() + o * c, c);
  });
  for (uint64_t b = 0; b < nb; ++b) {
    caches[b]->seq_len += 1;
    if (argmax) argmax[b] = po_argmax_logits(lg + b * v, v);
  }
  return PO_OK;
}

// ------------------------------------------------------------------ sampling
void po_default_generation_config(uint64_t max_new_tokens, po_generation_config* o) {
  *o = po_generation_config{max_new_tokens, -1, 0.0f, -1.0f, -1, 299792458ULL, 1.0f, 128};
}

int po_generation_config_validate(const po_generation_config* g) {  // generation.rs:92-116
  if (!std::isfinite(g->temperature) || g->temperature < 0.0f)
    return fail(PO_INVALID_CONFIG, "temperature must be finite and >= 0");
  if (!(g->top_p < 0.0f)) {  // a negative value encodes None; anything else is Some(top_p)
    if (!std::isfinite(g->top_p) || g->top_p <= 0.0f || g->top_p > 1.0f)
      return fail(PO_INVALID_CONFIG, "top_p must be finite and in (0, 1]");
  }
  if (g->top_k == 0) return fail(PO_INVALID_CONFIG, "top_k must be > 0");  // negative encodes None
  if (!std::isfinite(g->repeat_penalty) || g->repeat_penalty <= 0.0f)
    return fail(PO_INVALID_CONFIG, "repeat_penalty must be finite and > 0");
  return PO_OK;
}

po_sampler* po_sampler_new(uint64_t seed) { return new po_sampler(seed); }
void po_sampler_free(po_sampler* s) { delete s; }
uint64_t po_sampler_next_u64(po_sampler* s) { return s->rng.next_u64(); }

int po_sampler_select_next_token(po_sampler* s, const float* logits, size_t n, const uint64_t* history,
                                 size_t n_hist, const po_generation_config* g, uint64_t* out) {
  std::vector<float> adjusted(logits, logits + n);
  // generation.rs:281-298
  if (!(g->repeat_penalty == 1.0f || g->repeat_last_n == 0)) {
    std::vector<uint64_t> seen;
    size_t take = std::min<size_t>(g->repeat_last_n, n_hist);
    for (size_t i = 0; i < take; ++i) {
      uint64_t tok = history[n_hist - 1 - i];
      if (tok >= n || std::find(seen.begin(), seen.end(), tok) != seen.end()) continue;
      seen.push_back(tok);
      if (adjusted[tok] < 0.0f) adjusted[tok] *= g->repeat_penalty;
      else adjusted[tok] /= g->repeat_penalty;
    }
  }
  if (g->temperature <= 0.0f) {
    *out = po_argmax_logits(adjusted.data(), n);
    return PO_OK;
  }
  // generation.rs:300-362
  std::vector<std::pair<uint64_t, float>> cand;
  cand.reserve(n);
  for (size_t i = 0; i < n; ++i)
    if (std::isfinite(adjusted[i])) cand.emplace_back(i, adjusted[i]);
  if (cand.empty()) return fail(PO_INVALID_INPUT, "cannot sample from empty or non-finite logits");
  std::stable_sort(cand.begin(), cand.end(), [](const auto& l, const auto& r) {
    return total_order_key(l.second) > total_order_key(r.second);
  });
  if (g->top_k > 0) cand.resize(std::min<size_t>((size_t)g->top_k, cand.size()));
  double temp = (double)g->temperature;
  double max_logit = (double)cand[0].second / temp;
  std::vector<std::pair<uint64_t, double>> weighted;
  weighted.reserve(cand.size());
  for (auto& [id, l] : cand) weighted.emplace_back(id, std::exp((double)l / temp - max_logit));
  if (g->top_p > 0.0f) {
    double full = 0.0;
    for (auto& w : weighted) full += w.second;
    if (full > 0.0) {
      double cum = 0.0;
      size_t keep = 0;
      for (auto& w : weighted) {
        cum += w.second;
        keep += 1;
        if (cum / full >= (double)g->top_p) break;
      }
      weighted.resize(std::max<size_t>(keep, 1));
    }
  }
  double total = 0.0;
  for (auto& w : weighted) total += w.second;
  if (total <= 0.0 || !std::isfinite(total)) {
    *out = weighted[0].first;
    return PO_OK;
  }
  uint64_t fallback = weighted.back().first;
  double target = s->rng.next_unit_f64() * total;
  for (auto& w : weighted) {
    target -= w.second;
    if (target <= 0.0) {
      *out = w.first;
      return PO_OK;
    }
  }
  *out = fallback;
  return PO_OK;
}

uint64_t po_pool_worker_chunks(uint64_t threads, uint64_t len, uint64_t chunk_size, uint64_t worker,
                               uint64_t* out_chunks, uint64_t cap) {
  if (len == 0) return 0;
  chunk_size = std::max<uint64_t>(chunk_size, 1);
  uint64_t chunks = (len + chunk_size - 1) / chunk_size;
  threads = std::max<uint64_t>(threads, 1);
  uint64_t workers = (threads == 1 || chunks == 1) ? 1 : std::min(threads, chunks);
  uint64_t n = 0;
  for (uint64_t c = worker; c < chunks && worker < workers; c += workers)
    if (n < cap) out_chunks[n++] = c; else ++n;
  return n;
}

}  // extern "C"
