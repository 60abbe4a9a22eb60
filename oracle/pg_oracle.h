/* CPU oracle for the GPT-2 inference path: C ABI for ctypes.
 *
 * TEST INFRASTRUCTURE ONLY. This is a restatement, in C++17, of the reference's
 * CPU algorithm (puppygrad: src/models/cpu.rs, src/models/gpt2/rust.rs,
 * src/models/generation.rs, src/models/autoregressive.rs,
 * src/runtime/thread_pool.rs). The product library never links, loads or calls it;
 * only the tests, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Pinning status: the reference is Rust and no Rust toolchain exists where this is
 * built, so it cannot be executed beside this file, and its GPT-2 tests store no
 * numeric vectors. The oracle is pinned against every known-answer and relation test
 * the reference holds for this path (tests/test_oracle_reference_tests.py) and against
 * an independent float64 restatement; absolute logits are therefore "parity unpinned"
 * with respect to the reference binary itself.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct po_model po_model;
typedef struct po_cache po_cache;
typedef struct po_sampler po_sampler;

/* src/models/gpt2/rust.rs:31-39 */
typedef struct {
  uint64_t vocab_size, n_positions, n_embd, n_layer, n_head, n_inner;
  float layer_norm_epsilon;
} po_config;

/* src/models/gpt2/options.rs:52-96 (defaults 1, 262144, 48, 64, 128, 64, 256, 4096) */
typedef struct {
  uint64_t threads, dense_parallel_threshold, qkv_chunk_size, attention_projection_chunk_size,
      mlp_fc_chunk_size, mlp_projection_chunk_size, logits_chunk_size,
      attention_head_parallel_threshold;
} po_rust_config;

/* src/models/generation.rs:60-85 */
typedef struct {
  uint64_t max_new_tokens;
  int64_t eos_token_id; /* -1 = None */
  float temperature;
  float top_p;   /* < 0 = None */
  int64_t top_k; /* < 0 = None */
  uint64_t seed;
  float repeat_penalty;
  uint64_t repeat_last_n;
} po_generation_config;

enum { PO_OK = 0, PO_ASSET = 1, PO_INVALID_CONFIG = 2, PO_INVALID_INPUT = 3, PO_INVALID_WEIGHTS = 4 };

const char* po_last_error(void);
void po_default_rust_config(po_rust_config* out);

/* ---- src/models/cpu.rs kernels ---- */
float po_dot(const float* a, const float* b, size_t n);        /* cpu.rs:186-254 (AVX path) */
float po_dot_scalar(const float* a, const float* b, size_t n); /* cpu.rs:206-208 */
void po_transposed_dense_projection(const float* x, size_t rows, size_t in_f, size_t out_f,
                                    const float* w, const float* bias, float* out); /* cpu.rs:58-75 */
void po_dense_projection(const float* x, size_t rows, size_t in_f, size_t out_f, const float* w,
                         const float* bias, float* out);                            /* cpu.rs:77-97 */
void po_quantize_rows(const float* w, size_t rows, size_t cols, int8_t* q, float* scales);  /* cpu.rs:33-57 */
void po_quantized_projection(const float* x, size_t rows, size_t in_f, size_t out_f, const int8_t* q,
                             const float* scales, const float* bias, float* out);    /* cpu.rs:99-117, 173-184 */
void po_layer_norm_in_place(float* x, size_t rows, size_t cols, const float* gamma,
                            const float* beta, float eps);                          /* cpu.rs:119-143 */
void po_gelu_in_place(float* v, size_t n);                                          /* cpu.rs:145-150 */
void po_softmax_in_place(float* v, size_t n);                                       /* cpu.rs:152-165 */
void po_add_in_place(float* dst, const float* src, size_t n);                       /* cpu.rs:167-171 */
void po_transpose_in_out(const float* w, size_t in_f, size_t out_f, float* out);    /* cpu.rs:281-289 */

/* ---- model (rust.rs:798-1027) ----
 * tensors: 4 + 12*n_layer pointers, HF [in,out] layout for the four dense matrices:
 *   wte, wpe, ln_f.weight, ln_f.bias, then per layer
 *   ln_1.weight, ln_1.bias, c_attn.weight, c_attn.bias, attn.c_proj.weight, attn.c_proj.bias,
 *   ln_2.weight, ln_2.bias, c_fc.weight, c_fc.bias, mlp.c_proj.weight, mlp.c_proj.bias
 * lens: element count of each. */
int po_model_new(const po_config* cfg, const float* const* tensors, const uint64_t* lens,
                 uint64_t n_tensors, const po_rust_config* rc, po_model** out);
void po_model_free(po_model* m);
/* Gpt2RustConfig::quantized_weights = true (options.rs:62-104; quantize_weights, rust.rs:1354-1376;
 * quantized_linear_into, rust.rs:1535-1578; quantized_logits_from_hidden_into, rust.rs:1815-1849) */
void po_model_quantize_weights(po_model* m);
int po_config_validate(const po_config* cfg);

int po_cache_new(const po_model* m, po_cache** out); /* rust.rs:186-200 */
void po_cache_free(po_cache* c);
uint64_t po_cache_seq_len(const po_cache* c);
uint64_t po_cache_max_seq_len(const po_cache* c);
void po_cache_clear(po_cache* c);
void po_cache_set_seq_len(po_cache* c, uint64_t n); /* tests only (rust.rs:1958) */
/* copy keys/values of one layer, layout [head][max_seq_len][head_dim] (rust.rs:1851-1855) */
int po_cache_read_layer(const po_cache* c, uint64_t layer, float* keys, float* values);

int po_forward(const po_model* m, const uint64_t* ids, uint64_t t, float* logits /* t*V */);      /* rust.rs:831-882 */
int po_prefill(const po_model* m, const uint64_t* ids, uint64_t t, po_cache* c, float* logits);  /* rust.rs:906-927 */
int po_forward_one(const po_model* m, uint64_t token, po_cache* c, float* logits);               /* rust.rs:929-1006 */
/* out_tokens has room for t + max_new; *out_len receives the final length */
int po_generate_greedy(const po_model* m, const uint64_t* ids, uint64_t t, uint64_t max_new,
                       uint64_t* out_tokens, uint64_t* out_len); /* rust.rs:884-900 */
typedef int (*po_token_cb)(uint64_t token, void* user); /* non-zero aborts */
int po_generate_greedy_cached(const po_model* m, const uint64_t* ids, uint64_t t, uint64_t max_new,
                              po_token_cb cb, void* user, uint64_t* out_tokens,
                              uint64_t* out_len); /* rust.rs:1008-1027, autoregressive.rs:61-87 */

/* Same arithmetic per element as po_forward_one, for `b` independent sequences at once; the
 * weight row is reused across sequences (loop order only). Used to produce golden streams. */
int po_forward_one_batch(const po_model* m, const uint64_t* tokens, po_cache* const* caches,
                         uint64_t b, float* logits /* b*V, or NULL */, uint64_t* argmax /* b, or NULL */);

/* ---- sampling (generation.rs:209-362) ---- */
uint64_t po_argmax_logits(const float* v, size_t n); /* generation.rs:269-279 */
int po_generation_config_validate(const po_generation_config* g);
void po_default_generation_config(uint64_t max_new_tokens, po_generation_config* out);
po_sampler* po_sampler_new(uint64_t seed);
void po_sampler_free(po_sampler* s);
uint64_t po_sampler_next_u64(po_sampler* s); /* generation.rs:255-261 */
int po_sampler_select_next_token(po_sampler* s, const float* logits, size_t n,
                                 const uint64_t* history, size_t n_hist,
                                 const po_generation_config* g, uint64_t* out);

/* ---- thread pool (thread_pool.rs:107-170): chunk ids in the order worker `w` runs them ---- */
uint64_t po_pool_worker_chunks(uint64_t threads, uint64_t len, uint64_t chunk_size, uint64_t worker,
                               uint64_t* out_chunks, uint64_t cap);

#ifdef __cplusplus
}
#endif
