/* puppygrad_b200 — C ABI of the B200 (sm_100a) GPT-2 inference path.
 *
 * This is the boundary a host program binds to (Rust `extern "C"`, ctypes, cgo …): opaque
 * handles, plain pointers and sizes, `int` status codes. Every entry point names the interface
 * of the reference (J45k4/puppygrad, paths relative to that project) that it stands in for.
 *
 * Conventions
 *  - Return value: a pg_status. On failure the message is available from
 *    pg_last_error_message() on the calling thread. The four reference error classes
 *    (src/models/gpt2/error.rs:4-21) map to PG_ASSET, PG_INVALID_CONFIG, PG_INVALID_INPUT,
 *    PG_INVALID_WEIGHTS; PG_CUDA and PG_TIMEOUT have no reference counterpart.
 *  - Host buffers are borrowed for the duration of the call only.
 *  - A pg_model is immutable after creation and may be shared between threads
 *    (reference: Gpt2Model is Clone over Arc<Gpt2Weights>, src/models/gpt2/rust.rs:142-148).
 *    A pg_cache has one user at a time (reference: `&mut Gpt2KvCache`).
 *  - There is no CPU fallback: every compute entry point needs a CUDA device of compute
 *    capability 10.0 and fails with PG_CUDA otherwise.
 *  - Token ids and positions are int32 at this boundary (vocab and context fit easily).
 *  - A cache holds `max_batch` independent sequences ("slots"). Batch entry points act on slots
 *    0..batch-1. With max_batch = 1 the calls reduce exactly to the reference's single-sequence
 *    traits (src/models/autoregressive.rs:1-31).
 */
#ifndef PUPPYGRAD_B200_H
#define PUPPYGRAD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pg_model pg_model;
typedef struct pg_cache pg_cache;
typedef struct pg_sampler pg_sampler;

typedef enum {
  PG_OK = 0,
  PG_ASSET = 1,           /* Gpt2Error::Asset          */
  PG_INVALID_CONFIG = 2,  /* Gpt2Error::InvalidConfig  */
  PG_INVALID_INPUT = 3,   /* Gpt2Error::InvalidInput   */
  PG_INVALID_WEIGHTS = 4, /* Gpt2Error::InvalidWeights */
  PG_CUDA = 5,            /* a CUDA runtime call or a kernel launch failed; no device */
  PG_TIMEOUT = 6          /* a bounded device-side wait gave up */
} pg_status;

/* Gpt2Config, src/models/gpt2/rust.rs:31-39 */
typedef struct {
  uint64_t vocab_size, n_positions, n_embd, n_layer, n_head, n_inner;
  float layer_norm_epsilon;
} pg_gpt2_config;

/* Arithmetic of the linears. The reference is FP32 only (src/models/safetensors.rs:126-130);
 * the other modes are extensions with their own stated error bounds. */
typedef enum {
  PG_MATH_FP32 = 0,   /* FP32 FMA everywhere */
  PG_MATH_TF32X3 = 1, /* FP32-grade products on the tensor cores as three TF32 MMAs over hi and lo parts of both
                         operands (x.w + x.w_lo + x_lo.w) with FP32 accumulation: the decode linears of 9..64
                         sequences and prefill GEMMs of at least 128 rows; passes the same token-exact and
                         1e-3 / 1e-4 logit tests as PG_MATH_FP32. Everything else as PG_MATH_FP32 */
  PG_MATH_TF32 = 2,   /* as TF32X3 for decode; prefill GEMMs of at least 128 rows and prefill attention
                         (head_dim 64) as single TF32 passes: a speed mode, bound 5e-3 of the logit span */
  PG_MATH_BF16 = 3    /* BF16 WEIGHTS, FP32 activations and sums: the four dense matrices of every block and the
                         tied embedding are rounded to BF16 (nearest even) at load; what the model computes is
                         the FP32 path of the reference on those rounded weights. Decode steps of at most 8
                         sequences stream the 2-byte copies; prefill and larger batches multiply the rounded
                         values as PG_MATH_TF32X3 does. No reference counterpart (it rejects every dtype but F32,
                         src/models/safetensors.rs:126-130) */
} pg_math_mode;

/* Stands where Gpt2BackendConfig::Rust(Gpt2RustConfig) stands in the reference
 * (src/models/gpt2/options.rs:15-18, 52-96): the knobs of this backend. Zero = default. */
typedef struct {
  int32_t device;       /* CUDA ordinal */
  int32_t math_mode;    /* pg_math_mode */
  int32_t page_tokens;  /* KV page size in tokens: 16, 32 or 64 (default 32) */
  int32_t use_graphs;   /* 0 = default (on), 1 = on, 2 = off: one CUDA graph per decode step */
  int32_t attn_splits;  /* split-K factor of decode attention, 0 = choose from the batch */
  int32_t persistent_step; /* decode steps of at most 8 sequences (head_dim 64, n_positions <= 1024) can run as ONE
                              persistent cooperative kernel whose weight stream runs ahead of the dependent
                              operations and whose CTAs exchange activations as tagged words instead of meeting
                              at grid barriers. 0 = where it measured faster than one kernel per operation in a
                              CUDA graph (up to 4 sequences with FP32 weights; always with BF16 / int8 weights,
                              which only that kernel reads), 1 = whenever the shapes allow, 2 = never */
  int32_t quantized_weights; /* Gpt2RustConfig::quantized_weights (src/models/gpt2/options.rs:62-104): 1 = the four
                                dense matrices of every block and the lm_head as row-wise int8 (QuantizedRows,
                                src/models/cpu.rs:26-56; quantize_weights, rust.rs:1354-1376); the embedding lookup
                                keeps FP32 rows as in the reference. Decode steps of at most 8 sequences stream the
                                1-byte copies; prefill and larger batches multiply the dequantised values q * scale */
  int32_t reserved[1];
} pg_backend_config;

/* TextGenerationConfig, src/models/generation.rs:60-85. None is encoded as a negative value. */
typedef struct {
  uint64_t max_new_tokens;
  int64_t eos_token_id; /* < 0 = None */
  float temperature;
  float top_p;          /* < 0 = None */
  int64_t top_k;        /* < 0 = None */
  uint64_t seed;
  float repeat_penalty;
  uint64_t repeat_last_n;
} pg_generation_config;

/* GenerationStats, src/models/generation.rs:129-180 (times in seconds) */
typedef struct {
  uint64_t prompt_tokens, generated_tokens;
  double tokenize_time, prefill_time, decode_time, total_generation_time;
  double first_token_time; /* < 0 = None */
} pg_generation_stats;

/* Gpt2OperationProfile, src/models/gpt2/rust.rs:336-347: seconds per operation class of one
 * decode step, from CUDA events around every kernel. A LayerNorm fused into the linear that
 * consumes it is counted in that linear's bucket (layer_norm is then 0); tokenization and decoding
 * are text-side and always 0 here; `other` holds the embedding and the end-of-step kernel, which
 * the reference leaves untimed. launches[i] counts kernels in the order layer_norm, qkv_projection,
 * attention, attention_projection, mlp_fc_projection, mlp_projection, final_logits, other.
 * When the step runs as one persistent kernel (batched tensor-core path), fused_step_kernel is
 * that launch's duration from CUDA events, the buckets hold the durations of its phases from
 * time stamps the kernel writes itself (bias / residual / LayerNorm phases count as layer_norm, a
 * GEMM's reduce phase counts with the GEMM), launches[i] counts phases, and `other` keeps what the
 * stamps do not cover. No reference counterpart for the two fused_* fields. */
typedef struct {
  double tokenization, layer_norm, qkv_projection, attention, attention_projection, mlp_fc_projection,
      mlp_projection, final_logits, decoding, other;
  uint64_t launches[8];
  double fused_step_kernel;
  uint64_t fused_phases;
} pg_operation_profile;

/* Number of tensors pg_model_from_host_weights expects: 4 + 12 * n_layer. */
#define PG_TENSORS_PER_LAYER 12
#define PG_GLOBAL_TENSORS 4

/* ------------------------------------------------------------------ errors, library */
/* Display text of the last error on this thread ("" if none); valid until the next failing call
 * on the same thread. Reference: the String inside each Gpt2Error variant. */
const char* pg_last_error_message(void);
/* Library version string. No reference counterpart. */
const char* pg_version(void);
/* Number of usable CUDA devices (0 without a driver). No reference counterpart. */
int pg_device_count(void);

/* ------------------------------------------------------------------ configuration */
/* Gpt2Config::validate, src/models/gpt2/rust.rs:59-94 */
int pg_config_validate(const pg_gpt2_config* cfg);
/* load_config, src/models/gpt2/rust.rs:684-711: reads vocab_size, n_positions|n_ctx, n_embd,
 * n_layer, n_head, optional n_inner (default 4*n_embd) and layer_norm_epsilon (default 1e-5). */
int pg_config_load_json(const char* path, pg_gpt2_config* out);
/* TextGenerationConfig::new / validate, src/models/generation.rs:73-116 */
void pg_generation_config_default(uint64_t max_new_tokens, pg_generation_config* out);
int pg_generation_config_validate(const pg_generation_config* cfg);
void pg_backend_config_default(pg_backend_config* out);

/* ------------------------------------------------------------------ model */
/* Gpt2Runtime::from_dir_with_backend minus the tokenizer (src/models/gpt2/rust.rs:382-396):
 * reads <dir>/config.json and <dir>/model.safetensors (load_weights, rust.rs:713-772: HF key
 * names, optional "transformer." prefix, F32 only, shapes checked), uploads to the device. */
int pg_model_load_dir(const char* dir, const pg_backend_config* backend, pg_model** out);
/* Gpt2Model::new_with_rust_config, src/models/gpt2/rust.rs:803-825. `tensors` holds
 * 4 + 12*n_layer host pointers in the order
 *   wte, wpe, ln_f.weight, ln_f.bias, then for each layer
 *   ln_1.weight, ln_1.bias, attn.c_attn.weight, attn.c_attn.bias, attn.c_proj.weight,
 *   attn.c_proj.bias, ln_2.weight, ln_2.bias, mlp.c_fc.weight, mlp.c_fc.bias,
 *   mlp.c_proj.weight, mlp.c_proj.bias
 * with the dense matrices in the Hugging Face [in, out] layout (they are transposed to
 * [out, in] on the device, as transpose_dense_weights does, rust.rs:1345-1352). `lens` are
 * element counts, checked like validate_weights (rust.rs:1279-1343). */
int pg_model_from_host_weights(const pg_gpt2_config* cfg, const float* const* tensors,
                               const uint64_t* lens, uint64_t n_tensors,
                               const pg_backend_config* backend, pg_model** out);
/* Gpt2Model.config */
int pg_model_config(const pg_model* model, pg_gpt2_config* out);
/* AutoregressiveDecoder::max_context_len, src/models/gpt2/rust.rs:1258-1260 */
uint64_t pg_model_max_context_len(const pg_model* model);
/* Bytes of weights one decode step streams from HBM (for roofline arithmetic). No counterpart. */
uint64_t pg_model_weight_bytes_per_step(const pg_model* model);
/* Drop of Gpt2Model */
void pg_model_free(pg_model* model);

/* ------------------------------------------------------------------ KV cache */
/* Gpt2Model::new_kv_cache / Gpt2KvCache::new, src/models/gpt2/rust.rs:186-200, 902-904.
 * One paged, device-resident pool per layer shared by `max_batch` slots. */
int pg_cache_new(const pg_model* model, int32_t max_batch, pg_cache** out);
/* KvCache::clear, rust.rs:202-204, for every slot / for one slot */
int pg_cache_clear(pg_cache* cache);
int pg_cache_clear_slot(pg_cache* cache, int32_t slot);
/* KvCache::seq_len / max_seq_len, rust.rs:237-249 */
int pg_cache_seq_len(const pg_cache* cache, int32_t slot, uint64_t* out);
uint64_t pg_cache_max_seq_len(const pg_cache* cache);
int32_t pg_cache_max_batch(const pg_cache* cache);
/* Copies one slot's keys and values of one layer to the host in the reference layout
 * [head][max_seq_len][head_dim] (kv_index, rust.rs:1851-1855); positions >= seq_len read 0. */
int pg_cache_read_layer(const pg_cache* cache, int32_t slot, uint64_t layer, float* keys,
                        float* values);
/* Drop of Gpt2KvCache */
void pg_cache_free(pg_cache* cache);

/* ------------------------------------------------------------------ forward passes */
/* Gpt2Model::prefill, src/models/gpt2/rust.rs:906-927, for `batch` sequences at once: clears
 * slots 0..batch-1, runs the prompts (ids concatenated, lens[b] tokens each) and leaves
 * seq_len[b] = lens[b]. logits_out (batch * vocab_size floats) and argmax_out (batch) are
 * optional (NULL to skip); they hold the last position of each prompt. */
int pg_prefill(const pg_model* model, pg_cache* cache, const int32_t* ids, const int32_t* lens,
               int32_t batch, float* logits_out, int32_t* argmax_out);
/* Gpt2Model::forward_one, src/models/gpt2/rust.rs:929-1006, for slots 0..batch-1: appends
 * ids[b] to slot b. Optional outputs: logits_out (batch * vocab_size), argmax_out (batch; the
 * rule of argmax_logits, src/models/generation.rs:269-279: first strict maximum), and the k
 * largest logits of each row in descending order, ties by lower index first, as the stable sort
 * of sample_logits orders them (generation.rs:315-318): topk_vals / topk_idx (batch * k). */
int pg_forward_one(const pg_model* model, pg_cache* cache, const int32_t* ids, int32_t batch,
                   float* logits_out, int32_t* argmax_out, float* topk_vals, int32_t* topk_idx,
                   int32_t k);
/* Gpt2Model::forward, src/models/gpt2/rust.rs:831-882: logits for every position of one
 * sequence, no cache. logits_out holds t * vocab_size floats. */
int pg_forward(const pg_model* model, const int32_t* ids, int32_t t, float* logits_out);

/* Greedy decode with every step's token fed back on the device (no host round trip per step):
 * runs `steps` forward_one calls on slots 0..batch-1 starting from first_ids, each next id being
 * the argmax of the step before. tokens_out (steps * batch, step-major) receives the argmax of
 * each step. Equivalent to the loop of autoregressive::generate (src/models/autoregressive.rs:
 * 61-87) with select_next_token = argmax_logits. */
int pg_decode_greedy(const pg_model* model, pg_cache* cache, const int32_t* first_ids,
                     int32_t batch, int32_t steps, int32_t* tokens_out);

/* forward_one_profiled, src/models/gpt2/rust.rs:933-941: one decode step for slots 0..batch-1 run
 * kernel by kernel (no graph, no overlap) with its device time split into the reference's
 * operation buckets. Advances the cache like pg_forward_one. */
int pg_profile_forward_one(const pg_model* model, pg_cache* cache, const int32_t* ids, int32_t batch,
                           pg_operation_profile* out);
/* Device-side stopwatch on the cache's own stream (where every kernel of this cache runs):
 * begin drains the stream and records an event; end records a second event, waits for it and
 * returns the elapsed seconds. The reference times with Instant::now() around the same calls
 * (src/models/gpt2/rust.rs:470-531). */
int pg_cache_time_begin(pg_cache* cache);
int pg_cache_time_end(pg_cache* cache, double* seconds);
/* Kernels launched so far by decode steps on this cache. No reference counterpart. */
uint64_t pg_cache_kernel_launches(const pg_cache* cache);
/* Test hook, no reference counterpart: makes one bounded wait of the NEXT decode step on this cache
 * run out by its limit. The step's persistent kernel is launched with `spin_limit` polls per wait
 * (a few thousand: microseconds) and is made to wait for a hand-over that never comes; every CTA
 * gives up at the limit, records the error and ends, and the call that ran the step returns
 * PG_TIMEOUT. Nothing faults and nothing waits without a limit. After a PG_TIMEOUT the cache's
 * device-side synchronisation state is re-initialised by the library, but the sequences in it are
 * undefined: clear the cache (or prefill again) before the next use. */
int pg_cache_debug_expire_next_wait(pg_cache* cache, uint32_t spin_limit);

/* One linear on host buffers, out[m, n] = x[m, k] . w[n, k]^T (+ bias[n]) then epilogue
 * (0 none, 1 tanh-GELU, 2 out = resid + value): transposed_dense_projection_into,
 * src/models/cpu.rs:58-75, with gelu_in_place / add_in_place (cpu.rs:145-171) fused. `w` is
 * already [out, in]. math_mode selects the kernel family (pg_math_mode; the tensor-core modes need
 * k % 32 == 0; tf32x3 runs the decode kernel up to 64 rows and the prefill kernel above). With reps > 0 the kernel is launched reps more times,
 * L2 flushed before each, and *seconds_per_launch receives the mean device time. */
int pg_op_linear(const float* x, const float* w, const float* bias, const float* resid, int32_t m,
                 int32_t n, int32_t k, int32_t epilogue, int32_t math_mode, int32_t device,
                 int32_t reps, float* out, double* seconds_per_launch);
/* Attention of one new token per sequence over cached keys and values, on host buffers:
 * cached_self_attention_into, src/models/gpt2/rust.rs:1662-1741. qkv is [batch][3 * n_head *
 * head_dim] (q, k, v of the new token); keys / values are [batch][n_head][kv_len][head_dim], the
 * kv_len positions already cached (the reference's per-head layout, kv_index, rust.rs:1851-1855,
 * without the unused tail). out is [batch][n_head * head_dim]. The cache is laid out in pages of
 * `page_tokens` with a permuted page table; `splits` is the split-K factor (head_dim 64 only).
 * Timing as in pg_op_linear. */
int pg_op_decode_attention(const float* qkv, const float* keys, const float* values, int32_t batch,
                           int32_t n_head, int32_t head_dim, int32_t kv_len, int32_t page_tokens,
                           int32_t splits, int32_t device, int32_t reps, float* out,
                           double* seconds_per_launch);
/* LayerNorm of `rows` rows of `cols` values on host buffers: layer_norm_in_place, src/models/cpu.rs:119-143
 * (mean, biased variance of the centred values, (v - mean) / sqrt(var + eps) * gamma + beta). Timing as in
 * pg_op_linear. */
int pg_op_layernorm(const float* x, const float* gamma, const float* beta, float eps, int32_t rows, int32_t cols,
                    int32_t device, int32_t reps, float* out, double* seconds_per_launch);
/* The end of a decode step on host buffers: logits[m, vocab] = hidden[m, k] . wte[vocab, k]^T without bias
 * (logits_from_hidden_into, src/models/gpt2/rust.rs:1767-1813) with the row arg-max fused into the same pass
 * (argmax_logits, src/models/generation.rs:269-279: first strict maximum, NaN never wins). 1 <= m <= 8.
 * logits_out may be NULL. Timing as in pg_op_linear (both launches of the operator are inside the timed region). */
int pg_op_lm_head_argmax(const float* hidden, const float* wte, int32_t m, int32_t vocab, int32_t k, int32_t device,
                         int32_t reps, float* logits_out, int32_t* argmax_out, double* seconds_per_launch);
/* Row-wise symmetric int8 quantisation of a [rows, cols] FP32 matrix on the device:
 * QuantizedRows::from_f32, src/models/cpu.rs:33-57 (scale = max|w| / 127, 1 for an all-zero row;
 * q = clamp(round(w / scale), -127, 127)). q_out is [rows, cols] int8, scales_out [rows]. The bytes
 * and scales equal the reference's. */
int pg_op_quantize_rows(const float* w, int32_t rows, int32_t cols, int32_t device, int8_t* q_out,
                        float* scales_out);
/* out[m, n] = x[m, k] . dequant(q[n, k])^T + bias over int8 weights with one scale per output row:
 * quantized_transposed_dense_projection_into + quantized_dot, src/models/cpu.rs:99-117, 173-184
 * (the --quantized-weights variant of the four linears and of the lm_head,
 * src/models/gpt2/rust.rs:1535-1578, 1815-1849). Decode-sized: m <= 8, k % 16 == 0; bias may be
 * NULL (the lm_head has none). Timing as in pg_op_linear. */
int pg_op_linear_q8(const float* x, const int8_t* q, const float* scales, const float* bias, int32_t m,
                    int32_t n, int32_t k, int32_t device, int32_t reps, float* out,
                    double* seconds_per_launch);
/* No counterpart in the reference (its CPU path owns no device memory at all). The same decode
 * attention kernel as above for callers that must not allocate when they call it — a server
 * whose own pool already owns all of HBM, a plugin invoked where its embedder forbids cudaMalloc,
 * a latency-critical loop that wants no allocator call: this entry point calls no cudaMalloc,
 * cudaFree or any allocating library routine. All pointers are DEVICE pointers owned by the
 * caller: d_qkv [batch][3 * n_head * head_dim]; d_out [batch][n_head * head_dim]; d_kv_pool, one
 * layer's pages laid out [page][2 (K, V)][n_head][page_tokens][head_dim]; d_page_table
 * [batch][pages_per_seq] physical page of each logical page; d_pos [batch], the position of the
 * new token (= positions already cached). The kernel appends the new K, V at d_pos and writes
 * d_out; it is enqueued on `stream` (a cudaStream_t, NULL = the default stream) and not waited
 * for. The split-K partials live in an array inside the library image (4.1 MiB per GPU that loads
 * the library, held until exit), which bounds the sizes: batch * n_head <= 2048 and splits <= 8;
 * larger requests fail with PG_INVALID_INPUT. The first call on a device looks up that array's
 * address for the device and sets kernel attributes; make that first call before any stream
 * capture begins. Every call shares the one array: two calls whose kernels overlap on the GPU
 * (different streams, different threads) race on it, so keep calls on one device ordered.
 * Preconditions the host cannot check: every d_pos[b] < pages_per_seq * page_tokens (the page-table row is
 * indexed by it) and every page number in d_page_table lies inside d_kv_pool. `device` is current only for
 * the duration of the call; the calling thread's current device is restored before it returns. */
int pg_decode_attention_noalloc(const float* d_qkv, float* d_out, float* d_kv_pool,
                                const int32_t* d_page_table, const int32_t* d_pos, int32_t batch,
                                int32_t n_head, int32_t head_dim, int32_t page_tokens,
                                int32_t pages_per_seq, int32_t splits, int32_t device, void* stream);

/* ------------------------------------------------------------------ generation loops */
/* non-zero return aborts generation (the closure returning Err in the reference) */
typedef int (*pg_token_callback)(uint64_t token_id, void* user);
/* Gpt2Model::generate_greedy, rust.rs:884-900 (uncached: re-runs the full forward per token).
 * out_tokens has room for n_ids + max_new_tokens entries. */
int pg_generate_greedy(const pg_model* model, const int32_t* ids, int32_t n_ids,
                       uint64_t max_new_tokens, int32_t* out_tokens, uint64_t* out_len);
/* Gpt2Model::generate_greedy_cached / stream_greedy_tokens, rust.rs:1008-1027, i.e.
 * autoregressive::generate, src/models/autoregressive.rs:61-87. */
int pg_stream_greedy_tokens(const pg_model* model, const int32_t* ids, int32_t n_ids,
                            uint64_t max_new_tokens, pg_token_callback on_token, void* user,
                            int32_t* out_tokens, uint64_t* out_len);
/* Gpt2Runtime::stream_token_ids_with_stats without the tokenizer, rust.rs:548-635: prefill, then
 * per token: sampler (repeat penalty, greedy or temperature/top-k/top-p), EOS stop, callback,
 * forward_one unless it was the last token. out_tokens receives only the generated ids
 * (room for cfg->max_new_tokens). stats may be NULL. */
int pg_generate_with_config(const pg_model* model, const int32_t* ids, int32_t n_ids,
                            const pg_generation_config* cfg, pg_token_callback on_token, void* user,
                            int32_t* out_tokens, uint64_t* out_len, pg_generation_stats* stats);

/* ------------------------------------------------------------------ text streaming and statistics (host side) */
/* TokenDecoder::decode_tokens, src/models/streaming.rs:1-9, as a callback: writes the UTF-8 text of the `n` token
 * ids into out[0..cap) and the length it needs into *out_len (when that exceeds cap the library calls again with a
 * larger buffer); non-zero return = the decoder's error. The tokenizer itself stays with the caller
 * (Gpt2Tokenizer, rust.rs:270-302, wraps the `tokenizers` crate and a tokenizer.json). */
typedef int (*pg_decode_tokens_fn)(const uint64_t* token_ids, size_t n, char* out, size_t cap, size_t* out_len,
                                   void* user);
/* the `on_text` closure of stream_token; non-zero return aborts */
typedef int (*pg_text_callback)(const char* text, size_t len, void* user);
typedef struct pg_text_streamer pg_text_streamer;
/* IncrementalTextStreamer::new / decoded / stream_token, src/models/streaming.rs:32-74: emits the token's own text
 * when it is safe to (not empty, no U+FFFD), otherwise decodes all output ids and emits what was added. */
int pg_text_streamer_new(const char* decoded, size_t len, pg_text_streamer** out);
void pg_text_streamer_free(pg_text_streamer* streamer);
int pg_text_streamer_decoded(const pg_text_streamer* streamer, const char** text, size_t* len);
int pg_text_streamer_stream_token(pg_text_streamer* streamer, pg_decode_tokens_fn decoder, void* decoder_user,
                                  const uint64_t* output_ids, size_t n_ids, uint64_t token_id,
                                  pg_text_callback on_text, void* text_user);
/* is_incremental_decode_safe, streaming.rs:76-78 (1 = safe) */
int pg_is_incremental_decode_safe(const char* text, size_t len);
/* escape_raw_token, streaming.rs:17-30 (the --stream-raw-tokens output): *out_len receives the escaped length;
 * the text is written when it fits cap. */
int pg_escape_raw_token(const char* token, size_t len, char* out, size_t cap, size_t* out_len);
/* GenerationStats::{total_model_tokens, prefill_/decode_/total_tokens_per_second, average_decode_token_time},
 * src/models/generation.rs:140-181; the last returns seconds, < 0 = None. */
uint64_t pg_generation_stats_total_model_tokens(const pg_generation_stats* stats);
double pg_generation_stats_prefill_tokens_per_second(const pg_generation_stats* stats);
double pg_generation_stats_decode_tokens_per_second(const pg_generation_stats* stats);
double pg_generation_stats_total_tokens_per_second(const pg_generation_stats* stats);
double pg_generation_stats_average_decode_token_time(const pg_generation_stats* stats);

/* ------------------------------------------------------------------ sampling (host side) */
/* argmax_logits, src/models/generation.rs:269-279 */
uint64_t pg_argmax_logits(const float* logits, size_t n);
/* LogitsSampler::new / select_next_token, src/models/generation.rs:209-241 */
int pg_sampler_new(uint64_t seed, pg_sampler** out);
void pg_sampler_free(pg_sampler* sampler);
int pg_sampler_select_next_token(pg_sampler* sampler, const float* logits, size_t n,
                                 const uint64_t* history, size_t n_history,
                                 const pg_generation_config* cfg, uint64_t* out_token);
/* The same draw from a pre-sorted top-k list (values descending, ties by lower index) as
 * produced by pg_forward_one: valid when cfg->top_k is set, k >= top_k, and repeat penalty is
 * off. Consumes exactly one RNG draw like sample_logits (generation.rs:300-362). */
int pg_sampler_select_from_topk(pg_sampler* sampler, const float* topk_vals,
                                const int32_t* topk_idx, size_t k,
                                const pg_generation_config* cfg, uint64_t* out_token);
/* The same for a batch in one call: sampler i draws from row i of the [batch, k] top-k arrays that
 * pg_forward_one filled; out_tokens[i] receives its token. One RNG draw per sampler, as `batch` calls of
 * pg_sampler_select_from_topk in order (a serving loop pays one foreign call per step instead of one per
 * sequence). No reference counterpart: the reference samples one sequence at a time. */
int pg_sampler_select_from_topk_batch(pg_sampler* const* samplers, const float* topk_vals, const int32_t* topk_idx,
                                      size_t batch, size_t k, const pg_generation_config* cfg, uint64_t* out_tokens);

#ifdef __cplusplus
}
#endif
#endif /* PUPPYGRAD_B200_H */
