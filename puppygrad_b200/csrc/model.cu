// Host runtime of the GPT-2 path: device weights, the paged KV cache, the decode-step CUDA graph,
// batched prefill, and the C ABI entry points that drive them.
//
// Mirrors, for a CUDA device, what Gpt2Model / Gpt2KvCache do on the CPU in the reference
// (src/models/gpt2/rust.rs:142-267, 798-1027). There is no CPU compute path in this file: without
// a device every compute entry point returns PG_CUDA.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <numeric>

#include "common.h"
#include "kernels.cuh"
#include "sampler.h"

namespace pg {

#define PG_CUDA_TRY(expr)                                                                      \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return set_error(PG_CUDA, std::string("CUDA error: ") + cudaGetErrorString(_e) + " at " + \
                                    __FILE__ + ":" + std::to_string(__LINE__) + " (" #expr ")"); \
  } while (0)

struct LayerWeights {
  float *ln1_g, *ln1_b, *w_qkv, *b_qkv, *w_proj, *b_proj, *ln2_g, *ln2_b, *w_fc, *b_fc, *w_proj2, *b_proj2;
  // copies in the tiled layout of the tensor-core decode kernel (nullptr in fp32 mode)
  float *t_qkv = nullptr, *t_proj = nullptr, *t_fc = nullptr, *t_proj2 = nullptr;
  // lo parts (w - hi(w), hi = the upper 19 bits a TF32 tensor core reads) of the four matrices, [out, in] row-major:
  // second operand of the FP32-grade prefill GEMM (nullptr in fp32 mode)
  float *l_qkv = nullptr, *l_proj = nullptr, *l_fc = nullptr, *l_proj2 = nullptr;
  // packed copies for the single-kernel decode step (BF16 or row-quantised int8 weights), [out, in] rows, and,
  // for int8, one scale per output row
  void *p_qkv = nullptr, *p_proj = nullptr, *p_fc = nullptr, *p_proj2 = nullptr;
  float *s_qkv = nullptr, *s_proj = nullptr, *s_fc = nullptr, *s_proj2 = nullptr;
};

static bool env_flag(const char* name) {
  const char* v = getenv(name);
  return v && *v && strcmp(v, "0") != 0;
}

}  // namespace pg

using namespace pg;

// ------------------------------------------------------------------ model
struct pg_model {
  pg_gpt2_config cfg{};
  pg_backend_config backend{};
  int device = 0;
  int num_sms = 148;
  float* arena = nullptr;  // every weight tensor lives in this one allocation
  float* tiled_arena = nullptr;  // second copy of the dense matrices, tiled for TMA (tensor-core modes)
  size_t tiled_floats = 0;
  float* t_wte = nullptr;
  float* lo_arena = nullptr;
  size_t arena_floats = 0;
  int stream_weight_type = STREAM_W_F32;  // what the single-kernel decode step streams
  unsigned char* packed_arena = nullptr;  // BF16 / int8 copies of the dense matrices and of wte
  float* scale_arena = nullptr;           // int8: row scales
  void* p_wte = nullptr;
  float* s_wte = nullptr;
  float* head_w = nullptr;      // FP32 rows of the lm_head: wte itself, or (int8) its dequantised copy
  float* head_deq = nullptr;    // owned storage of that copy
  float *wte = nullptr, *wpe = nullptr, *lnf_g = nullptr, *lnf_b = nullptr;
  std::vector<LayerWeights> layers;
  bool fused_ok = false;  // LayerNorm/argmax fusion needs n_embd % 4 == 0 and n_embd <= 2048
  bool use_pdl = true;

  int c() const { return (int)cfg.n_embd; }
  int f() const { return (int)cfg.n_inner; }
  int v() const { return (int)cfg.vocab_size; }
  int heads() const { return (int)cfg.n_head; }
  int head_dim() const { return (int)(cfg.n_embd / cfg.n_head); }
  int layers_n() const { return (int)cfg.n_layer; }
  int positions() const { return (int)cfg.n_positions; }

  ~pg_model() {
    if (arena) {
      cudaSetDevice(device);
      cudaFree(arena);
      if (tiled_arena) cudaFree(tiled_arena);
      if (lo_arena) cudaFree(lo_arena);
      if (packed_arena) cudaFree(packed_arena);
      if (scale_arena) cudaFree(scale_arena);
      if (head_deq) cudaFree(head_deq);
    }
  }
};

namespace pg {

static std::mutex g_init_mu;
static std::map<int, bool> g_device_inited;

int ensure_device(int device) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return set_error(PG_CUDA, std::string("no CUDA device available: ") +
                                  (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
  }
  if (device < 0 || device >= count)
    return set_error(PG_CUDA, "CUDA device " + std::to_string(device) + " out of range (" + std::to_string(count) + " present)");
  PG_CUDA_TRY(cudaSetDevice(device));
  std::lock_guard<std::mutex> g(g_init_mu);
  if (!g_device_inited[device]) {
    cudaDeviceProp prop;
    PG_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
      return set_error(PG_CUDA, "device " + std::to_string(device) + " (" + prop.name + ") has compute capability " +
                                    std::to_string(prop.major) + "." + std::to_string(prop.minor) +
                                    "; this library is built for sm_100a only");
    PG_CUDA_TRY(init_kernel_attributes());
    PG_CUDA_TRY(init_tc_kernel_attributes());
    PG_CUDA_TRY(init_attn_tc_attributes());
    g_device_inited[device] = true;
  }
  return PG_OK;
}

static size_t align_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

static int build_model(const pg_gpt2_config& cfg, const float* const* tensors, const uint64_t* lens, uint64_t n,
                       const pg_backend_config* backend, pg_model** out) {
  if (int r = validate_config(cfg)) return r;
  if (int r = validate_weight_lens(cfg, lens, n)) return r;
  pg_backend_config be{};
  if (backend) be = *backend;
  if (be.page_tokens == 0) be.page_tokens = 32;
  if (be.page_tokens != 16 && be.page_tokens != 32 && be.page_tokens != 64)
    return set_error(PG_INVALID_CONFIG, "cuda page_tokens must be 16, 32 or 64");
  if (be.math_mode < PG_MATH_FP32 || be.math_mode > PG_MATH_BF16)
    return set_error(PG_INVALID_CONFIG, "cuda math_mode must be one of fp32, tf32x3, tf32, bf16");
  if (be.quantized_weights < 0 || be.quantized_weights > 1)
    return set_error(PG_INVALID_CONFIG, "cuda quantized_weights must be 0 or 1");
  if (be.math_mode == PG_MATH_BF16 && be.quantized_weights)
    return set_error(PG_INVALID_CONFIG, "cuda math_mode bf16 and quantized_weights exclude each other");
  if (be.attn_splits < 0 || be.attn_splits > 16)
    return set_error(PG_INVALID_CONFIG, "cuda attn_splits must be in 0..16");
  if (cfg.vocab_size > 0x7fffffffULL || cfg.n_positions > 65536 || cfg.n_embd > 65536 || cfg.n_inner > 262144)
    return set_error(PG_INVALID_CONFIG, "config dimensions exceed what this backend indexes with 32 bits");
  if (int r = ensure_device(be.device)) return r;

  auto m = std::make_unique<pg_model>();
  m->cfg = cfg;
  m->backend = be;
  m->device = be.device;
  PG_CUDA_TRY(cudaDeviceGetAttribute(&m->num_sms, cudaDevAttrMultiProcessorCount, be.device));
  m->fused_ok = (cfg.n_embd % 4 == 0) && cfg.n_embd <= 2048;
  m->use_pdl = !env_flag("PG_NO_PDL");

  // one arena, every tensor 256-byte aligned
  size_t total = 0;
  std::vector<size_t> offs(n);
  size_t max_dense = 0;
  for (uint64_t i = 0; i < n; ++i) {
    offs[i] = total;
    total += align_up(lens[i], 64);
  }
  for (uint64_t l = 0; l < cfg.n_layer; ++l)
    for (int k : {2, 4, 8, 10}) max_dense = std::max<size_t>(max_dense, lens[4 + 12 * l + k]);
  PG_CUDA_TRY(cudaMalloc(&m->arena, total * sizeof(float)));
  m->arena_floats = total;
  float* staging = nullptr;
  PG_CUDA_TRY(cudaMalloc(&staging, max_dense * sizeof(float)));
  auto dev = [&](uint64_t i) { return m->arena + offs[i]; };
  int rc = PG_OK;
  auto upload = [&](uint64_t i) -> int {
    PG_CUDA_TRY(cudaMemcpy(dev(i), tensors[i], lens[i] * sizeof(float), cudaMemcpyHostToDevice));
    return PG_OK;
  };
  // HF Conv1D [in, out] -> [out, in] on the device (transpose_dense_weights, rust.rs:1345-1352)
  auto upload_t = [&](uint64_t i, int in_f, int out_f) -> int {
    PG_CUDA_TRY(cudaMemcpy(staging, tensors[i], lens[i] * sizeof(float), cudaMemcpyHostToDevice));
    PG_CUDA_TRY(launch_transpose(staging, dev(i), in_f, out_f, 0));
    PG_CUDA_TRY(cudaDeviceSynchronize());
    return PG_OK;
  };
  for (uint64_t i = 0; i < 4 && rc == PG_OK; ++i) rc = upload(i);
  m->wte = dev(0); m->wpe = dev(1); m->lnf_g = dev(2); m->lnf_b = dev(3);
  m->layers.resize(cfg.n_layer);
  const int C = (int)cfg.n_embd, F = (int)cfg.n_inner;
  for (uint64_t l = 0; l < cfg.n_layer && rc == PG_OK; ++l) {
    uint64_t o = 4 + 12 * l;
    LayerWeights& w = m->layers[l];
    for (int k : {0, 1, 3, 5, 6, 7, 9, 11})
      if (rc == PG_OK) rc = upload(o + k);
    if (rc == PG_OK) rc = upload_t(o + 2, C, 3 * C);
    if (rc == PG_OK) rc = upload_t(o + 4, C, C);
    if (rc == PG_OK) rc = upload_t(o + 8, C, F);
    if (rc == PG_OK) rc = upload_t(o + 10, F, C);
    w.ln1_g = dev(o); w.ln1_b = dev(o + 1); w.w_qkv = dev(o + 2); w.b_qkv = dev(o + 3);
    w.w_proj = dev(o + 4); w.b_proj = dev(o + 5); w.ln2_g = dev(o + 6); w.ln2_b = dev(o + 7);
    w.w_fc = dev(o + 8); w.b_fc = dev(o + 9); w.w_proj2 = dev(o + 10); w.b_proj2 = dev(o + 11);
  }
  cudaFree(staging);
  if (rc != PG_OK) return rc;
  m->head_w = m->wte;
  if (be.math_mode == PG_MATH_BF16 || be.quantized_weights) {
    // A second, narrow copy of the dense matrices and of the tied lm_head, every layer laid out alike:
    //  int8: QuantizedRows::from_f32 of the transposed matrices (quantize_weights, rust.rs:1354-1376); the FP32
    //        arena then holds q * scale, what quantized_dot multiplies by (cpu.rs:173-184), so that every FP32
    //        kernel of this library (prefill, batches above 8) computes the quantised model too; wte keeps its
    //        FP32 rows for the embedding lookup and gets a dequantised twin for the lm_head;
    //  bf16: round-to-nearest-even of the same tensors, written back into the FP32 arena as well.
    const bool q8 = be.quantized_weights != 0;
    const size_t eb = q8 ? 1 : 2;
    const int V = (int)cfg.vocab_size;
    auto al = [](size_t n) { return (n + 255) / 256 * 256; };
    const size_t lay_bytes = al((size_t)3 * C * C * eb) + al((size_t)C * C * eb) + 2 * al((size_t)C * F * eb);
    const size_t lay_scales = (size_t)(3 * C + C + F + C + 63) / 64 * 64;
    PG_CUDA_TRY(cudaMalloc(&m->packed_arena, lay_bytes * cfg.n_layer + al((size_t)V * C * eb)));
    if (q8) {
      PG_CUDA_TRY(cudaMalloc(&m->scale_arena, (lay_scales * cfg.n_layer + (size_t)V) * sizeof(float)));
      PG_CUDA_TRY(cudaMalloc(&m->head_deq, (size_t)V * C * sizeof(float)));
      m->head_w = m->head_deq;
    }
    m->stream_weight_type = q8 ? STREAM_W_I8 : STREAM_W_BF16;
    auto pack = [&](float* w, int rows, int cols, void* packed, float* scales, float* deq_out) -> int {
      if (q8) {
        PG_CUDA_TRY(launch_quantize_rows(w, rows, cols, static_cast<int8_t*>(packed), scales, 0));
        PG_CUDA_TRY(launch_dequantize_rows(static_cast<const int8_t*>(packed), scales, rows, cols, deq_out, 0));
      } else {
        PG_CUDA_TRY(launch_round_bf16(w, (size_t)rows * cols, static_cast<uint16_t*>(packed), 0));
      }
      return PG_OK;
    };
    for (uint64_t l = 0; l < cfg.n_layer; ++l) {
      LayerWeights& w = m->layers[l];
      unsigned char* p = m->packed_arena + l * lay_bytes;
      float* sc = q8 ? m->scale_arena + l * lay_scales : nullptr;
      w.p_qkv = p; p += al((size_t)3 * C * C * eb);
      w.p_proj = p; p += al((size_t)C * C * eb);
      w.p_fc = p; p += al((size_t)C * F * eb);
      w.p_proj2 = p;
      if (q8) {
        w.s_qkv = sc; w.s_proj = sc + 3 * C; w.s_fc = sc + 4 * C; w.s_proj2 = sc + 4 * C + F;
      }
      if (int r = pack(w.w_qkv, 3 * C, C, w.p_qkv, w.s_qkv, w.w_qkv)) return r;
      if (int r = pack(w.w_proj, C, C, w.p_proj, w.s_proj, w.w_proj)) return r;
      if (int r = pack(w.w_fc, F, C, w.p_fc, w.s_fc, w.w_fc)) return r;
      if (int r = pack(w.w_proj2, C, F, w.p_proj2, w.s_proj2, w.w_proj2)) return r;
    }
    m->p_wte = m->packed_arena + lay_bytes * cfg.n_layer;
    if (q8) m->s_wte = m->scale_arena + lay_scales * cfg.n_layer;
    if (int r = pack(m->wte, V, C, m->p_wte, m->s_wte, m->head_deq)) return r;
    PG_CUDA_TRY(cudaDeviceSynchronize());
  }
  // BF16 mode: everything that is not the single-kernel step multiplies the rounded FP32 values, on the tensor
  // cores as three TF32 products where the FP32-grade mode would
  const bool tc_modes = be.math_mode != PG_MATH_FP32;
  if (tc_modes && C % 32 == 0 && F % 32 == 0) {
    const int V = (int)cfg.vocab_size;
    const size_t per_layer = tc_tiled_weight_floats(3 * C, C) + tc_tiled_weight_floats(C, C) +
                             tc_tiled_weight_floats(F, C) + tc_tiled_weight_floats(C, F);
    const size_t total_t = per_layer * cfg.n_layer + tc_tiled_weight_floats(V, C);
    PG_CUDA_TRY(cudaMalloc(&m->tiled_arena, total_t * sizeof(float)));
    m->tiled_floats = total_t;
    float* p = m->tiled_arena;
    auto tile = [&](const float* src, int n_rows, int k_cols, float** dst) -> int {
      *dst = p;
      PG_CUDA_TRY(launch_tile_weights(src, p, n_rows, k_cols, 0));
      p += tc_tiled_weight_floats(n_rows, k_cols);
      return PG_OK;
    };
    for (auto& w : m->layers) {
      if (int r = tile(w.w_qkv, 3 * C, C, &w.t_qkv)) return r;
      if (int r = tile(w.w_proj, C, C, &w.t_proj)) return r;
      if (int r = tile(w.w_fc, F, C, &w.t_fc)) return r;
      if (int r = tile(w.w_proj2, C, F, &w.t_proj2)) return r;
    }
    if (int r = tile(m->head_w, V, C, &m->t_wte)) return r;
    if (C % 4 == 0 && F % 4 == 0) {
      const size_t per_lo = (size_t)3 * C * C + (size_t)C * C + 2 * (size_t)C * F;
      PG_CUDA_TRY(cudaMalloc(&m->lo_arena, per_lo * cfg.n_layer * sizeof(float)));
      float* q = m->lo_arena;
      auto lo = [&](const float* src, size_t n, float** dst) -> int {
        *dst = q;
        PG_CUDA_TRY(launch_tf32_lo(src, q, n, 0));
        q += n;
        return PG_OK;
      };
      for (auto& w : m->layers) {
        if (int r = lo(w.w_qkv, (size_t)3 * C * C, &w.l_qkv)) return r;
        if (int r = lo(w.w_proj, (size_t)C * C, &w.l_proj)) return r;
        if (int r = lo(w.w_fc, (size_t)C * F, &w.l_fc)) return r;
        if (int r = lo(w.w_proj2, (size_t)C * F, &w.l_proj2)) return r;
      }
    }
    PG_CUDA_TRY(cudaDeviceSynchronize());
  }
  *out = m.release();
  return PG_OK;
}

}  // namespace pg

// ------------------------------------------------------------------ cache
struct pg_cache {
  const pg_model* model = nullptr;
  int max_batch = 0;
  cudaStream_t stream = nullptr;
  KvLayout kv{};
  size_t page_floats = 0;  // floats of one page of one layer
  int num_pages = 0;
  float* kv_pool = nullptr;  // [layer][page][2][head][page_tokens][head_dim]
  std::vector<int> free_pages;
  std::vector<int> h_table;    // [max_batch][pages_per_seq], -1 = unassigned
  std::vector<int> seq_len;    // host mirror of d_pos
  int* d_table = nullptr;
  bool table_dirty = true;
  int *d_ids = nullptr, *d_pos = nullptr, *d_argmax = nullptr, *d_token_log = nullptr;
  float *x = nullptr, *norm = nullptr, *qkv = nullptr, *attn = nullptr, *hbuf = nullptr, *logits = nullptr;
  float* part_val = nullptr;
  int* part_idx = nullptr;
  int part_stride = 0;
  float* attn_part = nullptr;
  unsigned* attn_counters = nullptr;
  float* topk_vals = nullptr;
  int* topk_idx = nullptr;
  // tensor-core decode path (9..64 sequences): TF32 hi/lo pairs of the GEMM inputs, split-K scratch
  float *norm_lo = nullptr, *attn_lo = nullptr, *h_lo = nullptr;
  int* d_error = nullptr;
  // persistent chain kernel of the tensor-core decode path: partial tiles, grid-barrier word
  float* chain_partials = nullptr;
  unsigned* d_chain_barrier = nullptr;
  unsigned long long* d_chain_best = nullptr;  // row arg-max accumulators of the lm_head phase
  unsigned long long* d_chain_trace = nullptr;  // developer aid: only allocated in builds with -DPG_DEV_TRACE
  int chain_ctas = 0;
  int chain_min_batch = 9;  // smallest batch whose decode step runs as the chain kernel in the tensor-core modes (measured on
                            // B200, GPT-2 medium, 8 sequences: 1.34 ms as the chain kernel, 1.09 ms as one kernel per operation)
  struct ChainProgram {  // whole-step phase list of the persistent chain kernel for one batch size
    ChainPhase* dev = nullptr;            // in device memory (nullptr: this batch size is not supported)
    ChainPhase* dev_argmax_only = nullptr;  // the same list whose lm_head reduce phase keeps the row arg-max but stores no logits
    int n = 0;
    std::vector<int> bucket;              // profile bucket of every phase
    unsigned long long* d_times = nullptr;  // n + 1 time stamps, written in profiling runs
  };
  std::map<int, ChainProgram> chain_programs;
  bool step_wants_logits = true;  // false: the caller of this step only reads the arg-max (greedy decoding)
  // single-kernel decode step (at most 8 sequences): layer table, tagged exchange buffers, tag counter
  unsigned long long* d_stream_ll = nullptr;  // ll_x | ll_qkv | ll_attn | ll_h | ll_part | ll_best
  unsigned* d_stream_epoch = nullptr;
  int stream_grid = 0;
  unsigned dbg_spin_limit = 0, dbg_poison = 0;  // pg_cache_debug_expire_next_wait: consumed by the next decode step
#ifdef PG_DEV_TRACE
  unsigned long long* d_stream_trace = nullptr;
#endif
  int *h_ids = nullptr, *h_out = nullptr;  // pinned staging
  // prefill workspace (grow-only)
  size_t pre_rows = 0;
  float *px = nullptr, *pnorm = nullptr, *pqkv = nullptr, *pattn = nullptr, *ph = nullptr, *plo = nullptr;
  int* prow = nullptr;  // [4][pre_rows]: ids, pos, slot, (batch+1 seq_start / last rows)
  std::map<std::pair<int, int>, cudaGraphExec_t> graphs;  // (batch, splits) -> decode-step graph
  std::map<std::pair<int, int>, uint64_t> graphs_launches;  // kernel nodes in each graph
  uint64_t decode_launches = 0;  // kernels launched by decode steps (for gpu_launches accounting)
  cudaEvent_t t0 = nullptr, t1 = nullptr;  // pg_cache_time_begin / pg_cache_time_end

  float* layer_pool(int l) const { return kv_pool + (size_t)l * num_pages * page_floats; }

  ~pg_cache() {
    if (!model) return;
    cudaSetDevice(model->device);
    if (stream) cudaStreamSynchronize(stream);
#ifdef PG_DEV_TRACE
    if (d_stream_trace) {
      const int L = model->layers_n();
      std::vector<unsigned long long> t((size_t)2 * (L + 1) * 16 + 128);
      if (cudaMemcpy(t.data(), d_stream_trace, t.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess) {
        for (int cta = 0; cta < 2; ++cta)
          for (int l = 0; l <= L; ++l) {
            const unsigned long long* r = t.data() + ((size_t)cta * (L + 1) + l) * 16;
            fprintf(stderr, "stream trace cta %d layer %2d:", cta ? 100 : 0, l);
            for (int p = 1; p < 10; ++p) fprintf(stderr, " %6lld", r[p] ? (long long)(r[p] - r[p - 1]) : -1LL);
            fprintf(stderr, "  | start %lld cycles\n", (long long)(r[0] - t[((size_t)cta * (L + 1)) * 16]));
          }
      }
      cudaFree(d_stream_trace);
    }
#endif
#ifdef PG_DEV_TRACE
    if (d_chain_trace) {
      std::vector<unsigned long long> t((size_t)chain_ctas * 32 + 512);
      if (cudaMemcpy(t.data(), d_chain_trace, t.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess) {
        unsigned long long t0 = ~0ULL;
        for (int i = 0; i < chain_ctas; ++i) t0 = std::min(t0, t[(size_t)i * 32 + 31]);
        for (int sl = 0; sl < 10; ++sl) {
          unsigned long long lo = ~0ULL, hi = 0, wlo = ~0ULL, whi = 0;
          for (int i = 0; i < chain_ctas; ++i) {
            const unsigned long long v = t[(size_t)i * 32 + sl] - t0, w = t[(size_t)i * 32 + 10 + sl] - t0;
            lo = std::min(lo, v); hi = std::max(hi, v); wlo = std::min(wlo, w); whi = std::max(whi, w);
          }
          fprintf(stderr, "chain trace phase %d: work done %6llu..%6llu ns, barrier passed %6llu..%6llu ns\n", sl, wlo, whi, lo, hi);
        }
        // the lm_head of the last step: per CTA its SM and the time its share took; then CTA 0's units (see unit_trace)
        for (int i = 0; i < chain_ctas; ++i) {
          const unsigned long long* r = t.data() + (size_t)i * 32;
          fprintf(stderr, "chain trace lm_head cta %3d sm %3llu work %7lld ns\n", i, r[22], (long long)(r[21] - r[20]));
        }
        const unsigned long long* u = t.data() + (size_t)chain_ctas * 32;
        for (int i = 0; i < 48; ++i) {
          fprintf(stderr, "chain trace unit %2d:", i);
          for (int e = 0; e < 8; ++e) fprintf(stderr, " %7lld", u[i * 8 + e] ? (long long)(u[i * 8 + e] - u[0]) : -1LL);
          fprintf(stderr, "\n");
        }
      }
    }
#endif
    for (auto& cp : chain_programs) {
      if (cp.second.dev) cudaFree(cp.second.dev);
      if (cp.second.dev_argmax_only) cudaFree(cp.second.dev_argmax_only);
      if (cp.second.d_times) cudaFree(cp.second.d_times);
    }
    for (auto& g : graphs) cudaGraphExecDestroy(g.second);
    for (void* p : {(void*)kv_pool, (void*)d_table, (void*)d_ids, (void*)d_pos, (void*)d_argmax, (void*)d_token_log,
                    (void*)x, (void*)norm, (void*)qkv, (void*)attn, (void*)hbuf, (void*)logits, (void*)part_val,
                    (void*)part_idx, (void*)attn_part, (void*)attn_counters, (void*)topk_vals, (void*)topk_idx,
                    (void*)px, (void*)pnorm, (void*)pqkv, (void*)pattn, (void*)ph, (void*)plo, (void*)prow, (void*)norm_lo,
                    (void*)attn_lo, (void*)h_lo, (void*)d_error, (void*)d_stream_ll, (void*)d_stream_epoch,
                    (void*)chain_partials, (void*)d_chain_barrier, (void*)d_chain_trace, (void*)d_chain_best})
      if (p) cudaFree(p);
    if (t0) cudaEventDestroy(t0);
    if (t1) cudaEventDestroy(t1);
    if (h_ids) cudaFreeHost(h_ids);
    if (h_out) cudaFreeHost(h_out);
    if (stream) cudaStreamDestroy(stream);
  }
};

namespace pg {

constexpr int MAX_SPLITS = 16;
constexpr int MAX_TOPK = 64;

// Words of the tagged exchange buffers of the single-kernel decode step, in the order
// ll_x [8][C], ll_qkv [8][3C], ll_attn [8][C], ll_h [8][F], ll_part [8 * H][8][66], ll_best [8][grid][2].
static size_t stream_ll_words(const pg_model* m, int grid) {
  const size_t C = m->c(), F = m->f(), H = m->heads();
  return 8 * (C + 3 * C + C + F) + 8 * H * 8 * 66 + 8 * (size_t)grid * 2;
}

static int cache_new(const pg_model* m, int max_batch, pg_cache** out) {
  if (max_batch <= 0 || max_batch > 4096)
    return set_error(PG_INVALID_INPUT, "max_batch " + std::to_string(max_batch) + " must be in 1..4096");
  if (int r = ensure_device(m->device)) return r;
  auto c = std::make_unique<pg_cache>();
  c->model = m;
  c->max_batch = max_batch;
  const int C = m->c(), F = m->f(), V = m->v(), P = m->positions(), H = m->heads(), D = m->head_dim();
  c->kv = KvLayout{H, D, m->backend.page_tokens, (P + m->backend.page_tokens - 1) / m->backend.page_tokens};
  c->page_floats = (size_t)2 * H * c->kv.page_tokens * D;
  c->num_pages = max_batch * c->kv.pages_per_seq;
  PG_CUDA_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  const size_t B = (size_t)max_batch;
  PG_CUDA_TRY(cudaMalloc(&c->kv_pool, (size_t)m->layers_n() * c->num_pages * c->page_floats * sizeof(float)));
  // KV pages start zeroed like the reference's vec![0.0; len] (rust.rs:258-266)
  PG_CUDA_TRY(cudaMemsetAsync(c->kv_pool, 0, (size_t)m->layers_n() * c->num_pages * c->page_floats * sizeof(float), c->stream));
  c->free_pages.resize(c->num_pages);
  for (int i = 0; i < c->num_pages; ++i) c->free_pages[i] = c->num_pages - 1 - i;  // pop_back hands out page 0 first
  c->h_table.assign(B * c->kv.pages_per_seq, -1);
  c->seq_len.assign(B, 0);
  PG_CUDA_TRY(cudaMalloc(&c->d_table, B * c->kv.pages_per_seq * sizeof(int)));
  PG_CUDA_TRY(cudaMemsetAsync(c->d_table, 0, B * c->kv.pages_per_seq * sizeof(int), c->stream));
  PG_CUDA_TRY(cudaMalloc(&c->d_ids, B * sizeof(int)));
  PG_CUDA_TRY(cudaMalloc(&c->d_pos, B * sizeof(int)));
  PG_CUDA_TRY(cudaMalloc(&c->d_argmax, B * sizeof(int)));
  PG_CUDA_TRY(cudaMalloc(&c->d_token_log, B * P * sizeof(int)));
  PG_CUDA_TRY(cudaMemsetAsync(c->d_ids, 0, B * sizeof(int), c->stream));
  PG_CUDA_TRY(cudaMemsetAsync(c->d_pos, 0, B * sizeof(int), c->stream));
  PG_CUDA_TRY(cudaMemsetAsync(c->d_token_log, 0, B * P * sizeof(int), c->stream));
  PG_CUDA_TRY(cudaMalloc(&c->x, B * C * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->norm, B * std::max(C, 4) * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->qkv, B * 3 * C * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->attn, B * C * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->hbuf, B * F * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->logits, B * V * sizeof(float)));
  c->part_stride = linear_decode_grid(V, m->num_sms);
  PG_CUDA_TRY(cudaMalloc(&c->part_val, B * c->part_stride * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->part_idx, B * c->part_stride * sizeof(int)));
  PG_CUDA_TRY(cudaMalloc(&c->attn_part, B * H * MAX_SPLITS * (D + 2) * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->attn_counters, B * H * sizeof(unsigned)));
  PG_CUDA_TRY(cudaMemsetAsync(c->attn_counters, 0, B * H * sizeof(unsigned), c->stream));
  PG_CUDA_TRY(cudaMalloc(&c->topk_vals, B * MAX_TOPK * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->topk_idx, B * MAX_TOPK * sizeof(int)));
  PG_CUDA_TRY(cudaMalloc(&c->d_error, sizeof(int)));
  PG_CUDA_TRY(cudaMemsetAsync(c->d_error, 0, sizeof(int), c->stream));
  if (const char* e = getenv("PG_CHAIN_MIN_BATCH")) c->chain_min_batch = std::max(1, std::min(65, atoi(e)));
  if (max_batch >= c->chain_min_batch && C % 32 == 0 && F % 32 == 0) {
    const int bmax = std::min(max_batch, 64);
    PG_CUDA_TRY(cudaMalloc(&c->norm_lo, (size_t)bmax * C * sizeof(float)));
    PG_CUDA_TRY(cudaMalloc(&c->attn_lo, (size_t)bmax * C * sizeof(float)));
    PG_CUDA_TRY(cudaMalloc(&c->h_lo, (size_t)bmax * F * sizeof(float)));
    if (m->t_wte && !env_flag("PG_NO_CHAIN") && chain_grid(m->num_sms) > 0) {
      c->chain_ctas = chain_grid(m->num_sms);
      PG_CUDA_TRY(cudaMalloc(&c->chain_partials, chain_partial_floats(c->chain_ctas) * sizeof(float)));
      PG_CUDA_TRY(cudaMalloc(&c->d_chain_barrier, sizeof(unsigned)));
      PG_CUDA_TRY(cudaMemsetAsync(c->d_chain_barrier, 0, sizeof(unsigned), c->stream));
      {
        const std::vector<unsigned long long> init(64, chain_argmax_init());
        PG_CUDA_TRY(cudaMalloc(&c->d_chain_best, init.size() * sizeof(unsigned long long)));
        PG_CUDA_TRY(cudaMemcpy(c->d_chain_best, init.data(), init.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice));
      }
#ifdef PG_DEV_TRACE
      if (env_flag("PG_CHAIN_TRACE")) {
        PG_CUDA_TRY(cudaMalloc(&c->d_chain_trace, ((size_t)c->chain_ctas * 32 + 512) * sizeof(unsigned long long)));
        PG_CUDA_TRY(cudaMemsetAsync(c->d_chain_trace, 0, ((size_t)c->chain_ctas * 32 + 512) * sizeof(unsigned long long), c->stream));
      }
#endif
    }
  }
  if (m->backend.persistent_step != 2 && !env_flag("PG_NO_STREAM")) {
    const int grid = decode_stream_grid(m->num_sms);
    if (decode_stream_supported(1, C, F, V, D, P, c->kv.page_tokens, m->stream_weight_type, grid)) {
      c->stream_grid = grid;
      const size_t words = stream_ll_words(m, grid);
      PG_CUDA_TRY(cudaMalloc(&c->d_stream_ll, words * sizeof(unsigned long long)));
      PG_CUDA_TRY(cudaMemsetAsync(c->d_stream_ll, 0, words * sizeof(unsigned long long), c->stream));
      PG_CUDA_TRY(cudaMalloc(&c->d_stream_epoch, sizeof(unsigned)));
      PG_CUDA_TRY(cudaMemsetAsync(c->d_stream_epoch, 0, sizeof(unsigned), c->stream));
#ifdef PG_DEV_TRACE
      PG_CUDA_TRY(cudaMalloc(&c->d_stream_trace, ((size_t)2 * (m->layers_n() + 1) * 16 + 128) * 8));
      PG_CUDA_TRY(cudaMemsetAsync(c->d_stream_trace, 0, ((size_t)2 * (m->layers_n() + 1) * 16 + 128) * 8, c->stream));
#endif
    }
  }
  PG_CUDA_TRY(cudaMallocHost(&c->h_ids, B * sizeof(int)));
  PG_CUDA_TRY(cudaMallocHost(&c->h_out, (B * (1 + 2 * MAX_TOPK) + 1) * sizeof(int)));
  PG_CUDA_TRY(cudaStreamSynchronize(c->stream));
  *out = c.release();
  return PG_OK;
}

static void release_slot_pages(pg_cache* c, int slot) {
  int* row = c->h_table.data() + (size_t)slot * c->kv.pages_per_seq;
  for (int p = c->kv.pages_per_seq - 1; p >= 0; --p)
    if (row[p] >= 0) {
      c->free_pages.push_back(row[p]);
      row[p] = -1;
      c->table_dirty = true;
    }
}

// Makes sure slot `slot` owns pages for positions [0, upto).
static int ensure_pages(pg_cache* c, int slot, int upto) {
  int need = (upto + c->kv.page_tokens - 1) / c->kv.page_tokens;
  int* row = c->h_table.data() + (size_t)slot * c->kv.pages_per_seq;
  for (int p = 0; p < need; ++p)
    if (row[p] < 0) {
      if (c->free_pages.empty()) return set_error(PG_INVALID_INPUT, "KV page pool exhausted");
      row[p] = c->free_pages.back();
      c->free_pages.pop_back();
      c->table_dirty = true;
    }
  return PG_OK;
}

static int sync_table(pg_cache* c) {
  if (!c->table_dirty) return PG_OK;
  // unassigned entries are uploaded as page 0; kernels never index past a slot's seq_len
  std::vector<int> up(c->h_table.size());
  for (size_t i = 0; i < up.size(); ++i) up[i] = std::max(c->h_table[i], 0);
  PG_CUDA_TRY(cudaMemcpyAsync(c->d_table, up.data(), up.size() * sizeof(int), cudaMemcpyHostToDevice, c->stream));
  PG_CUDA_TRY(cudaStreamSynchronize(c->stream));  // `up` is a pageable temporary
  c->table_dirty = false;
  return PG_OK;
}

static int choose_splits(const pg_cache* c, int batch, int max_len) {
  const pg_model* m = c->model;
  if (m->head_dim() != 64) return 1;
  if (m->backend.attn_splits > 0) return std::min(m->backend.attn_splits, MAX_SPLITS);
  // enough CTAs to cover the SMs twice, but at least 128 keys per split
  int by_fill = (2 * m->num_sms + batch * m->heads() - 1) / (batch * m->heads());
  int by_len = std::max(1, (max_len + 127) / 128);
  int s = std::max(1, std::min(std::min(by_fill, by_len), 8));
  return s;
}

// Per-operation device timing of one decode step: the buckets of Gpt2OperationProfile
// (rust.rs:336-347). Events around every launch serialise the step, so this is a profiling mode.
enum Bucket { B_LAYER_NORM = 0, B_QKV, B_ATTN, B_ATTN_PROJ, B_MLP_FC, B_MLP_PROJ, B_LOGITS, B_OTHER, B_COUNT };
struct StepProfiler {
  std::vector<cudaEvent_t> ev;
  std::vector<int> bucket;
  int chain_event = -1;  // index of the event pair around the persistent chain kernel, if it ran
  cudaError_t mark(cudaStream_t s, int b) {
    cudaEvent_t e;
    cudaError_t r = cudaEventCreate(&e);
    if (r != cudaSuccess) return r;
    ev.push_back(e);
    bucket.push_back(b);
    return cudaEventRecord(e, s);
  }
  ~StepProfiler() {
    for (auto e : ev) cudaEventDestroy(e);
  }
};

// Arguments of the chain kernel for `batch` sequences starting at slot 64 * chunk (steps of more than 64
// sequences run as one launch per 64: the activation buffers are reused, what belongs to a slot is offset).
static ChainArgs chain_base_args(const pg_cache* c, int batch, int chunk = 0) {
  const pg_model* m = c->model;
  const size_t s0 = (size_t)chunk * 64;
  ChainArgs base{};
  base.m = batch; base.eps = m->cfg.layer_norm_epsilon; base.arena = m->tiled_arena; base.arena_floats = m->tiled_floats;
  base.act_hi[CH_ACT_NORM] = c->norm; base.act_lo[CH_ACT_NORM] = c->norm_lo; base.act_k[CH_ACT_NORM] = m->c();
  base.act_hi[CH_ACT_ATTN] = c->attn; base.act_lo[CH_ACT_ATTN] = c->attn_lo; base.act_k[CH_ACT_ATTN] = m->c();
  base.act_hi[CH_ACT_H] = c->hbuf; base.act_lo[CH_ACT_H] = c->h_lo; base.act_k[CH_ACT_H] = m->f();
  base.partials = c->chain_partials; base.barrier = c->d_chain_barrier; base.error_flag = c->d_error;
  base.trace = c->d_chain_trace;
  base.kv = c->kv; base.page_table = c->d_table + s0 * c->kv.pages_per_seq; base.pos = c->d_pos + s0;
  base.wte = m->wte; base.wpe = m->wpe; base.ids = c->d_ids + s0; base.pos_rw = c->d_pos + s0;
  base.argmax_out = c->d_argmax + s0;
  base.token_log = c->d_token_log + s0 * m->positions(); base.n_positions = m->positions(); base.best = c->d_chain_best;
  { static const int f = getenv("PG_CHAIN_FENCE") ? atoi(getenv("PG_CHAIN_FENCE")) : 0; base.tune_fence = f; }
  return base;
}

// Builds (once per batch size) the phase list of a whole decode step for the persistent chain
// kernel and uploads it: per layer QKV projection, attention, attention-output projection with
// residual and LayerNorm, MLP with GELU, residual and the next LayerNorm; then the lm_head.
// block_forward_one_profiled (rust.rs:1136-1250), forward_one tail (rust.rs:981-1003).
static int chain_program_key(int rows, int chunk) { return rows + 100 * chunk; }

static int ensure_chain_program(pg_cache* c, int batch, int chunk = 0) {
  if (c->chain_ctas <= 0 || batch < 1 || batch > 64 || !c->norm_lo) return PG_OK;
  if (chunk == 0 && batch < c->chain_min_batch) return PG_OK;
  const int key = chain_program_key(batch, chunk);
  if (c->chain_programs.count(key)) return PG_OK;
  const pg_model* m = c->model;
  const int C = m->c(), F = m->f(), V = m->v(), L = m->layers_n();
  std::vector<ChainPhase> ph;
  std::vector<int> bucket;
  int cur_b = B_OTHER;  // bucket of the phases being appended
  auto block0 = [&](const float* t) { return (unsigned)((size_t)(t - m->tiled_arena) / 4096); };
  auto gemm = [&](const float* t, int n_out, int k, int act) {
    ChainPhase p{};
    p.kind = CH_GEMM; p.n = n_out; p.k = k; p.act = act; p.w_block0 = block0(t);
    ph.push_back(p);
    bucket.push_back(cur_b);
  };
  auto rows = [&](int n_out, int k, const float* bias, const float* g, const float* b) {
    ChainPhase p{};
    p.kind = CH_ROWS; p.n = n_out; p.k = k; p.bias = bias; p.x = c->x; p.ln_g = g; p.ln_b = b;
    p.out_hi = c->norm; p.out_lo = c->norm_lo;
    ph.push_back(p);
    bucket.push_back(B_LAYER_NORM);  // partial sums + bias + residual + LayerNorm
  };
  auto elem = [&](int n_out, int k, const float* bias, int gelu, float* out, float* ohi, float* olo) {
    ChainPhase p{};
    p.kind = CH_ELEM; p.n = n_out; p.k = k; p.bias = bias; p.gelu = gelu; p.out = out; p.out_hi = ohi; p.out_lo = olo;
    ph.push_back(p);
    bucket.push_back(cur_b);  // belongs to the GEMM it finishes
  };
  {
    ChainPhase p{};  // token + position embedding and the first LayerNorm
    p.kind = CH_EMBED; p.n = C; p.k = C; p.x = c->x; p.ln_g = m->layers[0].ln1_g; p.ln_b = m->layers[0].ln1_b;
    p.out_hi = c->norm; p.out_lo = c->norm_lo;
    ph.push_back(p);
    bucket.push_back(B_LAYER_NORM);
  }
  for (int l = 0; l < L; ++l) {
    const LayerWeights& w = m->layers[l];
    cur_b = B_QKV;
    gemm(w.t_qkv, 3 * C, C, CH_ACT_NORM);
    ChainPhase at{};  // reduces the QKV partials itself
    at.kind = CH_ATTN; at.n = 3 * C; at.k = C; at.bias = w.b_qkv; at.kv_pool = c->layer_pool(l);
    at.out_hi = c->attn; at.out_lo = c->attn_lo;
    ph.push_back(at);
    bucket.push_back(B_ATTN);
    cur_b = B_ATTN_PROJ;
    gemm(w.t_proj, C, C, CH_ACT_ATTN);
    rows(C, C, w.b_proj, w.ln2_g, w.ln2_b);
    cur_b = B_MLP_FC;
    gemm(w.t_fc, F, C, CH_ACT_NORM);
    elem(F, C, w.b_fc, 1, nullptr, c->hbuf, c->h_lo);
    cur_b = B_MLP_PROJ;
    gemm(w.t_proj2, C, F, CH_ACT_H);
    if (l + 1 < L) rows(C, F, w.b_proj2, m->layers[l + 1].ln1_g, m->layers[l + 1].ln1_b);
    else rows(C, F, w.b_proj2, m->lnf_g, m->lnf_b);
  }
  cur_b = B_LOGITS;
  gemm(m->t_wte, V, C, CH_ACT_NORM);
  // The lm_head in whole row tiles per CTA: its drain stores the logits and finds the row arg-max, and there is no
  // reduce phase (measured on GPT-2 medium, 64 sequences: 38 + 37 us for GEMM + reduce with equal shares).
  // PG_CHAIN_LM_HEAD_REDUCE=1 brings the equal shares and the reduce phase back.
  static const bool lm_head_reduce = getenv("PG_CHAIN_LM_HEAD_REDUCE") && atoi(getenv("PG_CHAIN_LM_HEAD_REDUCE")) != 0;
  if (lm_head_reduce) {
    elem(V, C, nullptr, 0, c->logits + (size_t)chunk * 64 * V, nullptr, nullptr);
  } else {
    ph.back().whole_tiles = 1;
    ph.back().out = c->logits + (size_t)chunk * 64 * V;
  }
  ph.back().best = c->d_chain_best;  // together with the row arg-max
  {
    ChainPhase p{};
    p.kind = CH_FINAL;
    ph.push_back(p);
    bucket.push_back(B_OTHER);
  }
  chain_prepare_phases(ph.data(), (int)ph.size(), c->chain_ctas);
  ChainArgs a = chain_base_args(c, batch, chunk);
  a.n_phases = (int)ph.size();
  pg_cache::ChainProgram prog;
  prog.n = (int)ph.size();
  prog.bucket = bucket;
  if (m->head_dim() == 64 && chain_supported(a, c->chain_ctas, ph.data())) {
    PG_CUDA_TRY(cudaMalloc(&prog.dev, ph.size() * sizeof(ChainPhase)));
    PG_CUDA_TRY(cudaMemcpy(prog.dev, ph.data(), ph.size() * sizeof(ChainPhase), cudaMemcpyHostToDevice));
    PG_CUDA_TRY(cudaMalloc(&prog.d_times, (ph.size() + 1) * sizeof(unsigned long long)));
    // 12.9 MB of logits per step of 64 sequences that greedy decoding never reads
    std::vector<ChainPhase> lean = ph;
    for (ChainPhase& p : lean)
      if (p.best) p.out = nullptr;
    PG_CUDA_TRY(cudaMalloc(&prog.dev_argmax_only, lean.size() * sizeof(ChainPhase)));
    PG_CUDA_TRY(cudaMemcpy(prog.dev_argmax_only, lean.data(), lean.size() * sizeof(ChainPhase), cudaMemcpyHostToDevice));
  }
  c->chain_programs[key] = prog;
  return PG_OK;
}

// More than 64 sequences: a program per chunk of 64 (the last one may be smaller).
static int ensure_chain_programs(pg_cache* c, int batch) {
  if (batch <= 64) return ensure_chain_program(c, batch);
  for (int k = 0; k * 64 < batch; ++k)
    if (int r = ensure_chain_program(c, std::min(64, batch - k * 64), k)) return r;
  return PG_OK;
}

// Enqueues the kernels of one decode step for slots 0..batch-1 on `s`.
// forward_one_profiled_with_scratch + block_forward_one_profiled (rust.rs:943-1006, 1136-1250).
static cudaError_t enqueue_decode_step(pg_cache* c, int batch, int splits, cudaStream_t s, uint64_t* launches,
                                       StepProfiler* prof = nullptr) {
  // FP32 weights: the single-kernel step wins up to 4 sequences (measured on B200: 279 against 306 us for one GPT-2
  // small sequence, 1014 against 1168 us for four GPT-2 medium ones; at eight it loses, 1806 against 1548 us);
  // packed weights (BF16, int8) are only read by that kernel
  const bool stream_wanted = c->model->stream_weight_type != STREAM_W_F32 || batch <= 4 || c->model->backend.persistent_step == 1;
  if (!prof && c->stream_grid > 0 && stream_wanted &&
      decode_stream_supported(batch, c->model->c(), c->model->f(), c->model->v(), c->model->head_dim(),
                              c->model->positions(), c->kv.page_tokens, c->model->stream_weight_type, c->stream_grid)) {
    // the whole step in one persistent cooperative kernel
    const pg_model* m = c->model;
    const size_t C = m->c(), F = m->f(), H = m->heads();
    const LayerWeights& w0 = m->layers[0];
    const LayerWeights& w1 = m->layers[m->layers_n() > 1 ? 1 : 0];
    const bool packed = m->stream_weight_type != STREAM_W_F32;
    StreamArgs a{};
    auto bytes = [](const void* p) { return reinterpret_cast<const unsigned char*>(p); };
    if (packed) {
      a.w[0] = bytes(w0.p_qkv); a.w[1] = bytes(w0.p_proj); a.w[2] = bytes(w0.p_fc); a.w[3] = bytes(w0.p_proj2);
      a.w_stride = bytes(w1.p_qkv) - bytes(w0.p_qkv);
      a.scale[0] = w0.s_qkv; a.scale[1] = w0.s_proj; a.scale[2] = w0.s_fc; a.scale[3] = w0.s_proj2;
      a.s_stride = w0.s_qkv ? w1.s_qkv - w0.s_qkv : 0;
      a.w_head = bytes(m->p_wte); a.s_head = m->s_wte;
    } else {
      a.w[0] = bytes(w0.w_qkv); a.w[1] = bytes(w0.w_proj); a.w[2] = bytes(w0.w_fc); a.w[3] = bytes(w0.w_proj2);
      a.w_stride = bytes(w1.w_qkv) - bytes(w0.w_qkv);
      a.w_head = bytes(m->head_w);
    }
    a.bias[0] = w0.b_qkv; a.bias[1] = w0.b_proj; a.bias[2] = w0.b_fc; a.bias[3] = w0.b_proj2;
    a.ln_g[0] = w0.ln1_g; a.ln_g[1] = w0.ln2_g; a.ln_b[0] = w0.ln1_b; a.ln_b[1] = w0.ln2_b;
    a.p_stride = w1.b_qkv - w0.b_qkv;
    a.kv_pool = c->layer_pool(0); a.kv_stride = (long long)c->num_pages * (long long)c->page_floats;
    a.wte = m->wte; a.wpe = m->wpe; a.lnf_g = m->lnf_g; a.lnf_b = m->lnf_b;
    a.n_layer = m->layers_n(); a.c = m->c(); a.f = m->f(); a.v = m->v(); a.n_positions = m->positions();
    a.eps = m->cfg.layer_norm_epsilon;
    a.ids = c->d_ids; a.pos = c->d_pos; a.argmax = c->d_argmax; a.token_log = c->d_token_log;
    a.logits = c->step_wants_logits ? c->logits : nullptr;
    a.page_table = c->d_table; a.kv = c->kv;
    a.ll_x = c->d_stream_ll; a.ll_qkv = a.ll_x + 8 * C; a.ll_attn = a.ll_qkv + 8 * 3 * C; a.ll_h = a.ll_attn + 8 * C;
    a.ll_part = a.ll_h + 8 * F; a.ll_best = a.ll_part + 8 * H * 8 * 66;
    a.epoch = c->d_stream_epoch; a.error_flag = c->d_error;
    a.m = batch; a.attn_splits = m->backend.attn_splits > 8 ? 8 : m->backend.attn_splits;
    a.spin_limit = c->dbg_spin_limit; a.poison = c->dbg_poison;
#ifdef PG_DEV_TRACE
    a.trace = c->d_stream_trace;
#endif
    if (launches) *launches = 1;
    return launch_decode_stream(a, m->stream_weight_type, c->stream_grid, s);
  }
  const pg_model* m = c->model;
  const int C = m->c(), F = m->f(), V = m->v();
  const bool pdl = m->use_pdl;
  const bool fuse = m->fused_ok && batch <= 8;
  const float eps = m->cfg.layer_norm_epsilon;
  cudaError_t e;
  uint64_t n = 0;
  int cur_bucket = B_OTHER;
#define PG_E(expr)                                                       \
  do {                                                                   \
    if (prof && (e = prof->mark(s, cur_bucket)) != cudaSuccess) return e; \
    e = (expr);                                                          \
    ++n;                                                                 \
    if (e != cudaSuccess) return e;                                      \
    if (prof && (e = prof->mark(s, -1)) != cudaSuccess) return e;        \
  } while (0)
  if (m->t_wte && batch > 64 && !prof) {
    // more than 64 sequences: the same kernel once per 64 sequences, one after the other (each launch streams
    // the weights again: a step is bound by its chain of phases, not by bytes)
    bool all = true;
    for (int k = 0; k * 64 < batch && all; ++k) {
      auto prog = c->chain_programs.find(chain_program_key(std::min(64, batch - k * 64), k));
      all = prog != c->chain_programs.end() && prog->second.dev;
    }
    if (all) {
      for (int k = 0; k * 64 < batch; ++k) {
        const int rows = std::min(64, batch - k * 64);
        const auto& prog = c->chain_programs[chain_program_key(rows, k)];
        ChainArgs a = chain_base_args(c, rows, k);
        a.phases_dev = c->step_wants_logits ? prog.dev : prog.dev_argmax_only;
        a.n_phases = prog.n;
        cur_bucket = B_OTHER;
        PG_E(launch_chain(a, c->chain_ctas, s));
      }
      if (launches) *launches = n;
      return cudaSuccess;
    }
  }
  {
    auto prog = c->chain_programs.find(batch <= 64 ? chain_program_key(batch, 0) : -1);
    if (m->t_wte && prog != c->chain_programs.end() && prog->second.dev) {
      // the whole step, from the embedding to the token fed back, as one persistent cooperative kernel
      ChainArgs a = chain_base_args(c, batch);
      a.phases_dev = (c->step_wants_logits || prof) ? prog->second.dev : prog->second.dev_argmax_only;
      a.n_phases = prog->second.n;
      if (prof) a.phase_times = prog->second.d_times;  // per-phase time stamps for the operation profile
      cur_bucket = B_OTHER;
      if (prof) prof->chain_event = (int)prof->ev.size();
      PG_E(launch_chain(a, c->chain_ctas, s));
      if (launches) *launches = n;
      return cudaSuccess;
    }
  }
  PG_E(launch_embed(m->wte, m->wpe, c->d_ids, c->d_pos, c->x, batch, C, pdl, s));
  if (m->t_wte && batch > 8 && batch <= 64 && c->norm_lo) {
    // tensor-core path: every linear is three TF32 products (hi*hi + hi*lo + lo*hi) accumulated
    // in FP32; LayerNorm, attention and the GELU epilogue hand their results over as hi/lo pairs
    auto x3 = [&](const float* w, const float* bias, const float* xhi, const float* xlo, float* out, float* ohi,
                  float* olo, int n_out, int k, int epi, const float* resid) -> cudaError_t {
      TcGemmArgs a{};
      a.x = xhi; a.x_lo = xlo; a.w = w; a.bias = bias; a.resid = resid; a.out = out; a.out_hi = ohi; a.out_lo = olo;
      a.error_flag = c->d_error;
      a.m = batch; a.n = n_out; a.k = k; a.epilogue = epi;
      return launch_tc_gemm_x3(a, tc_gemm_x3_splits(n_out, k, m->num_sms), pdl, s);
    };
    for (int l = 0; l < m->layers_n(); ++l) {
      const LayerWeights& w = m->layers[l];
      cur_bucket = B_LAYER_NORM;
      PG_E(launch_layernorm_rows_split(c->x, w.ln1_g, w.ln1_b, eps, c->norm, c->norm_lo, batch, C, pdl, s));
      cur_bucket = B_QKV;
      PG_E(x3(w.t_qkv, w.b_qkv, c->norm, c->norm_lo, c->qkv, nullptr, nullptr, 3 * C, C, EPI_NONE, nullptr));
      cur_bucket = B_ATTN;
      DecodeAttnArgs at{};
      at.qkv = c->qkv; at.out = c->attn; at.out_lo = c->attn_lo; at.kv_pool = c->layer_pool(l);
      at.page_table = c->d_table; at.pos = c->d_pos; at.part = c->attn_part; at.counters = c->attn_counters;
      at.kv = c->kv; at.batch = batch; at.splits = splits;
      PG_E(launch_decode_attention(at, pdl, s));
      cur_bucket = B_ATTN_PROJ;
      PG_E(x3(w.t_proj, w.b_proj, c->attn, c->attn_lo, c->x, nullptr, nullptr, C, C, EPI_RESID, c->x));
      cur_bucket = B_LAYER_NORM;
      PG_E(launch_layernorm_rows_split(c->x, w.ln2_g, w.ln2_b, eps, c->norm, c->norm_lo, batch, C, pdl, s));
      cur_bucket = B_MLP_FC;
      PG_E(x3(w.t_fc, w.b_fc, c->norm, c->norm_lo, nullptr, c->hbuf, c->h_lo, F, C, EPI_GELU, nullptr));
      cur_bucket = B_MLP_PROJ;
      PG_E(x3(w.t_proj2, w.b_proj2, c->hbuf, c->h_lo, c->x, nullptr, nullptr, C, F, EPI_RESID, c->x));
    }
    cur_bucket = B_LAYER_NORM;
    PG_E(launch_layernorm_rows_split(c->x, m->lnf_g, m->lnf_b, eps, c->norm, c->norm_lo, batch, C, pdl, s));
    cur_bucket = B_LOGITS;
    PG_E(x3(m->t_wte, nullptr, c->norm, c->norm_lo, c->logits, nullptr, nullptr, V, C, EPI_NONE, nullptr));
    PG_E(launch_argmax_rows(c->logits, batch, V, c->d_argmax, s));
    FinalizeArgs fx{};
    fx.m = batch; fx.argmax_out = c->d_argmax; fx.next_ids = c->d_ids; fx.pos = c->d_pos;
    fx.token_log = c->d_token_log; fx.n_positions = m->positions();
    cur_bucket = B_OTHER;
    PG_E(launch_finalize(fx, pdl, s));
    if (launches) *launches = n;
    return cudaSuccess;
  }
  auto linear = [&](const float* w, const float* bias, const float* x, float* out, int n_out, int k, int epi,
                    const float* resid, const float* g, const float* b) -> cudaError_t {
    LinearArgs a{};
    a.w = w; a.bias = bias; a.x = x; a.out = out; a.resid = resid; a.eps = eps;
    a.m = batch; a.n = n_out; a.k = k;
    if (g && fuse) {
      a.ln_g = g; a.ln_b = b;
    } else if (g) {
      cudaError_t e2 = launch_layernorm_rows(x, g, b, eps, c->norm, batch, k, pdl, s);
      ++n;
      if (e2 != cudaSuccess) return e2;
      a.x = c->norm;
    }
    if (batch > 64 && k % 4 == 0) return launch_gemm_f32(a, epi, s);
    return launch_linear_decode(a, epi, pdl, s, nullptr);
  };
  for (int l = 0; l < m->layers_n(); ++l) {
    const LayerWeights& w = m->layers[l];
    cur_bucket = B_QKV;
    PG_E(linear(w.w_qkv, w.b_qkv, c->x, c->qkv, 3 * C, C, EPI_NONE, nullptr, w.ln1_g, w.ln1_b));
    cur_bucket = B_ATTN;
    DecodeAttnArgs at{};
    at.qkv = c->qkv; at.out = c->attn; at.kv_pool = c->layer_pool(l); at.page_table = c->d_table;
    at.pos = c->d_pos; at.part = c->attn_part; at.counters = c->attn_counters; at.kv = c->kv;
    at.batch = batch; at.splits = splits;
    PG_E(launch_decode_attention(at, pdl, s));
    cur_bucket = B_ATTN_PROJ;
    PG_E(linear(w.w_proj, w.b_proj, c->attn, c->x, C, C, EPI_RESID, c->x, nullptr, nullptr));
    cur_bucket = B_MLP_FC;
    PG_E(linear(w.w_fc, w.b_fc, c->x, c->hbuf, F, C, EPI_GELU, nullptr, w.ln2_g, w.ln2_b));
    cur_bucket = B_MLP_PROJ;
    PG_E(linear(w.w_proj2, w.b_proj2, c->hbuf, c->x, C, F, EPI_RESID, c->x, nullptr, nullptr));
  }
  cur_bucket = B_LOGITS;
  // final LayerNorm + tied lm_head (no bias) + argmax (rust.rs:981-1003, generation.rs:269-279)
  FinalizeArgs fa{};
  fa.m = batch; fa.argmax_out = c->d_argmax; fa.next_ids = c->d_ids; fa.pos = c->d_pos;
  fa.token_log = c->d_token_log; fa.n_positions = m->positions();
  if (fuse) {
    LinearArgs a{};
    a.w = m->head_w; a.x = c->x; a.out = c->logits; a.ln_g = m->lnf_g; a.ln_b = m->lnf_b; a.eps = eps;
    a.m = batch; a.n = V; a.k = C; a.part_val = c->part_val; a.part_idx = c->part_idx;
    int grid = 0;
    PG_E(launch_linear_decode(a, EPI_NONE, pdl, s, &grid));
    fa.part_val = c->part_val; fa.part_idx = c->part_idx; fa.parts = grid;
  } else {
    PG_E(linear(m->head_w, nullptr, c->x, c->logits, V, C, EPI_NONE, nullptr, m->lnf_g, m->lnf_b));
    PG_E(launch_argmax_rows(c->logits, batch, V, c->d_argmax, s));
  }
  cur_bucket = B_OTHER;
  PG_E(launch_finalize(fa, pdl, s));
#undef PG_E
  if (launches) *launches = n;
  return cudaSuccess;
}

static int run_decode_step(pg_cache* c, int batch) {
  const pg_model* m = c->model;
  int max_len = 0;
  for (int b = 0; b < batch; ++b) max_len = std::max(max_len, c->seq_len[b] + 1);
  const int splits = choose_splits(c, batch, max_len);
  const bool graphs = m->backend.use_graphs != 2 && !env_flag("PG_NO_GRAPHS");
  uint64_t launches = 0;
  if (m->t_wte) {
    if (int r = ensure_chain_programs(c, batch)) return r;
  }
  if (!graphs || c->dbg_poison) {
    cudaError_t e = enqueue_decode_step(c, batch, splits, c->stream, &launches);
    c->dbg_poison = c->dbg_spin_limit = 0;  // the test hook covers one step
    PG_CUDA_TRY(e);
    c->decode_launches += launches;
    return PG_OK;
  }
  auto key = std::make_pair(batch, splits * 2 + (c->step_wants_logits ? 1 : 0));
  auto it = c->graphs.find(key);
  if (it == c->graphs.end()) {
    cudaGraph_t graph = nullptr;
    PG_CUDA_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    cudaError_t e = enqueue_decode_step(c, batch, splits, c->stream, &launches);
    cudaError_t e2 = cudaStreamEndCapture(c->stream, &graph);
    if (e != cudaSuccess || e2 != cudaSuccess) {
      if (graph) cudaGraphDestroy(graph);
      cudaGetLastError();
      return set_error(PG_CUDA, std::string("decode graph capture failed: ") +
                                    cudaGetErrorString(e != cudaSuccess ? e : e2));
    }
    cudaGraphExec_t exec = nullptr;
    cudaError_t e3 = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e3 != cudaSuccess) return set_error(PG_CUDA, std::string("cudaGraphInstantiate failed: ") + cudaGetErrorString(e3));
    it = c->graphs.emplace(key, exec).first;
    c->graphs_launches[key] = launches;
  }
  PG_CUDA_TRY(cudaGraphLaunch(it->second, c->stream));
  c->decode_launches += c->graphs_launches[key];
  return PG_OK;
}


// ------------------------------------------------------------------ prefill (batched, GEMM path)
struct PrefillPlan {
  int rows = 0, batch = 0, max_len = 0;
  std::vector<int> ids, pos, slot, seq_start, last_rows;
};

static int grow_prefill_workspace(pg_cache* c, size_t rows) {
  if (rows <= c->pre_rows) return PG_OK;
  const pg_model* m = c->model;
  for (void* p : {(void*)c->px, (void*)c->pnorm, (void*)c->pqkv, (void*)c->pattn, (void*)c->ph, (void*)c->plo, (void*)c->prow})
    if (p) cudaFree(p);
  c->px = c->pnorm = c->pqkv = c->pattn = c->ph = c->plo = nullptr;
  c->prow = nullptr;
  c->pre_rows = 0;
  const size_t C = m->c(), F = m->f();
  PG_CUDA_TRY(cudaMalloc(&c->px, rows * C * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->pnorm, rows * C * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->pqkv, rows * 3 * C * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->pattn, rows * C * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->ph, rows * F * sizeof(float)));
  if (m->lo_arena) PG_CUDA_TRY(cudaMalloc(&c->plo, rows * (size_t)(C + F) * sizeof(float)));
  PG_CUDA_TRY(cudaMalloc(&c->prow, (rows * 3 + 2 * (size_t)c->max_batch + 2) * sizeof(int)));
  c->pre_rows = rows;
  return PG_OK;
}

// Runs the transformer blocks over `rows` concatenated prompt rows held in ws.x; leaves the final
// hidden states (before ln_f) in ws.x. When kv_pool_of_layer is set, K and V are scattered into
// the paged cache. block_forward, rust.rs:1053-1134.
struct BlockWorkspace {
  float *x, *norm, *qkv, *attn, *h;
  float* lo;  // FP32-grade tensor-core prefill: lo parts of the GEMM inputs, [rows, C] then [rows, F], or nullptr
  const int *d_slot, *d_pos, *d_seq_start;
  int* d_error;  // error word of the tensor-core kernels (may be nullptr: then they are not used)
};

static int run_blocks(const pg_model* m, const BlockWorkspace& ws, const PrefillPlan& plan, pg_cache* cache,
                      cudaStream_t s) {
  const int C = m->c(), F = m->f(), rows = plan.rows;
  const float eps = m->cfg.layer_norm_epsilon;
  const bool x3_mode = m->backend.math_mode == PG_MATH_TF32X3 || m->backend.math_mode == PG_MATH_BF16;
  // The FP32-grade tensor-core GEMM reads x and x - hi(x); whoever produces x (LayerNorm, attention, the GELU
  // epilogue of the MLP's first GEMM) writes the lo part along with it, so no separate pass over x is needed.
  const bool x3_rows = x3_mode && ws.lo && ws.d_error && rows >= 128 && m->lo_arena && m->head_dim() == 64 &&
                       C % 4 == 0 && C <= 4096 && tc_gemm_supported(rows, C, C) && tc_gemm_supported(rows, C, F);
  float* lo_c = x3_rows ? ws.lo : nullptr;                    // [rows, C]: LayerNorm or attention output
  float* lo_f = x3_rows ? ws.lo + (size_t)rows * C : nullptr;  // [rows, F]: MLP hidden
  auto gemm = [&](const float* w, const float* w_lo, const float* bias, const float* x, const float* x_lo, float* out,
                  float* out_lo, int n_out, int k, int epi, const float* resid) -> cudaError_t {
    LinearArgs a{};
    a.w = w; a.bias = bias; a.x = x; a.out = out; a.resid = resid; a.eps = eps;
    a.m = rows; a.n = n_out; a.k = k;
    if (rows <= 16 && k % 4 == 0) return launch_linear_decode(a, epi, false, s, nullptr);
    if (x3_rows && w_lo && x_lo) {
      // FP32-grade product on the tensor cores: x.w + x.w_lo + x_lo.w as three TF32 MMAs per k step
      TcGemmArgs t{};
      t.x = x; t.x_lo = x_lo; t.w = w; t.w_lo = w_lo; t.bias = bias; t.resid = resid; t.out = out; t.out_lo = out_lo;
      t.error_flag = ws.d_error;
      t.m = rows; t.n = n_out; t.k = k; t.epilogue = epi;
      return launch_tc_gemm_tf32x3_rows(t, s);
    }
    if (m->backend.math_mode == PG_MATH_TF32 && ws.d_error && rows >= 128 && tc_gemm_supported(rows, n_out, k)) {
      // single TF32 pass on the tensor cores: the fast prefill variant with its own looser bound
      TcGemmArgs t{};
      t.x = x; t.w = w; t.bias = bias; t.resid = resid; t.out = out; t.error_flag = ws.d_error;
      t.m = rows; t.n = n_out; t.k = k; t.epilogue = epi;
      return launch_tc_gemm_tf32(t, s);
    }
    return launch_gemm_f32(a, epi, s);
  };
  static const bool no_tc_attn = getenv("PG_NO_TC_ATTN") != nullptr;
  for (int l = 0; l < m->layers_n(); ++l) {
    const LayerWeights& w = m->layers[l];
    PG_CUDA_TRY(launch_layernorm_rows(ws.x, w.ln1_g, w.ln1_b, eps, ws.norm, rows, C, false, s, lo_c));
    PG_CUDA_TRY(gemm(w.w_qkv, w.l_qkv, w.b_qkv, ws.norm, lo_c, ws.qkv, nullptr, 3 * C, C, EPI_NONE, nullptr));
    if (cache)
      PG_CUDA_TRY(launch_kv_scatter(ws.qkv, ws.d_slot, ws.d_pos, cache->layer_pool(l), cache->d_table, cache->kv,
                                    rows, s));
    PrefillAttnArgs pa{};
    pa.qkv = ws.qkv; pa.out = ws.attn; pa.seq_start = ws.d_seq_start;
    pa.n_head = m->heads(); pa.head_dim = m->head_dim(); pa.batch = plan.batch; pa.max_len = plan.max_len;
    if (m->backend.math_mode == PG_MATH_TF32 && ws.d_error && !no_tc_attn && prefill_attention_tc_supported(pa)) {
      PG_CUDA_TRY(launch_prefill_attention_tc(pa, rows, ws.d_error, s));
    } else if (x3_rows && !no_tc_attn && prefill_attention_tc_supported(pa)) {
      pa.out_lo = lo_c;
      PG_CUDA_TRY(launch_prefill_attention_x3(pa, rows, ws.d_error, s));
    } else {
      pa.out_lo = lo_c;
      PG_CUDA_TRY(launch_prefill_attention(pa, s));
    }
    PG_CUDA_TRY(gemm(w.w_proj, w.l_proj, w.b_proj, ws.attn, lo_c, ws.x, nullptr, C, C, EPI_RESID, ws.x));
    PG_CUDA_TRY(launch_layernorm_rows(ws.x, w.ln2_g, w.ln2_b, eps, ws.norm, rows, C, false, s, lo_c));
    PG_CUDA_TRY(gemm(w.w_fc, w.l_fc, w.b_fc, ws.norm, lo_c, ws.h, lo_f, F, C, EPI_GELU, nullptr));
    PG_CUDA_TRY(gemm(w.w_proj2, w.l_proj2, w.b_proj2, ws.h, lo_f, ws.x, nullptr, C, F, EPI_RESID, ws.x));
  }
  return PG_OK;
}

static int validate_ids(const pg_model* m, const int32_t* ids, int n, bool with_index) {
  for (int i = 0; i < n; ++i)
    if (ids[i] < 0 || (uint64_t)ids[i] >= m->cfg.vocab_size)
      return set_error(PG_INVALID_INPUT, "token id " + std::to_string(ids[i]) +
                                             (with_index ? " at index " + std::to_string(i) : std::string()) +
                                             " exceeds vocab_size " + std::to_string(m->cfg.vocab_size));
  return PG_OK;
}

// validate_input, rust.rs:1029-1051
static int validate_sequence(const pg_model* m, const int32_t* ids, int n) {
  if (n <= 0) return set_error(PG_INVALID_INPUT, "input_ids must not be empty");
  if ((uint64_t)n > m->cfg.n_positions)
    return set_error(PG_INVALID_INPUT, "sequence length " + std::to_string(n) + " exceeds n_positions " +
                                           std::to_string(m->cfg.n_positions));
  return validate_ids(m, ids, n, true);
}

static int check_cache(const pg_model* m, const pg_cache* c) {
  if (!m || !c) return set_error(PG_INVALID_INPUT, "null model or cache");
  const pg_gpt2_config &a = m->cfg, &b = c->model->cfg;
  // check_compatible, rust.rs:206-234
  if (b.n_layer != a.n_layer)
    return set_error(PG_INVALID_INPUT, "cache layer count " + std::to_string(b.n_layer) + " does not match n_layer " + std::to_string(a.n_layer));
  if (b.n_positions != a.n_positions)
    return set_error(PG_INVALID_INPUT, "cache max_seq_len " + std::to_string(b.n_positions) + " does not match n_positions " + std::to_string(a.n_positions));
  if (b.n_head != a.n_head)
    return set_error(PG_INVALID_INPUT, "cache n_head " + std::to_string(b.n_head) + " does not match n_head " + std::to_string(a.n_head));
  if (b.n_embd / b.n_head != a.n_embd / a.n_head)
    return set_error(PG_INVALID_INPUT, "cache head_dim " + std::to_string(b.n_embd / b.n_head) + " does not match head_dim " + std::to_string(a.n_embd / a.n_head));
  if (c->model->device != m->device) return set_error(PG_INVALID_INPUT, "cache and model live on different devices");
  return PG_OK;
}

// After a bounded device-side wait expired (the stream is idle, d_error holds the code): puts the
// device-side synchronisation state back to what a fresh cache has, so that later launches do not
// inherit a half-passed barrier or tags of the failed step, and reports PG_TIMEOUT. The sequences in
// the cache are undefined afterwards.
static int recover_after_timeout(pg_cache* c, int code) {
  cudaMemsetAsync(c->d_error, 0, sizeof(int), c->stream);
  if (c->d_chain_barrier) cudaMemsetAsync(c->d_chain_barrier, 0, sizeof(unsigned), c->stream);
  if (c->d_chain_best) {
    const std::vector<unsigned long long> init(64, chain_argmax_init());
    cudaMemcpyAsync(c->d_chain_best, init.data(), init.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice, c->stream);
  }
  cudaMemsetAsync(c->attn_counters, 0, (size_t)c->max_batch * c->model->heads() * sizeof(unsigned), c->stream);
  if (c->d_stream_epoch) {
    // tags of the failed step may sit in the exchange buffers: move the counter far past them
    unsigned e = 0;
    cudaMemcpyAsync(&e, c->d_stream_epoch, sizeof(unsigned), cudaMemcpyDeviceToHost, c->stream);
    cudaStreamSynchronize(c->stream);
    e += 1u << 20;
    cudaMemcpyAsync(c->d_stream_epoch, &e, sizeof(unsigned), cudaMemcpyHostToDevice, c->stream);
  }
  cudaStreamSynchronize(c->stream);
  cudaGetLastError();
  return set_error(PG_TIMEOUT, "a bounded wait inside a device kernel expired (code " + std::to_string(code) +
                                   "); the cache's sequences are undefined until it is cleared");
}

// Reads the error word of the finished stream work; PG_TIMEOUT (after recovery) when it is set.
static int check_device_error(pg_cache* c) {
  int* h_err = c->h_out + (size_t)c->max_batch * (1 + 2 * MAX_TOPK);
  PG_CUDA_TRY(cudaMemcpyAsync(h_err, c->d_error, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  PG_CUDA_TRY(cudaStreamSynchronize(c->stream));
  if (*h_err) return recover_after_timeout(c, *h_err);
  return PG_OK;
}

// Copies the requested results of the last step to the host and waits for the stream.
static int fetch_outputs(pg_cache* c, int batch, float* logits_out, int32_t* argmax_out, float* topk_vals,
                         int32_t* topk_idx, int k) {
  const int V = c->model->v();
  if (k > 0 && (topk_vals || topk_idx)) {
    PG_CUDA_TRY(launch_topk_rows(c->logits, batch, V, k, c->topk_vals, c->topk_idx, c->stream));
    float* hv = reinterpret_cast<float*>(c->h_out + c->max_batch);
    int* hi = c->h_out + c->max_batch + (size_t)c->max_batch * MAX_TOPK;
    PG_CUDA_TRY(cudaMemcpyAsync(hv, c->topk_vals, (size_t)batch * k * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    PG_CUDA_TRY(cudaMemcpyAsync(hi, c->topk_idx, (size_t)batch * k * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  }
  if (argmax_out)
    PG_CUDA_TRY(cudaMemcpyAsync(c->h_out, c->d_argmax, batch * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  if (logits_out)
    PG_CUDA_TRY(cudaMemcpyAsync(logits_out, c->logits, (size_t)batch * V * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  int* h_err = c->h_out + (size_t)c->max_batch * (1 + 2 * MAX_TOPK);
  PG_CUDA_TRY(cudaMemcpyAsync(h_err, c->d_error, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  PG_CUDA_TRY(cudaStreamSynchronize(c->stream));
  if (*h_err) return recover_after_timeout(c, *h_err);
  if (argmax_out) memcpy(argmax_out, c->h_out, batch * sizeof(int));
  if (k > 0 && topk_vals) memcpy(topk_vals, c->h_out + c->max_batch, (size_t)batch * k * sizeof(float));
  if (k > 0 && topk_idx) memcpy(topk_idx, c->h_out + c->max_batch + (size_t)c->max_batch * MAX_TOPK, (size_t)batch * k * sizeof(int));
  return PG_OK;
}

static int do_prefill(const pg_model* m, pg_cache* c, const int32_t* ids, const int32_t* lens, int batch,
                      float* logits_out, int32_t* argmax_out) {
  if (int r = check_cache(m, c)) return r;
  if (batch <= 0 || batch > c->max_batch)
    return set_error(PG_INVALID_INPUT, "batch " + std::to_string(batch) + " exceeds the cache's max_batch " + std::to_string(c->max_batch));
  if (!ids || !lens) return set_error(PG_INVALID_INPUT, "null ids or lens");
  PrefillPlan plan;
  plan.batch = batch;
  plan.seq_start.push_back(0);
  {
    int off = 0;
    for (int b = 0; b < batch; ++b) {
      if (int r = validate_sequence(m, ids + off, lens[b])) return r;
      off += lens[b];
      plan.seq_start.push_back(off);
      plan.max_len = std::max(plan.max_len, lens[b]);
      plan.last_rows.push_back(off - 1);
    }
    plan.rows = off;
  }
  PG_CUDA_TRY(cudaSetDevice(m->device));
  // KvCache::clear for these slots, then pages for the whole prompt
  for (int b = 0; b < batch; ++b) {
    release_slot_pages(c, b);
    c->seq_len[b] = 0;
  }
  for (int b = 0; b < batch; ++b)
    if (int r = ensure_pages(c, b, lens[b])) return r;
  if (int r = sync_table(c)) return r;
  if (int r = grow_prefill_workspace(c, plan.rows)) return r;
  plan.ids.assign(ids, ids + plan.rows);
  for (int b = 0; b < batch; ++b)
    for (int t = 0; t < lens[b]; ++t) {
      plan.pos.push_back(t);
      plan.slot.push_back(b);
    }
  const size_t R = plan.rows;
  int* d_ids = c->prow;
  int* d_pos = c->prow + R;
  int* d_slot = c->prow + 2 * R;
  int* d_start = c->prow + 3 * R;
  int* d_last = d_start + batch + 1;
  cudaStream_t s = c->stream;
  PG_CUDA_TRY(cudaMemcpyAsync(d_ids, plan.ids.data(), R * sizeof(int), cudaMemcpyHostToDevice, s));
  PG_CUDA_TRY(cudaMemcpyAsync(d_pos, plan.pos.data(), R * sizeof(int), cudaMemcpyHostToDevice, s));
  PG_CUDA_TRY(cudaMemcpyAsync(d_slot, plan.slot.data(), R * sizeof(int), cudaMemcpyHostToDevice, s));
  PG_CUDA_TRY(cudaMemcpyAsync(d_start, plan.seq_start.data(), (batch + 1) * sizeof(int), cudaMemcpyHostToDevice, s));
  PG_CUDA_TRY(cudaMemcpyAsync(d_last, plan.last_rows.data(), batch * sizeof(int), cudaMemcpyHostToDevice, s));
  PG_CUDA_TRY(launch_embed(m->wte, m->wpe, d_ids, d_pos, c->px, plan.rows, m->c(), false, s));
  BlockWorkspace ws{c->px, c->pnorm, c->pqkv, c->pattn, c->ph, c->plo, d_slot, d_pos, d_start, c->d_error};
  if (int r = run_blocks(m, ws, plan, c, s)) return r;
  // last position of each prompt -> ln_f -> lm_head (the reference computes logits for every
  // prompt token and keeps the last, rust.rs:920-926; only the last is observable)
  PG_CUDA_TRY(launch_gather_rows(c->px, d_last, c->x, batch, m->c(), s));
  PG_CUDA_TRY(launch_layernorm_rows(c->x, m->lnf_g, m->lnf_b, m->cfg.layer_norm_epsilon, c->norm, batch, m->c(), false, s));
  LinearArgs a{};
  a.w = m->head_w; a.x = c->norm; a.out = c->logits; a.m = batch; a.n = m->v(); a.k = m->c();
  if (batch > 64 && a.k % 4 == 0) PG_CUDA_TRY(launch_gemm_f32(a, EPI_NONE, s));
  else PG_CUDA_TRY(launch_linear_decode(a, EPI_NONE, false, s, nullptr));
  PG_CUDA_TRY(launch_argmax_rows(c->logits, batch, m->v(), c->d_argmax, s));
  // device-side sequence state: pos = lens, next id = argmax
  PG_CUDA_TRY(cudaMemcpyAsync(c->d_pos, lens, batch * sizeof(int), cudaMemcpyHostToDevice, s));
  PG_CUDA_TRY(cudaMemcpyAsync(c->d_ids, c->d_argmax, batch * sizeof(int), cudaMemcpyDeviceToDevice, s));
  if (int r = fetch_outputs(c, batch, logits_out, argmax_out, nullptr, nullptr, 0)) return r;
  for (int b = 0; b < batch; ++b) c->seq_len[b] = lens[b];
  return PG_OK;
}

// Validates and stages one decode step; `ids` may be null to keep the ids already on the device.
static int prepare_step(const pg_model* m, pg_cache* c, const int32_t* ids, int batch) {
  if (int r = check_cache(m, c)) return r;
  if (batch <= 0 || batch > c->max_batch)
    return set_error(PG_INVALID_INPUT, "batch " + std::to_string(batch) + " exceeds the cache's max_batch " + std::to_string(c->max_batch));
  if (ids)
    if (int r = validate_ids(m, ids, batch, false)) return r;
  for (int b = 0; b < batch; ++b)
    if (c->seq_len[b] >= m->positions())
      return set_error(PG_INVALID_INPUT, "cache is full at seq_len " + std::to_string(c->seq_len[b]));
  PG_CUDA_TRY(cudaSetDevice(m->device));
  for (int b = 0; b < batch; ++b)
    if (int r = ensure_pages(c, b, c->seq_len[b] + 1)) return r;
  if (int r = sync_table(c)) return r;
  if (ids) {
    memcpy(c->h_ids, ids, batch * sizeof(int));
    PG_CUDA_TRY(cudaMemcpyAsync(c->d_ids, c->h_ids, batch * sizeof(int), cudaMemcpyHostToDevice, c->stream));
  }
  return PG_OK;
}

static int do_forward_one(const pg_model* m, pg_cache* c, const int32_t* ids, int batch, float* logits_out,
                          int32_t* argmax_out, float* topk_vals, int32_t* topk_idx, int k) {
  if (!ids) return set_error(PG_INVALID_INPUT, "null ids");
  if (k < 0 || k > MAX_TOPK) return set_error(PG_INVALID_INPUT, "k must be in 0.." + std::to_string(MAX_TOPK));
  if (int r = prepare_step(m, c, ids, batch)) return r;
  c->step_wants_logits = logits_out != nullptr || k > 0;
  if (int r = run_decode_step(c, batch)) return r;
  for (int b = 0; b < batch; ++b) c->seq_len[b] += 1;
  return fetch_outputs(c, batch, logits_out, argmax_out, topk_vals, topk_idx, k);
}

// Device buffers and stream of the cache-less full-sequence forward, sized for `rows` positions and re-used
// from call to call (generate_greedy runs one forward per token).
struct ForwardWorkspace {
  size_t rows = 0, out_rows = 0;
  float *x = nullptr, *norm = nullptr, *qkv = nullptr, *attn = nullptr, *h = nullptr, *logits = nullptr;
  int* meta = nullptr;
  cudaStream_t s = nullptr;
  ~ForwardWorkspace() {
    if (s) cudaStreamSynchronize(s);
    for (void* p : {(void*)x, (void*)norm, (void*)qkv, (void*)attn, (void*)h, (void*)logits, (void*)meta})
      if (p) cudaFree(p);
    if (s) cudaStreamDestroy(s);
  }
  int reserve(const pg_model* m, size_t r, size_t o) {
    if (!s) PG_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    const size_t C = m->c(), F = m->f(), V = m->v();
    if (r > rows) {
      for (void* p : {(void*)x, (void*)norm, (void*)qkv, (void*)attn, (void*)h, (void*)meta})
        if (p) cudaFree(p);
      x = norm = qkv = attn = h = nullptr;
      meta = nullptr;
      rows = 0;
      PG_CUDA_TRY(cudaMalloc(&x, r * C * sizeof(float)));
      PG_CUDA_TRY(cudaMalloc(&norm, r * C * sizeof(float)));
      PG_CUDA_TRY(cudaMalloc(&qkv, r * 3 * C * sizeof(float)));
      PG_CUDA_TRY(cudaMalloc(&attn, r * C * sizeof(float)));
      PG_CUDA_TRY(cudaMalloc(&h, r * F * sizeof(float)));
      PG_CUDA_TRY(cudaMalloc(&meta, (2 * r + 2) * sizeof(int)));
      rows = r;
    }
    if (o > out_rows) {
      if (logits) cudaFree(logits);
      logits = nullptr;
      out_rows = 0;
      PG_CUDA_TRY(cudaMalloc(&logits, o * V * sizeof(float)));
      out_rows = o;
    }
    return PG_OK;
  }
};

// Full-sequence forward without a cache (Gpt2Model::forward, rust.rs:831-882). When
// `last_only`, only the last position's logits are produced (what generate_greedy consumes).
// `reserve_rows`: positions the workspace should be sized for when it has to grow.
static int do_forward(const pg_model* m, const int32_t* ids, int t, float* logits_out, bool last_only,
                      ForwardWorkspace& ws, size_t reserve_rows) {
  if (!m) return set_error(PG_INVALID_INPUT, "null model");
  if (int r = validate_sequence(m, ids, t)) return r;
  if (int r = ensure_device(m->device)) return r;
  const size_t C = m->c(), V = m->v(), R = t;
  const size_t out_rows = last_only ? 1 : R;
  if (int r = ws.reserve(m, std::max(R, reserve_rows), out_rows)) return r;
  cudaStream_t s = ws.s;
  PrefillPlan plan;
  plan.rows = t; plan.batch = 1; plan.max_len = t;
  std::vector<int> hm(2 * R + 2);
  for (int i = 0; i < t; ++i) {
    hm[i] = ids[i];
    hm[R + i] = i;
  }
  hm[2 * R] = 0;
  hm[2 * R + 1] = t;
  PG_CUDA_TRY(cudaMemcpyAsync(ws.meta, hm.data(), hm.size() * sizeof(int), cudaMemcpyHostToDevice, s));
  PG_CUDA_TRY(launch_embed(m->wte, m->wpe, ws.meta, ws.meta + R, ws.x, t, (int)C, false, s));
  BlockWorkspace bw{ws.x, ws.norm, ws.qkv, ws.attn, ws.h, nullptr, nullptr, ws.meta + R, ws.meta + 2 * R, nullptr};
  if (int r = run_blocks(m, bw, plan, nullptr, s)) return r;
  const float* hidden = last_only ? ws.x + (R - 1) * C : ws.x;
  PG_CUDA_TRY(launch_layernorm_rows(hidden, m->lnf_g, m->lnf_b, m->cfg.layer_norm_epsilon, ws.norm, (int)out_rows, (int)C, false, s));
  LinearArgs a{};
  a.w = m->head_w; a.x = ws.norm; a.out = ws.logits; a.m = (int)out_rows; a.n = (int)V; a.k = (int)C;
  if (out_rows > 16 && C % 4 == 0) PG_CUDA_TRY(launch_gemm_f32(a, EPI_NONE, s));
  else PG_CUDA_TRY(launch_linear_decode(a, EPI_NONE, false, s, nullptr));
  PG_CUDA_TRY(cudaMemcpyAsync(logits_out, ws.logits, out_rows * V * sizeof(float), cudaMemcpyDeviceToHost, s));
  PG_CUDA_TRY(cudaStreamSynchronize(s));  // also keeps `hm` alive long enough
  return PG_OK;
}

static double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace pg

// ================================================================== C ABI
extern "C" {

const char* pg_last_error_message(void) { return last_error_cstr(); }
const char* pg_version(void) { return "puppygrad_b200 0.1 (sm_100a)"; }

int pg_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int pg_config_validate(const pg_gpt2_config* cfg) {
  if (!cfg) return set_error(PG_INVALID_CONFIG, "null config");
  return validate_config(*cfg);
}

int pg_config_load_json(const char* path, pg_gpt2_config* out) {
  if (!path || !out) return set_error(PG_ASSET, "null path or output");
  return load_config_json(path, out);
}

void pg_backend_config_default(pg_backend_config* out) {
  if (!out) return;
  memset(out, 0, sizeof(*out));
  out->page_tokens = 32;
}

int pg_model_from_host_weights(const pg_gpt2_config* cfg, const float* const* tensors, const uint64_t* lens,
                               uint64_t n_tensors, const pg_backend_config* backend, pg_model** out) {
  if (!cfg || !tensors || !lens || !out) return set_error(PG_INVALID_INPUT, "null argument");
  return build_model(*cfg, tensors, lens, n_tensors, backend, out);
}

int pg_model_load_dir(const char* dir, const pg_backend_config* backend, pg_model** out) {
  if (!dir || !out) return set_error(PG_ASSET, "null directory or output");
  std::string d(dir);
  pg_gpt2_config cfg{};
  if (int r = load_config_json(d + "/config.json", &cfg)) return r;
  HostWeights hw;
  if (int r = load_weights_safetensors(d + "/model.safetensors", cfg, &hw)) return r;
  return build_model(cfg, hw.ptrs.data(), hw.lens.data(), hw.ptrs.size(), backend, out);
}

int pg_model_config(const pg_model* model, pg_gpt2_config* out) {
  if (!model || !out) return set_error(PG_INVALID_INPUT, "null argument");
  *out = model->cfg;
  return PG_OK;
}

uint64_t pg_model_max_context_len(const pg_model* model) { return model ? model->cfg.n_positions : 0; }

uint64_t pg_model_weight_bytes_per_step(const pg_model* model) {
  if (!model) return 0;
  const pg_gpt2_config& c = model->cfg;
  // every block matrix, bias and LayerNorm vector once; the tied embedding once as lm_head;
  // ln_f; one wte row and one wpe row are negligible and not counted. With BF16 / int8 weights the
  // matrices and the lm_head count at their narrow size (what decode steps of at most 8 sequences read),
  // int8 with one FP32 scale per row
  const uint64_t dense = c.n_embd * 3 * c.n_embd + c.n_embd * c.n_embd + 2 * c.n_embd * c.n_inner;
  const uint64_t dense_rows = 3 * c.n_embd + c.n_embd + c.n_inner + c.n_embd;
  const uint64_t vectors = 3 * c.n_embd + c.n_embd + c.n_inner + c.n_embd + 4 * c.n_embd;
  const uint64_t eb = model->stream_weight_type == STREAM_W_F32 ? 4 : model->stream_weight_type == STREAM_W_BF16 ? 2 : 1;
  const uint64_t scales = model->stream_weight_type == STREAM_W_I8 ? 4 : 0;
  return c.n_layer * (dense * eb + dense_rows * scales + vectors * 4) + c.vocab_size * (c.n_embd * eb + scales) +
         2 * c.n_embd * 4;
}

void pg_model_free(pg_model* model) { delete model; }

int pg_cache_new(const pg_model* model, int32_t max_batch, pg_cache** out) {
  if (!model || !out) return set_error(PG_INVALID_INPUT, "null argument");
  return cache_new(model, max_batch, out);
}

int pg_cache_clear(pg_cache* cache) {
  if (!cache) return set_error(PG_INVALID_INPUT, "null cache");
  for (int b = 0; b < cache->max_batch; ++b) {
    release_slot_pages(cache, b);
    cache->seq_len[b] = 0;
  }
  PG_CUDA_TRY(cudaSetDevice(cache->model->device));
  PG_CUDA_TRY(cudaMemsetAsync(cache->d_pos, 0, cache->max_batch * sizeof(int), cache->stream));
  PG_CUDA_TRY(cudaStreamSynchronize(cache->stream));
  return PG_OK;
}

int pg_cache_clear_slot(pg_cache* cache, int32_t slot) {
  if (!cache) return set_error(PG_INVALID_INPUT, "null cache");
  if (slot < 0 || slot >= cache->max_batch) return set_error(PG_INVALID_INPUT, "slot out of range");
  release_slot_pages(cache, slot);
  cache->seq_len[slot] = 0;
  PG_CUDA_TRY(cudaSetDevice(cache->model->device));
  PG_CUDA_TRY(cudaMemsetAsync(cache->d_pos + slot, 0, sizeof(int), cache->stream));
  PG_CUDA_TRY(cudaStreamSynchronize(cache->stream));
  return PG_OK;
}

int pg_cache_seq_len(const pg_cache* cache, int32_t slot, uint64_t* out) {
  if (!cache || !out) return set_error(PG_INVALID_INPUT, "null argument");
  if (slot < 0 || slot >= cache->max_batch) return set_error(PG_INVALID_INPUT, "slot out of range");
  *out = (uint64_t)cache->seq_len[slot];
  return PG_OK;
}

uint64_t pg_cache_max_seq_len(const pg_cache* cache) { return cache ? cache->model->cfg.n_positions : 0; }
int32_t pg_cache_max_batch(const pg_cache* cache) { return cache ? cache->max_batch : 0; }

int pg_cache_read_layer(const pg_cache* cache, int32_t slot, uint64_t layer, float* keys, float* values) {
  if (!cache || !keys || !values) return set_error(PG_INVALID_INPUT, "null argument");
  if (slot < 0 || slot >= cache->max_batch) return set_error(PG_INVALID_INPUT, "slot out of range");
  if (layer >= cache->model->cfg.n_layer) return set_error(PG_INVALID_INPUT, "layer out of range");
  const pg_model* m = cache->model;
  PG_CUDA_TRY(cudaSetDevice(m->device));
  size_t n = (size_t)m->positions() * m->c();
  float *dk = nullptr, *dv = nullptr;
  PG_CUDA_TRY(cudaMalloc(&dk, 2 * n * sizeof(float)));
  dv = dk + n;
  pg_cache* c = const_cast<pg_cache*>(cache);
  int rc = sync_table(c);
  cudaError_t e = cudaSuccess;
  if (rc == PG_OK) {
    e = launch_kv_gather(cache->layer_pool((int)layer), cache->d_table, cache->kv, slot, cache->seq_len[slot],
                         m->positions(), dk, dv, cache->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(keys, dk, n * sizeof(float), cudaMemcpyDeviceToHost, cache->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(values, dv, n * sizeof(float), cudaMemcpyDeviceToHost, cache->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(cache->stream);
  }
  cudaFree(dk);
  if (rc != PG_OK) return rc;
  if (e != cudaSuccess) return set_error(PG_CUDA, std::string("CUDA error: ") + cudaGetErrorString(e));
  return PG_OK;
}

void pg_cache_free(pg_cache* cache) { delete cache; }

int pg_prefill(const pg_model* model, pg_cache* cache, const int32_t* ids, const int32_t* lens, int32_t batch,
               float* logits_out, int32_t* argmax_out) {
  return do_prefill(model, cache, ids, lens, batch, logits_out, argmax_out);
}

int pg_forward_one(const pg_model* model, pg_cache* cache, const int32_t* ids, int32_t batch, float* logits_out,
                   int32_t* argmax_out, float* topk_vals, int32_t* topk_idx, int32_t k) {
  return do_forward_one(model, cache, ids, batch, logits_out, argmax_out, topk_vals, topk_idx, k);
}

int pg_forward(const pg_model* model, const int32_t* ids, int32_t t, float* logits_out) {
  if (!logits_out) return set_error(PG_INVALID_INPUT, "null logits_out");
  ForwardWorkspace ws;
  return do_forward(model, ids, t, logits_out, false, ws, 0);
}

int pg_decode_greedy(const pg_model* model, pg_cache* cache, const int32_t* first_ids, int32_t batch,
                     int32_t steps, int32_t* tokens_out) {
  if (!first_ids || !tokens_out) return set_error(PG_INVALID_INPUT, "null argument");
  if (steps <= 0) return set_error(PG_INVALID_INPUT, "steps must be > 0");
  if (int r = check_cache(model, cache)) return r;
  if (batch <= 0 || batch > cache->max_batch)
    return set_error(PG_INVALID_INPUT, "batch " + std::to_string(batch) + " exceeds the cache's max_batch " + std::to_string(cache->max_batch));
  for (int b = 0; b < batch; ++b)
    if (cache->seq_len[b] + steps > model->positions())
      return set_error(PG_INVALID_INPUT, "cache is full at seq_len " + std::to_string(model->positions()));
  std::vector<int> start(cache->seq_len.begin(), cache->seq_len.begin() + batch);
  // pages for the whole run now: one page-table upload instead of a host round trip at every page boundary
  PG_CUDA_TRY(cudaSetDevice(model->device));
  for (int b = 0; b < batch; ++b)
    if (int r = ensure_pages(cache, b, cache->seq_len[b] + steps)) return r;
  if (int r = sync_table(cache)) return r;
  for (int s = 0; s < steps; ++s) {
    if (int r = prepare_step(model, cache, s == 0 ? first_ids : nullptr, batch)) return r;
    cache->step_wants_logits = false;
    if (int r = run_decode_step(cache, batch)) return r;
    for (int b = 0; b < batch; ++b) cache->seq_len[b] += 1;
  }
  // the step at position p logs its argmax at token_log[b][p + 1]
  const int P = model->positions();
  std::vector<int> log((size_t)batch * P);
  PG_CUDA_TRY(cudaMemcpyAsync(log.data(), cache->d_token_log, log.size() * sizeof(int), cudaMemcpyDeviceToHost, cache->stream));
  if (int r = check_device_error(cache)) return r;  // also waits for the stream
  for (int s = 0; s < steps; ++s)
    for (int b = 0; b < batch; ++b) {
      int p = start[b] + s + 1;
      tokens_out[(size_t)s * batch + b] = p < P ? log[(size_t)b * P + p] : -1;
    }
  bool fills = false;
  for (int b = 0; b < batch; ++b) fills = fills || start[b] + steps >= P;
  if (fills) {
    // the last loggable position is P-1; a step that fills the cache reports its argmax directly
    std::vector<int> last(batch);
    PG_CUDA_TRY(cudaMemcpy(last.data(), cache->d_argmax, batch * sizeof(int), cudaMemcpyDeviceToHost));
    for (int b = 0; b < batch; ++b)
      if (start[b] + steps >= P) tokens_out[(size_t)(steps - 1) * batch + b] = last[b];
  }
  return PG_OK;
}

int pg_profile_forward_one(const pg_model* model, pg_cache* cache, const int32_t* ids, int32_t batch,
                           pg_operation_profile* out) {
  if (!ids || !out) return set_error(PG_INVALID_INPUT, "null argument");
  if (int r = prepare_step(model, cache, ids, batch)) return r;
  int max_len = 0;
  for (int b = 0; b < batch; ++b) max_len = std::max(max_len, cache->seq_len[b] + 1);
  StepProfiler prof;
  uint64_t launches = 0;
  PG_CUDA_TRY(enqueue_decode_step(cache, batch, choose_splits(cache, batch, max_len), cache->stream, &launches, &prof));
  for (int b = 0; b < batch; ++b) cache->seq_len[b] += 1;
  if (int r = check_device_error(cache)) return r;  // also waits for the stream
  cache->decode_launches += launches;
  double sec[B_COUNT] = {0};
  uint64_t cnt[B_COUNT] = {0};
  for (size_t i = 0; i + 1 < prof.ev.size(); i += 2) {
    float ms = 0.f;
    PG_CUDA_TRY(cudaEventElapsedTime(&ms, prof.ev[i], prof.ev[i + 1]));
    sec[prof.bucket[i]] += ms * 1e-3;
    cnt[prof.bucket[i]] += 1;
  }
  double fused_sec = 0.0;
  uint64_t fused_phases = 0;
  if (prof.chain_event >= 0) {
    {
      float ms = 0.f;
      PG_CUDA_TRY(cudaEventElapsedTime(&ms, prof.ev[prof.chain_event], prof.ev[prof.chain_event + 1]));
      fused_sec = ms * 1e-3;
    }
    // the chain kernel's own time stamps split its duration into the operation buckets; what the
    // stamps do not cover (launch, set-up, exit) stays in `other`
    auto it = cache->chain_programs.find(batch);
    if (it != cache->chain_programs.end() && it->second.d_times) {
      std::vector<unsigned long long> ts((size_t)it->second.n + 1);
      PG_CUDA_TRY(cudaMemcpy(ts.data(), it->second.d_times, ts.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
      double covered = 0.0;
#ifdef PG_DEV_TRACE
      const bool dump = env_flag("PG_PHASE_DUMP");  // tuning aid: every phase's duration
#else
      constexpr bool dump = false;
#endif
      for (int p = 0; p < it->second.n; ++p) {
        const double d = (double)(ts[p + 1] - ts[p]) * 1e-9;
        if (dump) fprintf(stderr, "phase %3d bucket %d %8.2f us\n", p, it->second.bucket[p], d * 1e6);
        sec[it->second.bucket[p]] += d;
        cnt[it->second.bucket[p]] += 1;
        covered += d;
      }
      sec[B_OTHER] = std::max(0.0, sec[B_OTHER] - covered);
      fused_phases = (uint64_t)it->second.n;
    }
  }
  memset(out, 0, sizeof(*out));
  out->layer_norm = sec[B_LAYER_NORM]; out->qkv_projection = sec[B_QKV]; out->attention = sec[B_ATTN];
  out->attention_projection = sec[B_ATTN_PROJ]; out->mlp_fc_projection = sec[B_MLP_FC];
  out->mlp_projection = sec[B_MLP_PROJ]; out->final_logits = sec[B_LOGITS]; out->other = sec[B_OTHER];
  const Bucket order[8] = {B_LAYER_NORM, B_QKV, B_ATTN, B_ATTN_PROJ, B_MLP_FC, B_MLP_PROJ, B_LOGITS, B_OTHER};
  for (int i = 0; i < 8; ++i) out->launches[i] = cnt[order[i]];
  out->fused_step_kernel = fused_sec;
  out->fused_phases = fused_phases;
  return PG_OK;
}

int pg_cache_time_begin(pg_cache* cache) {
  if (!cache) return set_error(PG_INVALID_INPUT, "null cache");
  PG_CUDA_TRY(cudaSetDevice(cache->model->device));
  if (!cache->t0) {
    PG_CUDA_TRY(cudaEventCreate(&cache->t0));
    PG_CUDA_TRY(cudaEventCreate(&cache->t1));
  }
  PG_CUDA_TRY(cudaStreamSynchronize(cache->stream));
  PG_CUDA_TRY(cudaEventRecord(cache->t0, cache->stream));
  return PG_OK;
}

int pg_cache_time_end(pg_cache* cache, double* seconds) {
  if (!cache || !seconds) return set_error(PG_INVALID_INPUT, "null argument");
  if (!cache->t0) return set_error(PG_INVALID_INPUT, "pg_cache_time_begin was not called");
  PG_CUDA_TRY(cudaEventRecord(cache->t1, cache->stream));
  PG_CUDA_TRY(cudaEventSynchronize(cache->t1));
  float ms = 0.f;
  PG_CUDA_TRY(cudaEventElapsedTime(&ms, cache->t0, cache->t1));
  *seconds = ms * 1e-3;
  return PG_OK;
}

uint64_t pg_cache_kernel_launches(const pg_cache* cache) { return cache ? cache->decode_launches : 0; }

int pg_cache_debug_expire_next_wait(pg_cache* cache, uint32_t spin_limit) {
  if (!cache) return set_error(PG_INVALID_INPUT, "null cache");
  if (spin_limit == 0 || spin_limit > (1u << 20))
    return set_error(PG_INVALID_INPUT, "spin_limit must be in 1..1048576");
  cache->dbg_spin_limit = spin_limit;
  cache->dbg_poison = 0x5a5a5a5au;
  return PG_OK;
}

int pg_generate_greedy(const pg_model* model, const int32_t* ids, int32_t n_ids, uint64_t max_new_tokens,
                       int32_t* out_tokens, uint64_t* out_len) {
  if (!model || !out_tokens || !out_len) return set_error(PG_INVALID_INPUT, "null argument");
  if (int r = validate_sequence(model, ids, n_ids)) return r;
  std::vector<int32_t> tokens(ids, ids + n_ids);
  std::vector<float> logits(model->cfg.vocab_size);
  ForwardWorkspace ws;  // one set of buffers for every token of this call
  const size_t longest = std::min<uint64_t>(model->cfg.n_positions, (uint64_t)n_ids + max_new_tokens);
  for (uint64_t i = 0; i < max_new_tokens; ++i) {
    if (tokens.size() >= model->cfg.n_positions) break;
    if (int r = do_forward(model, tokens.data(), (int)tokens.size(), logits.data(), true, ws, longest)) return r;
    tokens.push_back((int32_t)argmax_logits(logits.data(), logits.size()));
  }
  memcpy(out_tokens, tokens.data(), tokens.size() * sizeof(int32_t));
  *out_len = tokens.size();
  return PG_OK;
}

int pg_stream_greedy_tokens(const pg_model* model, const int32_t* ids, int32_t n_ids, uint64_t max_new_tokens,
                            pg_token_callback on_token, void* user, int32_t* out_tokens, uint64_t* out_len) {
  if (!model || !out_tokens || !out_len) return set_error(PG_INVALID_INPUT, "null argument");
  pg_cache* cache = nullptr;
  if (int r = cache_new(model, 1, &cache)) return r;
  std::unique_ptr<pg_cache> guard(cache);
  int32_t next = 0;
  if (int r = do_prefill(model, cache, ids, &n_ids, 1, nullptr, &next)) return r;
  std::vector<int32_t> tokens(ids, ids + n_ids);
  for (uint64_t i = 0; i < max_new_tokens; ++i) {
    if (tokens.size() >= model->cfg.n_positions) break;
    tokens.push_back(next);
    if (on_token && on_token((uint64_t)next, user)) return set_error(PG_INVALID_INPUT, "token callback aborted generation");
    // the reference also runs forward_one after the final token; its logits are never used
    if (i + 1 < max_new_tokens && tokens.size() < model->cfg.n_positions) {
      int32_t cur = next;
      if (int r = do_forward_one(model, cache, &cur, 1, nullptr, &next, nullptr, nullptr, 0)) return r;
    }
  }
  memcpy(out_tokens, tokens.data(), tokens.size() * sizeof(int32_t));
  *out_len = tokens.size();
  return PG_OK;
}

int pg_generate_with_config(const pg_model* model, const int32_t* ids, int32_t n_ids, const pg_generation_config* cfg,
                            pg_token_callback on_token, void* user, int32_t* out_tokens, uint64_t* out_len,
                            pg_generation_stats* stats) {
  if (!model || !cfg || !out_tokens || !out_len) return set_error(PG_INVALID_INPUT, "null argument");
  if (int r = validate_generation_config(*cfg)) return r;
  const double t_start = now_s();
  pg_cache* cache = nullptr;
  if (int r = cache_new(model, 1, &cache)) return r;
  std::unique_ptr<pg_cache> guard(cache);
  const size_t V = model->cfg.vocab_size;
  const bool penalty = !(cfg->repeat_penalty == 1.0f || cfg->repeat_last_n == 0);
  const bool greedy = cfg->temperature <= 0.0f;
  // what each step must bring back from the device
  const bool use_argmax = greedy && !penalty;
  // the device top-k keeps one key per vocabulary entry in shared memory; larger vocabularies sample on the host
  const bool use_topk = !greedy && !penalty && cfg->top_k > 0 && cfg->top_k <= MAX_TOPK && V * sizeof(int) <= 220 * 1024;
  const int k = use_topk ? (int)cfg->top_k : 0;
  std::vector<float> logits(use_argmax || use_topk ? 0 : V);
  std::vector<float> tv(k);
  std::vector<int32_t> ti(k);
  int32_t am = 0;
  pg_sampler sampler(cfg->seed);
  std::vector<uint64_t> history(ids, ids + std::max(n_ids, 0));
  const double t_prefill = now_s();
  if (int r = do_prefill(model, cache, ids, &n_ids, 1, logits.empty() ? nullptr : logits.data(), &am)) return r;
  if (use_topk)
    if (int r = fetch_outputs(cache, 1, nullptr, nullptr, tv.data(), ti.data(), k)) return r;
  const double t_decode = now_s();
  double first_token = -1.0;
  uint64_t generated = 0;
  for (uint64_t i = 0; i < cfg->max_new_tokens; ++i) {
    if (history.size() >= model->cfg.n_positions) break;
    uint64_t next = 0;
    if (use_argmax) next = (uint64_t)am;
    else if (use_topk) {
      if (int r = sampler.select_from_sorted(tv.data(), ti.data(), k, *cfg, &next)) return r;
    } else if (int r = sampler.select_next_token(logits.data(), V, history.data(), history.size(), *cfg, &next)) return r;
    if (cfg->eos_token_id >= 0 && next == (uint64_t)cfg->eos_token_id) break;
    history.push_back(next);
    out_tokens[generated++] = (int32_t)next;
    if (first_token < 0) first_token = now_s() - t_start;
    if (on_token && on_token(next, user)) return set_error(PG_INVALID_INPUT, "token callback aborted generation");
    const bool needs_next = i + 1 < cfg->max_new_tokens && history.size() < model->cfg.n_positions;
    if (needs_next) {
      int32_t cur = (int32_t)next;
      if (int r = do_forward_one(model, cache, &cur, 1, logits.empty() ? nullptr : logits.data(), &am,
                                 use_topk ? tv.data() : nullptr, use_topk ? ti.data() : nullptr, k))
        return r;
    }
  }
  *out_len = generated;
  if (stats) {
    const double t_end = now_s();
    stats->prompt_tokens = (uint64_t)n_ids;
    stats->generated_tokens = generated;
    stats->tokenize_time = 0.0;
    stats->prefill_time = t_decode - t_prefill;
    stats->decode_time = t_end - t_decode;
    stats->total_generation_time = t_end - t_start;
    stats->first_token_time = first_token;
  }
  return PG_OK;
}

}  // extern "C"
