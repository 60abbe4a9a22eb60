// Launch wrappers of the sm_100a kernels (definitions in kernels.cu). Pointers are device
// pointers. Every wrapper returns the cudaError_t of its launch.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace pg {

enum Epilogue { EPI_NONE = 0, EPI_GELU = 1, EPI_RESID = 2 };

// KV page pool of one layer: [page][2 (K,V)][head][page_tokens][head_dim] floats.
struct KvLayout {
  int n_head, head_dim, page_tokens, pages_per_seq;  // pages_per_seq = ceil(n_positions / page_tokens)
};

struct LinearArgs {
  const float* w;      // [n, k] row-major ([out, in])
  const float* bias;   // [n] or nullptr
  const float* x;      // [m, k]
  float* out;          // [m, n]
  const float* resid;  // [m, n], EPI_RESID only (may alias out)
  const float* ln_g;   // LayerNorm gamma/beta over k, or nullptr for no LayerNorm prologue
  const float* ln_b;
  float eps;
  int m, n, k;
  float* part_val;     // optional per-CTA argmax partials: [m][grid] (lm_head)
  int* part_idx;
};

// Decode-time linear for a few activation rows (m <= 64): streams W once per 8 rows of x with
// 128-bit loads, optional fused LayerNorm prologue (m <= 8, k <= 2048) and bias/GELU/residual
// epilogue. `pdl` launches with programmatic dependent launch. Returns the grid size used in
// *grid_out (the stride of part_val / part_idx).
cudaError_t launch_linear_decode(const LinearArgs& a, int epilogue, bool pdl, cudaStream_t s, int* grid_out);
int linear_decode_grid(int n, int num_sms);

// out[r, :] = wte[ids[r]] + wpe[pos[r]]
cudaError_t launch_embed(const float* wte, const float* wpe, const int* ids, const int* pos, float* out,
                         int rows, int c, bool pdl, cudaStream_t s);
// out = LayerNorm(x) row-wise; lo (optional; needs c % 4 == 0 and c <= 4096) = out - hi(out), the TF32 lo part of the result
cudaError_t launch_layernorm_rows(const float* x, const float* g, const float* b, float eps, float* out,
                                  int rows, int c, bool pdl, cudaStream_t s, float* lo = nullptr);
// General FP32 GEMM out[m,n] = x[m,k] . w[n,k]^T (+bias)(+GELU | +resid), CUDA-core FMA.
cudaError_t launch_gemm_f32(const LinearArgs& a, int epilogue, cudaStream_t s);
// dst[o, i] = src[i, o]
cudaError_t launch_transpose(const float* src, float* dst, int in_f, int out_f, cudaStream_t s);

struct DecodeAttnArgs {
  const float* qkv;       // [batch, 3c]
  float* out;             // [batch, c]
  float* out_lo;          // optional: out receives the TF32 hi part and out_lo the remainder
  float* kv_pool;         // this layer's page pool
  const int* page_table;  // [max_batch, pages_per_seq]
  const int* pos;         // [batch]: position of the new token (= keys already cached)
  float* part;            // split-K partials [batch*head][splits][head_dim + 2]
  unsigned* counters;     // [batch*head], zero between launches
  KvLayout kv;
  int batch, splits;
};
// Causal attention of one new token per sequence over the paged cache; also appends the new K,V.
cudaError_t launch_decode_attention(const DecodeAttnArgs& a, bool pdl, cudaStream_t s);

struct PrefillAttnArgs {
  const float* qkv;      // [rows, 3c], sequences concatenated
  float* out;            // [rows, c]
  float* out_lo;         // optional (head_dim 64, FP32 kernel): out - hi(out), the lo part the FP32-grade GEMM after it reads
  const int* seq_start;  // [batch + 1] row offsets
  int n_head, head_dim, batch, max_len;
};
cudaError_t launch_prefill_attention(const PrefillAttnArgs& a, cudaStream_t s);
// The same attention with TF32 products on the tensor cores (head_dim 64; used by the TF32 prefill mode).
// rows = rows of the QKV matrix; error_flag receives a code when a bounded wait runs out.
bool prefill_attention_tc_supported(const PrefillAttnArgs& a);
cudaError_t launch_prefill_attention_tc(const PrefillAttnArgs& a, int rows, int* error_flag, cudaStream_t s);
// The same at FP32 grade (three TF32 products per term, lo parts formed inside the kernel): the FP32-parity modes.
cudaError_t launch_prefill_attention_x3(const PrefillAttnArgs& a, int rows, int* error_flag, cudaStream_t s);
cudaError_t init_attn_tc_attributes();
// Copies K,V of every prompt row into the paged cache.
cudaError_t launch_kv_scatter(const float* qkv, const int* row_slot, const int* row_pos, float* kv_pool,
                              const int* page_table, KvLayout kv, int rows, cudaStream_t s);
// Reads one slot's K,V of one layer back in [head][n_positions][head_dim] order.
cudaError_t launch_kv_gather(const float* kv_pool, const int* page_table, KvLayout kv, int slot, int seq_len,
                             int n_positions, float* keys, float* values, cudaStream_t s);
// dst[r, :] = src[rows[r], :]
cudaError_t launch_gather_rows(const float* src, const int* rows, float* dst, int n, int c, cudaStream_t s);

// End of a decode step. Reduces the per-CTA argmax partials of the lm_head into argmax_out[m]
// (when part_val is nullptr, argmax_out already holds the row argmax), feeds the token back as
// next_ids[m], advances pos[m] by one and records the token at its position in
// token_log[m * n_positions + new_pos].
struct FinalizeArgs {
  const float* part_val;
  const int* part_idx;
  int parts, m;
  int* argmax_out;  // [m]
  int* next_ids;    // [m]
  int* pos;         // [m]
  int* token_log;   // [m][n_positions]
  int n_positions;
};
// Sets the opt-in shared-memory limits of the kernels; once per device before the first launch.
cudaError_t init_kernel_attributes();
cudaError_t init_tc_kernel_attributes();

// hi = x with the 13 low mantissa bits cleared (exactly representable in TF32), lo = x - hi
cudaError_t launch_split_tf32(const float* x, float* hi, float* lo, size_t n, bool pdl, cudaStream_t s);
// LayerNorm rows whose result is written as a TF32 hi/lo pair
cudaError_t launch_layernorm_rows_split(const float* x, const float* g, const float* b, float eps, float* hi,
                                        float* lo, int rows, int c, bool pdl, cudaStream_t s);

// Tensor-core GEMM out[m, n] = x[m, k] . w[n, k]^T (+bias)(+GELU | +resid); k % 32 == 0.
struct TcGemmArgs {
  const float* x;     // [m, k] activations (x3: the hi part)
  const float* x_lo;  // [m, k] lo part (x3 only)
  const float* w;     // [n, k] row-major; for the x3 kernel the tiled copy made by launch_tile_weights
  const float* w_lo;  // [n, k] row-major lo parts of w (launch_tc_gemm_tf32x3_rows only)
  const float* bias;  // [n] or nullptr
  const float* resid; // [m, n], EPI_RESID
  float* out;         // [m, n] (may be nullptr in x3 when only the split outputs are wanted)
  float* out_hi;      // x3: optional TF32 hi/lo pair of the result, [m, n] each
  float* out_lo;      // launch_tc_gemm_tf32x3_rows: optional, out - hi(out) (out_hi unused there)
  int* error_flag;    // set non-zero if a bounded wait inside the kernel expired
  unsigned long long* trace;  // optional tuning aid (x3 kernel): 16 words per CTA, phase timestamps and cycle counts
  int m, n, k, epilogue;
};
bool tc_gemm_supported(int m, int n, int k);
// Tiled weight layout of the x3 kernel: [n / 128][k / 32][128 rows][32 floats], every TMA tile one
// contiguous 16 KB run in HBM (row-major tiles would be 128 scattered 128-byte pieces, which costs
// most of the DRAM bandwidth). Rows are padded with zeros to a multiple of 128.
size_t tc_tiled_weight_floats(int n, int k);
cudaError_t launch_tile_weights(const float* src, float* dst, int n, int k, cudaStream_t s);
// single TF32 pass, any m (prefill)
cudaError_t launch_tc_gemm_tf32(const TcGemmArgs& a, cudaStream_t s);
// three TF32 passes (FP32-grade), any m (prefill): x_lo and w_lo hold v - hi(v) of x and w (launch_tf32_lo)
cudaError_t launch_tc_gemm_tf32x3_rows(const TcGemmArgs& a, cudaStream_t s);
cudaError_t launch_tf32_lo(const float* x, float* lo, size_t n, cudaStream_t s);
// three TF32 passes (FP32-grade), m <= 64 (decode)
int tc_gemm_x3_splits(int n, int k, int num_sms);
cudaError_t launch_tc_gemm_x3(const TcGemmArgs& a, int splits, bool pdl, cudaStream_t s);
cudaError_t launch_finalize(const FinalizeArgs& a, bool pdl, cudaStream_t s);

// A chain of dependent decode linears (m <= 64 tokens, three TF32 products each) as ONE persistent
// cooperative kernel (gemm_chain.cu), one CTA per SM. The weights of every GEMM phase are one
// contiguous run of 16 KB blocks of the tiled arena, cut into equal shares per CTA whatever the
// matrix shape; a CTA's share may cross row tiles, and it writes one partial accumulator per tile
// it touched. The phase after a GEMM adds the partials in k order and applies the bias with either
// a residual update (+ LayerNorm, written as a TF32 hi/lo pair) or an element-wise epilogue (GELU,
// hi/lo pair and/or plain FP32). Phases are separated by a bounded grid barrier that only the
// worker warps take part in: the weight stream of later phases keeps running through it.
enum ChainKind { CH_GEMM = 0, CH_ROWS = 1, CH_ELEM = 2, CH_ATTN = 3, CH_EMBED = 4, CH_FINAL = 5 };
enum ChainAct { CH_ACT_NORM = 0, CH_ACT_ATTN = 1, CH_ACT_H = 2 };
struct ChainPhase {
  int kind;
  int n, k;           // GEMM: output features and reduction length; ROWS / ELEM / ATTN: those of the GEMM being reduced
  int act;            // GEMM: which hi/lo activation pair is the input (ChainAct)
  unsigned w_block0;  // GEMM: index of the first 16 KB block of this matrix inside the tiled arena
  int gelu;           // ELEM: tanh-GELU after the bias
  const float* bias;  // ROWS / ELEM: [n] or nullptr
  float* x;           // ROWS: residual stream [m, n], updated in place
  const float* ln_g;  // ROWS: LayerNorm over the updated row (nullptr: none) ...
  const float* ln_b;
  float* out;         // ELEM: plain FP32 result [m, n] or nullptr
  float* out_hi;      // ROWS: LayerNorm result, ELEM / ATTN: result, as a TF32 hi/lo pair (or nullptr)
  float* out_lo;
  float* kv_pool;     // ATTN: this layer's page pool (n, k, bias: those of the QKV GEMM right before it)
  unsigned long long* best;  // ELEM, whole-tile GEMM: optional row arg-max accumulator [m] (packed value | index, see CH_FINAL)
  // derived by chain_prepare_phases (share arithmetic of the phase's GEMM for the launch grid, so that no thread
  // divides when a phase starts): 32 KB weight units per row tile, units per CTA, multiply-high reciprocals of both
  int r_nkb, r_per;
  unsigned r_magic_per, r_magic_nkb;
  // GEMM without a reduce phase behind it (the lm_head): every CTA takes whole row tiles, so an accumulator holds
  // finished sums, and the drain stores them to `out` (or nowhere) and folds them into `best`; no bias, no partial tiles
  int whole_tiles;
  int reserved_;
};
constexpr int CHAIN_MAX_PHASES = 10;
struct ChainArgs {
  ChainPhase ph[CHAIN_MAX_PHASES];  // the phases, when phases_dev is nullptr
  const ChainPhase* phases_dev;     // or: the phases in device memory (any number of them)
  int n_phases;
  // ATTN phases: causal attention of one new token per sequence over the paged cache (head_dim 64),
  // appending the new K and V; key / value rows are staged in shared memory by bulk async copies
  KvLayout kv;
  const int* page_table;  // [max_batch, pages_per_seq]
  const int* pos;         // [m] position of the new token (= keys already cached)
  // EMBED phase (x[j] = wte[ids[j]] + wpe[pos[j]], then the first LayerNorm as in a ROWS phase) and FINAL phase
  // (end of a decode step, as FinalizeArgs: row arg-max from the accumulator the lm_head's ELEM phase filled,
  // token fed back as the next id, position advanced, token logged; the accumulator is reset)
  const float* wte;
  const float* wpe;
  int* ids;          // [m]
  int* pos_rw;       // the same array as `pos`
  int* argmax_out;   // [m]
  int* token_log;    // [m][n_positions]
  int n_positions;
  unsigned long long* best;  // [m], holds chain_argmax_init() between launches
  int m;               // tokens (rows of every activation matrix), <= 64
  float eps;
  const float* arena;  // tiled weight arena (all matrices of the model)
  size_t arena_floats;
  const float* act_hi[3];  // activation pairs by ChainAct: [m, k] each
  const float* act_lo[3];
  int act_k[3];
  float* partials;     // chain_partial_floats(grid) floats
  unsigned* barrier;   // one word, zero before the first launch (the kernel leaves it zero)
  int* error_flag;     // set non-zero when a bounded wait expired
  int tune_fence;      // tuning: bit 0 = a separate __threadfence(), bit 1 = a proxy fence before the arrival at the grid barrier
                       // (0: the release alone); bit 2 = phase descriptors read from global memory instead of the staged copy;
                       // bit 3 = weight loads without the L2 evict-first hint; bit 4 = the activation producer of a GEMM phase is
                       // told by the first worker thread after the barrier instead of by the polling thread inside it
  unsigned long long* phase_times;  // optional: n_phases + 1 %globaltimer stamps written by CTA 0 (start, then after each phase)
  unsigned long long* trace;  // optional tuning aid, 32 words per CTA: [p] when worker thread 0 left phase p, [10 + p]
                              // when its work of phase p was done, [20..25] wait / issue cycle counts, [31] start
};
// Cooperative grid of the chain kernel on this device (0: not launchable) and the scratch it needs.
int chain_grid(int num_sms);
size_t chain_partial_floats(int grid);
// Value of an empty row arg-max accumulator: (-inf, index 0), the start of argmax_logits (generation.rs:269-279).
unsigned long long chain_argmax_init();
// True when every phase fits the kernel's limits for a grid of `grid` CTAs. `host_phases` is the
// host copy of the phase list (a.ph when nullptr).
bool chain_supported(const ChainArgs& a, int grid, const ChainPhase* host_phases = nullptr);
// Fills the derived fields of a phase list for a grid of `grid` CTAs (before chain_supported / the upload).
void chain_prepare_phases(ChainPhase* phases, int n_phases, int grid);
cudaError_t launch_chain(const ChainArgs& a, int grid, cudaStream_t s);

// Whole decode step for at most 8 sequences (head_dim 64) as one persistent cooperative kernel
// (decode_stream.cu): a producer warp per CTA streams that CTA's share of every weight matrix into a
// shared-memory ring without ever waiting for a dependency, and activations move between CTAs as
// 8-byte {value, tag} words, so there is no grid barrier. Weights: FP32, BF16 or row-quantised int8.
enum StreamWeightType { STREAM_W_F32 = 0, STREAM_W_BF16 = 1, STREAM_W_I8 = 2 };
struct StreamArgs {
  // Layer 0's tensors; layer l's are `l * stride` further on (the arenas hold every layer in the same layout).
  const unsigned char* w[4];  // weight rows [out, in] of c_attn, attn.c_proj, mlp.c_fc, mlp.c_proj in the weight type of the launch
  const float* scale[4];      // int8: one scale per output row (else unused)
  const float* bias[4];       // FP32
  const float* ln_g[2];       // ln_1, ln_2
  const float* ln_b[2];
  long long w_stride;         // bytes from a layer's matrix to the next layer's
  long long s_stride;         // floats from a layer's row scales to the next layer's
  long long p_stride;         // floats from a layer's bias / LayerNorm vector to the next layer's
  float* kv_pool;             // layer 0's page pool
  long long kv_stride;        // floats of one layer's pool
  const float *wte, *wpe;     // FP32 embedding tables
  const unsigned char* w_head;  // the tied lm_head in the weight type of the launch ([vocab, n_embd])
  const float* s_head;          // int8: row scales of the lm_head
  const float *lnf_g, *lnf_b;
  int n_layer, c, f, v, n_positions;
  float eps;
  int *ids, *pos, *argmax, *token_log;  // [m] / [m][n_positions]
  float* logits;                        // [m, v] or nullptr (greedy steps read only the arg-max)
  const int* page_table;
  KvLayout kv;
  // exchange buffers of 8-byte words (value | tag << 32), zero before the first launch
  unsigned long long *ll_x, *ll_qkv, *ll_attn, *ll_h;  // [8][c], [8][3c], [8][c], [8][f]
  unsigned long long* ll_part;                         // attention split partials [8 * n_head][8][66]
  unsigned long long* ll_best;                         // lm_head arg-max partials [8][grid][2]
  unsigned* epoch;            // one word: last tag used, carried from launch to launch
  int* error_flag;            // set non-zero when a bounded wait expired
  int m, attn_splits;         // attn_splits 0: chosen from the context length
  unsigned spin_limit;        // polls before a wait gives up (0: default)
  unsigned poison;            // test hook: XORed into one expected tag, so that the wait for it runs out
  unsigned long long* trace;  // developer aid (builds with -DPG_DEV_TRACE only), else nullptr
};
// Cooperative grid of the kernel on this device (0: not launchable).
int decode_stream_grid(int num_sms);
int decode_stream_elem_bytes(int weight_type);
bool decode_stream_supported(int m, int c, int f, int v, int head_dim, int n_positions, int page_tokens, int weight_type,
                             int grid);
cudaError_t launch_decode_stream(const StreamArgs& a, int weight_type, int grid, cudaStream_t s);
// Row-wise int8 quantisation (QuantizedRows::from_f32, cpu.rs:33-57), its inverse w = q * scale, and BF16 rounding
// (nearest even) of an FP32 array in place with a packed 2-byte copy: the narrow weight copies made at model load.
cudaError_t launch_quantize_rows(const float* w, int rows, int cols, int8_t* q, float* scales, cudaStream_t s);
cudaError_t launch_dequantize_rows(const int8_t* q, const float* scales, int rows, int cols, float* w, cudaStream_t s);
cudaError_t launch_round_bf16(float* w, size_t n, uint16_t* packed, cudaStream_t s);
// Plain argmax over rows of a [m, n] matrix (first strict maximum).
cudaError_t launch_argmax_rows(const float* logits, int m, int n, int* out, cudaStream_t s);
// k largest per row, descending, ties by lower index; k <= 64.
cudaError_t launch_topk_rows(const float* logits, int m, int n, int k, float* vals, int* idx, cudaStream_t s);

}  // namespace pg
