// Kernel-level entry points of the C ABI: one operator on host buffers, timed on the device.
// They exist for the kernel sweeps (shapes of GPT-2 XL) and for operator-level parity tests; the
// model path in model.cu launches the same kernels directly.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "common.h"
#include "kernels.cuh"

namespace pg {
int ensure_device(int device);  // model.cu
}
using namespace pg;

#define PG_OP_TRY(expr)                                                                                     \
  do {                                                                                                      \
    cudaError_t _e = (expr);                                                                                \
    if (_e != cudaSuccess) {                                                                                \
      rc = set_error(PG_CUDA, std::string("CUDA error: ") + cudaGetErrorString(_e) + " (" #expr ")");       \
      goto done;                                                                                            \
    }                                                                                                       \
  } while (0)

namespace {
struct DeviceBuf {
  void* p = nullptr;
  ~DeviceBuf() {
    if (p) cudaFree(p);
  }
  template <typename T>
  T* as() { return static_cast<T*>(p); }
};
constexpr size_t FLUSH_BYTES = 256u << 20;  // larger than the 126 MB L2
}  // namespace

extern "C" int pg_op_linear(const float* x, const float* w, const float* bias, const float* resid, int32_t m,
                            int32_t n, int32_t k, int32_t epilogue, int32_t math_mode, int32_t device, int32_t reps,
                            float* out, double* seconds_per_launch) {
  if (!x || !w || !out) return set_error(PG_INVALID_INPUT, "null argument");
  if (m <= 0 || n <= 0 || k <= 0) return set_error(PG_INVALID_INPUT, "m, n, k must be > 0");
  if (epilogue < EPI_NONE || epilogue > EPI_RESID) return set_error(PG_INVALID_INPUT, "unknown epilogue");
  if (epilogue == EPI_RESID && !resid) return set_error(PG_INVALID_INPUT, "residual epilogue needs resid");
  if (math_mode < PG_MATH_FP32 || math_mode > PG_MATH_TF32) return set_error(PG_INVALID_CONFIG, "math_mode must be fp32, tf32x3 or tf32");
  if (math_mode != PG_MATH_FP32 && !tc_gemm_supported(m, n, k))
    return set_error(PG_INVALID_INPUT, "tensor-core modes need k to be a multiple of 32");
  const bool x3_rows = math_mode == PG_MATH_TF32X3 && m > 64;  // the FP32-grade prefill GEMM (both operands as hi + lo)
  if (int r = ensure_device(device)) return r;
  int rc = PG_OK;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const size_t xs = (size_t)m * k, ws = (size_t)n * k, os = (size_t)m * n;
  DeviceBuf dx, dw, dwt, db, dr, dout, dhi, dlo, derr, dflush, dtrace, dpart, dbar, dwlo;
#ifdef PG_DEV_TRACE
  const bool want_trace = getenv("PG_TRACE") != nullptr;  // developer aid: phase time stamps of the kernel, printed below
#else
  constexpr bool want_trace = false;
#endif
  // tf32x3 runs on the persistent chain kernel (one GEMM phase + its reduce phase) unless PG_NO_CHAIN is set
  int chain_ctas = 0;
  ChainArgs chain{};
  cudaStream_t s = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  int splits = 1;
  auto run = [&](cudaStream_t st) -> cudaError_t {
    if (math_mode == PG_MATH_FP32) {
      LinearArgs a{};
      a.w = dw.as<float>(); a.bias = db.as<float>(); a.x = dx.as<float>(); a.out = dout.as<float>();
      a.resid = dr.as<float>(); a.m = m; a.n = n; a.k = k;
      if (m <= 64 || k % 4 != 0) return launch_linear_decode(a, epilogue, false, st, nullptr);
      return launch_gemm_f32(a, epilogue, st);
    }
    TcGemmArgs a{};
    a.w = dw.as<float>(); a.bias = db.as<float>(); a.resid = dr.as<float>(); a.out = dout.as<float>();
    a.error_flag = derr.as<int>(); a.m = m; a.n = n; a.k = k; a.epilogue = epilogue;
    if (math_mode == PG_MATH_TF32) {
      a.x = dx.as<float>();
      return launch_tc_gemm_tf32(a, st);
    }
    if (x3_rows) {  // the lo parts of the activations are made per call, as the prefill does; those of the weights once
      cudaError_t e = launch_tf32_lo(dx.as<float>(), dlo.as<float>(), xs, st);
      if (e != cudaSuccess) return e;
      a.x = dx.as<float>(); a.x_lo = dlo.as<float>(); a.w_lo = dwlo.as<float>();
      return launch_tc_gemm_tf32x3_rows(a, st);
    }
    cudaError_t e = launch_split_tf32(dx.as<float>(), dhi.as<float>(), dlo.as<float>(), xs, false, st);
    if (e != cudaSuccess) return e;
    if (chain_ctas > 0) {
      if (epilogue == EPI_RESID) {
        e = cudaMemcpyAsync(dout.p, dr.p, os * 4, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return e;
      }
      return launch_chain(chain, chain_ctas, st);
    }
    a.x = dhi.as<float>(); a.x_lo = dlo.as<float>(); a.w = dwt.as<float>();
    a.trace = dtrace.as<unsigned long long>();
    return launch_tc_gemm_x3(a, splits, false, st);
  };
  PG_OP_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  PG_OP_TRY(cudaMalloc(&dx.p, xs * 4));
  PG_OP_TRY(cudaMalloc(&dw.p, ws * 4));
  PG_OP_TRY(cudaMalloc(&dout.p, os * 4));
  PG_OP_TRY(cudaMalloc(&derr.p, 4));
  PG_OP_TRY(cudaMemsetAsync(derr.p, 0, 4, s));
  PG_OP_TRY(cudaMemcpyAsync(dx.p, x, xs * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(cudaMemcpyAsync(dw.p, w, ws * 4, cudaMemcpyHostToDevice, s));
  if (bias) {
    PG_OP_TRY(cudaMalloc(&db.p, (size_t)n * 4));
    PG_OP_TRY(cudaMemcpyAsync(db.p, bias, (size_t)n * 4, cudaMemcpyHostToDevice, s));
  }
  if (resid && epilogue == EPI_RESID) {
    PG_OP_TRY(cudaMalloc(&dr.p, os * 4));
    PG_OP_TRY(cudaMemcpyAsync(dr.p, resid, os * 4, cudaMemcpyHostToDevice, s));
  }
  if (x3_rows) {
    if (xs % 4 || ws % 4) {
      rc = set_error(PG_INVALID_INPUT, "tf32x3 with more than 64 rows needs m * k and n * k to be multiples of 4");
      goto done;
    }
    PG_OP_TRY(cudaMalloc(&dlo.p, xs * 4));
    PG_OP_TRY(cudaMalloc(&dwlo.p, ws * 4));
    PG_OP_TRY(launch_tf32_lo(dw.as<float>(), dwlo.as<float>(), ws, s));
  } else if (math_mode == PG_MATH_TF32X3) {
    splits = tc_gemm_x3_splits(n, k, sms);
    PG_OP_TRY(cudaMalloc(&dhi.p, xs * 4));
    PG_OP_TRY(cudaMalloc(&dlo.p, xs * 4));
    PG_OP_TRY(cudaMalloc(&dwt.p, tc_tiled_weight_floats(n, k) * 4));
    PG_OP_TRY(launch_tile_weights(dw.as<float>(), dwt.as<float>(), n, k, s));
    if (!getenv("PG_NO_CHAIN") && chain_grid(sms) > 0) {
      const int g = chain_grid(sms);
      chain.n_phases = 2;
      chain.ph[0].kind = CH_GEMM; chain.ph[0].n = n; chain.ph[0].k = k; chain.ph[0].act = CH_ACT_NORM;
      chain.ph[0].w_block0 = 0;
      chain.ph[1].kind = epilogue == EPI_RESID ? CH_ROWS : CH_ELEM;
      chain.ph[1].n = n; chain.ph[1].k = k; chain.ph[1].bias = db.as<float>();
      chain.ph[1].gelu = epilogue == EPI_GELU; chain.ph[1].x = dout.as<float>(); chain.ph[1].out = dout.as<float>();
      chain.m = m; chain.eps = 1e-5f; chain.arena = dwt.as<float>(); chain.arena_floats = tc_tiled_weight_floats(n, k);
      chain.act_hi[0] = dhi.as<float>(); chain.act_lo[0] = dlo.as<float>(); chain.act_k[0] = k;
      chain.error_flag = derr.as<int>();
      PG_OP_TRY(cudaMalloc(&dpart.p, chain_partial_floats(g) * 4));
      PG_OP_TRY(cudaMalloc(&dbar.p, 4));
      PG_OP_TRY(cudaMemsetAsync(dbar.p, 0, 4, s));
      chain.partials = dpart.as<float>(); chain.barrier = dbar.as<unsigned>();
      if (want_trace) {
        PG_OP_TRY(cudaMalloc(&dtrace.p, (size_t)g * 256 + 4096));
        PG_OP_TRY(cudaMemset(dtrace.p, 0, (size_t)g * 256 + 4096));
        chain.trace = dtrace.as<unsigned long long>();
      }
      if (chain_supported(chain, g)) chain_ctas = g;
    }
    if (want_trace && chain_ctas == 0) {
      PG_OP_TRY(cudaMalloc(&dtrace.p, (size_t)((n + 127) / 128) * splits * 128));
      PG_OP_TRY(cudaMemset(dtrace.p, 0, (size_t)((n + 127) / 128) * splits * 128));
    }
  }
  PG_OP_TRY(run(s));
  PG_OP_TRY(cudaMemcpyAsync(out, dout.p, os * 4, cudaMemcpyDeviceToHost, s));
  PG_OP_TRY(cudaStreamSynchronize(s));
  {
    int flag = 0;
    PG_OP_TRY(cudaMemcpy(&flag, derr.p, 4, cudaMemcpyDeviceToHost));
    if (flag) {
      rc = set_error(PG_TIMEOUT, "a bounded wait inside the tensor-core GEMM expired (role code " + std::to_string(flag) + ")");
      goto done;
    }
  }
  if (reps > 0 && seconds_per_launch) {
    PG_OP_TRY(cudaMalloc(&dflush.p, FLUSH_BYTES));
    PG_OP_TRY(cudaEventCreate(&e0));
    PG_OP_TRY(cudaEventCreate(&e1));
    double total = 0.0;
    for (int i = 0; i < reps + 3; ++i) {
      PG_OP_TRY(cudaMemsetAsync(dflush.p, i, FLUSH_BYTES, s));  // evict the operands from L2
      PG_OP_TRY(cudaEventRecord(e0, s));
      PG_OP_TRY(run(s));
      PG_OP_TRY(cudaEventRecord(e1, s));
      PG_OP_TRY(cudaEventSynchronize(e1));
      float ms = 0.f;
      PG_OP_TRY(cudaEventElapsedTime(&ms, e0, e1));
      if (i >= 3) total += ms * 1e-3;
    }
    *seconds_per_launch = total / reps;
  }
  if (want_trace && dtrace.p && chain_ctas > 0) {
    // tuning aid: when worker thread 0 of each CTA left each phase, relative to the earliest start
    std::vector<unsigned long long> t((size_t)chain_ctas * 32 + 512);
    PG_OP_TRY(cudaMemcpy(t.data(), dtrace.p, t.size() * 8, cudaMemcpyDeviceToHost));
    unsigned long long t0 = ~0ULL;
    for (int i = 0; i < chain_ctas; ++i) t0 = std::min(t0, t[(size_t)i * 32 + 31]);
    for (int sl = 0; sl < chain.n_phases; ++sl) {
      unsigned long long lo = ~0ULL, hi = 0, wlo = ~0ULL, whi = 0;
      for (int i = 0; i < chain_ctas; ++i) {
        const unsigned long long v = t[(size_t)i * 32 + sl] - t0, w = t[(size_t)i * 32 + 10 + sl] - t0;
        lo = std::min(lo, v); hi = std::max(hi, v); wlo = std::min(wlo, w); whi = std::max(whi, w);
      }
      fprintf(stderr, "chain trace phase %d: work done %6llu..%6llu ns, barrier passed %6llu..%6llu ns\n", sl, wlo, whi, lo, hi);
    }
    const char* cn[6] = {"split wait w_full", "split wait tmem", "mma wait ready", "(unused)", "mma issue", "mma wait d_empty"};
    for (int sl = 0; sl < 6; ++sl) {
      double mean = 0;
      for (int i = 0; i < chain_ctas; ++i) mean += (double)t[(size_t)i * 32 + 20 + sl];
      fprintf(stderr, "chain trace %-18s mean %8.0f cycles per CTA\n", cn[sl], mean / chain_ctas);
    }
  } else if (want_trace && dtrace.p) {
    // tuning aid: phase timestamps of the last launch, relative to the earliest CTA start
    const size_t ctas = (size_t)((n + 127) / 128) * splits;
    std::vector<unsigned long long> t(ctas * 16);
    PG_OP_TRY(cudaMemcpy(t.data(), dtrace.p, t.size() * 8, cudaMemcpyDeviceToHost));
    unsigned long long t0 = ~0ULL;
    for (size_t i = 0; i < ctas; ++i) t0 = std::min(t0, t[i * 16]);
    const char* names[8] = {"start", "setup", "first_full", "d_full", "pre_cluster", "post_cluster", "epi_done", "end"};
    for (int sl = 0; sl < 8; ++sl) {
      unsigned long long lo = ~0ULL, hi = 0;
      double mean = 0;
      for (size_t i = 0; i < ctas; ++i) {
        unsigned long long v = t[i * 16 + sl] - t0;
        lo = std::min(lo, v); hi = std::max(hi, v); mean += (double)v;
      }
      fprintf(stderr, "trace %-13s min %6llu ns  mean %8.0f ns  max %6llu ns\n", names[sl], lo, mean / ctas, hi);
    }
    const char* cn[8] = {"split_wait", "split_ld_alu", "split_st", "mma_wait", "mma_issue", "blk5_fence", "blk5_mmas", "blk5_commit"};
    for (int sl = 0; sl < 8; ++sl) {
      double mean = 0;
      for (size_t i = 0; i < ctas; ++i) mean += (double)t[i * 16 + 8 + sl];
      fprintf(stderr, "trace %-13s mean %8.0f cycles per CTA\n", cn[sl], mean / ctas);
    }
  }
done:
  if (s) cudaStreamSynchronize(s);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (s) cudaStreamDestroy(s);
  return rc;
}

// Decode attention of one new token per sequence on host buffers (cached_self_attention_into,
// src/models/gpt2/rust.rs:1662-1741). keys/values: [batch][head][kv_len][head_dim], the positions
// already cached; qkv: [batch][3c], the new token's q, k, v. The entry point lays the cache out in
// pages (with a permuted page table), runs the kernel and returns out[batch][c].
extern "C" int pg_op_decode_attention(const float* qkv, const float* keys, const float* values, int32_t batch,
                                      int32_t n_head, int32_t head_dim, int32_t kv_len, int32_t page_tokens,
                                      int32_t splits, int32_t device, int32_t reps, float* out,
                                      double* seconds_per_launch) {
  if (!qkv || !out || (kv_len > 0 && (!keys || !values))) return set_error(PG_INVALID_INPUT, "null argument");
  if (batch <= 0 || n_head <= 0 || head_dim <= 0 || kv_len < 0) return set_error(PG_INVALID_INPUT, "bad shape");
  if (page_tokens != 16 && page_tokens != 32 && page_tokens != 64) return set_error(PG_INVALID_CONFIG, "cuda page_tokens must be 16, 32 or 64");
  if (splits < 1 || splits > 16) return set_error(PG_INVALID_CONFIG, "cuda attn_splits must be in 1..16");
  if (head_dim != 64) splits = 1;
  if (int r = ensure_device(device)) return r;
  int rc = PG_OK;
  const int c = n_head * head_dim;
  KvLayout kv{n_head, head_dim, page_tokens, (kv_len + 1 + page_tokens - 1) / page_tokens};
  const int pages = batch * kv.pages_per_seq;
  const size_t page_floats = (size_t)2 * n_head * page_tokens * head_dim;
  // page p of sequence b lives at physical page (b + p * batch) * 7919 % pages-ish: any bijection
  std::vector<int> table((size_t)pages);
  {
    std::vector<int> perm(pages);
    for (int i = 0; i < pages; ++i) perm[i] = i;
    uint64_t st = 0x9e3779b97f4a7c15ULL;
    for (int i = pages - 1; i > 0; --i) {
      st = st * 6364136223846793005ULL + 1442695040888963407ULL;
      std::swap(perm[i], perm[(int)((st >> 33) % (uint64_t)(i + 1))]);
    }
    for (int i = 0; i < pages; ++i) table[i] = perm[i];
  }
  std::vector<float> pool((size_t)pages * page_floats, 0.f);
  for (int b = 0; b < batch; ++b)
    for (int h = 0; h < n_head; ++h)
      for (int p = 0; p < kv_len; ++p) {
        const int page = table[(size_t)b * kv.pages_per_seq + p / page_tokens], off = p % page_tokens;
        const size_t src = (((size_t)b * n_head + h) * kv_len + p) * head_dim;
        const size_t kd = ((((size_t)page * 2 + 0) * n_head + h) * page_tokens + off) * head_dim;
        const size_t vd = ((((size_t)page * 2 + 1) * n_head + h) * page_tokens + off) * head_dim;
        for (int d = 0; d < head_dim; ++d) {
          pool[kd + d] = keys[src + d];
          pool[vd + d] = values[src + d];
        }
      }
  std::vector<int> pos((size_t)batch, kv_len);
  DeviceBuf dq, dout, dpool, dtab, dpos, dpart, dcnt, dflush;
  cudaStream_t s = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  DecodeAttnArgs a{};
  PG_OP_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  PG_OP_TRY(cudaMalloc(&dq.p, (size_t)batch * 3 * c * 4));
  PG_OP_TRY(cudaMalloc(&dout.p, (size_t)batch * c * 4));
  PG_OP_TRY(cudaMalloc(&dpool.p, pool.size() * 4));
  PG_OP_TRY(cudaMalloc(&dtab.p, table.size() * 4));
  PG_OP_TRY(cudaMalloc(&dpos.p, pos.size() * 4));
  PG_OP_TRY(cudaMalloc(&dpart.p, (size_t)batch * n_head * splits * (head_dim + 2) * 4));
  PG_OP_TRY(cudaMalloc(&dcnt.p, (size_t)batch * n_head * 4));
  PG_OP_TRY(cudaMemsetAsync(dcnt.p, 0, (size_t)batch * n_head * 4, s));
  PG_OP_TRY(cudaMemcpyAsync(dq.p, qkv, (size_t)batch * 3 * c * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(cudaMemcpyAsync(dpool.p, pool.data(), pool.size() * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(cudaMemcpyAsync(dtab.p, table.data(), table.size() * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(cudaMemcpyAsync(dpos.p, pos.data(), pos.size() * 4, cudaMemcpyHostToDevice, s));
  a.qkv = dq.as<float>(); a.out = dout.as<float>(); a.kv_pool = dpool.as<float>(); a.page_table = dtab.as<int>();
  a.pos = dpos.as<int>(); a.part = dpart.as<float>(); a.counters = dcnt.as<unsigned>(); a.kv = kv;
  a.batch = batch; a.splits = splits;
  PG_OP_TRY(launch_decode_attention(a, false, s));
  PG_OP_TRY(cudaMemcpyAsync(out, dout.p, (size_t)batch * c * 4, cudaMemcpyDeviceToHost, s));
  PG_OP_TRY(cudaStreamSynchronize(s));
  if (reps > 0 && seconds_per_launch) {
    PG_OP_TRY(cudaMalloc(&dflush.p, FLUSH_BYTES));
    PG_OP_TRY(cudaEventCreate(&e0));
    PG_OP_TRY(cudaEventCreate(&e1));
    double total = 0.0;
    for (int i = 0; i < reps + 3; ++i) {
      PG_OP_TRY(cudaMemsetAsync(dflush.p, i, FLUSH_BYTES, s));
      PG_OP_TRY(cudaEventRecord(e0, s));
      PG_OP_TRY(launch_decode_attention(a, false, s));
      PG_OP_TRY(cudaEventRecord(e1, s));
      PG_OP_TRY(cudaEventSynchronize(e1));
      float ms = 0.f;
      PG_OP_TRY(cudaEventElapsedTime(&ms, e0, e1));
      if (i >= 3) total += ms * 1e-3;
    }
    *seconds_per_launch = total / reps;
  }
done:
  if (s) cudaStreamSynchronize(s);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (s) cudaStreamDestroy(s);
  return rc;
}

// Times `run` reps times on `s` with the operands evicted from L2 before each launch; mean seconds.
template <typename F>
static cudaError_t time_launches(F&& run, cudaStream_t s, int reps, double* seconds) {
  void* flush = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaError_t e = cudaMalloc(&flush, FLUSH_BYTES);
  if (e == cudaSuccess) e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  double total = 0.0;
  for (int i = 0; i < reps + 3 && e == cudaSuccess; ++i) {
    e = cudaMemsetAsync(flush, i, FLUSH_BYTES, s);
    if (e == cudaSuccess) e = cudaEventRecord(e0, s);
    if (e == cudaSuccess) e = run(s);
    if (e == cudaSuccess) e = cudaEventRecord(e1, s);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (i >= 3) total += ms * 1e-3;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (flush) cudaFree(flush);
  if (e == cudaSuccess) *seconds = total / reps;
  return e;
}

extern "C" int pg_op_layernorm(const float* x, const float* gamma, const float* beta, float eps, int32_t rows,
                               int32_t cols, int32_t device, int32_t reps, float* out, double* seconds_per_launch) {
  if (!x || !gamma || !beta || !out) return set_error(PG_INVALID_INPUT, "null argument");
  if (rows <= 0 || cols <= 0) return set_error(PG_INVALID_INPUT, "rows and cols must be > 0");
  if (int r = ensure_device(device)) return r;
  int rc = PG_OK;
  const size_t n = (size_t)rows * cols;
  DeviceBuf dx, dg, db, dout;
  cudaStream_t s = nullptr;
  auto run = [&](cudaStream_t st) {
    return launch_layernorm_rows(dx.as<float>(), dg.as<float>(), db.as<float>(), eps, dout.as<float>(), rows, cols, false, st);
  };
  PG_OP_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  PG_OP_TRY(cudaMalloc(&dx.p, n * 4));
  PG_OP_TRY(cudaMalloc(&dout.p, n * 4));
  PG_OP_TRY(cudaMalloc(&dg.p, (size_t)cols * 4));
  PG_OP_TRY(cudaMalloc(&db.p, (size_t)cols * 4));
  PG_OP_TRY(cudaMemcpyAsync(dx.p, x, n * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(cudaMemcpyAsync(dg.p, gamma, (size_t)cols * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(cudaMemcpyAsync(db.p, beta, (size_t)cols * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(run(s));
  PG_OP_TRY(cudaMemcpyAsync(out, dout.p, n * 4, cudaMemcpyDeviceToHost, s));
  PG_OP_TRY(cudaStreamSynchronize(s));
  if (reps > 0 && seconds_per_launch) PG_OP_TRY(time_launches(run, s, reps, seconds_per_launch));
done:
  if (s) {
    cudaStreamSynchronize(s);
    cudaStreamDestroy(s);
  }
  return rc;
}

extern "C" int pg_op_lm_head_argmax(const float* hidden, const float* wte, int32_t m, int32_t vocab, int32_t k,
                                    int32_t device, int32_t reps, float* logits_out, int32_t* argmax_out,
                                    double* seconds_per_launch) {
  if (!hidden || !wte || !argmax_out) return set_error(PG_INVALID_INPUT, "null argument");
  if (m <= 0 || m > 8 || vocab <= 0 || k <= 0 || k % 4 != 0)
    return set_error(PG_INVALID_INPUT, "lm_head with fused arg-max is the decode operator: 1 <= m <= 8, k a multiple of 4");
  if (int r = ensure_device(device)) return r;
  int rc = PG_OK;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int stride = linear_decode_grid(vocab, sms);
  DeviceBuf dx, dw, dlog, dpv, dpi, dam, dids, dpos, dtok;
  cudaStream_t s = nullptr;
  // the same two launches that end a decode step: the lm_head GEMV that also writes one (value, index) candidate
  // per CTA and row, and the kernel that reduces the candidates (first strict maximum, generation.rs:269-279)
  auto run = [&](cudaStream_t st) -> cudaError_t {
    LinearArgs a{};
    a.w = dw.as<float>(); a.x = dx.as<float>(); a.out = dlog.as<float>(); a.m = m; a.n = vocab; a.k = k;
    a.part_val = dpv.as<float>(); a.part_idx = dpi.as<int>();
    int grid = 0;
    cudaError_t e = launch_linear_decode(a, EPI_NONE, false, st, &grid);
    if (e != cudaSuccess) return e;
    FinalizeArgs f{};
    f.part_val = dpv.as<float>(); f.part_idx = dpi.as<int>(); f.parts = grid; f.m = m;
    f.argmax_out = dam.as<int>(); f.next_ids = dids.as<int>(); f.pos = dpos.as<int>(); f.token_log = dtok.as<int>();
    f.n_positions = 1;
    return launch_finalize(f, false, st);
  };
  PG_OP_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  PG_OP_TRY(cudaMalloc(&dx.p, (size_t)m * k * 4));
  PG_OP_TRY(cudaMalloc(&dw.p, (size_t)vocab * k * 4));
  PG_OP_TRY(cudaMalloc(&dlog.p, (size_t)m * vocab * 4));
  PG_OP_TRY(cudaMalloc(&dpv.p, (size_t)m * stride * 4));
  PG_OP_TRY(cudaMalloc(&dpi.p, (size_t)m * stride * 4));
  PG_OP_TRY(cudaMalloc(&dam.p, (size_t)m * 4));
  PG_OP_TRY(cudaMalloc(&dids.p, (size_t)m * 4));
  PG_OP_TRY(cudaMalloc(&dpos.p, (size_t)m * 4));
  PG_OP_TRY(cudaMalloc(&dtok.p, (size_t)m * 4));
  PG_OP_TRY(cudaMemsetAsync(dpos.p, 0, (size_t)m * 4, s));
  PG_OP_TRY(cudaMemcpyAsync(dx.p, hidden, (size_t)m * k * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(cudaMemcpyAsync(dw.p, wte, (size_t)vocab * k * 4, cudaMemcpyHostToDevice, s));
  PG_OP_TRY(run(s));
  PG_OP_TRY(cudaMemcpyAsync(argmax_out, dam.p, (size_t)m * 4, cudaMemcpyDeviceToHost, s));
  if (logits_out) PG_OP_TRY(cudaMemcpyAsync(logits_out, dlog.p, (size_t)m * vocab * 4, cudaMemcpyDeviceToHost, s));
  PG_OP_TRY(cudaStreamSynchronize(s));
  if (reps > 0 && seconds_per_launch) PG_OP_TRY(time_launches(run, s, reps, seconds_per_launch));
done:
  if (s) {
    cudaStreamSynchronize(s);
    cudaStreamDestroy(s);
  }
  return rc;
}
