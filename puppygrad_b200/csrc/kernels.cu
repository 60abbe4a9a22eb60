// sm_100a CUDA kernels of the GPT-2 inference path (FP32 parity path).
//
// Decode is HBM-bound weight streaming: every linear reads its [out, in] matrix once with 128-bit
// non-allocating loads, keeps the few activation rows on chip, and fuses LayerNorm (prologue) and
// bias / GELU / residual (epilogue). Kernels of one decode step are chained with programmatic
// dependent launch: each CTA issues its first weight loads *before* griddepcontrol.wait, so the
// weight stream of kernel N+1 overlaps the tail of kernel N.
#include <algorithm>
#include <cfloat>
#include <climits>

#include <mutex>

#include "common.h"
#include "kernels.cuh"

namespace pg {
namespace {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 128-bit streaming load of read-only weights: bypass L1 allocation so activations stay cached.
__device__ __forceinline__ float4 ldg_stream(const float4* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float dot4(float4 a, float4 b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  acc = fmaf(a.w, b.w, acc);
  return acc;
}

__device__ __forceinline__ float tf32_trunc(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
  return v;
}

// Reduces N (power of two, <= 32) per-lane values across the warp with N-1 + log2(32/N)
// shuffles. Afterwards v[0] of lane l holds the total of value index l >> (5 - log2 N).
template <int N, int OFF>
struct WarpMultiReduce {
  static __device__ __forceinline__ void run(float* v, int lane) {
    const bool up = (lane & OFF) != 0;
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
      float send = up ? v[j] : v[j + N / 2];
      float keep = up ? v[j + N / 2] : v[j];
      v[j] = keep + __shfl_xor_sync(FULL, send, OFF);
    }
    WarpMultiReduce<N / 2, OFF / 2>::run(v, lane);
  }
};
template <int OFF>
struct WarpMultiReduce<1, OFF> {
  static __device__ __forceinline__ void run(float* v, int lane) {
    v[0] += __shfl_xor_sync(FULL, v[0], OFF);
    WarpMultiReduce<1, OFF / 2>::run(v, lane);
  }
};
template <>
struct WarpMultiReduce<1, 0> {
  static __device__ __forceinline__ void run(float*, int) {}
};

// tanh-GELU in the reference's evaluation order (src/models/cpu.rs:145-150)
__device__ __forceinline__ float gelu_ref(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978846f * (x + 0.044715f * x * x * x)));
}

constexpr int LIN_THREADS = 128;
constexpr int LIN_WARPS = LIN_THREADS / 32;
constexpr int LIN_ROWS = 4;

// ------------------------------------------------------------------ decode linear
// CTA: LIN_ROWS weight rows per group, the 128 threads split K; grid-stride over row groups.
// Replaces linear_block_into / transposed_dense_projection_into / logits_from_hidden_into
// (src/models/gpt2/rust.rs:1481-1532, 1767-1813; src/models/cpu.rs:58-75) and, fused,
// layer_norm_in_place, gelu_in_place, add_in_place (cpu.rs:119-171).
template <int MT, int EPI, bool LN>
__global__ void __launch_bounds__(LIN_THREADS) linear_decode_kernel(LinearArgs a) {
  extern __shared__ float4 dyn_smem4[];
  float4* xs4 = dyn_smem4;  // [MT][k/4] normalised rows (LN only)
  __shared__ float red[LIN_WARPS][LIN_ROWS * MT];
  __shared__ float lnred[2][LIN_WARPS][MT];
  __shared__ float best_v[LIN_ROWS * MT];
  __shared__ int best_i[LIN_ROWS * MT];

  constexpr int NV = LIN_ROWS * MT;
  // 128-bit chunks per weight row that every thread requests before the dependency wait
  constexpr int PRE = MT <= 2 ? 3 : 2;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int k4 = a.k >> 2;
  const int groups = (a.n + LIN_ROWS - 1) / LIN_ROWS;
  const float4* w4 = reinterpret_cast<const float4*>(a.w);

  pdl_launch();

  // Weights and bias do not depend on the previous kernel: the first row group's loads go out
  // before the dependency wait, so their HBM latency overlaps the tail of the previous kernel.
  float4 wpre[PRE][LIN_ROWS];
  {
    const int g0 = blockIdx.x;
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
      const int c = tid + j * LIN_THREADS;
#pragma unroll
      for (int r = 0; r < LIN_ROWS; ++r) {
        const int row = min(g0 * LIN_ROWS + r, a.n - 1);
        wpre[j][r] = (g0 < groups && c < k4) ? ldg_stream(w4 + (size_t)row * k4 + c) : make_float4(0, 0, 0, 0);
      }
    }
  }
  float bias_pre = 0.f;
  if (tid < NV && a.bias) bias_pre = a.bias[min((int)blockIdx.x * LIN_ROWS + tid / MT, a.n - 1)];

  pdl_wait();

  float resid_pre = 0.f;
  if (EPI == EPI_RESID && tid < NV) {
    const int row = blockIdx.x * LIN_ROWS + tid / MT, m = tid % MT;
    if (row < a.n && m < a.m) resid_pre = a.resid[(size_t)m * a.n + row];
  }

  if (LN) {
    // LayerNorm of the (at most MT) rows into shared memory; every thread owns the chunks
    // c = tid (mod 128) of every row through all three passes
    const float4* x4 = reinterpret_cast<const float4*>(a.x);
    float s[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) s[m] = 0.f;
    for (int c = tid; c < k4; c += LIN_THREADS) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float4 v = m < a.m ? x4[(size_t)m * k4 + c] : make_float4(0, 0, 0, 0);
        xs4[(size_t)m * k4 + c] = v;
        s[m] += (v.x + v.y) + (v.z + v.w);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      s[m] = warp_sum(s[m]);
      if (lane == 0) lnred[0][warp][m] = s[m];
    }
    __syncthreads();
    float mean[MT], q[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      mean[m] = ((lnred[0][0][m] + lnred[0][1][m]) + (lnred[0][2][m] + lnred[0][3][m])) / (float)a.k;
      q[m] = 0.f;
    }
    for (int c = tid; c < k4; c += LIN_THREADS) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float4 v = xs4[(size_t)m * k4 + c];
        const float d0 = v.x - mean[m], d1 = v.y - mean[m], d2 = v.z - mean[m], d3 = v.w - mean[m];
        q[m] += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      q[m] = warp_sum(q[m]);
      if (lane == 0) lnred[1][warp][m] = q[m];
    }
    __syncthreads();
    const float4* g4 = reinterpret_cast<const float4*>(a.ln_g);
    const float4* b4 = reinterpret_cast<const float4*>(a.ln_b);
    for (int c = tid; c < k4; c += LIN_THREADS) {
      const float4 g = g4[c], b = b4[c];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float var = ((lnred[1][0][m] + lnred[1][1][m]) + (lnred[1][2][m] + lnred[1][3][m])) / (float)a.k;
        const float inv_std = 1.0f / sqrtf(var + a.eps);
        float4 v = xs4[(size_t)m * k4 + c];
        v.x = (v.x - mean[m]) * inv_std * g.x + b.x;
        v.y = (v.y - mean[m]) * inv_std * g.y + b.y;
        v.z = (v.z - mean[m]) * inv_std * g.z + b.z;
        v.w = (v.w - mean[m]) * inv_std * g.w + b.w;
        xs4[(size_t)m * k4 + c] = m < a.m ? v : make_float4(0, 0, 0, 0);
      }
    }
    // no barrier needed: the main loop below reads only the chunks this thread wrote
  }

  float run_best = -INFINITY;  // lm_head argmax partial of this thread's (row-in-group, m) pair
  int run_idx = INT_MAX;

  for (int g = blockIdx.x; g < groups; g += gridDim.x) {
    const int row0 = g * LIN_ROWS;
    const bool first_group = g == (int)blockIdx.x;
    const float4* wrow[LIN_ROWS];
#pragma unroll
    for (int r = 0; r < LIN_ROWS; ++r) wrow[r] = w4 + (size_t)min(row0 + r, a.n - 1) * k4;

    for (int m0 = 0; m0 < a.m; m0 += MT) {
      float acc[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[i] = 0.f;
      const float4* xbase = LN ? xs4 : reinterpret_cast<const float4*>(a.x) + (size_t)m0 * k4;

      auto accumulate = [&](const float4 (&w)[LIN_ROWS], int c) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float4 xv;
          if (LN) xv = xbase[(size_t)m * k4 + c];
          else xv = (m0 + m < a.m) ? xbase[(size_t)m * k4 + c] : make_float4(0, 0, 0, 0);
#pragma unroll
          for (int r = 0; r < LIN_ROWS; ++r) acc[r * MT + m] = dot4(w[r], xv, acc[r * MT + m]);
        }
      };

      int cstart = tid;
      if (first_group && m0 == 0) {
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
          const int c = tid + j * LIN_THREADS;
          if (c < k4) accumulate(wpre[j], c);
        }
        cstart = tid + PRE * LIN_THREADS;
      }
#pragma unroll 2
      for (int c = cstart; c < k4; c += LIN_THREADS) {
        float4 w[LIN_ROWS];
#pragma unroll
        for (int r = 0; r < LIN_ROWS; ++r) w[r] = ldg_stream(wrow[r] + c);
        accumulate(w, c);
      }

      WarpMultiReduce<NV, 16>::run(acc, lane);
      constexpr int SH = (NV == 32) ? 0 : (NV == 16) ? 1 : (NV == 8) ? 2 : 3;  // 5 - log2(NV)
      if ((lane & ((1 << SH) - 1)) == 0) red[warp][lane >> SH] = acc[0];
      __syncthreads();
      if (tid < NV) {
        const int r = tid / MT, m = m0 + tid % MT, row = row0 + r;
        if (row < a.n && m < a.m) {
          const float dotv = ((red[0][tid] + red[1][tid]) + red[2][tid]) + red[3][tid];
          const float b = (first_group || !a.bias) ? bias_pre : a.bias[row];
          float v = a.bias ? b + dotv : dotv;
          if (EPI == EPI_GELU) v = gelu_ref(v);
          if (EPI == EPI_RESID) v = ((first_group && m0 == 0) ? resid_pre : a.resid[(size_t)m * a.n + row]) + v;
          a.out[(size_t)m * a.n + row] = v;
          if (a.part_val && v > run_best) {
            run_best = v;
            run_idx = row;
          }
        }
      }
      __syncthreads();
    }
  }

  if (a.part_val) {  // m <= MT here: one (r, m) pair per thread
    if (tid < NV) {
      best_v[tid] = run_best;
      best_i[tid] = run_idx;
    }
    __syncthreads();
    if (tid < MT && tid < a.m) {
      float bv = -INFINITY;
      int bi = INT_MAX;
#pragma unroll
      for (int r = 0; r < LIN_ROWS; ++r) {
        float v = best_v[r * MT + tid];
        int i = best_i[r * MT + tid];
        if (v > bv || (v == bv && i < bi)) {
          bv = v;
          bi = i;
        }
      }
      a.part_val[(size_t)tid * gridDim.x + blockIdx.x] = bv;
      a.part_idx[(size_t)tid * gridDim.x + blockIdx.x] = bi;
    }
  }
}


// ------------------------------------------------------------------ decode linear, activations in shared memory
// The same operator as one persistent CTA of 16 warps per SM: with several input rows the kernel above
// re-reads the activations from L1 once per input row and 16 weights, and starts a CTA (and, fused, a
// LayerNorm) per four weight rows. Here a CTA stages the input rows once ([MT][k] floats, LayerNorm applied
// in place when asked for) and its warps then walk units of (four weight rows, one of `kparts` parts of
// k): 128-bit streaming loads of the weights, activations from shared memory (consecutive lanes,
// consecutive 16-byte units: no bank conflict), one folding warp reduction per unit. With kparts = 1 the
// lanes that hold the sums finish the rows; otherwise the parts of a row group, which are neighbouring
// warps of one CTA, leave their sums in shared memory and after a CTA barrier the first threads add them
// in part order. kparts is chosen so that all 16 x 148 warps have a unit when the matrix has few rows.
constexpr int LR_THREADS = 512;
constexpr int LR_WARPS = LR_THREADS / 32;
constexpr int LR_ROWS = 4;
constexpr size_t LR_MAX_SMEM = 208 * 1024;  // [MT][k] floats
constexpr int LR_ONE_ROW_MIN_N = 16384;      // one input row takes this kernel only for the lm_head

template <int MT, int EPI>
__global__ void __launch_bounds__(LR_THREADS, 1) linear_rows_smem_kernel(LinearArgs a, int kp_shift) {
  extern __shared__ float4 dyn_smem4[];
  float4* xs4 = dyn_smem4;  // [MT][k / 4]
  constexpr int NV = LR_ROWS * MT;
  constexpr int SH = (NV == 32) ? 0 : (NV == 16) ? 1 : (NV == 8) ? 2 : 3;  // 5 - log2(NV)
  __shared__ float part[LR_WARPS][NV];
  __shared__ float best_v[LR_WARPS][NV];
  __shared__ int best_i[LR_WARPS][NV];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int k4 = a.k >> 2;
  const int groups = (a.n + LR_ROWS - 1) / LR_ROWS;
  const int kparts = 1 << kp_shift;
  const int gpc = LR_WARPS >> kp_shift;           // row groups a CTA works on at a time
  const int wg = warp >> kp_shift, kp = warp & (kparts - 1);  // this warp's group slot and part of k
  const int c_beg = (int)(((long long)k4 * kp) >> kp_shift), c_end = (int)(((long long)k4 * (kp + 1)) >> kp_shift);
  const float4* w4 = reinterpret_cast<const float4*>(a.w);
  const int g_first = (int)blockIdx.x * gpc + wg, g_stride = (int)gridDim.x * gpc;

  pdl_launch();
  // weights do not depend on the previous kernel: the warp's first loads go out before the dependency wait
  float4 wpre[LR_ROWS];
#pragma unroll
  for (int r = 0; r < LR_ROWS; ++r)
    wpre[r] = (g_first < groups && c_beg + lane < c_end)
                  ? ldg_stream(w4 + (size_t)min(g_first * LR_ROWS + r, a.n - 1) * k4 + c_beg + lane)
                  : make_float4(0, 0, 0, 0);
  pdl_wait();

  {
    const float4* x4 = reinterpret_cast<const float4*>(a.x);
    for (int idx = tid; idx < MT * k4; idx += LR_THREADS) {
      const int r = idx / k4;
      xs4[idx] = r < a.m ? x4[idx] : make_float4(0, 0, 0, 0);
    }
  }
  __syncthreads();
  if (a.ln_g) {  // LayerNorm of each row, by one warp (layer_norm_in_place, src/models/cpu.rs:119-143, tree sums)
    const float4* g4 = reinterpret_cast<const float4*>(a.ln_g);
    const float4* b4 = reinterpret_cast<const float4*>(a.ln_b);
    for (int r = warp; r < a.m && r < MT; r += LR_WARPS) {
      float4* row = xs4 + (size_t)r * k4;
      float sum = 0.f;
      for (int c = lane; c < k4; c += 32) {
        const float4 v = row[c];
        sum += (v.x + v.y) + (v.z + v.w);
      }
      const float mean = warp_sum(sum) / (float)a.k;
      float q = 0.f;
      for (int c = lane; c < k4; c += 32) {
        const float4 v = row[c];
        const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
        q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      }
      const float inv_std = 1.0f / sqrtf(warp_sum(q) / (float)a.k + a.eps);
      for (int c = lane; c < k4; c += 32) {
        const float4 g = g4[c], b = b4[c];
        float4 v = row[c];
        v.x = (v.x - mean) * inv_std * g.x + b.x;
        v.y = (v.y - mean) * inv_std * g.y + b.y;
        v.z = (v.z - mean) * inv_std * g.z + b.z;
        v.w = (v.w - mean) * inv_std * g.w + b.w;
        row[c] = v;
      }
    }
    __syncthreads();
  }

  // after the warp reduction the lanes with (lane & (2^SH - 1)) == 0 hold sum number lane >> SH = r * MT + m
  const bool holder = (lane & ((1 << SH) - 1)) == 0;
  // who finishes a sum: with kparts = 1 the holder lanes of the warp, else thread t < gpc * NV for (group slot, sum)
  const bool finisher = kparts == 1 ? holder : tid < gpc * NV;
  const int fs = kparts == 1 ? (lane >> SH) : tid % NV;  // sum number
  const int fslot = kparts == 1 ? wg : tid / NV;         // group slot
  const int fr = fs / MT, fm = fs % MT;
  float run_best = -INFINITY;  // lm_head arg-max partial of this finisher's (row in group, input row) pair
  int run_idx = INT_MAX;

  // every warp of the CTA makes the same number of rounds (the CTA barrier inside needs all of them)
  const int rounds = (groups - (int)blockIdx.x * gpc + g_stride - 1) / g_stride;
  for (int it = 0; it < rounds; ++it) {
    const int g = g_first + it * g_stride;
    const bool live = g < groups;
    const int row0 = g * LR_ROWS;
    // what the epilogue needs from memory, asked for before the loop
    const int orow = ((int)blockIdx.x * gpc + fslot + it * g_stride) * LR_ROWS + fr;
    const bool fin = finisher && orow < a.n && fm < a.m && ((int)blockIdx.x * gpc + fslot + it * g_stride) < groups;
    float bias_v = 0.f, resid_v = 0.f;
    if (fin) {
      if (a.bias) bias_v = a.bias[orow];
      if (EPI == EPI_RESID) resid_v = a.resid[(size_t)fm * a.n + orow];
    }
    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = 0.f;
    if (live) {
      const float4* wrow[LR_ROWS];
#pragma unroll
      for (int r = 0; r < LR_ROWS; ++r) wrow[r] = w4 + (size_t)min(row0 + r, a.n - 1) * k4;
      auto accumulate = [&](const float4 (&w)[LR_ROWS], int c) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float4 xv = xs4[(size_t)m * k4 + c];
#pragma unroll
          for (int r = 0; r < LR_ROWS; ++r) acc[r * MT + m] = dot4(w[r], xv, acc[r * MT + m]);
        }
      };
      int c = c_beg + lane;
      if (it == 0) {
        if (c < c_end) accumulate(wpre, c);
        c += 32;
      }
      constexpr int UNR = MT >= 4 ? 2 : 4;  // iterations whose loads are in flight together (registers permitting)
#pragma unroll(UNR)
      for (; c < c_end; c += 32) {
        float4 w[LR_ROWS];
#pragma unroll
        for (int r = 0; r < LR_ROWS; ++r) w[r] = ldg_stream(wrow[r] + c);
        accumulate(w, c);
      }
      WarpMultiReduce<NV, 16>::run(acc, lane);
    }
    float total = acc[0];
    if (kparts > 1) {
      if (holder) part[warp][lane >> SH] = acc[0];
      __syncthreads();
      if (fin) {
        total = 0.f;
        for (int q = 0; q < kparts; ++q) total += part[(fslot << kp_shift) + q][fs];  // in part order
      }
    }
    if (fin) {
      float v = a.bias ? bias_v + total : total;
      if (EPI == EPI_GELU) v = gelu_ref(v);
      if (EPI == EPI_RESID) v = resid_v + v;
      a.out[(size_t)fm * a.n + orow] = v;
      if (a.part_val && v > run_best) {
        run_best = v;
        run_idx = orow;
      }
    }
    if (kparts > 1) __syncthreads();  // `part` is rewritten in the next round
  }

  if (a.part_val) {
    // finishers: kparts = 1: holder lanes of every warp, sum number lane >> SH; else threads t < gpc * NV
    if (kparts == 1) {
      if (holder) {
        best_v[warp][lane >> SH] = run_best;
        best_i[warp][lane >> SH] = run_idx;
      }
    } else if (tid < gpc * NV) {
      best_v[tid / NV][tid % NV] = run_best;
      best_i[tid / NV][tid % NV] = run_idx;
    }
    __syncthreads();
    if (tid < MT && tid < a.m) {
      float bv = -INFINITY;
      int bi = INT_MAX;
      for (int w = 0; w < gpc; ++w)
#pragma unroll
        for (int r = 0; r < LR_ROWS; ++r) {
          const float v = best_v[w][r * MT + tid];
          const int i = best_i[w][r * MT + tid];
          if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
          }
        }
      a.part_val[(size_t)tid * gridDim.x + blockIdx.x] = bv;
      a.part_idx[(size_t)tid * gridDim.x + blockIdx.x] = bi;
    }
  }
}

// Any k (no alignment requirement): one thread per output element. Only shapes whose inner
// dimension is not a multiple of 4 take this path.
__global__ void linear_generic_kernel(LinearArgs a, int epi) {
  pdl_launch();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)a.m * a.n) return;
  int m = (int)(idx / a.n), o = (int)(idx % a.n);
  const float* xr = a.x + (size_t)m * a.k;
  const float* wr = a.w + (size_t)o * a.k;
  float acc = 0.f;
  for (int i = 0; i < a.k; ++i) acc = fmaf(xr[i], wr[i], acc);
  float v = a.bias ? a.bias[o] + acc : acc;
  if (epi == EPI_GELU) v = gelu_ref(v);
  if (epi == EPI_RESID) v = a.resid[idx] + v;
  a.out[idx] = v;
}

// ------------------------------------------------------------------ small row kernels
__global__ void embed_kernel(const float* __restrict__ wte, const float* __restrict__ wpe, const int* ids,
                             const int* pos, float* out, int rows, int c) {
  pdl_launch();
  pdl_wait();
  int r = blockIdx.x;
  if (r >= rows) return;
  const float* t = wte + (size_t)ids[r] * c;
  const float* p = wpe + (size_t)pos[r] * c;
  for (int i = threadIdx.x; i < c; i += blockDim.x) out[(size_t)r * c + i] = t[i] + p[i];
}

// One warp per row (src/models/cpu.rs:119-143 with tree sums).
__global__ void layernorm_rows_kernel(const float* x, const float* __restrict__ g, const float* __restrict__ b,
                                      float eps, float* out, int rows, int c) {
  pdl_launch();
  pdl_wait();
  int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float* xr = x + (size_t)r * c;
  float s = 0.f;
  for (int i = lane; i < c; i += 32) s += xr[i];
  s = warp_sum(s);
  float mean = s / (float)c;
  float q = 0.f;
  for (int i = lane; i < c; i += 32) {
    float d = xr[i] - mean;
    q += d * d;
  }
  q = warp_sum(q);
  float inv_std = 1.0f / sqrtf(q / (float)c + eps);
  for (int i = lane; i < c; i += 32) out[(size_t)r * c + i] = (xr[i] - mean) * inv_std * g[i] + b[i];
}

// One 128-thread CTA per row, 128-bit loads, row kept in registers between the passes (c % 4 == 0, c <= 4096):
// the row is read from memory once. `lo` (optional) receives y - hi(y), hi = the upper 19 bits a TF32 tensor
// core reads, for the FP32-grade GEMM that consumes the row.
__global__ void __launch_bounds__(128) layernorm_rows_vec_kernel(const float* x, const float* __restrict__ g,
                                                                 const float* __restrict__ b, float eps, float* out,
                                                                 float* lo, int rows, int c) {
  __shared__ float red[4];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  if (r >= rows) return;
  const int c4 = c >> 2;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * c);
  float4 v[8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = tid + i * 128;
    v[i] = idx < c4 ? xr[idx] : make_float4(0, 0, 0, 0);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  s = warp_sum(s);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  const float mean = ((red[0] + red[1]) + (red[2] + red[3])) / (float)c;
  __syncthreads();
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (tid + i * 128 < c4) {
      const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
      q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  q = warp_sum(q);
  if ((tid & 31) == 0) red[tid >> 5] = q;
  __syncthreads();
  const float inv_std = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)c + eps);
  const float4* g4 = reinterpret_cast<const float4*>(g);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* o4 = reinterpret_cast<float4*>(out + (size_t)r * c);
  float4* lo4 = lo ? reinterpret_cast<float4*>(lo + (size_t)r * c) : nullptr;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = tid + i * 128;
    if (idx < c4) {
      const float4 gg = g4[idx], bb = b4[idx];
      const float4 y = make_float4((v[i].x - mean) * inv_std * gg.x + bb.x, (v[i].y - mean) * inv_std * gg.y + bb.y,
                                   (v[i].z - mean) * inv_std * gg.z + bb.z, (v[i].w - mean) * inv_std * gg.w + bb.w);
      o4[idx] = y;
      if (lo4) lo4[idx] = make_float4(y.x - tf32_trunc(y.x), y.y - tf32_trunc(y.y), y.z - tf32_trunc(y.z), y.w - tf32_trunc(y.w));
    }
  }
}

__global__ void split_tf32_kernel(const float* x, float* hi, float* lo, size_t n) {
  pdl_launch();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = x[i];
    const float h = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    hi[i] = h;
    lo[i] = v - h;
  }
}

// One 128-thread CTA per row, 128-bit loads, row kept in registers (c <= 4096) between the passes.
__global__ void __launch_bounds__(128) layernorm_rows_split_kernel(const float* x, const float* __restrict__ g,
                                                                   const float* __restrict__ b, float eps, float* hi,
                                                                   float* lo, int rows, int c) {
  __shared__ float red[4];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  if (r >= rows) return;
  const int c4 = c >> 2;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * c);
  float4 v[8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = tid + i * 128;
    v[i] = idx < c4 ? xr[idx] : make_float4(0, 0, 0, 0);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  s = warp_sum(s);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  const float mean = ((red[0] + red[1]) + (red[2] + red[3])) / (float)c;
  __syncthreads();
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (tid + i * 128 < c4) {
      const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
      q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  q = warp_sum(q);
  if ((tid & 31) == 0) red[tid >> 5] = q;
  __syncthreads();
  const float inv_std = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)c + eps);
  const float4* g4 = reinterpret_cast<const float4*>(g);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* hi4 = reinterpret_cast<float4*>(hi + (size_t)r * c);
  float4* lo4 = reinterpret_cast<float4*>(lo + (size_t)r * c);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = tid + i * 128;
    if (idx < c4) {
      const float4 gg = g4[idx], bb = b4[idx];
      const float y[4] = {(v[i].x - mean) * inv_std * gg.x + bb.x, (v[i].y - mean) * inv_std * gg.y + bb.y,
                          (v[i].z - mean) * inv_std * gg.z + bb.z, (v[i].w - mean) * inv_std * gg.w + bb.w};
      float h[4], l[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        h[e] = __uint_as_float(__float_as_uint(y[e]) & 0xFFFFE000u);
        l[e] = y[e] - h[e];
      }
      hi4[idx] = make_float4(h[0], h[1], h[2], h[3]);
      lo4[idx] = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
}

__global__ void transpose_kernel(const float* __restrict__ src, float* __restrict__ dst, int in_f, int out_f) {
  __shared__ float tile[32][33];
  int o0 = blockIdx.x * 32, i0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int i = i0 + j, o = o0 + threadIdx.x;
    if (i < in_f && o < out_f) tile[j][threadIdx.x] = src[(size_t)i * out_f + o];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int o = o0 + j, i = i0 + threadIdx.x;
    if (i < in_f && o < out_f) dst[(size_t)o * in_f + i] = tile[threadIdx.x][j];
  }
}

__global__ void gather_rows_kernel(const float* src, const int* rows, float* dst, int n, int c) {
  int r = blockIdx.x;
  if (r >= n) return;
  const float* s = src + (size_t)rows[r] * c;
  for (int i = threadIdx.x; i < c; i += blockDim.x) dst[(size_t)r * c + i] = s[i];
}

// ------------------------------------------------------------------ FP32 GEMM (prefill parity path)
// 128x128x8 tiles, 256 threads, 8x8 outputs per thread.
constexpr int GB = 128, GK = 8;
__global__ void __launch_bounds__(256) gemm_f32_kernel(LinearArgs a, int epi) {
  __shared__ __align__(16) float As[GK][GB + 4];
  __shared__ __align__(16) float Ws[GK][GB + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GB, n0 = blockIdx.x * GB;
  const int lr = tid >> 1, lk = (tid & 1) * 4;  // loader: row within tile, k offset
  const int ty = tid >> 4, tx = tid & 15;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const bool arow_ok = (m0 + lr) < a.m, wrow_ok = (n0 + lr) < a.n;
  const float* ap = a.x + (size_t)(m0 + lr) * a.k + lk;
  const float* wp = a.w + (size_t)(n0 + lr) * a.k + lk;
  for (int k0 = 0; k0 < a.k; k0 += GK) {
    float4 av = make_float4(0, 0, 0, 0), wv = make_float4(0, 0, 0, 0);
    if (k0 + lk < a.k) {  // k is a multiple of 4
      if (arow_ok) av = *reinterpret_cast<const float4*>(ap + k0);
      if (wrow_ok) wv = *reinterpret_cast<const float4*>(wp + k0);
    }
    As[lk + 0][lr] = av.x; As[lk + 1][lr] = av.y; As[lk + 2][lr] = av.z; As[lk + 3][lr] = av.w;
    Ws[lk + 0][lr] = wv.x; Ws[lk + 1][lr] = wv.y; Ws[lk + 2][lr] = wv.z; Ws[lk + 3][lr] = wv.w;
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      float4 a1 = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
      float4 b0 = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      float4 b1 = *reinterpret_cast<const float4*>(&Ws[kk][64 + tx * 4]);
      float af[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float bf[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(af[i], bf[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= a.m) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (n >= a.n) continue;
      float v = a.bias ? a.bias[n] + acc[i][j] : acc[i][j];
      if (epi == EPI_GELU) v = gelu_ref(v);
      if (epi == EPI_RESID) v = a.resid[(size_t)m * a.n + n] + v;
      a.out[(size_t)m * a.n + n] = v;
    }
  }
}

// ------------------------------------------------------------------ paged KV helpers
__device__ __forceinline__ size_t kv_row_offset(const KvLayout& kv, int page, int which, int head, int off) {
  // [page][2][head][page_tokens][head_dim]
  return ((((size_t)page * 2 + which) * kv.n_head + head) * kv.page_tokens + off) * kv.head_dim;
}

// One piece of VEC floats of a K or V row per thread (VEC = 4 when head_dim is a multiple of 4:
// rows are 256-byte segments of the page for head_dim 64, and 16 consecutive threads fill one).
template <int VEC>
__global__ void kv_scatter_kernel(const float* __restrict__ qkv, const int* __restrict__ row_slot,
                                  const int* __restrict__ row_pos, float* __restrict__ pool,
                                  const int* __restrict__ page_table, KvLayout kv, int rows) {
  const int c = kv.n_head * kv.head_dim;
  const int per_row = 2 * c / VEC;
  const size_t total = (size_t)rows * per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(idx / per_row), i = (int)(idx % per_row) * VEC;
    const int slot = __ldg(row_slot + r), pos = __ldg(row_pos + r);
    const int page = __ldg(page_table + (size_t)slot * kv.pages_per_seq + pos / kv.page_tokens);
    const int off = pos % kv.page_tokens;
    const int which = i / c, j = i % c, h = j / kv.head_dim, d = j % kv.head_dim;
    const float* src = qkv + (size_t)r * 3 * c + c + i;
    float* dst = pool + kv_row_offset(kv, page, which, h, off) + d;
    if (VEC == 4)
      *reinterpret_cast<float4*>(dst) = __ldg(reinterpret_cast<const float4*>(src));
    else
      *dst = __ldg(src);
  }
}

__global__ void kv_gather_kernel(const float* pool, const int* page_table, KvLayout kv, int slot, int seq_len,
                                 int n_positions, float* keys, float* values) {
  // output layout (head * n_positions + pos) * head_dim + dim
  size_t total = (size_t)kv.n_head * n_positions * kv.head_dim;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    int d = (int)(idx % kv.head_dim);
    int pos = (int)((idx / kv.head_dim) % n_positions);
    int h = (int)(idx / ((size_t)kv.head_dim * n_positions));
    float k = 0.f, v = 0.f;
    if (pos < seq_len) {
      int page = page_table[(size_t)slot * kv.pages_per_seq + pos / kv.page_tokens];
      int off = pos % kv.page_tokens;
      k = pool[kv_row_offset(kv, page, 0, h, off) + d];
      v = pool[kv_row_offset(kv, page, 1, h, off) + d];
    }
    keys[idx] = k;
    values[idx] = v;
  }
}

// ------------------------------------------------------------------ decode attention
// cached_self_attention_into (src/models/gpt2/rust.rs:1662-1741): append K,V of the new token,
// scores over the cached keys, softmax, weighted sum of values. One CTA per (head, sequence,
// split); the split partials are merged by whichever CTA of the (head, sequence) finishes last.
constexpr int ATT_THREADS = 128;

__device__ __forceinline__ float block_max_128(float v, float* sm) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum_128(float v, float* sm) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = (sm[0] + sm[1]) + (sm[2] + sm[3]);
  __syncthreads();
  return r;
}

// Merges split partials (m, l, acc[D]) in split order and writes the normalised head output.
// Writes one attention output value, optionally as a TF32 hi/lo pair for the tensor-core linears.
__device__ __forceinline__ void store_split(float* out, float* out_lo, size_t idx, float v) {
  if (out_lo) {
    const float h = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    out[idx] = h;
    out_lo[idx] = v - h;
  } else {
    out[idx] = v;
  }
}

__device__ void merge_splits(const float* part, int splits, int d_len, float* out, float* out_lo, size_t base) {
  for (int d = threadIdx.x; d < d_len; d += blockDim.x) {
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part[(size_t)s * (d_len + 2)]);
    float l = 0.f, o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* p = part + (size_t)s * (d_len + 2);
      float sc = (p[0] == -INFINITY) ? 0.f : expf(p[0] - mx);
      l += p[1] * sc;
      o += p[2 + d] * sc;
    }
    store_split(out, out_lo, base + d, o / l);
  }
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS) decode_attention_kernel(DecodeAttnArgs a) {
  static_assert(D == 64, "fast path is written for head_dim 64");
  extern __shared__ float4 dyn_smem4[];
  float* scores = reinterpret_cast<float*>(dyn_smem4);  // [keys of this split]
  __shared__ float red4[4];
  __shared__ __align__(16) float pv[8][D];
  __shared__ int is_last;

  const int h = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = a.kv.n_head * D;
  pdl_launch();
  pdl_wait();

  const int pos = a.pos[b];
  const int nkeys = pos + 1;
  const int per = (nkeys + a.splits - 1) / a.splits;
  const int k0 = min(sp * per, nkeys), k1 = min(k0 + per, nkeys);
  const int* table = a.page_table + (size_t)b * a.kv.pages_per_seq;
  const float* row = a.qkv + (size_t)b * 3 * c;

  if (k0 <= pos && pos < k1) {  // this split owns the new position: append K,V
    if (tid < 32) {
      const int page = table[pos / a.kv.page_tokens], off = pos % a.kv.page_tokens;
      const int which = tid >> 4, j = tid & 15;
      float4 v = reinterpret_cast<const float4*>(row + c + which * c + h * D)[j];
      reinterpret_cast<float4*>(a.kv_pool + kv_row_offset(a.kv, page, which, h, off))[j] = v;
    }
    __syncthreads();
  }

  // scores: four lanes per key, lane part p owns float4 i*4+p (i = 0..3) of the 64 dims
  const int part = lane & 3;
  float4 q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = reinterpret_cast<const float4*>(row + h * D)[i * 4 + part];
  const float scale = 1.0f / sqrtf((float)D);
  float lmax = -INFINITY;
  for (int kb = k0 + warp * 8; kb < k1; kb += 32) {
    const int key = kb + (lane >> 2);
    float s = 0.f;
    if (key < k1) {
      const int page = table[key / a.kv.page_tokens], off = key % a.kv.page_tokens;
      const float4* kr = reinterpret_cast<const float4*>(a.kv_pool + kv_row_offset(a.kv, page, 0, h, off));
#pragma unroll
      for (int i = 0; i < 4; ++i) s = dot4(q[i], kr[i * 4 + part], s);
    }
    s += __shfl_xor_sync(FULL, s, 1);
    s += __shfl_xor_sync(FULL, s, 2);
    s *= scale;
    if (key < k1) {
      if (part == 0) scores[key - k0] = s;
      lmax = fmaxf(lmax, s);
    }
  }
  const float mx = block_max_128(lmax, red4);  // also orders the score writes
  float lsum = 0.f;
  for (int k = k0 + tid; k < k1; k += ATT_THREADS) {
    float e = expf(scores[k - k0] - mx);
    scores[k - k0] = e;
    lsum += e;
  }
  const float total = block_sum_128(lsum, red4);

  // weighted values: 16 lanes cover one 64-float row, 8 key groups
  const int dg = tid & 15, kg = tid >> 4;
  float4 acc = make_float4(0, 0, 0, 0);
  for (int k = k0 + kg; k < k1; k += 8) {
    const int page = table[k / a.kv.page_tokens], off = k % a.kv.page_tokens;
    const float4 v = reinterpret_cast<const float4*>(a.kv_pool + kv_row_offset(a.kv, page, 1, h, off))[dg];
    const float p = scores[k - k0];
    acc.x = fmaf(p, v.x, acc.x);
    acc.y = fmaf(p, v.y, acc.y);
    acc.z = fmaf(p, v.z, acc.z);
    acc.w = fmaf(p, v.w, acc.w);
  }
  reinterpret_cast<float4*>(&pv[kg][0])[dg] = acc;
  __syncthreads();
  float o = 0.f;
  if (tid < D) {
#pragma unroll
    for (int g = 0; g < 8; ++g) o += pv[g][tid];
  }

  if (a.splits == 1) {
    if (tid < D) store_split(a.out, a.out_lo, (size_t)b * c + h * D + tid, o / total);
    return;
  }
  float* mypart = a.part + ((size_t)(b * a.kv.n_head + h) * a.splits + sp) * (D + 2);
  if (tid < D) mypart[2 + tid] = o;
  if (tid == 0) {
    mypart[0] = (k1 > k0) ? mx : -INFINITY;
    mypart[1] = (k1 > k0) ? total : 0.f;
  }
  // The arrival is an acquire-release atomic at GPU scope: with the CTA barriers around it, it orders this
  // CTA's partial before the arrival and, for the last arriver, every other split's partial before the merge
  // (a separate fence by every thread cost more than the atomic).
  __syncthreads();
  if (tid == 0) {
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(&a.counters[b * a.kv.n_head + h]) : "memory");
    is_last = (old == (unsigned)a.splits - 1);
  }
  __syncthreads();
  if (is_last) {
    merge_splits(a.part + (size_t)(b * a.kv.n_head + h) * a.splits * (D + 2), a.splits, D, a.out, a.out_lo,
                 (size_t)b * c + h * D);
    if (tid == 0) a.counters[b * a.kv.n_head + h] = 0;
  }
}

// Any head_dim, one CTA per (head, sequence), no split. Same arithmetic, simple indexing.
__global__ void decode_attention_generic_kernel(DecodeAttnArgs a) {
  extern __shared__ float4 dyn_smem4[];
  float* scores = reinterpret_cast<float*>(dyn_smem4);
  __shared__ float red4[4];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int D = a.kv.head_dim, c = a.kv.n_head * D;
  pdl_launch();
  pdl_wait();
  const int pos = a.pos[b], nkeys = pos + 1;
  const int* table = a.page_table + (size_t)b * a.kv.pages_per_seq;
  const float* row = a.qkv + (size_t)b * 3 * c;
  {
    const int page = table[pos / a.kv.page_tokens], off = pos % a.kv.page_tokens;
    for (int i = tid; i < 2 * D; i += blockDim.x) {
      int which = i / D, d = i % D;
      a.kv_pool[kv_row_offset(a.kv, page, which, h, off) + d] = row[c + which * c + h * D + d];
    }
  }
  __syncthreads();
  const float scale = 1.0f / sqrtf((float)D);
  float lmax = -INFINITY;
  for (int k = tid; k < nkeys; k += blockDim.x) {
    const int page = table[k / a.kv.page_tokens], off = k % a.kv.page_tokens;
    const float* kr = a.kv_pool + kv_row_offset(a.kv, page, 0, h, off);
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(row[h * D + d], kr[d], s);
    s *= scale;
    scores[k] = s;
    lmax = fmaxf(lmax, s);
  }
  const float mx = block_max_128(lmax, red4);
  float lsum = 0.f;
  for (int k = tid; k < nkeys; k += blockDim.x) {
    float e = expf(scores[k] - mx);
    scores[k] = e;
    lsum += e;
  }
  const float total = block_sum_128(lsum, red4);
  for (int d = tid; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int k = 0; k < nkeys; ++k) {
      const int page = table[k / a.kv.page_tokens], off = k % a.kv.page_tokens;
      o = fmaf(scores[k], a.kv_pool[kv_row_offset(a.kv, page, 1, h, off) + d], o);
    }
    store_split(a.out, a.out_lo, (size_t)b * c + h * D + d, o / total);
  }
}

// ------------------------------------------------------------------ prefill attention
// causal_self_attention (src/models/gpt2/rust.rs:1580-1659) over concatenated sequences.
// CTA = 64 queries of one (head, sequence), 128 threads, keys / values in tiles of 64. Both products
// are register-tiled FP32 GEMMs out of shared memory: S = Q K^T with a 4 x 8 tile per thread
// (rows ty + 16 i, key columns tx + 8 j: consecutive lanes read consecutive rows, conflict-free
// with the 68-float row pitch), online softmax per row across the eight threads that share it,
// P staged in shared memory, O += P V with a 4 x 8 tile per thread (value dims 4 tx .. and
// 32 + 4 tx ..). About ten FMAs per 128-bit shared-memory load.
constexpr int PA_Q = 64, PA_K = 64, PA_PITCH = 68;
constexpr int PA_SMEM = (3 * PA_Q * PA_PITCH + PA_K * 64) * 4;  // Q, K, P padded; V unpadded
template <int D>
__global__ void __launch_bounds__(128) prefill_attention_kernel(PrefillAttnArgs a) {
  static_assert(D == 64, "fast path is written for head_dim 64");
  extern __shared__ float4 pa_smem4[];
  float* Qs = reinterpret_cast<float*>(pa_smem4);  // [64][68]
  float* Ks = Qs + PA_Q * PA_PITCH;                // [64][68]
  float* Ps = Ks + PA_K * PA_PITCH;                // [64][68]
  float* Vs = Ps + PA_Q * PA_PITCH;                // [64][64]
  const int h = blockIdx.x, qb = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, tx = tid & 7, ty = tid >> 3;
  const int c = a.n_head * D;
  const int r0 = a.seq_start[b], len = a.seq_start[b + 1] - r0;
  const int q0 = qb * PA_Q;
  if (q0 >= len) return;
  const float scale = 1.0f / sqrtf((float)D);

  // Q tile: 64 rows x 16 float4 (rows past the sequence end are zero)
  for (int i = tid; i < PA_Q * (D / 4); i += 128) {
    const int r = i >> 4, d4 = i & 15;
    float4 v = make_float4(0, 0, 0, 0);
    if (q0 + r < len) v = reinterpret_cast<const float4*>(a.qkv + (size_t)(r0 + q0 + r) * 3 * c + h * D)[d4];
    *reinterpret_cast<float4*>(Qs + r * PA_PITCH + d4 * 4) = v;
  }
  float m[4], l[4], o[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) o[i][j] = 0.f;
  }

  const int kend = min(len, q0 + PA_Q);  // keys needed by the last query of this CTA
  for (int kt = 0; kt < kend; kt += PA_K) {
    __syncthreads();  // previous tile's P and V reads are done (and Q is written, first time round)
    for (int i = tid; i < PA_K * (D / 4); i += 128) {
      const int r = i >> 4, d4 = i & 15;
      float4 kv = make_float4(0, 0, 0, 0), vv = kv;
      if (kt + r < len) {
        const float* base = a.qkv + (size_t)(r0 + kt + r) * 3 * c + h * D;
        kv = reinterpret_cast<const float4*>(base + c)[d4];
        vv = reinterpret_cast<const float4*>(base + 2 * c)[d4];
      }
      *reinterpret_cast<float4*>(Ks + r * PA_PITCH + d4 * 4) = kv;
      *reinterpret_cast<float4*>(Vs + r * D + d4 * 4) = vv;
    }
    __syncthreads();
    // ---- S = Q K^T
    float s[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) s[i][j] = 0.f;
#pragma unroll 4
    for (int d4 = 0; d4 < D / 4; ++d4) {
      float4 qv[4], kv[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty + 16 * i) * PA_PITCH + d4 * 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) kv[j] = *reinterpret_cast<const float4*>(Ks + (tx + 8 * j) * PA_PITCH + d4 * 4);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) s[i][j] = dot4(qv[i], kv[j], s[i][j]);
    }
    // ---- scale, causal mask, online softmax per query row (shared by the 8 lanes tx = 0..7)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qpos = q0 + ty + 16 * i;
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int kpos = kt + tx + 8 * j;
        s[i][j] = (kpos <= qpos && qpos < len) ? s[i][j] * scale : -INFINITY;
        tmax = fmaxf(tmax, s[i][j]);
      }
      tmax = fmaxf(tmax, __shfl_xor_sync(FULL, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(FULL, tmax, 2));
      tmax = fmaxf(tmax, __shfl_xor_sync(FULL, tmax, 4));
      const float mn = fmaxf(m[i], tmax);
      const float mref = (mn == -INFINITY) ? 0.f : mn;  // nothing unmasked yet: every term below is 0
      const float corr = expf(m[i] - mref);             // m = -inf before the first unmasked key: 0
      float ps = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p = expf(s[i][j] - mref);  // masked: expf(-inf) = 0
        ps += p;
        Ps[(ty + 16 * i) * PA_PITCH + tx + 8 * j] = p;
      }
      ps += __shfl_xor_sync(FULL, ps, 1);
      ps += __shfl_xor_sync(FULL, ps, 2);
      ps += __shfl_xor_sync(FULL, ps, 4);
      l[i] = l[i] * corr + ps;
      m[i] = mn;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[i][j] *= corr;
    }
    __syncthreads();
    // ---- O += P V
#pragma unroll 4
    for (int k4 = 0; k4 < PA_K / 4; ++k4) {
      float4 pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * i) * PA_PITCH + k4 * 4);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float4 va = *reinterpret_cast<const float4*>(Vs + (k4 * 4 + kk) * D + tx * 4);
        const float4 vb = *reinterpret_cast<const float4*>(Vs + (k4 * 4 + kk) * D + 32 + tx * 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float p = kk == 0 ? pv[i].x : kk == 1 ? pv[i].y : kk == 2 ? pv[i].z : pv[i].w;
          o[i][0] = fmaf(p, va.x, o[i][0]); o[i][1] = fmaf(p, va.y, o[i][1]);
          o[i][2] = fmaf(p, va.z, o[i][2]); o[i][3] = fmaf(p, va.w, o[i][3]);
          o[i][4] = fmaf(p, vb.x, o[i][4]); o[i][5] = fmaf(p, vb.y, o[i][5]);
          o[i][6] = fmaf(p, vb.z, o[i][6]); o[i][7] = fmaf(p, vb.w, o[i][7]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qpos = q0 + ty + 16 * i;
    if (qpos < len) {
      const float inv = 1.0f / l[i];
      float* orow = a.out + (size_t)(r0 + qpos) * c + h * D;
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = o[i][e] * inv;
      *reinterpret_cast<float4*>(orow + tx * 4) = make_float4(y[0], y[1], y[2], y[3]);
      *reinterpret_cast<float4*>(orow + 32 + tx * 4) = make_float4(y[4], y[5], y[6], y[7]);
      if (a.out_lo) {
        float* lrow = a.out_lo + (size_t)(r0 + qpos) * c + h * D;
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] -= tf32_trunc(y[e]);
        *reinterpret_cast<float4*>(lrow + tx * 4) = make_float4(y[0], y[1], y[2], y[3]);
        *reinterpret_cast<float4*>(lrow + 32 + tx * 4) = make_float4(y[4], y[5], y[6], y[7]);
      }
    }
  }
}

// Any head_dim <= 128: one thread per query, two passes over the keys.
__global__ void prefill_attention_generic_kernel(PrefillAttnArgs a) {
  const int h = blockIdx.x, b = blockIdx.z;
  const int D = a.head_dim, c = a.n_head * D;
  const int r0 = a.seq_start[b], len = a.seq_start[b + 1] - r0;
  const int qpos = blockIdx.y * blockDim.x + threadIdx.x;
  if (qpos >= len) return;
  const float* qr = a.qkv + (size_t)(r0 + qpos) * 3 * c + h * D;
  const float scale = 1.0f / sqrtf((float)D);
  float mx = -INFINITY;
  for (int k = 0; k <= qpos; ++k) {
    const float* kr = a.qkv + (size_t)(r0 + k) * 3 * c + c + h * D;
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
    mx = fmaxf(mx, s * scale);
  }
  float acc[128];
  for (int d = 0; d < D; ++d) acc[d] = 0.f;
  float l = 0.f;
  for (int k = 0; k <= qpos; ++k) {
    const float* kr = a.qkv + (size_t)(r0 + k) * 3 * c + c + h * D;
    const float* vr = kr + c;
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
    float p = expf(s * scale - mx);
    l += p;
    for (int d = 0; d < D; ++d) acc[d] = fmaf(p, vr[d], acc[d]);
  }
  for (int d = 0; d < D; ++d) a.out[(size_t)(r0 + qpos) * c + h * D + d] = acc[d] / l;
}

// ------------------------------------------------------------------ argmax / top-k
// argmax_logits (src/models/generation.rs:269-279): first strict maximum from -inf.
__global__ void finalize_kernel(FinalizeArgs a) {
  pdl_launch();
  pdl_wait();
  const int m = blockIdx.x;
  __shared__ float sv[32];
  __shared__ int si[32];
  float bv = -INFINITY;
  int bi = INT_MAX;
  for (int p = threadIdx.x; p < a.parts; p += blockDim.x) {
    float v = a.part_val[(size_t)m * a.parts + p];
    int i = a.part_idx[(size_t)m * a.parts + p];
    if (v > bv || (v == bv && i < bi)) {
      bv = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(FULL, bv, o);
    int oi = __shfl_xor_sync(FULL, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) {
        bv = sv[w];
        bi = si[w];
      }
    int tok;
    if (a.part_val) {
      tok = (bi == INT_MAX) ? 0 : bi;
      a.argmax_out[m] = tok;
    } else {
      tok = a.argmax_out[m];
    }
    a.next_ids[m] = tok;
    const int np = a.pos[m] + 1;
    a.pos[m] = np;
    if (np < a.n_positions) a.token_log[(size_t)m * a.n_positions + np] = tok;
  }
}

__global__ void argmax_rows_kernel(const float* logits, int m, int n, int* out) {
  const int r = blockIdx.x;
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (size_t)r * n;
  float bv = -INFINITY;
  int bi = INT_MAX;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = row[i];
    if (v > bv) {  // increasing i per thread: strict > keeps the lowest index
      bv = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(FULL, bv, o);
    int oi = __shfl_xor_sync(FULL, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) {
        bv = sv[w];
        bi = si[w];
      }
    out[r] = (bi == INT_MAX) ? 0 : bi;
  }
}

// Order of f32::total_cmp as a signed key; larger key = larger value.
__device__ __forceinline__ int total_key(float f) {
  int b = __float_as_int(f);
  return b ^ (int)(((unsigned)(b >> 31)) >> 1);
}

// k rounds of block-wide arg-max over the row held in shared memory. Candidates are the finite
// logits; order is descending total_cmp, ties by lower index (the stable sort of sample_logits,
// src/models/generation.rs:305-318). Rows shorter than k are padded with -inf / -1. Every thread keeps the
// best of its own keys (i = tid, tid + 1024, ...) in registers; a round reduces those 1024 candidates and only
// the thread that owned the winner scans its keys again.
__global__ void __launch_bounds__(1024) topk_rows_kernel(const float* logits, int m, int n, int k, float* vals,
                                                         int* idx) {
  extern __shared__ float4 dyn_smem4[];
  int* keys = reinterpret_cast<int*>(dyn_smem4);  // [n] total-order keys, INT_MIN = removed
  __shared__ int sk[32];
  __shared__ int si[32];
  __shared__ int win_i;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * n;
  int my_k = INT_MIN, my_i = INT_MAX;  // best of this thread's keys; scanning upwards keeps the lower index on ties
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = row[i];
    const int kk = isfinite(v) ? total_key(v) : INT_MIN;
    keys[i] = kk;
    if (kk > my_k) {
      my_k = kk;
      my_i = i;
    }
  }
  for (int round = 0; round < k; ++round) {
    int bk = my_k, bi = my_i;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      int ok = __shfl_xor_sync(FULL, bk, o);
      int oi = __shfl_xor_sync(FULL, bi, o);
      if (ok > bk || (ok == bk && oi < bi)) {
        bk = ok;
        bi = oi;
      }
    }
    if ((threadIdx.x & 31) == 0) {
      sk[threadIdx.x >> 5] = bk;
      si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      bk = threadIdx.x < (blockDim.x >> 5) ? sk[threadIdx.x] : INT_MIN;
      bi = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : INT_MAX;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        int ok = __shfl_xor_sync(FULL, bk, o);
        int oi = __shfl_xor_sync(FULL, bi, o);
        if (ok > bk || (ok == bk && oi < bi)) {
          bk = ok;
          bi = oi;
        }
      }
      if (threadIdx.x == 0) {
        if (bk == INT_MIN) {
          vals[(size_t)r * k + round] = -INFINITY;
          idx[(size_t)r * k + round] = -1;
          win_i = -1;
        } else {
          vals[(size_t)r * k + round] = row[bi];
          idx[(size_t)r * k + round] = bi;
          win_i = bi;
        }
      }
    }
    __syncthreads();
    const int w = win_i;
    if (w >= 0 && (w % (int)blockDim.x) == (int)threadIdx.x) {  // the owner removes it and looks for its next best
      keys[w] = INT_MIN;
      my_k = INT_MIN;
      my_i = INT_MAX;
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int kk = keys[i];
        if (kk > my_k) {
          my_k = kk;
          my_i = i;
        }
      }
    }
    // sk / si / win_i are rewritten only after the next round's first barrier has been passed by everyone who read them
  }
}

// ------------------------------------------------------------------ launch helper
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                   Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int MT, int EPI>
cudaError_t launch_linear_mt(const LinearArgs& a, bool ln, int grid, bool pdl, cudaStream_t s) {
  if (ln) {
    size_t smem = (size_t)MT * a.k * sizeof(float);
    auto kern = linear_decode_kernel<MT, EPI, true>;
    return launch(kern, dim3(grid), dim3(LIN_THREADS), smem, s, pdl, a);
  }
  return launch(linear_decode_kernel<MT, EPI, false>, dim3(grid), dim3(LIN_THREADS), 0, s, pdl, a);
}

template <int EPI>
cudaError_t launch_linear_epi(const LinearArgs& a, bool ln, int mt, int grid, bool pdl, cudaStream_t s) {
  switch (mt) {
    case 1: return launch_linear_mt<1, EPI>(a, ln, grid, pdl, s);
    case 2: return launch_linear_mt<2, EPI>(a, ln, grid, pdl, s);
    case 4: return launch_linear_mt<4, EPI>(a, ln, grid, pdl, s);
    default: return launch_linear_mt<8, EPI>(a, ln, grid, pdl, s);
  }
}

int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

}  // namespace

int linear_decode_grid(int n, int sms) {
  int groups = (n + LIN_ROWS - 1) / LIN_ROWS;
  int cap = sms * 8;  // eight 128-thread CTAs per SM keep >= 32 KB of weight loads in flight
  return groups < cap ? groups : cap;
}

// smallest row count class (1, 2, 4, 8) that takes the shared-memory kernel (one input row is faster on the
// kernel above: GPT-2 medium steps of 1 / 2 / 4 / 8 sequences took 747 / 893 / 1113 / 1580 us with it and
// 758 / 789 / 921 / 1091 us with the shared-memory kernel); PG_LR_MIN_MT overrides it for tuning
static int g_lr_min_mt = [] { const char* e = getenv("PG_LR_MIN_MT"); return e ? atoi(e) : 2; }();

cudaError_t launch_linear_decode(const LinearArgs& a, int epilogue, bool pdl, cudaStream_t s, int* grid_out) {
  if (a.k % 4 != 0 || (a.ln_g && (a.m > 8 || a.k > 2048)) || (a.part_val && a.m > 8)) {
    if (a.ln_g || a.part_val) return cudaErrorInvalidValue;  // callers un-fuse these cases
    size_t total = (size_t)a.m * a.n;
    if (grid_out) *grid_out = 0;
    return launch(linear_generic_kernel, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, s, pdl, a, epilogue);
  }
  int mt = a.m <= 1 ? 1 : a.m <= 2 ? 2 : a.m <= 4 ? 4 : 8;
  if (a.m <= 8 && (mt >= g_lr_min_mt || a.n >= LR_ONE_ROW_MIN_N) && (size_t)mt * a.k * sizeof(float) <= LR_MAX_SMEM) {
    // activations staged in shared memory, one persistent CTA per SM; k is shared out over the warps of a
    // CTA when the matrix has too few rows to give every warp of the chip a row group
    const int groups = (a.n + LR_ROWS - 1) / LR_ROWS, k4 = a.k / 4;
    int kp_shift = 0;
    while (kp_shift < 4 && (groups << (kp_shift + 1)) <= num_sms() * LR_WARPS && (k4 >> (kp_shift + 1)) >= 32) ++kp_shift;
    const int gpc = LR_WARPS >> kp_shift;
    const int grid = std::max(1, std::min(num_sms(), (groups + gpc - 1) / gpc));
    if (grid_out) *grid_out = grid;
    const size_t smem = (size_t)mt * a.k * sizeof(float);
#define PG_LR(MT_)                                                                                                        \
  switch (epilogue) {                                                                                                      \
    case EPI_GELU: return launch(linear_rows_smem_kernel<MT_, EPI_GELU>, dim3(grid), dim3(LR_THREADS), smem, s, pdl, a, kp_shift);   \
    case EPI_RESID: return launch(linear_rows_smem_kernel<MT_, EPI_RESID>, dim3(grid), dim3(LR_THREADS), smem, s, pdl, a, kp_shift); \
    default: return launch(linear_rows_smem_kernel<MT_, EPI_NONE>, dim3(grid), dim3(LR_THREADS), smem, s, pdl, a, kp_shift);         \
  }
    if (mt == 1) { PG_LR(1) }
    if (mt == 2) { PG_LR(2) }
    if (mt == 4) { PG_LR(4) }
    PG_LR(8)
#undef PG_LR
  }
  int grid = linear_decode_grid(a.n, num_sms());
  if (grid_out) *grid_out = grid;
  bool ln = a.ln_g != nullptr;
  switch (epilogue) {
    case EPI_GELU: return launch_linear_epi<EPI_GELU>(a, ln, mt, grid, pdl, s);
    case EPI_RESID: return launch_linear_epi<EPI_RESID>(a, ln, mt, grid, pdl, s);
    default: return launch_linear_epi<EPI_NONE>(a, ln, mt, grid, pdl, s);
  }
}

cudaError_t launch_embed(const float* wte, const float* wpe, const int* ids, const int* pos, float* out, int rows,
                         int c, bool pdl, cudaStream_t s) {
  return launch(embed_kernel, dim3(rows), dim3(256), 0, s, pdl, wte, wpe, ids, pos, out, rows, c);
}

cudaError_t launch_layernorm_rows(const float* x, const float* g, const float* b, float eps, float* out, int rows,
                                  int c, bool pdl, cudaStream_t s, float* lo) {
  if (c % 4 == 0 && c <= 4096)
    return launch(layernorm_rows_vec_kernel, dim3(rows), dim3(128), 0, s, pdl, x, g, b, eps, out, lo, rows, c);
  if (lo) return cudaErrorInvalidValue;
  return launch(layernorm_rows_kernel, dim3((rows + 3) / 4), dim3(128), 0, s, pdl, x, g, b, eps, out, rows, c);
}

cudaError_t launch_split_tf32(const float* x, float* hi, float* lo, size_t n, bool pdl, cudaStream_t s) {
  int grid = (int)std::min<size_t>((n + 255) / 256, 1184);
  return launch(split_tf32_kernel, dim3(grid), dim3(256), 0, s, pdl, x, hi, lo, n);
}

cudaError_t launch_layernorm_rows_split(const float* x, const float* g, const float* b, float eps, float* hi,
                                        float* lo, int rows, int c, bool pdl, cudaStream_t s) {
  if (c % 4 != 0 || c > 4096) return cudaErrorInvalidValue;
  return launch(layernorm_rows_split_kernel, dim3(rows), dim3(128), 0, s, pdl, x, g, b, eps, hi, lo, rows, c);
}

cudaError_t launch_gemm_f32(const LinearArgs& a, int epilogue, cudaStream_t s) {
  if (a.k % 4 != 0) {
    size_t total = (size_t)a.m * a.n;
    return launch(linear_generic_kernel, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, s, false, a, epilogue);
  }
  dim3 grid((a.n + GB - 1) / GB, (a.m + GB - 1) / GB);
  return launch(gemm_f32_kernel, grid, dim3(256), 0, s, false, a, epilogue);
}

cudaError_t launch_transpose(const float* src, float* dst, int in_f, int out_f, cudaStream_t s) {
  dim3 grid((out_f + 31) / 32, (in_f + 31) / 32);
  transpose_kernel<<<grid, dim3(32, 8), 0, s>>>(src, dst, in_f, out_f);
  return cudaGetLastError();
}

cudaError_t launch_decode_attention(const DecodeAttnArgs& a, bool pdl, cudaStream_t s) {
  const int max_keys = a.kv.pages_per_seq * a.kv.page_tokens;
  if (a.kv.head_dim == 64) {
    size_t smem = (size_t)((max_keys + a.splits - 1) / a.splits + 1) * sizeof(float);
    smem = (smem + 15) & ~(size_t)15;
    auto kern = decode_attention_kernel<64>;
    if (smem > 64 * 1024) return cudaErrorInvalidValue;
    return launch(kern, dim3(a.kv.n_head, a.batch, a.splits), dim3(ATT_THREADS), smem, s, pdl, a);
  }
  size_t smem = ((size_t)max_keys * sizeof(float) + 15) & ~(size_t)15;
  auto kern = decode_attention_generic_kernel;
  if (smem > 64 * 1024) return cudaErrorInvalidValue;
  return launch(kern, dim3(a.kv.n_head, a.batch, 1), dim3(ATT_THREADS), smem, s, pdl, a);
}

cudaError_t launch_prefill_attention(const PrefillAttnArgs& a, cudaStream_t s) {
  if (a.head_dim == 64) {
    dim3 grid(a.n_head, (a.max_len + PA_Q - 1) / PA_Q, a.batch);
    prefill_attention_kernel<64><<<grid, 128, PA_SMEM, s>>>(a);
  } else {
    if (a.head_dim > 128) return cudaErrorInvalidValue;
    dim3 grid(a.n_head, (a.max_len + 63) / 64, a.batch);
    prefill_attention_generic_kernel<<<grid, 64, 0, s>>>(a);
  }
  return cudaGetLastError();
}

cudaError_t launch_kv_scatter(const float* qkv, const int* row_slot, const int* row_pos, float* kv_pool,
                              const int* page_table, KvLayout kv, int rows, cudaStream_t s) {
  const int vec = kv.head_dim % 4 == 0 ? 4 : 1;
  const size_t total = (size_t)rows * (2 * kv.n_head * kv.head_dim / vec);
  const unsigned blocks = std::max(1u, (unsigned)std::min<size_t>((total + 255) / 256, (size_t)148 * 16));
  if (vec == 4)
    kv_scatter_kernel<4><<<blocks, 256, 0, s>>>(qkv, row_slot, row_pos, kv_pool, page_table, kv, rows);
  else
    kv_scatter_kernel<1><<<blocks, 256, 0, s>>>(qkv, row_slot, row_pos, kv_pool, page_table, kv, rows);
  return cudaGetLastError();
}

cudaError_t launch_kv_gather(const float* kv_pool, const int* page_table, KvLayout kv, int slot, int seq_len,
                             int n_positions, float* keys, float* values, cudaStream_t s) {
  kv_gather_kernel<<<296, 256, 0, s>>>(kv_pool, page_table, kv, slot, seq_len, n_positions, keys, values);
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const float* src, const int* rows, float* dst, int n, int c, cudaStream_t s) {
  gather_rows_kernel<<<n, 256, 0, s>>>(src, rows, dst, n, c);
  return cudaGetLastError();
}

cudaError_t launch_finalize(const FinalizeArgs& a, bool pdl, cudaStream_t s) {
  return launch(finalize_kernel, dim3(a.m), dim3(256), 0, s, pdl, a);
}

cudaError_t init_kernel_attributes() {
  const int ln_smem = 8 * 2048 * (int)sizeof(float);
  cudaError_t e;
#define PG_SET(kern, bytes)                                                                 \
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes)); \
  if (e != cudaSuccess) return e;
  PG_SET((linear_decode_kernel<8, EPI_NONE, true>), ln_smem)
  PG_SET((linear_decode_kernel<8, EPI_GELU, true>), ln_smem)
  PG_SET((linear_decode_kernel<8, EPI_RESID, true>), ln_smem)
  PG_SET((linear_decode_kernel<4, EPI_NONE, true>), ln_smem / 2)
  PG_SET((linear_decode_kernel<4, EPI_GELU, true>), ln_smem / 2)
  PG_SET((linear_decode_kernel<4, EPI_RESID, true>), ln_smem / 2)
#define PG_SET_LR(MT_)                                              \
  PG_SET((linear_rows_smem_kernel<MT_, EPI_NONE>), LR_MAX_SMEM)    \
  PG_SET((linear_rows_smem_kernel<MT_, EPI_GELU>), LR_MAX_SMEM)    \
  PG_SET((linear_rows_smem_kernel<MT_, EPI_RESID>), LR_MAX_SMEM)
  PG_SET_LR(1) PG_SET_LR(2) PG_SET_LR(4) PG_SET_LR(8)
#undef PG_SET_LR
  PG_SET(decode_attention_kernel<64>, 64 * 1024)
  PG_SET(prefill_attention_kernel<64>, PA_SMEM)
  PG_SET(decode_attention_generic_kernel, 64 * 1024)
  PG_SET(topk_rows_kernel, 220 * 1024)
#undef PG_SET
  // The tensor-core GEMMs of a batched decode step need the largest shared-memory carve-out. If
  // the small kernels between them asked for the default (L1-heavy) split, every switch would
  // drain and reconfigure the SMs; they do not depend on L1, so they all request the same split.
#define PG_CARVE(kern)                                                                                      \
  e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared); \
  if (e != cudaSuccess) return e;
  PG_CARVE(layernorm_rows_split_kernel)
  PG_CARVE(decode_attention_kernel<64>)
  PG_CARVE(argmax_rows_kernel)
  PG_CARVE(finalize_kernel)
  PG_CARVE(embed_kernel)
  PG_CARVE(split_tf32_kernel)
#undef PG_CARVE
  return cudaSuccess;
}

cudaError_t launch_argmax_rows(const float* logits, int m, int n, int* out, cudaStream_t s) {
  argmax_rows_kernel<<<m, 1024, 0, s>>>(logits, m, n, out);
  return cudaGetLastError();
}

cudaError_t launch_topk_rows(const float* logits, int m, int n, int k, float* vals, int* idx, cudaStream_t s) {
  size_t smem = ((size_t)n * sizeof(int) + 15) & ~(size_t)15;
  if (smem > 220 * 1024) return cudaErrorInvalidValue;
  topk_rows_kernel<<<m, 1024, smem, s>>>(logits, m, n, k, vals, idx);
  return cudaGetLastError();
}

}  // namespace pg

// ================================================================== decode attention without allocation
// Some hosts of this library may not allocate device memory at the point where they run a decode
// step: a serving loop that has handed every byte of HBM to its own pool allocator, a plugin that
// is called inside a region where its embedder forbids cudaMalloc (allocation synchronises the
// device and can fail late), or a real-time path that wants no allocator call at all. For them
// the split-K scratch of the decode attention kernel lives in the library image itself.
namespace pg {
int ensure_device(int device);  // model.cu
}

namespace {

constexpr int NOALLOC_MAX_PAIRS = 2048;   // batch * n_head
constexpr int NOALLOC_MAX_SPLITS = 8;
constexpr int NOALLOC_HEAD_DIM = 64;
constexpr size_t NOALLOC_PART_FLOATS = (size_t)NOALLOC_MAX_PAIRS * NOALLOC_MAX_SPLITS * (NOALLOC_HEAD_DIM + 2);
// [partials: pairs x splits x (64 + 2) floats][arrival counters: one 32-bit word per pair], 4.1 MiB.
// Every GPU that loads the library holds one copy until the process exits.
static __device__ __align__(256) float g_attn_static_scratch[NOALLOC_PART_FLOATS + NOALLOC_MAX_PAIRS];

constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};

// In host code `g_attn_static_scratch` is only a handle for the symbol, not a device address:
// the address on the current device has to be asked for, once per device.
int noalloc_scratch(int device, float** out) {
  std::lock_guard<std::mutex> g(g_noalloc_mu);
  if (!g_noalloc_ptr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
    if (e != cudaSuccess)
      return pg::set_error(PG_CUDA, std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
    g_noalloc_ptr[device] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[device];
  return PG_OK;
}

}  // namespace

extern "C" int pg_decode_attention_noalloc(const float* d_qkv, float* d_out, float* d_kv_pool,
                                           const int32_t* d_page_table, const int32_t* d_pos, int32_t batch,
                                           int32_t n_head, int32_t head_dim, int32_t page_tokens,
                                           int32_t pages_per_seq, int32_t splits, int32_t device, void* stream) {
  using namespace pg;
  if (!d_qkv || !d_out || !d_kv_pool || !d_page_table || !d_pos) return set_error(PG_INVALID_INPUT, "null argument");
  if (batch <= 0 || n_head <= 0 || head_dim <= 0 || pages_per_seq <= 0) return set_error(PG_INVALID_INPUT, "bad shape");
  if (page_tokens != 16 && page_tokens != 32 && page_tokens != 64)
    return set_error(PG_INVALID_CONFIG, "cuda page_tokens must be 16, 32 or 64");
  if (device < 0 || device >= NOALLOC_MAX_DEVICES) return set_error(PG_INVALID_INPUT, "device ordinal out of range");
  if (head_dim != NOALLOC_HEAD_DIM) splits = 1;  // only the head_dim 64 kernel splits (and uses scratch)
  if (splits < 1 || splits > NOALLOC_MAX_SPLITS)
    return set_error(PG_INVALID_INPUT, "splits " + std::to_string(splits) + " exceeds the built-in scratch limit of " +
                                           std::to_string(NOALLOC_MAX_SPLITS));
  if ((int64_t)batch * n_head > NOALLOC_MAX_PAIRS)
    return set_error(PG_INVALID_INPUT, "batch * n_head = " + std::to_string((int64_t)batch * n_head) +
                                           " exceeds the built-in scratch limit of " + std::to_string(NOALLOC_MAX_PAIRS));
  if ((int64_t)pages_per_seq * page_tokens > 16320 * (int64_t)splits)
    return set_error(PG_INVALID_INPUT, "context too long for the kernel's score buffer");
  // `device` is made current for the launch and the caller's current device is put back on every way out: an
  // embedder that calls this from a thread bound to another device must not find it changed
  struct DeviceGuard {
    int prev = -1;
    DeviceGuard() {
      if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    }
    ~DeviceGuard() {
      if (prev >= 0) cudaSetDevice(prev);
    }
  } guard;
  if (int r = ensure_device(device)) return r;  // allocates nothing
  float* scratch = nullptr;
  if (int r = noalloc_scratch(device, &scratch)) return r;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned* counters = reinterpret_cast<unsigned*>(scratch + NOALLOC_PART_FLOATS);
  // the array keeps whatever the last call left: the arrival counters must start at zero
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)batch * n_head * sizeof(unsigned), s);
  if (e != cudaSuccess) return set_error(PG_CUDA, std::string("CUDA error: ") + cudaGetErrorString(e));
  DecodeAttnArgs a{};
  a.qkv = d_qkv; a.out = d_out; a.kv_pool = d_kv_pool; a.page_table = d_page_table; a.pos = d_pos;
  a.part = scratch; a.counters = counters;
  a.kv = KvLayout{n_head, head_dim, page_tokens, pages_per_seq};
  a.batch = batch; a.splits = splits;
  e = launch_decode_attention(a, false, s);
  if (e != cudaSuccess) return set_error(PG_CUDA, std::string("CUDA error: ") + cudaGetErrorString(e));
  return PG_OK;
}

