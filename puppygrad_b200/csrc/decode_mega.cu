// One decode step as a single persistent cooperative kernel (FP32, at most 8 sequences).
//
// At one sequence a GPT-2 small step is 62 dependent matrix-vector phases of a few megabytes each;
// as separate kernels every phase pays a launch, a cold first load and a drain. Here all CTAs stay
// resident for the whole step: a phase ends in a grid-wide barrier (bounded spin on a generation
// word), and before a warp arrives at the barrier it has already requested the first weight rows
// of its next phase into registers, so HBM keeps streaming while the barrier resolves.
//
// Phases per layer (block_forward_one_profiled, src/models/gpt2/rust.rs:1136-1250):
//   qkv = LN1(x) Wqkv^T + b | attention over the paged cache (+append) | x += attn Wproj^T + b |
//   h = gelu(LN2(x) Wfc^T + b) | x += h Wproj2^T + b ;  then logits = LN_f(x) wte^T, argmax.
// Work split of a linear phase: weight row r belongs to warp (r mod total_warps); the 32 lanes
// split K with 128-bit loads; no shared-memory reduction is needed.
#include <algorithm>
#include <climits>

#include "kernels.cuh"

namespace pg {
namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr int MG_THREADS = 512;
constexpr int MG_WARPS = MG_THREADS / 32;
constexpr int PFJ = 6;                       // prefetched 128-bit chunks per lane and row (k <= 768 fully)
constexpr unsigned BARRIER_SPIN_LIMIT = 1u << 21;

__device__ __forceinline__ float4 ldg_stream(const float4* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
// Activations written by other SMs earlier in this kernel: read through L2, never a stale L1 line.
__device__ __forceinline__ float4 ld_act4(const float4* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_act(const float* p) { return __ldcg(p); }

__device__ __forceinline__ float dot4(float4 a, float4 b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  acc = fmaf(a.w, b.w, acc);
  return acc;
}
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
__device__ __forceinline__ float gelu_ref(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978846f * (x + 0.044715f * x * x * x)));
}

// N per-lane values -> totals; lane l ends with the total of value index l >> (5 - log2 N).
template <int N, int OFF>
struct MultiReduce {
  static __device__ __forceinline__ void run(float* v, int lane) {
    const bool up = (lane & OFF) != 0;
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
      float send = up ? v[j] : v[j + N / 2];
      float keep = up ? v[j + N / 2] : v[j];
      v[j] = keep + __shfl_xor_sync(FULL, send, OFF);
    }
    MultiReduce<N / 2, OFF / 2>::run(v, lane);
  }
};
template <int OFF>
struct MultiReduce<1, OFF> {
  static __device__ __forceinline__ void run(float* v, int lane) {
    v[0] += __shfl_xor_sync(FULL, v[0], OFF);
    MultiReduce<1, OFF / 2>::run(v, lane);
  }
};
template <>
struct MultiReduce<1, 0> {
  static __device__ __forceinline__ void run(float*, int) {}
};

// Grid-wide barrier. Every CTA of the cooperative launch is resident, so the wait ends as soon as
// the last CTA arrives; the spin is bounded all the same and records an error instead of hanging.
__device__ __forceinline__ void grid_barrier(unsigned* bar, unsigned nblocks, int* err) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned gen, prev, cur;
    // the generation cannot advance before this CTA has arrived, so reading it first is safe
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(bar + 1) : "memory");
    // release: this CTA's earlier writes (made visible to thread 0 by the CTA barrier) are
    // ordered before the arrival
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(bar) : "memory");
    if (prev == nblocks - 1) {
      asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(bar), "r"(0u) : "memory");
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + 1), "r"(gen + 1) : "memory");
    } else {
      unsigned spins = 0;
      for (;;) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(cur) : "l"(bar + 1) : "memory");
        if (cur != gen) break;
        if (++spins > BARRIER_SPIN_LIMIT) {
          atomicCAS(err, 0, 21);
          break;
        }
      }
    }
  }
  __syncthreads();
}

// Weights (and biases) of the first two rows a warp owns in its next linear phase.
struct Prefetch {
  float4 w[2][PFJ];
  float b[2];
};

// Work split of a linear phase inside the grid: `ks` warps of a CTA share one weight row (each a
// contiguous slice of k, so that a slice fits the prefetch registers), a CTA covers
// MG_WARPS / ks rows per pass, pass p of CTA b covers rows (p * gridDim.x + b) * rows_per_cta + ...
__device__ __forceinline__ int k_slices(int k4) {
  int ks = 1;
  while (ks < MG_WARPS && k4 > ks * 32 * PFJ) ks *= 2;
  return ks;
}
struct Split {
  int ks, slice, rsub, rpc, cbeg, cend;
};
__device__ __forceinline__ Split make_split(int k4, int warp) {
  Split s;
  s.ks = k_slices(k4);
  s.slice = warp % s.ks;
  s.rsub = warp / s.ks;
  s.rpc = MG_WARPS / s.ks;
  const int per = (k4 + s.ks - 1) / s.ks;
  s.cbeg = min(s.slice * per, k4);
  s.cend = min(s.cbeg + per, k4);
  return s;
}

__device__ __forceinline__ void prefetch_rows(Prefetch& p, const float* w, const float* bias, int k4, int n, int warp,
                                              int lane) {
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const Split sp = make_split(k4, warp);
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = (rr * (int)gridDim.x + (int)blockIdx.x) * sp.rpc + sp.rsub;
#pragma unroll
    for (int j = 0; j < PFJ; ++j) {
      const int c = sp.cbeg + lane + 32 * j;
      p.w[rr][j] = (row < n && c < sp.cend) ? ldg_stream(w4 + (size_t)row * k4 + c) : make_float4(0, 0, 0, 0);
    }
    p.b[rr] = (bias && row < n) ? bias[row] : 0.f;
  }
}

// LayerNorm of the step's rows into shared memory, by the whole CTA (cpu.rs:119-143, tree sums).
// `from_embedding`: the rows are wte[id] + wpe[pos] (first layer); CTA 0 also stores them to x.
template <int MT>
__device__ void stage_layernorm(const MegaArgs& a, const float* g, const float* b, float4* xs4, float* red,
                                bool from_embedding) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c4 = a.c >> 2;
  float s[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) s[m] = 0.f;
  for (int c = tid; c < c4; c += MG_THREADS) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float4 v = make_float4(0, 0, 0, 0);
      if (m < a.m) {
        if (from_embedding) {
          const float4 t = reinterpret_cast<const float4*>(a.wte + (size_t)a.ids[m] * a.c)[c];
          const float4 p = reinterpret_cast<const float4*>(a.wpe + (size_t)a.pos[m] * a.c)[c];
          v = make_float4(t.x + p.x, t.y + p.y, t.z + p.z, t.w + p.w);
          if (blockIdx.x == 0) reinterpret_cast<float4*>(a.x + (size_t)m * a.c)[c] = v;
        } else {
          v = ld_act4(reinterpret_cast<const float4*>(a.x + (size_t)m * a.c) + c);
        }
      }
      xs4[(size_t)m * c4 + c] = v;
      s[m] += (v.x + v.y) + (v.z + v.w);
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    s[m] = warp_sum(s[m]);
    if (lane == 0) red[warp * MT + m] = s[m];
  }
  __syncthreads();
  float mean[MT], q[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < MG_WARPS; ++w) t += red[w * MT + m];
    mean[m] = t / (float)a.c;
    q[m] = 0.f;
  }
  for (int c = tid; c < c4; c += MG_THREADS) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float4 v = xs4[(size_t)m * c4 + c];
      const float d0 = v.x - mean[m], d1 = v.y - mean[m], d2 = v.z - mean[m], d3 = v.w - mean[m];
      q[m] += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  float* red2 = red + MG_WARPS * MT;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    q[m] = warp_sum(q[m]);
    if (lane == 0) red2[warp * MT + m] = q[m];
  }
  __syncthreads();
  const float4* g4 = reinterpret_cast<const float4*>(g);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  for (int c = tid; c < c4; c += MG_THREADS) {
    const float4 gg = g4[c], bb = b4[c];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < MG_WARPS; ++w) t += red2[w * MT + m];
      const float inv_std = 1.0f / sqrtf(t / (float)a.c + a.eps);
      float4 v = xs4[(size_t)m * c4 + c];
      v.x = (v.x - mean[m]) * inv_std * gg.x + bb.x;
      v.y = (v.y - mean[m]) * inv_std * gg.y + bb.y;
      v.z = (v.z - mean[m]) * inv_std * gg.z + bb.z;
      v.w = (v.w - mean[m]) * inv_std * gg.w + bb.w;
      xs4[(size_t)m * c4 + c] = m < a.m ? v : make_float4(0, 0, 0, 0);
    }
  }
  __syncthreads();
}

// Plain copy of the step's input rows [m, k] into shared memory (inputs written by other SMs).
template <int MT>
__device__ void stage_copy(const MegaArgs& a, const float* src, int k, float4* xs4) {
  const int k4 = k >> 2;
  for (int c = threadIdx.x; c < k4; c += MG_THREADS) {
#pragma unroll
    for (int m = 0; m < MT; ++m)
      xs4[(size_t)m * k4 + c] = m < a.m ? ld_act4(reinterpret_cast<const float4*>(src + (size_t)m * k) + c)
                                        : make_float4(0, 0, 0, 0);
  }
  __syncthreads();
}

// out[m, row] = epilogue(bias[row] + dot(x[m, :], w[row, :])) for the rows this CTA owns
// (linear_block_into, rust.rs:1481-1532; logits_from_hidden_into, rust.rs:1767-1813).
// XS: the input rows are in shared memory; otherwise they are read from global memory through L2.
// Must be called by every warp of the CTA (it contains CTA barriers when k is sliced).
template <int MT, int EPI, bool XS>
__device__ __forceinline__ void linear_phase(const MegaArgs& a, const float* w, const float* bias, const float4* xs4,
                                             const float* xg, int k, int n, float* out, const float* resid,
                                             Prefetch& pre, float* kpart, int warp, int lane, float* best_v,
                                             int* best_i) {
  constexpr int NV = 2 * MT;
  constexpr int SH = (NV == 16) ? 1 : (NV == 8) ? 2 : (NV == 4) ? 3 : 4;  // 5 - log2(NV)
  const int k4 = k >> 2;
  const Split sp = make_split(k4, warp);
  const int nj = (sp.cend - sp.cbeg + 31) >> 5;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const float4* x4 = reinterpret_cast<const float4*>(xg);
  const int my = lane >> SH, my_rr = my / MT, my_m = my % MT;
  const bool lane_writes = (lane & ((1 << SH) - 1)) == 0;
  const bool writer = lane_writes && sp.slice == 0 && my_m < a.m;
  const int pass_rows = (int)gridDim.x * sp.rpc;
  bool first = true;
  for (int base = (int)blockIdx.x * sp.rpc; base < n; base += 2 * pass_rows) {  // CTA-uniform trip count
    const int row0 = base + sp.rsub, row1 = row0 + pass_rows;
    const int my_row = my_rr ? row1 : row0;
    float rv = 0.f;
    if (EPI == EPI_RESID && writer && my_row < n) rv = ld_act(resid + (size_t)my_m * n + my_row);
    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = 0.f;
    auto step = [&](const float4& w0, const float4& w1, int c) {
      if (c < sp.cend) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float4 xv;
          if (XS) xv = xs4[(size_t)m * k4 + c];
          else xv = m < a.m ? ld_act4(x4 + (size_t)m * k4 + c) : make_float4(0, 0, 0, 0);
          acc[m] = dot4(w0, xv, acc[m]);
          acc[MT + m] = dot4(w1, xv, acc[MT + m]);
        }
      }
    };
    int j0 = 0;
    if (first) {
#pragma unroll
      for (int j = 0; j < PFJ; ++j) step(pre.w[0][j], pre.w[1][j], sp.cbeg + lane + 32 * j);
      j0 = PFJ;
    }
#pragma unroll 2
    for (int j = j0; j < nj; ++j) {
      const int c = sp.cbeg + lane + 32 * j;
      const float4 w0 = (c < sp.cend && row0 < n) ? ldg_stream(w4 + (size_t)row0 * k4 + c) : make_float4(0, 0, 0, 0);
      const float4 w1 = (c < sp.cend && row1 < n) ? ldg_stream(w4 + (size_t)row1 * k4 + c) : make_float4(0, 0, 0, 0);
      step(w0, w1, c);
    }
    MultiReduce<NV, 16>::run(acc, lane);
    float total = acc[0];
    if (sp.ks > 1) {  // add the k slices of a row in slice order
      if (lane_writes) kpart[warp * NV + my] = acc[0];
      __syncthreads();
      if (sp.slice == 0 && lane_writes) {
        total = 0.f;
        for (int s2 = 0; s2 < sp.ks; ++s2) total += kpart[(warp + s2) * NV + my];
      }
      __syncthreads();
    }
    if (writer && my_row < n) {
      float v = total;
      if (bias) v = (first ? (my_rr ? pre.b[1] : pre.b[0]) : bias[my_row]) + v;
      if (EPI == EPI_GELU) v = gelu_ref(v);
      if (EPI == EPI_RESID) v = rv + v;
      out[(size_t)my_m * n + my_row] = v;
      if (best_v && v > *best_v) {
        *best_v = v;
        *best_i = my_row;
      }
    }
    first = false;
  }
}

__device__ __forceinline__ size_t kv_off(const KvLayout& kv, int page, int which, int head, int off) {
  return ((((size_t)page * 2 + which) * kv.n_head + head) * kv.page_tokens + off) * kv.head_dim;
}

// One (sequence, head, split) of cached_self_attention_into (rust.rs:1662-1741), head_dim 64,
// by the whole CTA. `sm` is the CTA's dynamic shared memory (scores, then the value partials).
__device__ void attention_item(const MegaArgs& a, float* kv_pool, int b, int h, int sp, float* sm, float* red) {
  constexpr int D = 64;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = a.c, splits = a.attn_splits;
  const int pos = a.pos[b], nkeys = pos + 1;
  const int per = (nkeys + splits - 1) / splits;
  const int k0 = min(sp * per, nkeys), k1 = min(k0 + per, nkeys);
  const int* table = a.page_table + (size_t)b * a.kv.pages_per_seq;
  const float* row = a.qkv + (size_t)b * 3 * c;
  float* scores = sm;
  float* pv = sm + ((per + 3) & ~3);  // [MG_THREADS / 16][64]
  __shared__ int is_last;

  if (k0 <= pos && pos < k1) {  // this split owns the new position: append K, V
    if (tid < 32) {
      const int page = table[pos / a.kv.page_tokens], off = pos % a.kv.page_tokens;
      const int which = tid >> 4, j = tid & 15;
      const float4 v = ld_act4(reinterpret_cast<const float4*>(row + c + which * c + h * D) + j);
      reinterpret_cast<float4*>(kv_pool + kv_off(a.kv, page, which, h, off))[j] = v;
    }
    __syncthreads();
  }
  const int part = lane & 3;
  float4 q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = ld_act4(reinterpret_cast<const float4*>(row + h * D) + i * 4 + part);
  const float scale = 1.0f / sqrtf((float)D);
  float lmax = -INFINITY;
  for (int kb = k0 + warp * 8; kb < k1; kb += 8 * MG_WARPS) {
    const int key = kb + (lane >> 2);
    float s = 0.f;
    if (key < k1) {
      const int page = table[key / a.kv.page_tokens], off = key % a.kv.page_tokens;
      const float4* kr = reinterpret_cast<const float4*>(kv_pool + kv_off(a.kv, page, 0, h, off));
#pragma unroll
      for (int i = 0; i < 4; ++i) s = dot4(q[i], ld_act4(kr + i * 4 + part), s);
    }
    s += __shfl_xor_sync(FULL, s, 1);
    s += __shfl_xor_sync(FULL, s, 2);
    s *= scale;
    if (key < k1) {
      if (part == 0) scores[key - k0] = s;
      lmax = fmaxf(lmax, s);
    }
  }
  lmax = warp_max(lmax);
  if (lane == 0) red[warp] = lmax;
  __syncthreads();
  float mx = red[0];
#pragma unroll
  for (int w = 1; w < MG_WARPS; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float lsum = 0.f;
  for (int k = k0 + tid; k < k1; k += MG_THREADS) {
    const float e = expf(scores[k - k0] - mx);
    scores[k - k0] = e;
    lsum += e;
  }
  lsum = warp_sum(lsum);
  if (lane == 0) red[warp] = lsum;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < MG_WARPS; ++w) total += red[w];
  constexpr int KG = MG_THREADS / 16;
  const int dg = tid & 15, kg = tid >> 4;  // 16 lanes per value row, KG key groups
  float4 acc = make_float4(0, 0, 0, 0);
  for (int k = k0 + kg; k < k1; k += KG) {
    const int page = table[k / a.kv.page_tokens], off = k % a.kv.page_tokens;
    const float4 v = ld_act4(reinterpret_cast<const float4*>(kv_pool + kv_off(a.kv, page, 1, h, off)) + dg);
    const float p = scores[k - k0];
    acc.x = fmaf(p, v.x, acc.x);
    acc.y = fmaf(p, v.y, acc.y);
    acc.z = fmaf(p, v.z, acc.z);
    acc.w = fmaf(p, v.w, acc.w);
  }
  reinterpret_cast<float4*>(pv + kg * D)[dg] = acc;
  __syncthreads();
  float o = 0.f;
  if (tid < D) {
#pragma unroll
    for (int g = 0; g < KG; ++g) o += pv[g * D + tid];
  }
  float* out = a.attn + (size_t)b * c + h * D;
  if (splits == 1) {
    if (tid < D) out[tid] = o / total;
    __syncthreads();
    return;
  }
  const int pair = b * a.kv.n_head + h;
  float* mypart = a.attn_part + ((size_t)pair * splits + sp) * (D + 2);
  if (tid < D) mypart[2 + tid] = o;
  if (tid == 0) {
    mypart[0] = (k1 > k0) ? mx : -INFINITY;
    mypart[1] = (k1 > k0) ? total : 0.f;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = (atomicAdd(&a.attn_counters[pair], 1u) == (unsigned)splits - 1);
  __syncthreads();
  if (is_last) {
    __threadfence();
    const float* part_base = a.attn_part + (size_t)pair * splits * (D + 2);
    if (tid < D) {
      float m2 = -INFINITY;
      for (int s = 0; s < splits; ++s) m2 = fmaxf(m2, ld_act(part_base + (size_t)s * (D + 2)));
      float l = 0.f, acc2 = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float* p = part_base + (size_t)s * (D + 2);
        const float pm = ld_act(p);
        const float sc = (pm == -INFINITY) ? 0.f : expf(pm - m2);
        l += ld_act(p + 1) * sc;
        acc2 += ld_act(p + 2 + tid) * sc;
      }
      out[tid] = acc2 / l;
    }
    if (tid == 0) a.attn_counters[pair] = 0;
  }
  __syncthreads();
}

template <int MT>
__global__ void __launch_bounds__(MG_THREADS, 1) decode_step_mega_kernel(MegaArgs a, int xs_floats) {
  extern __shared__ float4 mega_smem4[];
  float4* xs4 = mega_smem4;  // staged input rows of the current phase; attention scratch
  __shared__ float red[2 * MG_WARPS * MT + MG_WARPS];
  __shared__ float kpart[MG_WARPS * 2 * MT];
  __shared__ float cta_best_v[MG_WARPS * 2 * MT];
  __shared__ int cta_best_i[MG_WARPS * 2 * MT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned nblocks = gridDim.x;
  const int c = a.c, f = a.f, c4 = c >> 2, f4 = f >> 2;
  const bool stage_h = (size_t)MT * f <= (size_t)xs_floats;

  long long t_start = clock64(), t_bar = 0, t_att = 0, t_stage = 0, t_head = 0, t_lin = 0, t0;
#define MG_T0() t0 = clock64()
#define MG_ACC(var) var += clock64() - t0
  Prefetch pre;
  prefetch_rows(pre, a.layers[0].w_qkv, a.layers[0].b_qkv, c4, 3 * c, warp, lane);

  for (int l = 0; l < a.n_layer; ++l) {
    const MegaLayer L = a.layers[l];
    // ---- qkv = LN1(x) Wqkv^T + b
    MG_T0(); stage_layernorm<MT>(a, L.ln1_g, L.ln1_b, xs4, red, l == 0); MG_ACC(t_stage);
    MG_T0();
    linear_phase<MT, EPI_NONE, true>(a, L.w_qkv, L.b_qkv, xs4, nullptr, c, 3 * c, a.qkv, nullptr, pre, kpart, warp, lane,
                                     nullptr, nullptr);
    MG_ACC(t_lin);
    prefetch_rows(pre, L.w_proj, L.b_proj, c4, c, warp, lane);
    MG_T0(); grid_barrier(a.barrier, nblocks, a.error_flag); MG_ACC(t_bar);
    // ---- attention over the cache (+ append of the new K, V)
    MG_T0();
    {
      const int items = a.m * a.kv.n_head * a.attn_splits;
      for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int sp = it % a.attn_splits, pair = it / a.attn_splits;
        attention_item(a, L.kv_pool, pair / a.kv.n_head, pair % a.kv.n_head, sp, reinterpret_cast<float*>(xs4), red);
      }
    }
    MG_ACC(t_att);
    MG_T0(); grid_barrier(a.barrier, nblocks, a.error_flag); MG_ACC(t_bar);
    // ---- x += attn Wproj^T + b
    MG_T0(); stage_copy<MT>(a, a.attn, c, xs4); MG_ACC(t_stage);
    linear_phase<MT, EPI_RESID, true>(a, L.w_proj, L.b_proj, xs4, nullptr, c, c, a.x, a.x, pre, kpart, warp, lane, nullptr,
                                      nullptr);
    prefetch_rows(pre, L.w_fc, L.b_fc, c4, f, warp, lane);
    MG_T0(); grid_barrier(a.barrier, nblocks, a.error_flag); MG_ACC(t_bar);
    // ---- h = gelu(LN2(x) Wfc^T + b)
    MG_T0(); stage_layernorm<MT>(a, L.ln2_g, L.ln2_b, xs4, red, false); MG_ACC(t_stage);
    linear_phase<MT, EPI_GELU, true>(a, L.w_fc, L.b_fc, xs4, nullptr, c, f, a.h, nullptr, pre, kpart, warp, lane, nullptr,
                                     nullptr);
    prefetch_rows(pre, L.w_proj2, L.b_proj2, f4, c, warp, lane);
    MG_T0(); grid_barrier(a.barrier, nblocks, a.error_flag); MG_ACC(t_bar);
    // ---- x += h Wproj2^T + b
    if (stage_h) {
      MG_T0(); stage_copy<MT>(a, a.h, f, xs4); MG_ACC(t_stage);
      linear_phase<MT, EPI_RESID, true>(a, L.w_proj2, L.b_proj2, xs4, nullptr, f, c, a.x, a.x, pre, kpart, warp, lane,
                                        nullptr, nullptr);
    } else {
      linear_phase<MT, EPI_RESID, false>(a, L.w_proj2, L.b_proj2, nullptr, a.h, f, c, a.x, a.x, pre, kpart, warp, lane,
                                         nullptr, nullptr);
    }
    if (l + 1 < a.n_layer) prefetch_rows(pre, a.layers[l + 1].w_qkv, a.layers[l + 1].b_qkv, c4, 3 * c, warp, lane);
    else prefetch_rows(pre, a.wte, nullptr, c4, a.v, warp, lane);
    MG_T0(); grid_barrier(a.barrier, nblocks, a.error_flag); MG_ACC(t_bar);
  }

  // ---- logits = LN_f(x) wte^T (no bias), arg-max partials (rust.rs:981-1003, generation.rs:269-279)
  constexpr int NV = 2 * MT;
  constexpr int SH = (NV == 16) ? 1 : (NV == 8) ? 2 : (NV == 4) ? 3 : 4;
  MG_T0();
  stage_layernorm<MT>(a, a.lnf_g, a.lnf_b, xs4, red, false);
  float best_v = -INFINITY;
  int best_i = INT_MAX;
  linear_phase<MT, EPI_NONE, true>(a, a.wte, nullptr, xs4, nullptr, c, a.v, a.logits, nullptr, pre, kpart, warp, lane,
                                   &best_v, &best_i);
  if ((lane & ((1 << SH) - 1)) == 0) {
    cta_best_v[warp * NV + (lane >> SH)] = best_v;
    cta_best_i[warp * NV + (lane >> SH)] = best_i;
  }
  __syncthreads();
  if (tid < MT && tid < a.m) {
    float bv = -INFINITY;
    int bi = INT_MAX;
    for (int w = 0; w < MG_WARPS; ++w)
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const float v = cta_best_v[w * NV + rr * MT + tid];
        const int i = cta_best_i[w * NV + rr * MT + tid];
        if (v > bv || (v == bv && i < bi)) {
          bv = v;
          bi = i;
        }
      }
    a.part_val[(size_t)tid * gridDim.x + blockIdx.x] = bv;
    a.part_idx[(size_t)tid * gridDim.x + blockIdx.x] = bi;
  }
  MG_ACC(t_head);
  MG_T0(); grid_barrier(a.barrier, nblocks, a.error_flag); MG_ACC(t_bar);
  if (a.trace && blockIdx.x == 0 && tid == 0) {
    a.trace[0] += (unsigned long long)(clock64() - t_start);
    a.trace[1] += (unsigned long long)t_bar;
    a.trace[2] += (unsigned long long)t_att;
    a.trace[3] += (unsigned long long)t_stage;
    a.trace[4] += (unsigned long long)t_head;
    a.trace[5] += 1;
    a.trace[6] += (unsigned long long)t_lin;
  }
  // ---- end of step: CTA 0, warp m finishes sequence m
  if (blockIdx.x == 0 && warp < a.m) {
    float bv = -INFINITY;
    int bi = INT_MAX;
    for (int p = lane; p < (int)gridDim.x; p += 32) {
      const float v = ld_act(a.part_val + (size_t)warp * gridDim.x + p);
      const int i = __ldcg(a.part_idx + (size_t)warp * gridDim.x + p);
      if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(FULL, bv, o);
      const int oi = __shfl_xor_sync(FULL, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      const int tok = (bi == INT_MAX) ? 0 : bi;
      a.argmax[warp] = tok;
      a.ids[warp] = tok;
      const int np = a.pos[warp] + 1;
      a.pos[warp] = np;
      if (np < a.n_positions) a.token_log[(size_t)warp * a.n_positions + np] = tok;
    }
  }
}

template <int MT>
cudaError_t launch_mt(const MegaArgs& a, int grid, size_t smem, int xs_floats, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(MG_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // the runtime checks that the whole grid is co-resident
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_step_mega_kernel<MT>, a, xs_floats);
}

constexpr size_t MEGA_SMEM_BYTES = 160 * 1024;  // one 512-thread CTA per SM

template <int MT>
int max_grid(int num_sms) {
  int per_sm = 0;
  if (cudaFuncSetAttribute(decode_step_mega_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)MEGA_SMEM_BYTES) != cudaSuccess)
    return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_mega_kernel<MT>, MG_THREADS,
                                                    MEGA_SMEM_BYTES) != cudaSuccess)
    return 0;
  return num_sms * (per_sm > 1 ? 1 : per_sm);
}

}  // namespace

bool decode_mega_supported(int m, int c, int f, int head_dim) {
  return m >= 1 && m <= 8 && head_dim == 64 && c % 4 == 0 && f % 4 == 0 &&
         (size_t)8 * c * sizeof(float) <= MEGA_SMEM_BYTES;
}

int decode_mega_grid(int num_sms) {
  int g = max_grid<1>(num_sms);
  g = std::min(g, max_grid<2>(num_sms));
  g = std::min(g, max_grid<4>(num_sms));
  g = std::min(g, max_grid<8>(num_sms));
  return g;
}

cudaError_t launch_decode_mega(const MegaArgs& a, int grid, cudaStream_t s) {
  if (!decode_mega_supported(a.m, a.c, a.f, a.kv.head_dim) || grid <= 0) return cudaErrorInvalidValue;
  const int xs_floats = (int)(MEGA_SMEM_BYTES / sizeof(float));
  if (a.m <= 1) return launch_mt<1>(a, grid, MEGA_SMEM_BYTES, xs_floats, s);
  if (a.m <= 2) return launch_mt<2>(a, grid, MEGA_SMEM_BYTES, xs_floats, s);
  if (a.m <= 4) return launch_mt<4>(a, grid, MEGA_SMEM_BYTES, xs_floats, s);
  return launch_mt<8>(a, grid, MEGA_SMEM_BYTES, xs_floats, s);
}

}  // namespace pg
