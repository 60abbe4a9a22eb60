// The batched decode step as one persistent cooperative kernel for sm_100a.
//
// One decode step of a transformer for m <= 64 tokens is a chain of small operations that depend
// on each other through row-wise work (bias, residual, LayerNorm, GELU, attention). Launched one
// by one, each pays its launch, its pipeline fill and its epilogue, which together cost several
// times the streaming time of its weights. Here one CTA per SM stays resident for a whole list of
// phases (GEMM, ROWS, ELEM, ATTN, EMBED, FINAL; see kernels.cuh), separated by grid barriers:
//
//   warp 0      weight producer: TMA loads of 32 KB weight units (two 128 x 32 blocks of the tiled
//               weight copy) into a ring of shared-memory stages. Weights do not depend on
//               activations, so this warp never waits for a phase to begin: while the other warps
//               reduce, normalise, attend or wait at the grid barrier it already fetches the next
//               GEMM's units.
//   warps 4-7   splitters: FP32 weight tile -> TF32 hi/lo pair in tensor memory (tcgen05.st); they
//               run ahead as far as tensor memory stages are free.
//   warp 2      activation producer: after the phase's inputs exist (grid barrier), TMA loads of
//               the 64-token x 32 hi and lo tiles.
//   warps 1, 3  MMA issuers, one per k block of a unit, a 64-column accumulator in tensor memory each:
//               per 8-wide k slice three tcgen05.mma of N = 64 into it (w_hi . x_hi, w_lo . x_hi,
//               w_hi . x_lo). One accumulator for the three products leaves tensor memory for three
//               stages of split weights (two stages and separate columns for w_hi . x_lo measured
//               1% slower: a stage comes back only when its MMAs have completed).
//   warps 8-15  workers: drain the accumulators into per-CTA partial tiles (global memory, L2
//               resident), take part in the grid barrier, run the reduce phases, the attention
//               phases (one warp per sequence-head pair), the embedding and the end-of-step phase.
//
// Every GEMM's units (row tile major, k minor) are cut into equal contiguous shares, one per CTA,
// so all SMs stream the same number of bytes whatever the matrix shape. Partials are added in k
// order by the following phase: results do not depend on scheduling.
//
// Every wait is bounded. On expiry the CTA raises the error word; every role then falls through
// its remaining loops without touching memory, tensor memory is freed and the kernel ends.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace pg {
namespace {

constexpr int CH_THREADS = 512;
// The pipelines move units of CH_UB consecutive k blocks (128 weight rows x 32 floats each): a wait
// on an mbarrier or a tcgen05.commit costs the single MMA-issuing thread as much as several MMAs,
// so fewer, larger hand-overs keep the tensor pipe busier.
constexpr int CH_UB = 2;
constexpr int CH_W_STAGES = 3;    // weight units in flight per SM (32 KB each)
constexpr int CH_X_STAGES = 3;    // units whose activation tiles (shared memory) and split weights (tensor memory) are staged
constexpr int CH_BN = 64;
constexpr int CH_W_BYTES = CH_UB * TILE_M * BK * 4;
constexpr int CH_ACT_BYTES = CH_UB * 2 * CH_BN * BK * 4;  // per block: x_hi tile then x_lo tile
constexpr int CH_MAX_SEG = 4;     // row tiles one CTA's share may touch
constexpr int CH_WORKERS = 256;
// tensor memory: two accumulators of CH_BN columns, then CH_X_STAGES stages of w_hi | w_lo for the unit's two k blocks
constexpr uint32_t CH_D_COLS = 64, CH_A_COL0 = 128, CH_TMEM_COLS = 512;
static_assert(CH_D_COLS == CH_BN && CH_A_COL0 == 2 * CH_D_COLS && CH_A_COL0 + CH_X_STAGES * 64 * CH_UB <= CH_TMEM_COLS, "tensor memory columns");
// Attention phases stage key / value rows in the (then idle) activation ring plus an extra region:
// each of the eight worker warps has AT_SLOTS slots, each holding AT_ROWS key rows and the AT_ROWS
// value rows of the same positions (one mbarrier per slot: one wait per block of keys).
constexpr int AT_ROWS = 16;
constexpr int AT_SLOTS = 2;
constexpr int AT_SLOT_BYTES = 2 * AT_ROWS * 64 * 4;
constexpr int AT_EXTRA_BYTES = 8 * AT_SLOTS * AT_SLOT_BYTES - CH_X_STAGES * CH_ACT_BYTES;
constexpr int AT_SCRATCH_FLOATS = 4 * 64;  // per group of four warps: one 64-float query per warp
static_assert(AT_EXTRA_BYTES >= 0, "the activation ring is part of the attention staging area");
// 227 KB, the most a CTA can have: the dynamic shared memory must start 1024-byte aligned (checked at run time)
constexpr size_t CH_SMEM = (size_t)CH_W_STAGES * CH_W_BYTES + (size_t)CH_X_STAGES * CH_ACT_BYTES + AT_EXTRA_BYTES +
                           2 * AT_SCRATCH_FLOATS * 4 + 1024;
static_assert(CH_SMEM <= 232448, "shared memory of one CTA");
static_assert(CH_UB == 2, "one MMA issuer per k block of a unit");
static_assert(sizeof(ChainPhase) % 8 == 0 && 384 + 2 * sizeof(ChainPhase) <= 1024, "two phase descriptors behind the barriers");
constexpr size_t CH_PART_TILE = (size_t)CH_BN * TILE_M;  // floats of one partial tile: [token][row]

// Share of one CTA in units: [g0, g1) of the phase's tiles * nkb units (row tile major); per = units per CTA.
struct ChRange {
  int g0, g1, nkb, per;
};
__device__ __host__ inline ChRange chain_range(int n, int k, int cta, int grid, bool whole_tiles = false) {
  const int tiles = (n + TILE_M - 1) / TILE_M, nkb = k / (BK * CH_UB);  // units per row tile
  const int total = tiles * nkb;
  int per = (total + grid - 1) / grid;
  // one block more per CTA when that makes shares line up with row tiles: fewer partial tiles to
  // write and to add, at the price of a few idle SMs
  if (nkb % per != 0 && nkb % (per + 1) == 0) per += 1;
  if (whole_tiles) per = nkb * ((tiles + grid - 1) / grid);
  ChRange r;
  r.nkb = nkb;
  r.per = per;
  r.g0 = cta * per < total ? cta * per : total;
  r.g1 = r.g0 + per < total ? r.g0 + per : total;
  return r;
}

// The same share from the fields chain_prepare_phases filled in: no division.
__device__ __forceinline__ ChRange chain_range_ph(const ChainPhase& ph, int cta) {
  ChRange r;
  r.nkb = ph.r_nkb;
  r.per = ph.r_per;
  const int total = ((ph.n + TILE_M - 1) >> 7) * r.nkb;
  r.g0 = min(cta * r.per, total);
  r.g1 = min(r.g0 + r.per, total);
  return r;
}
static_assert(TILE_M == 128, "row tiles by shift");

__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// All lanes wait (one polling lane with a shuffle behind it measured 2.5% slower here); the verdict is made
// warp-uniform because aligned tcgen05 instructions follow.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* failed, int* err, int code) {
  const bool ok = mbar_wait(bar, parity, failed, err, code);
  return __all_sync(0xffffffffu, ok);
}

// Grid barrier of the worker warps: arrival count only grows during a launch, barrier b (1-based)
// is passed when it reaches grid * b. Returns the same verdict to every worker thread.
__device__ __forceinline__ bool chain_grid_barrier(unsigned* counter, unsigned target, volatile int* failed, int* err,
                                                   int wt, volatile int* verdict, int fence_first, uint64_t* go,
                                                   const int* next_kind) {
  // thread 0 alone needs to know whether a GEMM follows; the load overlaps the CTA barrier
  uint64_t* go_next = nullptr;
  if (wt == 0 && next_kind && !(fence_first & 16) && *next_kind == CH_GEMM) go_next = go;
  workers_sync();
  if (wt == 0) {
    if (!*failed) {
      // The arrival is a release at GPU scope and release is cumulative: what the other workers of this CTA
      // wrote before the CTA barrier above is ordered before it, so no separate fence is needed for them.
      // Results that other CTAs read with TMA loads cross from the generic to the async proxy on the reading
      // side: the activation producer executes fence.proxy.async after it has seen `go` (measured: a second
      // proxy fence here cost 2% of the step, a separate __threadfence() another 4.5%).
      if (fence_first & 1) __threadfence();
      if (fence_first & 2) asm volatile("fence.proxy.async;" ::: "memory");
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
      uint32_t spins = 0;
      for (;;) {
        unsigned v;
        // (polling with relaxed loads and one acquire fence at the end measured 4% slower)
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= target) {
          // the next phase is a GEMM: its activation producer may start before the other workers have been told
          if (go_next) mbar_arrive(go_next);
          break;
        }
        if (++spins > (1u << 22) || *failed) {
          *failed = 1;
          atomicCAS(err, 0, 30);
          break;
        }
      }
    }
    *verdict = *failed;  // one read, so that all workers agree
  }
  workers_sync();
  return *verdict == 0;
}

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// Row arg-max as one 64-bit maximum: high word = the float mapped to an unsigned that orders like the
// float, low word = ~index, so the larger key is the larger value and, among equal values, the lower
// index; the maximum over any order of updates is the first strict maximum of a sequential scan.
__device__ __host__ inline unsigned long long argmax_key(unsigned int float_bits, unsigned int index) {
  const unsigned int ord = (float_bits & 0x80000000u) ? ~float_bits : (float_bits | 0x80000000u);
  return ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - index);
}

__device__ __forceinline__ void chain_trace(const ChainArgs& a, int slot) {
  if (a.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.trace[(size_t)blockIdx.x * 32 + slot] = t;
  }
}

// Developer aid, compiled in only with -DPG_DEV_TRACE (and then active only when the trace buffer exists): clock64()
// stamps of the first 48 weight units of CTA 0 in the whole-tile GEMM (the lm_head), eight events per unit, behind the
// per-CTA slots of the buffer: 0 weight copy issued, 1 splitters saw the weights, 2 ... the free tensor-memory stage,
// 3 split weights stored, 4 activation copy issued, 5 issuer saw the unit ready, 6 its MMAs committed, 7 issuer began
// to wait. Slots 20-22 of every CTA: globaltimer at the start and at the end of its lm_head work, and its SM.
#ifdef PG_DEV_TRACE
__device__ __forceinline__ void unit_trace(const ChainArgs& a, bool on, int u, int e) {
  if (on && a.trace && u < 48) a.trace[(size_t)gridDim.x * 32 + (size_t)u * 8 + e] = (unsigned long long)clock64();
}
#else
__device__ __forceinline__ void unit_trace(const ChainArgs&, bool, int, int) {}
#endif
__device__ __forceinline__ const ChainPhase& phase_at(const ChainArgs& a, int p) {
  return a.phases_dev ? a.phases_dev[p] : a.ph[p];
}

// Tiled load with an L2 eviction-priority hint: the weight stream is read once per step and should not push
// the partial tiles, activations and keys / values of the running step out of L2.
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Sum of the partial tiles covering features [f, f + 4) of token j, in k order. Loads go out in
// batches of NB before the first add, so that their L2 latencies overlap.
// x / d for the small non-negative operands of the share arithmetic (x * d < 2^32): one multiply-high with the
// reciprocal chain_prepare_phases computed on the host (ceil(2^32 / d); d = 1 divides by nothing).
struct FastDiv {
  unsigned magic, d;
};
__device__ __forceinline__ int div_by(int x, FastDiv f) { return f.d > 1 ? (int)__umulhi((unsigned)x, f.magic) : x; }

template <int NB>
__device__ __forceinline__ float4 sum_partials(const float* partials, int f, int j, int nkb, FastDiv by_per, FastDiv by_nkb) {
  const int per = (int)by_per.d;
  const int tile = f >> 7, row = f & 127;
  const int c_lo = div_by(tile * nkb, by_per), c_hi = div_by((tile + 1) * nkb - 1, by_per);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = c_lo; c0 <= c_hi; c0 += NB) {
    float4 v[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      const int c = c0 + i;
      v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c <= c_hi) {
        const int seg = tile - div_by(c * per, by_nkb);
        v[i] = ldcg4(partials + ((size_t)(c * CH_MAX_SEG + seg) * CH_BN + j) * TILE_M + row);
      }
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      if (c0 + i <= c_hi) {
        acc.x += v[i].x;
        acc.y += v[i].y;
        acc.z += v[i].z;
        acc.w += v[i].w;
      }
    }
  }
  return acc;
}

// The same sum when every share lies inside one row tile (nkb % per == 0): the tile's `cnt` = nkb / per
// partial tiles belong to consecutive CTAs and are each CTA's first segment, so the addresses are an
// arithmetic sequence and need no division.
template <int NB>
__device__ __forceinline__ float4 sum_partials_aligned(const float* partials, int f, int j, int cnt) {
  const int tile = f >> 7, row = f & 127;
  const float* p0 = partials + ((size_t)(tile * cnt) * CH_MAX_SEG * CH_BN + j) * TILE_M + row;
  constexpr size_t STRIDE = (size_t)CH_MAX_SEG * CH_BN * TILE_M;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = 0; c0 < cnt; c0 += NB) {
    float4 v[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c0 + i < cnt) v[i] = ldcg4(p0 + (size_t)(c0 + i) * STRIDE);
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      if (c0 + i < cnt) {
        acc.x += v[i].x;
        acc.y += v[i].y;
        acc.z += v[i].z;
        acc.w += v[i].w;
      }
    }
  }
  return acc;
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ROWS phase: x[j, :] += bias + sum of partials, then optional LayerNorm of the updated row written
// as a TF32 hi/lo pair. One CTA per token; wt = worker thread 0..255; n % 4 == 0, n <= 4096.
__device__ __forceinline__ void chain_rows_phase(const ChainArgs& a, const ChainPhase& ph, int j, int wt, float* red, bool embed) {
  const int n = ph.n, n4 = n >> 2;
  const ChRange r = chain_range_ph(ph, 0);
  const bool aligned = r.nkb % r.per == 0;
  const int cnt = r.nkb / r.per;
  float4 v[4];
  float s = 0.f;
  float4* xrow = reinterpret_cast<float4*>(ph.x + (size_t)j * n);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int u = wt + i * CH_WORKERS;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (u < n4 && embed) {  // x = token embedding + position embedding
      const float4 te = __ldg(reinterpret_cast<const float4*>(a.wte + (size_t)__ldg(a.ids + j) * n) + u);
      const float4 pe = __ldg(reinterpret_cast<const float4*>(a.wpe + (size_t)__ldg(a.pos + j) * n) + u);
      v[i] = make_float4(te.x + pe.x, te.y + pe.y, te.z + pe.z, te.w + pe.w);
      xrow[u] = v[i];
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    } else if (u < n4) {
      const float4 xv = __ldcg(xrow + u);
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ph.bias) b = __ldg(reinterpret_cast<const float4*>(ph.bias) + u);
      const float4 acc = aligned ? sum_partials_aligned<16>(a.partials, u * 4, j, cnt)
                                 : sum_partials<16>(a.partials, u * 4, j, r.nkb, FastDiv{ph.r_magic_per, (unsigned)r.per}, FastDiv{ph.r_magic_nkb, (unsigned)r.nkb});
      v[i].x = xv.x + (b.x + acc.x);
      v[i].y = xv.y + (b.y + acc.y);
      v[i].z = xv.z + (b.z + acc.z);
      v[i].w = xv.w + (b.w + acc.w);
      xrow[u] = v[i];
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  if (!ph.ln_g) return;
  const int warp = wt >> 5, lane = wt & 31;
  s = warp_sum_f(s);
  if (lane == 0) red[warp] = s;
  workers_sync();
  const float mean = (((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]))) / (float)n;
  workers_sync();
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (wt + i * CH_WORKERS < n4) {
      const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
      q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  q = warp_sum_f(q);
  if (lane == 0) red[warp] = q;
  workers_sync();
  const float var = (((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]))) / (float)n;
  const float inv_std = 1.0f / sqrtf(var + a.eps);
  float4* hi4 = reinterpret_cast<float4*>(ph.out_hi + (size_t)j * n);
  float4* lo4 = reinterpret_cast<float4*>(ph.out_lo + (size_t)j * n);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int u = wt + i * CH_WORKERS;
    if (u < n4) {
      const float4 g = __ldg(reinterpret_cast<const float4*>(ph.ln_g) + u);
      const float4 b = __ldg(reinterpret_cast<const float4*>(ph.ln_b) + u);
      const float y[4] = {(v[i].x - mean) * inv_std * g.x + b.x, (v[i].y - mean) * inv_std * g.y + b.y,
                          (v[i].z - mean) * inv_std * g.z + b.z, (v[i].w - mean) * inv_std * g.w + b.w};
      float h[4], l[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        h[e] = tf32_hi(y[e]);
        l[e] = y[e] - h[e];
      }
      hi4[u] = make_float4(h[0], h[1], h[2], h[3]);
      lo4[u] = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
  workers_sync();  // `red` is reused by the next phase
}

// ELEM phase: out[j, f] = act(bias[f] + sum of partials), all CTAs, four features per thread.
__device__ __forceinline__ void chain_elem_phase(const ChainArgs& a, const ChainPhase& ph, int wt, unsigned long long* best_s) {
  const int n = ph.n, n4 = (n + 3) >> 2;
  const ChRange r = chain_range_ph(ph, 0);
  const int total = a.m * n4;
  const bool vec = (n & 3) == 0;
  const bool aligned = r.nkb % r.per == 0;
  const int cnt = r.nkb / r.per;
  const FastDiv by_per = {ph.r_magic_per, (unsigned)r.per}, by_nkb = {ph.r_magic_nkb, (unsigned)r.nkb};
  // Every CTA takes one contiguous run of (token, four features) units, its threads interleaved over
  // it: a thread's units then lie in one row, rarely two, so the row arg-max is a running maximum
  // per thread that goes to shared memory only when the row changes.
  const int chunk = (total + (int)gridDim.x - 1) / (int)gridDim.x;
  const int begin = (int)blockIdx.x * chunk, end = min(begin + chunk, total);
  int best_row = -1;
  unsigned long long best_key = 0ull;
  if (ph.best) {
    if (wt < CH_BN) best_s[wt] = 0ull;
    workers_sync();
  }
  // (row, unit in row) of this thread's next unit, advanced without divisions
  int j0 = begin / n4, u0 = begin - j0 * n4 + wt;
  while (u0 >= n4) {
    u0 -= n4;
    ++j0;
  }
  for (int id0 = begin + wt; id0 < end; id0 += 2 * CH_WORKERS) {
    // two units per pass: the second one's loads are in flight while the first is finished
    const int id1 = id0 + CH_WORKERS;
    int j1 = j0, u1 = u0 + CH_WORKERS;
    while (u1 >= n4) {
      u1 -= n4;
      ++j1;
    }
    const int f0 = u0 * 4, f1 = id1 < end ? u1 * 4 : f0;
    if (id1 >= end) j1 = j0;
    const float4 acc0 = aligned ? sum_partials_aligned<8>(a.partials, f0, j0, cnt) : sum_partials<8>(a.partials, f0, j0, r.nkb, by_per, by_nkb);
    const float4 acc1 = aligned ? sum_partials_aligned<8>(a.partials, f1, j1, cnt) : sum_partials<8>(a.partials, f1, j1, r.nkb, by_per, by_nkb);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
    if (half == 1 && id1 >= end) break;
    const int j = half ? j1 : j0, f = half ? f1 : f0;
    const float4 acc = half ? acc1 : acc0;
    float y[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (f + e < n) {
        if (ph.bias) y[e] = __ldg(ph.bias + f + e) + y[e];
        if (ph.gelu) y[e] = gelu_ref(y[e]);
      }
    }
    if (ph.best) {
      if (j != best_row) {
        if (best_row >= 0 && best_key) atomicMax(best_s + best_row, best_key);
        best_row = j;
        best_key = 0ull;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (f + e < n && y[e] == y[e])  // NaN never wins; -0 counts as +0 (neither is greater than the other)
          best_key = max(best_key, argmax_key(y[e] == 0.f ? 0u : __float_as_uint(y[e]), (unsigned)(f + e)));
    }
    const size_t o = (size_t)j * n + f;
    if (vec) {
      if (ph.out) *reinterpret_cast<float4*>(ph.out + o) = make_float4(y[0], y[1], y[2], y[3]);
      if (ph.out_hi) {
        float h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          h[e] = tf32_hi(y[e]);
          l[e] = y[e] - h[e];
        }
        *reinterpret_cast<float4*>(ph.out_hi + o) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(ph.out_lo + o) = make_float4(l[0], l[1], l[2], l[3]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (f + e < n) {
          if (ph.out) ph.out[o + e] = y[e];
          if (ph.out_hi) {
            const float h = tf32_hi(y[e]);
            ph.out_hi[o + e] = h;
            ph.out_lo[o + e] = y[e] - h;
          }
        }
      }
    }
    }
    u0 += 2 * CH_WORKERS;
    while (u0 >= n4) {
      u0 -= n4;
      ++j0;
    }
  }
  if (ph.best) {
    if (best_row >= 0 && best_key) atomicMax(best_s + best_row, best_key);
    workers_sync();
    if (wt < a.m && best_s[wt]) atomicMax(ph.best + wt, best_s[wt]);
  }
}

// FINAL phase: end of a decode step for token j (finalize_kernel's work): the row arg-max the lm_head's
// ELEM phase accumulated becomes the next input id, the position advances, the token is logged.
__device__ __forceinline__ void chain_final_phase(const ChainArgs& a, int j) {
  const unsigned long long key = __ldcg(a.best + j);
  const int tok = (int)(0xffffffffu - (unsigned)(key & 0xffffffffull));
  a.argmax_out[j] = tok;
  a.ids[j] = tok;
  const int np = a.pos_rw[j] + 1;
  a.pos_rw[j] = np;
  if (np < a.n_positions) a.token_log[(size_t)j * a.n_positions + np] = tok;
  a.best[j] = argmax_key(0xff800000u, 0u);  // (-inf, index 0) for the next step
}

// ATTN phase: causal attention of one new token per sequence over the paged cache, head_dim 64.
// One worker WARP per (sequence, head) pair, eight pairs in flight per SM, no block-level barrier.
// The pair's q, k, v come straight from the partial tiles of the QKV GEMM before it (sum in k
// order + bias, as an ELEM phase would do), so that GEMM needs no reduce phase of its own.
// Keys and values are pulled into shared memory in blocks of 16 rows by bulk async copies issued
// up to AT_SLOTS chunks ahead of their use, across pair boundaries. Scores use two lanes per key,
// the weighted sum sixteen lanes per value row, with a running maximum (one pass over the cache).
// The new token's own key and value are appended to the cache.

struct AtCursor {  // where the warp is in issuing its block sequence; the same in every lane, except pg0 / pg1
  int item, blk, nblk, t, b, h;  // item = pair * parts + part; the warp walks blocks part, part + parts, ...
  int pg0, pg1;  // page table entries lane and lane + 32 of sequence b
  uint32_t issued;
};

__device__ __forceinline__ float4 attn_feature4(const ChainArgs& a, const ChainPhase& ph, const ChRange& r, int f, int j) {
  const float4 acc = (r.nkb % r.per == 0) ? sum_partials_aligned<8>(a.partials, f, j, r.nkb / r.per)
                                          : sum_partials<8>(a.partials, f, j, r.nkb, FastDiv{ph.r_magic_per, (unsigned)r.per}, FastDiv{ph.r_magic_nkb, (unsigned)r.nkb});
  float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
  if (ph.bias) b = __ldg(reinterpret_cast<const float4*>(ph.bias + f));
  return make_float4(b.x + acc.x, b.y + acc.y, b.z + acc.z, b.w + acc.w);
}

// q, k and v features [f, f + 4), [c + f, ...), [2c + f, ...) of token j. With at most four partial
// tiles per feature (shares aligned to row tiles) all twelve loads and the three bias loads go out
// before the first add: one L2 round trip instead of three.
__device__ __forceinline__ void attn_qkv4(const ChainArgs& a, const ChainPhase& ph, const ChRange& r, int f, int c, int j,
                                          float4& q, float4& k, float4& v) {
  const int cnt = r.nkb / r.per;
  if (r.nkb % r.per != 0 || cnt > 4) {
    q = attn_feature4(a, ph, r, f, j);
    k = attn_feature4(a, ph, r, c + f, j);
    v = attn_feature4(a, ph, r, 2 * c + f, j);
    return;
  }
  constexpr size_t STRIDE = (size_t)CH_MAX_SEG * CH_BN * TILE_M;
  const float* base[3];
  float4 part[3][4], bias[3];
#pragma unroll
  for (int w = 0; w < 3; ++w) {
    const int ff = w * c + f;
    const int tile = ff >> 7, row = ff & 127;
    base[w] = a.partials + ((size_t)(tile * cnt) * CH_MAX_SEG * CH_BN + j) * TILE_M + row;
    bias[w] = ph.bias ? __ldg(reinterpret_cast<const float4*>(ph.bias + ff)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int w = 0; w < 3; ++w)
      part[w][i] = i < cnt ? ldcg4(base[w] + (size_t)i * STRIDE) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 out[3];
#pragma unroll
  for (int w = 0; w < 3; ++w) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < cnt) {
        acc.x += part[w][i].x;
        acc.y += part[w][i].y;
        acc.z += part[w][i].z;
        acc.w += part[w][i].w;
      }
    }
    out[w] = make_float4(bias[w].x + acc.x, bias[w].y + acc.y, bias[w].z + acc.z, bias[w].w + acc.w);
  }
  q = out[0];
  k = out[1];
  v = out[2];
}

// With few pairs (small batches) the keys of one pair are shared out over `parts` = 2, 4 or 8 warps of one
// CTA, block i of the pair going to part i mod parts, so that no warp idles while another walks a whole
// context alone: parts = the largest power of two with pairs * parts <= worker warps of the grid.
__device__ __forceinline__ int at_parts_shift(int pairs, int grid) {
  int sh = 0;
  while (sh < 3 && (pairs << (sh + 1)) <= grid * 8) ++sh;
  return sh;
}

// Moves the issuing cursor of an attention warp to `item` (all lanes, identical control flow).
__device__ __forceinline__ void at_cursor_load(const ChainArgs& a, AtCursor& cur, int item, int items, int lane, int psh) {
  const int H = a.kv.n_head, pps = a.kv.pages_per_seq;
  cur.item = item;
  cur.blk = 0;
  cur.nblk = 0;
  if (item >= items) return;
  const int pair = item >> psh;
  cur.b = pair / H;
  cur.h = pair - cur.b * H;
  cur.blk = item & ((1 << psh) - 1);
  cur.t = __ldg(a.pos + cur.b);
  cur.nblk = (cur.t + AT_ROWS - 1) / AT_ROWS;
  const int* table = a.page_table + (size_t)cur.b * pps;
  cur.pg0 = lane < pps ? __ldg(table + lane) : 0;
  cur.pg1 = lane + 32 < pps ? __ldg(table + lane + 32) : 0;
}

// Called by the attention warps while they have nothing to do in the GEMM phase before an attention
// phase: position and page table entries of the warp's first pair come in (two dependent global
// loads), so that the attention phase starts with its first copies. (Asking L2 for the pair's first
// key / value blocks here with cp.async.bulk.prefetch.L2 measured slower, twice, and is not done.)
__device__ __forceinline__ void chain_attn_prepare(const ChainArgs& a, int w8, int lane, AtCursor& cur, uint32_t consumed) {
  const int psh = at_parts_shift(a.m * a.kv.n_head, (int)gridDim.x);
  at_cursor_load(a, cur, (int)blockIdx.x * 8 + w8, (a.m * a.kv.n_head) << psh, lane, psh);
  cur.issued = consumed;
}

__device__ __forceinline__ void chain_attn_phase(const ChainArgs& a, const ChainPhase& ph, int wt, uint8_t* stage_all,
                                                 uint64_t* kv_full_all, float* scratch_all, uint32_t& consumed, AtCursor& cur,
                                                 bool prepared, volatile int* failed, bool live) {
  constexpr int D = 64, RB = AT_ROWS;
  const int w8 = wt >> 5, lane = wt & 31;
  uint8_t* stage = stage_all + (size_t)w8 * AT_SLOTS * AT_SLOT_BYTES;
  uint64_t* kv_full = kv_full_all + w8 * AT_SLOTS;
  float4* qs = reinterpret_cast<float4*>(scratch_all + w8 * D);  // this pair's query, 16 float4
  const int H = a.kv.n_head, C = H * D, pt = a.kv.page_tokens, pps = a.kv.pages_per_seq;
  const int pt_shift = pt == 16 ? 4 : pt == 32 ? 5 : 6;
  const int psh = at_parts_shift(a.m * H, (int)gridDim.x), parts = 1 << psh;
  const int items = (a.m * H) << psh, step = (int)gridDim.x * 8, first = (int)blockIdx.x * 8 + w8;
  const ChRange r = chain_range_ph(ph, 0);  // shares of the QKV GEMM whose partials are read
  const float scale = 0.125f;  // 1 / sqrt(64)
  bool ok = live;

  if (!prepared) {
    at_cursor_load(a, cur, first, items, lane, psh);
    cur.issued = consumed;
  }
  // executed by all lanes with identical control flow; only lane 0 starts copies
  auto issue_upto = [&](uint32_t limit) {  // blocks with index < limit may be in flight
    while (cur.issued < limit) {
      if (cur.blk >= cur.nblk) {
        if (cur.item >= items) break;
        at_cursor_load(a, cur, cur.item + step, items, lane, psh);
        if (cur.item >= items) break;
        continue;
      }
      const int rows = min(RB, cur.t - cur.blk * RB);
      const int p0 = cur.blk * RB;
      const int pidx = p0 >> pt_shift, off = p0 & (pt - 1);
      const int page = __shfl_sync(0xffffffffu, pidx < 32 ? cur.pg0 : cur.pg1, pidx & 31);
      {
        // lane 0 copies the key rows, lane 1 the value rows: both copies leave in one instruction
        const uint32_t slot = cur.issued % AT_SLOTS;
        const uint32_t bytes = (uint32_t)rows * D * 4;
        const float* src = ph.kv_pool + ((((size_t)page * 2 + lane) * H + cur.h) * pt + off) * D;  // lane = 0: K, 1: V
        uint8_t* dst = stage + (size_t)slot * AT_SLOT_BYTES + (size_t)lane * (AT_SLOT_BYTES / 2);
        if (lane == 0) mbar_expect_tx(&kv_full[slot], 2 * bytes);
        __syncwarp();
        if (lane < 2) bulk_load(dst, src, bytes, &kv_full[slot]);
      }
      ++cur.issued;
      cur.blk += parts;
    }
  };
  if (ok) issue_upto(consumed + AT_SLOTS);

  const int key = lane >> 1, half = lane & 1;  // scores: two lanes per key, 32 dims each
  const int d4 = lane & 15, kh = lane >> 4;    // values: sixteen lanes per row, two key halves
  for (int item = first; item < items; item += step) {
    const int pair = item >> psh, part = item & (parts - 1);
    const int b = pair / H, h = pair - b * H;
    const int t = __ldg(a.pos + b);
    const int nblk = (t + RB - 1) / RB;
    // q, k, v of the new token: lanes 0-15 each own four of the head's 64 features
    float sn = 0.f;
    float4 vn = make_float4(0.f, 0.f, 0.f, 0.f), kn = vn;
    const int app_page = __ldg(a.page_table + (size_t)b * pps + (t >> pt_shift));  // used after the walk
    if (lane < 16) {
      float4 qv;
      attn_qkv4(a, ph, r, h * D + lane * 4, C, b, qv, kn, vn);
      qs[lane] = qv;
      sn = fmaf(qv.x, kn.x, fmaf(qv.y, kn.y, fmaf(qv.z, kn.z, qv.w * kn.w)));
    }
    sn = warp_sum_f(sn) * scale;
    __syncwarp();
    float m = -INFINITY, l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = part; i < nblk; i += parts) {
      const int rows = min(RB, t - i * RB);
      const uint32_t slot = consumed % AT_SLOTS;
      const uint8_t* blk = stage + (size_t)slot * AT_SLOT_BYTES;  // key rows, then value rows
      // ---- scores of this block's keys
      if (ok) ok = warp_wait(&kv_full[slot], (consumed / AT_SLOTS) & 1, failed, a.error_flag, 31);
      float s0 = 0.f, s1 = 0.f;
      if (ok && key < rows) {
        const float4* kr = reinterpret_cast<const float4*>(blk) + key * 16 + half * 8;
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          // rotate: the eight lanes of a quarter warp hit eight different bank groups
          const int e2 = (e + lane) & 7, e3 = (e + 1 + lane) & 7;
          const float4 ka = kr[e2], kb = kr[e3];
          const float4 qa = qs[half * 8 + e2], qb = qs[half * 8 + e3];
          s0 = fmaf(qa.x, ka.x, s0);
          s1 = fmaf(qb.x, kb.x, s1);
          s0 = fmaf(qa.y, ka.y, s0);
          s1 = fmaf(qb.y, kb.y, s1);
          s0 = fmaf(qa.z, ka.z, s0);
          s1 = fmaf(qb.z, kb.z, s1);
          s0 = fmaf(qa.w, ka.w, s0);
          s1 = fmaf(qb.w, kb.w, s1);
        }
      }
      float s = s0 + s1;
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s = key < rows ? s * scale : -INFINITY;
      float pm = s;
#pragma unroll
      for (int o = 16; o > 1; o >>= 1) pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, o));
      if (pm > m) {  // the running maximum moves (the same decision in every lane): rescale what was summed so far
        const float corr = (m == -INFINITY) ? 0.f : expf(m - pm);
        l *= corr;
        acc.x *= corr;
        acc.y *= corr;
        acc.z *= corr;
        acc.w *= corr;
        m = pm;
      }
      const float p = key < rows ? expf(s - m) : 0.f;
      l += half == 0 ? p : 0.f;
      // ---- weighted values
      const float4* vr = reinterpret_cast<const float4*>(blk + AT_SLOT_BYTES / 2);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int kk = kh * 8 + e;
        const float pk = __shfl_sync(0xffffffffu, p, kk * 2);
        if (ok && kk < rows) {
          const float4 v = vr[kk * 16 + d4];
          acc.x = fmaf(pk, v.x, acc.x);
          acc.y = fmaf(pk, v.y, acc.y);
          acc.z = fmaf(pk, v.z, acc.z);
          acc.w = fmaf(pk, v.w, acc.w);
        }
      }
      consumed += 1;
      __syncwarp();
      if (ok) issue_upto(consumed + AT_SLOTS);  // this block's slot is free
    }
    float ls, pn;
    if (parts > 1) {
      // ---- the two key halves and the lanes' partial sums of this warp's share
      acc.x += __shfl_xor_sync(0xffffffffu, acc.x, 16);
      acc.y += __shfl_xor_sync(0xffffffffu, acc.y, 16);
      acc.z += __shfl_xor_sync(0xffffffffu, acc.z, 16);
      acc.w += __shfl_xor_sync(0xffffffffu, acc.w, 16);
      l = warp_sum_f(l);
      // The parts of a pair are neighbouring warps of this CTA. Every warp has at most one item per phase
      // here (that is how `parts` is chosen), so no copy is in flight and the warp's own staging area is
      // free: (m, l, acc) go there, the warps of the pair meet at a named barrier, and part 0 adds the
      // shares in part order (the same result whichever warp finishes first), then the new token itself.
      float* mine = reinterpret_cast<float*>(stage);
      if (lane < 16) reinterpret_cast<float4*>(mine)[lane] = acc;
      if (lane == 0) {
        mine[64] = m;
        mine[65] = l;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(2 + (w8 >> psh)), "r"(32 << psh) : "memory");
      float mm = fmaxf(m, sn);
      if (part == 0) {
        for (int q = 1; q < parts; ++q)
          mm = fmaxf(mm, reinterpret_cast<const float*>(stage + (size_t)q * AT_SLOTS * AT_SLOT_BYTES)[64]);
        const float c0 = (m == -INFINITY) ? 0.f : expf(m - mm);
        acc.x *= c0;
        acc.y *= c0;
        acc.z *= c0;
        acc.w *= c0;
        l *= c0;
        for (int q = 1; q < parts; ++q) {
          const float* other = reinterpret_cast<const float*>(stage + (size_t)q * AT_SLOTS * AT_SLOT_BYTES);
          const float mq = other[64];
          const float cq = (mq == -INFINITY) ? 0.f : expf(mq - mm);
          const float4 aq = reinterpret_cast<const float4*>(other)[lane & 15];
          acc.x = fmaf(cq, aq.x, acc.x);
          acc.y = fmaf(cq, aq.y, acc.y);
          acc.z = fmaf(cq, aq.z, acc.z);
          acc.w = fmaf(cq, aq.w, acc.w);
          l = fmaf(cq, other[65], l);
        }
      }
      pn = expf(sn - mm);
      ls = l + pn;
    } else {
      // ---- the new token itself, then the two key halves and the lanes' partial sums
      const float m_fin = fmaxf(m, sn);
      const float corr = (m == -INFINITY) ? 0.f : expf(m - m_fin);
      pn = expf(sn - m_fin);
      acc.x *= corr;
      acc.y *= corr;
      acc.z *= corr;
      acc.w *= corr;
      acc.x += __shfl_xor_sync(0xffffffffu, acc.x, 16);
      acc.y += __shfl_xor_sync(0xffffffffu, acc.y, 16);
      acc.z += __shfl_xor_sync(0xffffffffu, acc.z, 16);
      acc.w += __shfl_xor_sync(0xffffffffu, acc.w, 16);
      ls = warp_sum_f(l) * corr + pn;
    }
    if (lane < 16 && ok && part == 0) {
      const float inv = 1.0f / ls;
      const float y[4] = {fmaf(pn, vn.x, acc.x) * inv, fmaf(pn, vn.y, acc.y) * inv, fmaf(pn, vn.z, acc.z) * inv,
                          fmaf(pn, vn.w, acc.w) * inv};
      float hi[4], lo[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        hi[e] = tf32_hi(y[e]);
        lo[e] = y[e] - hi[e];
      }
      const size_t idx = (size_t)b * C + h * D + lane * 4;
      *reinterpret_cast<float4*>(ph.out_hi + idx) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<float4*>(ph.out_lo + idx) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
    if (lane < 16 && part == 0) {  // append the new K and V rows
      const int off = t & (pt - 1);
      reinterpret_cast<float4*>(ph.kv_pool + ((((size_t)app_page * 2 + 0) * H + h) * pt + off) * D)[lane] = kn;
      reinterpret_cast<float4*>(ph.kv_pool + ((((size_t)app_page * 2 + 1) * H + h) * pt + off) * D)[lane] = vn;
    }
    __syncwarp();  // qs is rewritten by the next pair
  }
}

__global__ void __launch_bounds__(CH_THREADS, 1)
    chain_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_hi0,
                 const __grid_constant__ CUtensorMap map_lo0, const __grid_constant__ CUtensorMap map_hi1,
                 const __grid_constant__ CUtensorMap map_lo1, const __grid_constant__ CUtensorMap map_hi2,
                 const __grid_constant__ CUtensorMap map_lo2, const __grid_constant__ ChainArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = smem_raw;
  if ((smem_u32(base) & 1023u) != 0) {  // swizzled TMA tiles need it; every thread takes the same way out
    if (threadIdx.x == 0) atomicCAS(a.error_flag, 0, 35);
    return;
  }
  uint8_t* w_ring = base;
  uint8_t* act_ring = base + (size_t)CH_W_STAGES * CH_W_BYTES;
  // attention staging = the activation ring and the region after it; then the attention scratch
  float* at_scratch = reinterpret_cast<float*>(act_ring + (size_t)CH_X_STAGES * CH_ACT_BYTES + AT_EXTRA_BYTES);
  uint64_t* w_full = reinterpret_cast<uint64_t*>(at_scratch + 2 * AT_SCRATCH_FLOATS);
  uint64_t* w_empty = w_full + CH_W_STAGES;
  uint64_t* ready = w_empty + CH_W_STAGES;  // split weights in tensor memory AND activation tiles in shared memory
  uint64_t* done = ready + CH_X_STAGES;     // the MMAs that read them have completed
  uint64_t* d_full = done + CH_X_STAGES;
  uint64_t* d_empty = d_full + 2;
  uint64_t* go = d_empty + 2;
  uint64_t* kv_full = go + 1;  // [8 worker warps][AT_SLOTS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_full + 8 * AT_SLOTS);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* verdict = reinterpret_cast<volatile int*>(tmem_slot + 2);
  float* red = reinterpret_cast<float*>(tmem_slot + 4);  // 8 floats
  // the descriptor of the current and of the next phase, copied here ahead of the barrier before the phase: what a
  // phase needs first is then a shared-memory read away instead of a chain of L2 reads
  ChainPhase* ph_s = reinterpret_cast<ChainPhase*>(reinterpret_cast<uint8_t*>(w_full) + 384);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = (int)blockIdx.x, grid = (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CH_W_STAGES; ++s) {
      mbar_init(&w_full[s], 1);
      mbar_init(&w_empty[s], 4);
    }
    for (int s = 0; s < CH_X_STAGES; ++s) {
      mbar_init(&ready[s], 5);  // four splitter warps + the activation producer's expect_tx arrival
      mbar_init(&done[s], 2);  // both MMA issuers commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&d_full[s], 2);  // both MMA issuers commit ([0] is used; accumulators are not double-buffered)
      mbar_init(&d_empty[s], 8);
    }
    mbar_init(go, 1);
    for (int s = 0; s < 8 * AT_SLOTS; ++s) mbar_init(&kv_full[s], 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, CH_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Registers follow the work: the producer / issuer warps (one busy lane each) and the splitters
  // give registers back, the worker warps, whose reduce and attention code wants many loads in
  // flight, take them (per warp group of four warps; 128 * (40 + 128) + 256 * 168 = 64 K).

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ---------------------------------------------------------------- weight producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      uint64_t evict_first;
      asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(evict_first));
      const bool hint = (a.tune_fence & 8) == 0;
      uint32_t wi = 0;
      bool ok = true;
      for (int p = 0; p < a.n_phases && ok; ++p) {
        if (phase_at(a, p).kind != CH_GEMM) continue;
        const ChRange r = chain_range_ph(phase_at(a, p), cta);
        const uint32_t b0 = phase_at(a, p).w_block0;
        const bool tr = cta == 0 && phase_at(a, p).whole_tiles;
        for (int g = r.g0; g < r.g1 && ok; ++g, ++wi) {
          const uint32_t s = wi % CH_W_STAGES;
          if (wi >= CH_W_STAGES) ok = mbar_wait(&w_empty[s], ((wi / CH_W_STAGES) - 1) & 1, failed, a.error_flag, 21);
          if (!ok) break;
          unit_trace(a, tr, g - r.g0, 0);
          // one unit = CH_UB consecutive 16 KB blocks of the tiled arena = one box of CH_UB * 128 rows
          mbar_expect_tx(&w_full[s], CH_W_BYTES);
          if (hint)
            tma_load_2d_hint(w_ring + (size_t)s * CH_W_BYTES, &map_w, 0, (int)((b0 + (uint32_t)g * CH_UB) * TILE_M), &w_full[s], evict_first);
          else
            tma_load_2d(w_ring + (size_t)s * CH_W_BYTES, &map_w, 0, (int)((b0 + (uint32_t)g * CH_UB) * TILE_M), &w_full[s]);
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ---------------------------------------------------------------- MMA issuers
    // Issuing one tcgen05.mma costs its thread ~60 clocks whatever the tile, so two threads share the
    // work: the issuer of warp 1 takes k block 0 of every unit, the one of warp 3 k block 1, each
    // into an accumulator of its own; the drain adds the two.
    if (lane == 0) {
      const int b = warp == 1 ? 0 : 1;
      const uint32_t idesc1 = umma_idesc_tf32(TILE_M, CH_BN);
      const uint32_t dcol = tmem_base + (uint32_t)b * CH_D_COLS;
      uint32_t wi = 0, si = 0;
      bool ok = true;
      for (int p = 0; p < a.n_phases && ok; ++p) {
        if (phase_at(a, p).kind != CH_GEMM) continue;
        const ChRange r = chain_range_ph(phase_at(a, p), cta);
        for (int g = r.g0; g < r.g1 && ok;) {
          const int tile = g / r.nkb;
          const int gend = min(r.g1, (tile + 1) * r.nkb);
          if (si >= 1) ok = mbar_wait(d_empty, (si - 1) & 1, failed, a.error_flag, 22);  // the previous row tile is drained
          if (!ok) break;
          tc_fence_after();
          for (int gb = g; gb < gend && ok; ++gb, ++wi) {
            const uint32_t xs = wi % CH_X_STAGES;
            const bool tr = cta == 0 && b == 0 && phase_at(a, p).whole_tiles;
            unit_trace(a, tr, gb - r.g0, 7);
            ok = mbar_wait(&ready[xs], (wi / CH_X_STAGES) & 1, failed, a.error_flag, 23);
            if (!ok) break;
            unit_trace(a, tr, gb - r.g0, 5);
            tc_fence_after();
            // block b of the unit: x_hi rows then x_lo rows in shared memory, w_hi | w_lo columns in tensor memory
            const uint64_t dx = umma_desc_sw128(act_ring + (size_t)xs * CH_ACT_BYTES + (size_t)b * (CH_ACT_BYTES / CH_UB));
            const uint64_t dxl = umma_desc_sw128(act_ring + (size_t)xs * CH_ACT_BYTES + (size_t)b * (CH_ACT_BYTES / CH_UB) + CH_BN * BK * 4);
            const uint32_t ahi = tmem_base + CH_A_COL0 + xs * (64 * CH_UB) + b * 64, alo = ahi + 32;
#pragma unroll
            for (int k = 0; k < BK / 8; ++k) {
              umma_tf32_ts(dcol, ahi + k * 8, dx + (uint64_t)(k * 2), idesc1, (gb != g || k != 0) ? 1u : 0u);
              umma_tf32_ts(dcol, alo + k * 8, dx + (uint64_t)(k * 2), idesc1, 1u);
              umma_tf32_ts(dcol, ahi + k * 8, dxl + (uint64_t)(k * 2), idesc1, 1u);
            }
            umma_commit(&done[xs]);
            unit_trace(a, tr, gb - r.g0, 6);
          }
          if (ok) umma_commit(d_full);
          ++si;
          g = gend;
        }
      }
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------------- activation producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_hi0) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_lo0) : "memory");
      uint32_t wi = 0, gp = 0;
      bool ok = true;
      for (int p = 0; p < a.n_phases && ok; ++p) {
        if (phase_at(a, p).kind != CH_GEMM) continue;
        const ChRange r = chain_range_ph(phase_at(a, p), cta);
        const int act = phase_at(a, p).act;
        const CUtensorMap* mh = act == 0 ? &map_hi0 : act == 1 ? &map_hi1 : &map_hi2;
        const CUtensorMap* ml = act == 0 ? &map_lo0 : act == 1 ? &map_lo1 : &map_lo2;
        ok = mbar_wait(go, gp & 1, failed, a.error_flag, 25);
        ++gp;
        if (!ok) break;
        asm volatile("fence.proxy.async;" ::: "memory");
        for (int g = r.g0; g < r.g1 && ok; ++g, ++wi) {
          const uint32_t s = wi % CH_X_STAGES;
          if (wi >= CH_X_STAGES) ok = mbar_wait(&done[s], ((wi / CH_X_STAGES) - 1) & 1, failed, a.error_flag, 26);
          if (!ok) break;
          unit_trace(a, cta == 0 && phase_at(a, p).whole_tiles, g - r.g0, 4);
          const int kb = (g % r.nkb) * CH_UB;
          uint8_t* dst = act_ring + (size_t)s * CH_ACT_BYTES;
          mbar_expect_tx(&ready[s], CH_ACT_BYTES);
#pragma unroll
          for (int b = 0; b < CH_UB; ++b) {
            tma_load_2d(dst + (size_t)b * (CH_ACT_BYTES / CH_UB), mh, (kb + b) * BK, 0, &ready[s]);
            tma_load_2d(dst + (size_t)b * (CH_ACT_BYTES / CH_UB) + CH_BN * BK * 4, ml, (kb + b) * BK, 0, &ready[s]);
          }
        }
      }
    }
  }
  } else if (warp < 8) {
    // ---------------------------------------------------------------- splitters
    const int q = warp & 3;
    const int row = q * 32 + lane;  // row of the weight tile == tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    uint32_t wi = 0;
    bool ok = true;
    for (int p = 0; p < a.n_phases && ok; ++p) {
      if (phase_at(a, p).kind != CH_GEMM) continue;
      const ChRange r = chain_range_ph(phase_at(a, p), cta);
      for (int g = r.g0; g < r.g1 && ok; ++g, ++wi) {
        const uint32_t s = wi % CH_W_STAGES, xs = wi % CH_X_STAGES;
        const bool tr = cta == 0 && warp == 4 && lane == 0 && phase_at(a, p).whole_tiles;
        ok = warp_wait(&w_full[s], (wi / CH_W_STAGES) & 1, failed, a.error_flag, 27);
        if (!ok) break;
        unit_trace(a, tr, g - r.g0, 1);
        // the tensor-memory stage is free once the MMAs of the unit that used it last have completed
        if (wi >= CH_X_STAGES) ok = warp_wait(&done[xs], ((wi / CH_X_STAGES) - 1) & 1, failed, a.error_flag, 28);
        if (!ok) break;
        unit_trace(a, tr, g - r.g0, 2);
        tc_fence_after();
#pragma unroll
        for (int b = 0; b < CH_UB; ++b) {
          const float4* rowp = reinterpret_cast<const float4*>(w_ring + (size_t)s * CH_W_BYTES + (size_t)b * (TILE_M * BK * 4) +
                                                               (size_t)row * 128);
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = rowp[j ^ (row & 7)];  // undo the 128-byte swizzle: conflict-free per quarter warp
            const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float h = tf32_hi(f[e]);
              hi[j * 4 + e] = __float_as_uint(h);
              lo[j * 4 + e] = __float_as_uint(f[e] - h);
            }
          }
          const uint32_t col = tmem_base + CH_A_COL0 + xs * (64 * CH_UB) + b * 64 + lane_addr;
          tmem_st32(col, hi);
          tmem_st32(col + 32, lo);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&w_empty[s]);  // the unit is in registers / tensor memory: the stage may be refilled
        tmem_wait_st();
        unit_trace(a, tr, g - r.g0, 3);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready[xs]);
      }
    }
  } else {
    // ---------------------------------------------------------------- workers
    asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
    const int wt = (int)threadIdx.x - 256;
    const int ww = wt >> 5;
    const int q = ww & 3, half = ww >> 2;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int row = q * 32 + lane;
    uint32_t si = 0, barriers = 0;
    bool ok = true;     // this warp's drains
    bool live = true;   // same for all workers of the CTA: decided at the grid barriers
    if (wt == 0) chain_trace(a, 31);
    if (wt == 0 && cta == 0 && a.phase_times) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      a.phase_times[0] = t;
    }
    uint32_t at_consumed = 0;  // key / value blocks this warp has used so far (all attention phases)
    AtCursor at_cur;
    bool at_prepared = false;
    at_cur.item = at_cur.blk = at_cur.nblk = at_cur.t = at_cur.b = at_cur.h = at_cur.pg0 = at_cur.pg1 = 0;
    at_cur.issued = 0;
    // Sums of token columns [c0, c0 + 16) of this thread's row: two accumulators (k block 0 and 1 of every unit);
    // the two loads are in flight together
    auto ld_acc = [&](int c0, float* y) {
      uint32_t v[16], u[16];
      tmem_ld16_issue(tmem_base + lane_addr + (uint32_t)c0, v);
      tmem_ld16_issue(tmem_base + CH_D_COLS + lane_addr + (uint32_t)c0, u);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) y[j] = __uint_as_float(v[j]) + __uint_as_float(u[j]);
    };
    constexpr int PH_WORDS = (int)(sizeof(ChainPhase) / 4);
    const bool ph_staged = !(a.tune_fence & 4);
    if (wt < PH_WORDS) reinterpret_cast<uint32_t*>(&ph_s[0])[wt] = reinterpret_cast<const uint32_t*>(&phase_at(a, 0))[wt];
    workers_sync();
    for (int p = 0; p < a.n_phases; ++p) {
      const ChainPhase& ph = ph_staged ? ph_s[p & 1] : phase_at(a, p);
      const int kind = ph.kind;
      if (kind == CH_GEMM) {
        // inputs of this phase exist: previous kernel (first phase), or the barrier just passed, whose polling
        // thread has told the activation producer already
        if (wt == 0 && (p == 0 || (a.tune_fence & 16))) mbar_arrive(go);
        if (live && p + 1 < a.n_phases && phase_at(a, p + 1).kind == CH_ATTN) {
          chain_attn_prepare(a, ww, lane, at_cur, at_consumed);
          at_prepared = true;
        }
        const ChRange r = chain_range_ph(ph, cta);
        unsigned long long* best_s = reinterpret_cast<unsigned long long*>(at_scratch);
        if (ph.whole_tiles && ph.best) {
          if (wt < CH_BN) best_s[wt] = 0ull;
          workers_sync();
        }
        int seg = 0;
        for (int g = r.g0; g < r.g1; ++seg) {
          const int tile = g / r.nkb;
          const int gend = min(r.g1, (tile + 1) * r.nkb);
          if (ok) ok = warp_wait(d_full, si & 1, failed, a.error_flag, 29);
          if (ok && ph.whole_tiles) {
            // finished sums (the share is whole row tiles): store them and fold them into the row arg-max;
            // the accumulator is handed back as soon as it is in registers, so the next tile's MMAs overlap the rest
            tc_fence_after();
            const int feat = tile * TILE_M + row;
            const bool valid = feat < ph.n;
            float y[32];
#pragma unroll
            for (int cc = 0; cc < 32; cc += 16) {
              const int c0 = half * 32 + cc;
              ld_acc(c0, &y[cc]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(d_empty);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int tok = half * 32 + j;
              if (tok >= a.m) continue;  // the same for the whole warp
              if (ph.out && valid) ph.out[(size_t)tok * ph.n + feat] = y[j];
              if (!ph.best) continue;
              // NaN never wins; -0 counts as +0; 0 = no candidate (the high word of a key is never 0 for a number)
              const unsigned bits = y[j] == 0.f ? 0u : __float_as_uint(y[j]);
              const unsigned ord = (valid && y[j] == y[j]) ? ((bits & 0x80000000u) ? ~bits : (bits | 0x80000000u)) : 0u;
              const unsigned mx = __reduce_max_sync(0xffffffffu, ord);
              const unsigned who = __ballot_sync(0xffffffffu, ord == mx);
              if (mx != 0u && lane == 0)  // lowest lane = lowest feature among equals
                atomicMax(best_s + tok, ((unsigned long long)mx << 32) |
                                            (unsigned long long)(0xffffffffu - (unsigned)(tile * TILE_M + q * 32 + __ffs((int)who) - 1)));
            }
          } else if (ok) {
            tc_fence_after();
            float* dst = a.partials + ((size_t)(cta * CH_MAX_SEG + seg) * CH_BN) * TILE_M + row;
#pragma unroll
            for (int cc = 0; cc < 32; cc += 16) {
              const int c0 = half * 32 + cc;
              float y[16];
              ld_acc(c0, y);
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c0 + j < a.m) dst[(size_t)(c0 + j) * TILE_M] = y[j];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(d_empty);
          }
          ++si;
          g = gend;
        }
        if (ph.whole_tiles && ph.best) {
          workers_sync();
          if (live && wt < a.m && best_s[wt]) atomicMax(ph.best + wt, best_s[wt]);
        }
      } else if (kind == CH_ATTN) {
        chain_attn_phase(a, ph, wt, act_ring, kv_full, at_scratch, at_consumed, at_cur, at_prepared, failed, live);
        at_prepared = false;
      } else if (kind == CH_ROWS || kind == CH_EMBED) {
        if (live && cta < a.m) chain_rows_phase(a, ph, cta, wt, red, kind == CH_EMBED);
      } else if (kind == CH_FINAL) {
        if (live && cta == 0 && wt < a.m) chain_final_phase(a, wt);
      } else {
        if (live) chain_elem_phase(a, ph, wt, reinterpret_cast<unsigned long long*>(at_scratch));
      }
      if (wt == 0 && p < 10) chain_trace(a, 10 + p);
#ifdef PG_DEV_TRACE
      if (wt == 0 && a.trace && kind == CH_GEMM && ph.whole_tiles) {
        chain_trace(a, 21);
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        a.trace[(size_t)blockIdx.x * 32 + 22] = smid;
      }
#endif
      if (p + 1 < a.n_phases) {
        if (wt < PH_WORDS)  // the next phase's descriptor; the barrier's first CTA barrier orders it before its readers
          reinterpret_cast<uint32_t*>(&ph_s[(p + 1) & 1])[wt] = reinterpret_cast<const uint32_t*>(&phase_at(a, p + 1))[wt];
        ++barriers;
        live = chain_grid_barrier(a.barrier, (unsigned)grid * barriers, failed, a.error_flag, wt, verdict, a.tune_fence, go,
                                  &phase_at(a, p + 1).kind);
        ok = ok && live;
      }
      if (wt == 0 && p < 10) chain_trace(a, p);
#ifdef PG_DEV_TRACE
      if (wt == 0 && p + 1 < a.n_phases && phase_at(a, p + 1).kind == CH_GEMM && phase_at(a, p + 1).whole_tiles) chain_trace(a, 20);
#endif
      if (wt == 0 && cta == 0 && a.phase_times) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.phase_times[p + 1] = t;
      }
    }
    // leave the barrier word zero for the next launch: the last CTA to get here resets it
    if (wt == 0 && !*failed) {
      const unsigned old = atomicAdd(a.barrier, 1u);
      if (old == (unsigned)grid * (barriers + 1) - 1) atomicExch(a.barrier, 0u);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, CH_TMEM_COLS);
}

}  // namespace

int chain_grid(int num_sms) {
  static int cached = -1;
  if (cached >= 0) return cached;
  cached = 0;
  if (!encode_fn()) return 0;
  if (cudaFuncSetAttribute(chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CH_SMEM) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, chain_kernel, CH_THREADS, CH_SMEM) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int coop = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (per_sm >= 1 && coop) cached = num_sms;
  return cached;
}

size_t chain_partial_floats(int grid) { return (size_t)grid * CH_MAX_SEG * CH_PART_TILE; }

unsigned long long chain_argmax_init() { return argmax_key(0xff800000u, 0u); }

void chain_prepare_phases(ChainPhase* phases, int n_phases, int grid) {
  for (int p = 0; p < n_phases; ++p) {
    ChainPhase& ph = phases[p];
    ph.r_nkb = ph.r_per = 0;
    ph.r_magic_per = ph.r_magic_nkb = 0;
    if (ph.kind == CH_FINAL || ph.k < BK * CH_UB || ph.n < 1) continue;
    const ChRange r = chain_range(ph.n, ph.k, 0, grid, ph.kind == CH_GEMM && ph.whole_tiles);
    ph.r_nkb = r.nkb;
    ph.r_per = r.per;
    ph.r_magic_per = r.per > 1 ? (unsigned)((0x100000000ull + (unsigned)r.per - 1) / (unsigned)r.per) : 0u;
    ph.r_magic_nkb = r.nkb > 1 ? (unsigned)((0x100000000ull + (unsigned)r.nkb - 1) / (unsigned)r.nkb) : 0u;
  }
}

bool chain_supported(const ChainArgs& a, int grid, const ChainPhase* host_phases) {
  const ChainPhase* phs = host_phases ? host_phases : a.ph;
  if (grid <= 0 || a.m < 1 || a.m > CH_BN || a.n_phases < 1) return false;
  if (!host_phases && (a.n_phases > CHAIN_MAX_PHASES || a.phases_dev)) return false;
  for (int p = 0; p < a.n_phases; ++p) {
    const ChainPhase& ph = phs[p];
    if (ph.kind == CH_ATTN) {
      if (a.kv.head_dim != 64 || (a.kv.page_tokens != 16 && a.kv.page_tokens != 32 && a.kv.page_tokens != 64)) return false;
      if (!a.page_table || !a.pos || !ph.kv_pool || !ph.out_hi || !ph.out_lo || a.kv.pages_per_seq > 64) return false;
      if (p == 0 || phs[p - 1].kind != CH_GEMM || phs[p - 1].n != ph.n || phs[p - 1].k != ph.k) return false;
      if (ph.n != 3 * a.kv.n_head * 64) return false;
      continue;
    }
    if (ph.kind == CH_FINAL) {
      if (!a.best || !a.argmax_out || !a.ids || !a.pos_rw || !a.token_log || a.n_positions < 1) return false;
      if (p == 0 || phs[p - 1].best != a.best) return false;
      if (phs[p - 1].kind != CH_ELEM && !(phs[p - 1].kind == CH_GEMM && phs[p - 1].whole_tiles)) return false;
      continue;
    }
    if (ph.k < BK * CH_UB || ph.k % (BK * CH_UB) != 0 || ph.n < 1) return false;
    if (ph.kind == CH_EMBED) {
      if (ph.n % 4 != 0 || ph.n > 4 * 4 * CH_WORKERS || !ph.x || !ph.ln_g || !ph.ln_b || !ph.out_hi || !ph.out_lo) return false;
      if (!a.wte || !a.wpe || !a.ids || !a.pos) return false;
      continue;
    }
    const bool whole = ph.kind == CH_GEMM && ph.whole_tiles;
    const ChRange r = chain_range(ph.n, ph.k, 0, grid, whole);
    if (!whole && (r.per + r.nkb - 2) / r.nkb + 1 > CH_MAX_SEG) return false;  // partial tiles of one CTA
    if (whole && (ph.bias || ph.gelu || ph.out_hi || (p + 1 < a.n_phases && phs[p + 1].kind != CH_FINAL))) return false;
    if (!whole && ph.kind == CH_GEMM && (ph.best || ph.out)) return false;
    if (ph.kind == CH_GEMM) {
      if (ph.act < 0 || ph.act > 2 || !a.act_hi[ph.act] || !a.act_lo[ph.act] || a.act_k[ph.act] != ph.k) return false;
      const unsigned long long rows = ((unsigned long long)ph.w_block0 + (unsigned long long)((ph.n + TILE_M - 1) / TILE_M) * r.nkb * CH_UB) * TILE_M;
      if (rows > 0x7fffffffull || rows * BK > a.arena_floats) return false;
    } else if (ph.kind == CH_ROWS) {
      if (ph.n % 4 != 0 || ph.n > 4 * 4 * CH_WORKERS || !ph.x) return false;
      if (ph.ln_g && (!ph.ln_b || !ph.out_hi || !ph.out_lo)) return false;
      if (p == 0 || phs[p - 1].kind != CH_GEMM || phs[p - 1].n != ph.n || phs[p - 1].k != ph.k) return false;
    } else if (ph.kind == CH_ELEM) {
      if (ph.out_hi && !ph.out_lo) return false;
      if (p == 0 || phs[p - 1].kind != CH_GEMM || phs[p - 1].n != ph.n || phs[p - 1].k != ph.k) return false;
    } else {
      return false;
    }
  }
  return true;
}

// When a.phases_dev is set the caller has validated the phase list with chain_supported already.
cudaError_t launch_chain(const ChainArgs& a, int grid, cudaStream_t s) {
  if (!a.phases_dev && !chain_supported(a, grid)) return cudaErrorInvalidValue;
  CUtensorMap maps[7];
  memset(maps, 0, sizeof(maps));
  if (!make_map(&maps[0], a.arena, a.arena_floats / BK, BK, CH_UB * TILE_M)) return cudaErrorInvalidValue;
  for (int i = 0; i < 3; ++i) {
    if (!a.act_hi[i]) continue;
    if (!make_map(&maps[1 + 2 * i], a.act_hi[i], (uint64_t)a.m, (uint64_t)a.act_k[i], CH_BN) ||
        !make_map(&maps[2 + 2 * i], a.act_lo[i], (uint64_t)a.m, (uint64_t)a.act_k[i], CH_BN))
      return cudaErrorInvalidValue;
  }
  ChainArgs args = a;
  if (!args.phases_dev) chain_prepare_phases(args.ph, args.n_phases, grid);
  void* params[8] = {&maps[0], &maps[1], &maps[2], &maps[3], &maps[4], &maps[5], &maps[6], &args};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(CH_THREADS);
  cfg.dynamicSmemBytes = CH_SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // the runtime checks that the whole grid is co-resident
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(chain_kernel), params);
}

}  // namespace pg
