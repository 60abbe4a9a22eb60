// One decode step for at most 8 sequences as ONE persistent kernel whose weight stream never stops.
//
// At one sequence a GPT-2 small step is 62 dependent matrix-vector products of a few megabytes
// each (forward_one, src/models/gpt2/rust.rs:943-1006; block_forward_one_profiled, rust.rs:1136-1250).
// What bounds such a step is not bandwidth but the hand-over between dependent operations and the
// serial instruction count of each of them. Here:
//
//  * One CTA per SM stays resident for the whole step (cooperative launch: co-residency checked).
//    Every linear is cut into equal contiguous row ranges, one per CTA, so every SM streams the
//    same number of bytes of every matrix. The ranges depend only on the kind of linear, so they
//    are worked out once per launch and kept in shared memory.
//  * The step's whole list of weight ranges of this CTA is copied, 16 KB at a time, into a ring in
//    shared memory with cp.async.bulk (global -> shared, a full and an empty mbarrier per ring slot,
//    L2 evict-first) by warp 15, the producer. Weights do not depend on activations, so the copies
//    run ahead of the arithmetic by as much as the ring holds (about one layer of GPT-2 small):
//    every slot is refilled the moment the rows in it have been used, whatever phase the refill
//    belongs to, and HBM keeps streaming while the dependent chain of the step resolves. The
//    producer joins none of the other warps' barriers, so its bookkeeping delays nobody.
//  * Warps 0..14 compute: four weight rows x 128 columns per warp step from shared memory, FP32 FMA,
//    k split over warps, partial sums added in a fixed order (deterministic).
//  * There is no grid barrier. Activations travel between CTAs as 8-byte words {value, tag} written
//    with one relaxed 64-bit store and polled with relaxed 64-bit loads (single-copy atomic, so the
//    tag vouches for the value next to it; no fence, no flag round trip). The tag is a counter that
//    is unique per phase and step, kept in device memory across launches. A consumer needs the
//    complete input vector of its phase, which every CTA contributes to, so every phase is also a
//    barrier in effect, which is what makes the re-use of the exchange buffers safe.
//  * Every wait (mbarrier, tag poll) is bounded; on expiry the CTA records an error code, skips the
//    rest of the step, waits (bounded) for its copies in flight, and the host returns PG_TIMEOUT.
//
// Weights may be FP32, BF16 (2 bytes) or row-quantised int8 (1 byte + one FP32 scale per row:
// QuantizedRows, src/models/cpu.rs:26-56); activations and sums are FP32 in all three.
#include <algorithm>
#include <climits>

#include "kernels.cuh"

namespace pg {
namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr int ST_THREADS = 512;            // launched: 15 computing warps and the producer warp
constexpr int ST_WARPS = 15;               // computing warps
constexpr int ST_CT = ST_WARPS * 32;       // computing threads
constexpr int ST_LN_THREADS = 256;         // threads that stage a LayerNorm input (warps 0..7)
constexpr int ST_RELEASER = ST_CT - 1;     // the computing thread that hands ring slots back (it has no epilogue rows)
constexpr int ST_STAGE = 16384;            // bytes of one ring slot
constexpr int ST_STAGE_SHIFT = 14;
constexpr int ST_MAX_STAGES = 13;
constexpr int ST_BLOCK_ROWS = 32;          // most weight rows handed over at once (16 unless a block may span five or six ring slots)
constexpr int ST_MAX_SPLITS = 8;
constexpr int ST_PART_WORDS = 66;          // attention partial: max, sum, 64 values
constexpr int ST_KEEP = 16;                // residual values a CTA keeps per sequence: its rows of the next residual phase
constexpr int ST_MAX_PAGES = 64;           // page-table entries per sequence (1024 positions / 16)

typedef unsigned long long u64;

// Developer aid, compiled in only with -DPG_DEV_TRACE: CTAs 0 and 100 stamp clock64() at the phase
// boundaries of every layer into StreamArgs::trace ([2][n_layer + 1][16] words).
#ifdef PG_DEV_TRACE
#define ST_TRACE(layer, point)                                                                              \
  do {                                                                                                      \
    if (sh.args.trace && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == 100))                        \
      sh.args.trace[((blockIdx.x ? 1 : 0) * (sh.args.n_layer + 1) + (layer)) * 16 + (point)] = (u64)clock64(); \
  } while (0)
#else
#define ST_TRACE(layer, point) \
  do {                         \
  } while (0)
#endif

// ------------------------------------------------------------------ shared state of one CTA
enum { LIN_QKV = 0, LIN_PROJ = 1, LIN_FC = 2, LIN_PROJ2 = 3, LIN_HEAD = 4 };

struct LinInfo {   // this CTA's share of one kind of linear; the same in every layer
  int r0, nrows;   // first row and number of rows
  int n;           // rows of the whole matrix
  int k4;          // row length / 4
  int row_bytes;   // row length in bytes of the weight type
  int rb;          // rows per block (what is handed from the copies to the arithmetic at once)
  int ls;          // floor(log2(128-column slices per row))
};

struct Shared {
  StreamArgs args;           // the kernel's arguments, where every function reads them at shared-memory speed
  u64 full[ST_MAX_STAGES];   // ring slot filled (the producer arms it with the byte count, the copy completes it)
  u64 empty[ST_MAX_STAGES];  // ring slot free again (one computing thread arrives per hand-over)
  LinInfo lin[5];
  int failed;                // a bounded wait of this CTA expired, or another CTA reported one
  unsigned limit;            // polls before a wait gives up
  int splits;                // attention: CTAs per (sequence, head)
  float inv_c;               // 1 / n_embd
  int pos[8];
  int ids[8];
  int table[8][ST_MAX_PAGES];  // this step's page-table rows
  float red[2][ST_LN_THREADS / 32];
  float best_v[ST_BLOCK_ROWS * 8];
  int best_i[ST_BLOCK_ROWS * 8];
  alignas(16) float qs[64];  // q, and the new token's k and v, of the attention item in progress (read as float4)
  alignas(16) float kn[64];
  alignas(16) float vn[64];
  alignas(16) float att[ST_WARPS][68];  // per warp: max, sum, (pad), 64 weighted values
};

__shared__ Shared sh;
extern __shared__ __align__(128) unsigned char st_smem[];

// ------------------------------------------------------------------ small device helpers
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// barriers of the computing warps (the producer warp never joins them)
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, 480;" ::: "memory"); }
__device__ __forceinline__ void ln_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
static_assert(ST_CT == 480 && ST_LN_THREADS == 256, "thread counts of the named barriers");

__device__ __forceinline__ u64 ll_ld(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ll_st(u64* p, float val, unsigned tag) {
  const u64 v = ((u64)tag << 32) | (u64)__float_as_uint(val);
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int ld_flag(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ldg_nc4(const float4* p) {
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
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}

// N per-lane values -> totals over the warp; lane l ends with the total of value index l >> (5 - log2 N).
template <int N, int OFF>
struct LaneReduce {
  static __device__ __forceinline__ void run(float* v, int lane) {
    const bool up = (lane & OFF) != 0;
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
      const float send = up ? v[j] : v[j + N / 2];
      const float keep = up ? v[j + N / 2] : v[j];
      v[j] = keep + __shfl_xor_sync(FULL, send, OFF);
    }
    LaneReduce<N / 2, OFF / 2>::run(v, lane);
  }
};
template <int OFF>
struct LaneReduce<1, OFF> {
  static __device__ __forceinline__ void run(float* v, int lane) {
    v[0] += __shfl_xor_sync(FULL, v[0], OFF);
    LaneReduce<1, OFF / 2>::run(v, lane);
  }
};
template <>
struct LaneReduce<1, 0> {
  static __device__ __forceinline__ void run(float*, int) {}
};

// ------------------------------------------------------------------ bounded waits
__device__ __noinline__ void fail_with(int code) {
  sh.failed = 1;
  atomicCAS(sh.args.error_flag, 0, code);
}
// true when this CTA must stop: its own flag, or (looked at now and then) the launch-wide error word
__device__ __forceinline__ bool should_stop(unsigned spins) {
  if (*(volatile int*)&sh.failed) return true;
  if ((spins & 255u) == 255u && ld_flag(sh.args.error_flag) != 0) {
    sh.failed = 1;
    return true;
  }
  return false;
}

__device__ __forceinline__ bool mbar_try(u64* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// non-blocking look at a barrier's phase (try_wait may suspend the thread for a while even when the
// phase it asks about is long complete)
__device__ __forceinline__ bool mbar_test(u64* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __noinline__ bool mbar_wait_slow(u64* bar, uint32_t parity, int code) {
  const unsigned limit = sh.limit;
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try(bar, parity)) return true;
    if (should_stop(i)) return false;
  }
  fail_with(code);
  return false;
}
// One lane per warp watches the slot's barrier (thirty-two lanes polling one mbarrier serialise); the
// warp-wide exchange of the verdict orders the other lanes after the observation.
__device__ __forceinline__ bool wait_full(int slot, uint32_t parity) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_test(&sh.full[slot], parity) || mbar_wait_slow(&sh.full[slot], parity, 42);
  return __shfl_sync(FULL, ok, 0) != 0;
}

// Polls up to four tagged words base[j * stride], j < n, until each carries `tag`; words not asked for
// (and, after a failure, words that never came) read as zero. One copy of this code serves every phase.
__device__ __noinline__ float4 ll_poll4(const u64* base, int stride, int n, unsigned tag, int code) {
  float r[4] = {0.f, 0.f, 0.f, 0.f};
  unsigned pending = (1u << n) - 1u;
  unsigned spins = 0;
  while (pending) {
    u64 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if ((pending >> j) & 1u) v[j] = ll_ld(base + j * stride);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (((pending >> j) & 1u) && (unsigned)(v[j] >> 32) == tag) {
        r[j] = __uint_as_float((unsigned)v[j]);
        pending &= ~(1u << j);
      }
    if (pending) {
      if (++spins > sh.limit) {
        fail_with(code);
        break;
      }
      if (should_stop(spins)) break;
    }
  }
  return make_float4(r[0], r[1], r[2], r[3]);
}

// ------------------------------------------------------------------ the weight stream
__device__ __host__ inline int rows_per_block(int k, int elem_bytes, int block_stages) {
  int rb = (block_stages * ST_STAGE) / (k * elem_bytes);
  const int cap = block_stages >= 5 ? ST_BLOCK_ROWS : ST_BLOCK_ROWS / 2;
  if (rb > cap) rb = cap;
  if (rb >= 4) rb &= ~3;
  return rb;
}

struct RingPos {
  int slot;        // next ring slot
  uint32_t phase;  // parity of the round that slot is in
  __device__ __forceinline__ void advance(int ns) {
    if (++slot == ns) {
      slot = 0;
      phase ^= 1u;
    }
  }
};

// The producer (lane 0 of warp 15): walks this CTA's list of weight copies (every linear of the step in
// order, this CTA's rows of it block by block, 16 KB per copy), waiting only for ring slots to come
// back, then waits (bounded) until its last copies have landed.
__device__ __noinline__ void producer_run(unsigned char* ring, int ns) {
  u64 policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  RingPos rp{0, 0};
  int issued = 0;
  bool ok = true;
  const int L = sh.args.n_layer;
  for (int lin = 0; lin <= 4 * L && ok; ++lin) {
    const int kind = lin == 4 * L ? LIN_HEAD : (lin & 3), l = lin >> 2;
    const LinInfo li = sh.lin[kind];
    const unsigned char* w = kind == LIN_HEAD ? sh.args.w_head : sh.args.w[kind] + (long long)l * sh.args.w_stride;
    w += (long long)li.r0 * li.row_bytes;
    for (int rbase = 0; rbase < li.nrows && ok; rbase += li.rb) {
      const int bytes = min(li.rb, li.nrows - rbase) * li.row_bytes;
      const unsigned char* src = w + (long long)rbase * li.row_bytes;
      for (int off = 0; off < bytes; off += ST_STAGE) {
        if (issued >= ns && !mbar_try(&sh.empty[rp.slot], rp.phase ^ 1u)) {  // the slot's last readers are not done yet
          if (!mbar_wait_slow(&sh.empty[rp.slot], rp.phase ^ 1u, 41)) {
            ok = false;
            break;
          }
        }
        const int chunk = min(ST_STAGE, bytes - off);
        u64* bar = &sh.full[rp.slot];
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(chunk) : "memory");
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                smem_addr(ring + ((size_t)rp.slot << ST_STAGE_SHIFT))),
            "l"(src + off), "r"(chunk), "r"(smem_addr(bar)), "l"(policy)
            : "memory");
        ++issued;
        rp.advance(ns);
      }
    }
  }
  // before the CTA ends every copy still in flight must have landed: walk back over the slots armed last
  const int back = min(issued, ns);
  for (int i = 0; i < back; ++i) {
    if (rp.slot == 0) {
      rp.slot = ns - 1;
      rp.phase ^= 1u;
    } else {
      --rp.slot;
    }
    for (unsigned s = 0; s < (1u << 22); ++s)
      if (mbar_try(&sh.full[rp.slot], rp.phase)) break;
  }
}

// ------------------------------------------------------------------ arithmetic on a block of rows in the ring
enum { WT_F32 = 0, WT_BF16 = 1, WT_I8 = 2 };
template <int WT>
struct Elem {};
template <>
struct Elem<WT_F32> {
  static constexpr int BYTES = 4;
  static __device__ __forceinline__ float4 load4(const unsigned char* p) { return *reinterpret_cast<const float4*>(p); }
};
template <>
struct Elem<WT_BF16> {
  static constexpr int BYTES = 2;
  static __device__ __forceinline__ float4 load4(const unsigned char* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
  }
};
template <>
struct Elem<WT_I8> {
  static constexpr int BYTES = 1;
  // int8 -> float without the conversion unit: the byte, biased to unsigned, becomes the low mantissa
  // bits of 2^23; subtracting 2^23 + 128 leaves the signed value
  static __device__ __forceinline__ float4 load4(const unsigned char* p) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(p) ^ 0x80808080u;
    const float off = 8388736.0f;  // 2^23 + 128
    return make_float4(__uint_as_float(__byte_perm(u, 0x4b000000u, 0x7650)) - off,
                       __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7651)) - off,
                       __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7652)) - off,
                       __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7653)) - off);
  }
};

// log2 of the k parts a block of `rows` rows is cut into: (row groups of four) x parts <= 15 warps.
__device__ __forceinline__ int block_lkp(int rows, int ls) {
  // row groups of four x parts of k = items, one per warp, at most 15: 1 group -> 8 parts, 2 or 3 -> 4,
  // 4..7 -> 2, 8 -> 1
  const int rg_n = (rows + 3) >> 2;
  const int l = rg_n == 1 ? 3 : rg_n <= 3 ? 2 : rg_n <= 7 ? 1 : 0;
  return min(l, ls);
}

// Partial dot products of `rows` weight rows (in the ring from slot s0 on, row-major) with the MT
// input rows in xs: one warp per (group of four rows, part of k); part[item][r * MT + b].
template <int MT, int WT>
__device__ __forceinline__ void block_dots(const unsigned char* ring, int ns, int s0, int rows, const LinInfo& li,
                                           const float4* xs4, float* part, int warp, int lane) {
  constexpr int NV = 4 * MT;
  constexpr int SH = (NV == 32) ? 0 : (NV == 16) ? 1 : (NV == 8) ? 2 : 3;  // 5 - log2(NV)
  constexpr int GB = 4 * Elem<WT>::BYTES;                                  // bytes of four weights
  const int lkp = block_lkp(rows, li.ls);
  const int item = warp;
  if (item >= (((rows + 3) >> 2) << lkp)) return;
  const int k4 = li.k4;
  const int S = (k4 + 31) >> 5;
  const int rg = item >> lkp, kp = item & ((1 << lkp) - 1);
  const int s_beg = (kp * S) >> lkp, s_end = ((kp + 1) * S) >> lkp;
  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
  const int ring_bytes = ns << ST_STAGE_SHIFT;
  // byte offset of this lane's first column in each of the four rows (rows past the block's end repeat
  // its last row: their sums are never read); the block is contiguous in the ring, modulo its size
  int roff[4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
    roff[r] = (s0 << ST_STAGE_SHIFT) + (min(rg * 4 + r, rows - 1) * k4 + (s_beg << 5) + lane) * GB;
  const float4* xp = xs4 + (s_beg << 5) + lane;
  int c4 = (s_beg << 5) + lane;
#pragma unroll 2
  for (int s = s_beg; s < s_end; ++s, c4 += 32, xp += 32) {
    if (c4 < k4) {
      float4 xv[MT];
#pragma unroll
      for (int b = 0; b < MT; ++b) xv[b] = xp[b * k4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        int off = roff[r];
        if (off >= ring_bytes) off -= ring_bytes;
        const float4 w = Elem<WT>::load4(ring + off);
#pragma unroll
        for (int b = 0; b < MT; ++b) acc[r * MT + b] = dot4(w, xv[b], acc[r * MT + b]);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) roff[r] += 32 * GB;
  }
  LaneReduce<NV, 16>::run(acc, lane);
  if ((lane & ((1 << SH) - 1)) == 0) part[item * NV + (lane >> SH)] = acc[0];
}

// tanh-GELU (gelu_in_place, cpu.rs:145-150) with tanh(u) = 1 - 2 / (1 + e^(2u)); hardware exponential
// (2 ulp) and a Newton-refined reciprocal: well inside the FP32 tolerance of the logits, and a tenth
// of the instructions of the library tanhf, which matters in code that runs once per hand-over.
__device__ __forceinline__ float gelu_fast(float x) {
  const float u = 0.7978846f * (x + 0.044715f * x * x * x);
  const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
  return 0.5f * x * (1.0f + t);
}

// What the threads that finish rows need from global memory, requested before the phase's input is
// waited for: bias and (int8) row scale of their row in the first two blocks.
struct EpiPre {
  float bias0, bias1, scale0, scale1;
};
template <int MT, int WT>
__device__ __forceinline__ EpiPre epilogue_prefetch(int kind, int l) {
  EpiPre p;
  p.bias0 = p.bias1 = 0.f;
  p.scale0 = p.scale1 = 1.f;
  const int tid = threadIdx.x;
  if (tid < ST_BLOCK_ROWS * MT) {
    const LinInfo& li = sh.lin[kind];
    const int rr = tid / MT;
    const float* bias = kind == LIN_HEAD ? nullptr : sh.args.bias[kind] + (long long)l * sh.args.p_stride;
    const float* scale = nullptr;
    if (WT == WT_I8) scale = kind == LIN_HEAD ? sh.args.s_head : sh.args.scale[kind] + (long long)l * sh.args.s_stride;
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int r = blk * li.rb + rr;
      if (rr < li.rb && r < li.nrows) {
        if (bias) (blk ? p.bias1 : p.bias0) = bias[li.r0 + r];
        if (WT == WT_I8) (blk ? p.scale1 : p.scale0) = scale[li.r0 + r];
      }
    }
  }
  return p;
}

// One linear phase of this CTA: waits for each block of its weight rows, multiplies, finishes the sums
// in a fixed order and hands the results on (linear_block_into, rust.rs:1481-1532; with
// quantised weights quantized_linear_into, rust.rs:1535-1578).
template <int MT, int WT>
__device__ __forceinline__ bool linear_phase(unsigned char* ring, int ns, RingPos& rp, int kind, int l,
                                             const EpiPre& pre, const float4* xs4, const float* xkeep, float* part,
                                             u64* out_ll, unsigned out_tag, float& best_v, int& best_i) {
  constexpr int NV = 4 * MT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const LinInfo li = sh.lin[kind];
  int buf = 0, blk = 0;
#pragma unroll 1
  for (int rbase = 0; rbase < li.nrows; rbase += li.rb, ++blk) {
    const int rows = min(li.rb, li.nrows - rbase);
    const int nst = (rows * li.row_bytes + ST_STAGE - 1) >> ST_STAGE_SHIFT;
    const int s0 = rp.slot;
    bool got = true;
#pragma unroll 1
    for (int s = 0; s < nst; ++s) {
      if (got) got = wait_full(rp.slot, rp.phase);
      rp.advance(ns);
    }
    float* pb = part + buf * (ST_WARPS * NV);
    if (got) block_dots<MT, WT>(ring, ns, s0, rows, li, xs4, pb, warp, lane);
    compute_sync();
    if (sh.failed) return false;
    if (tid == ST_RELEASER) {  // every warp is done with these slots: the producer may refill them
      int slot = s0;
      for (int s = 0; s < nst; ++s) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&sh.empty[slot])) : "memory");
        if (++slot == ns) slot = 0;
      }
    }
    if (tid < rows * MT) {
      const int rr = tid / MT, b = tid - rr * MT;
      if (b < sh.args.m) {
        const int lkp = block_lkp(rows, li.ls);
        const int rg = rr >> 2, j = (rr & 3) * MT + b, row = li.r0 + rbase + rr;
        float sum = 0.f;
        const float* pp = pb + (rg << lkp) * NV + j;
#pragma unroll
        for (int kp = 0; kp < 8; ++kp)  // at most eight parts (block_lkp), added in order
          if (kp < (1 << lkp)) sum += pp[kp * NV];
        float bias = 0.f;
        if (blk < 2) {
          bias = blk ? pre.bias1 : pre.bias0;
          if (WT == WT_I8) sum *= blk ? pre.scale1 : pre.scale0;
        } else {
          if (kind != LIN_HEAD) bias = (sh.args.bias[kind] + (long long)l * sh.args.p_stride)[row];
          if (WT == WT_I8)
            sum *= (kind == LIN_HEAD ? sh.args.s_head : sh.args.scale[kind] + (long long)l * sh.args.s_stride)[row];
        }
        float v = bias + sum;
        if (kind == LIN_FC) v = gelu_fast(v);
        if (kind == LIN_PROJ || kind == LIN_PROJ2) v = xkeep[b * ST_KEEP + rbase + rr] + v;
        if (kind == LIN_HEAD) {
          if (sh.args.logits) sh.args.logits[(size_t)b * li.n + row] = v;
          if (v > best_v) {  // first strict maximum: rows ascend within a thread (generation.rs:269-279)
            best_v = v;
            best_i = row;
          }
        } else {
          ll_st(out_ll + (size_t)b * li.n + row, v, out_tag);
        }
      }
    }
    buf ^= 1;
  }
  return true;
}

// ------------------------------------------------------------------ inputs of a phase
// The complete rows [m][k] of an exchange buffer (or, first layer, of the embedding tables:
// wte[id] + wpe[pos], rust.rs:970-974) into xs, as they are; unused rows of the tile read as zero.
template <int MT>
__device__ __forceinline__ void stage_input(const u64* ll, unsigned tag, int k, bool from_embedding, float* xs) {
  const int tid = threadIdx.x;
  const int total = sh.args.m * k;
  if (from_embedding) {
    for (int b = 0; b < sh.args.m; ++b) {
      const float* te = sh.args.wte + (size_t)sh.ids[b] * k;
      const float* pe = sh.args.wpe + (size_t)sh.pos[b] * k;
      for (int col = tid; col < k; col += ST_CT) xs[b * k + col] = te[col] + pe[col];
    }
  } else {
    // sixteen words per thread in flight while there are that many (eight sequences of 4096 values are 68
    // words per thread: four words at a time would be seventeen dependent round trips to L2)
#pragma unroll 1
    for (int base = tid; base < total; base += ST_CT * 16) {
      const int n = min(16, (total - base + ST_CT - 1) / ST_CT);
      if (n == 16) {
        u64 v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = ll_ld(ll + base + j * ST_CT);
        bool all = true;
#pragma unroll
        for (int j = 0; j < 16; ++j) all = all && (unsigned)(v[j] >> 32) == tag;
        if (all) {
#pragma unroll
          for (int j = 0; j < 16; ++j) xs[base + j * ST_CT] = __uint_as_float((unsigned)v[j]);
          continue;
        }
      }
#pragma unroll 1
      for (int j0 = 0; j0 < n; j0 += 4) {  // not all there yet (or a short tail): four at a time, waiting
        const int m4 = min(4, n - j0);
        const float4 r = ll_poll4(ll + base + j0 * ST_CT, ST_CT, m4, tag, 44);
        float* dst = xs + base + j0 * ST_CT;
        dst[0] = r.x;
        if (m4 > 1) dst[ST_CT] = r.y;
        if (m4 > 2) dst[2 * ST_CT] = r.z;
        if (m4 > 3) dst[3 * ST_CT] = r.w;
      }
    }
  }
  for (int i = total + tid; i < MT * k; i += ST_CT) xs[i] = 0.f;
  compute_sync();
}

// LayerNorm scale and shift of the coming phase into shared memory (gb[0..c) = gamma, gb[c..2c) = beta),
// requested before the phase's input is waited for.
__device__ __forceinline__ void ln_params_prefetch(const float* g, const float* bt, float* gb) {
  const int c = sh.args.c;
  for (int col = threadIdx.x; col < c; col += ST_CT) {
    gb[col] = g[col];
    gb[c + col] = bt[col];
  }
}

// LayerNorm of the rows in xs, in place (layer_norm_in_place, cpu.rs:119-143: mean, then the biased
// variance of the centred values; sums as trees), by the first 256 threads. The residual values of
// columns [keep0, keep0 + keepn) (this CTA's rows of the next residual phase) are kept in xkeep.
template <int MT>
__device__ __forceinline__ void ln_in_place(const float* gb, int keep0, int keepn, float* xkeep, float* xs) {
  constexpr int TPR = ST_LN_THREADS / MT;         // threads per row
  constexpr int WPR = (ST_LN_THREADS / 32) / MT;  // warps per row
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < ST_LN_THREADS) {
    const int b = tid / TPR, i0 = tid - b * TPR, c = sh.args.c;
    float* row = xs + b * c;
    float s = 0.f;
#pragma unroll 1
    for (int col = i0; col < c; col += TPR) s += row[col];
    s = warp_sum(s);
    if (lane == 0) sh.red[0][warp] = s;
    ln_sync();
    float mean = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) mean += sh.red[0][b * WPR + w];
    mean *= sh.inv_c;
    float q = 0.f;
#pragma unroll 1
    for (int col = i0; col < c; col += TPR) {
      const float d = row[col] - mean;
      q = fmaf(d, d, q);
    }
    q = warp_sum(q);
    if (lane == 0) sh.red[1][warp] = q;
    ln_sync();
    float var = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) var += sh.red[1][b * WPR + w];
    const float inv_std = rsqrtf(var * sh.inv_c + sh.args.eps);
#pragma unroll 1
    for (int col = i0; col < c; col += TPR) {
      const float v = row[col];
      const unsigned kc = (unsigned)(col - keep0);
      if (kc < (unsigned)keepn) xkeep[b * ST_KEEP + kc] = v;
      row[col] = (v - mean) * inv_std * gb[col] + gb[c + col];
    }
  }
  compute_sync();
}

// ------------------------------------------------------------------ attention
// One (sequence, head, split) of cached_self_attention_into (rust.rs:1662-1741), head_dim 64, by the
// 15 computing warps. Four lanes share a key: lane part p holds floats [16 i + 4 p, 16 i + 4 p + 4), i < 4,
// of q, of the key and of the value row, so one sweep computes the score and adds the weighted value
// (running maximum per warp; the warps' partial results are merged through shared memory). Keys and
// values of the warp's first cached position are requested before q is waited for: they do not depend
// on this step. The new token's k and v come from the exchange buffer and are appended to the cache
// by the split that owns the position.
__device__ __noinline__ void attention_item(int l, int b, int h, int sp, unsigned tag_qkv, unsigned tag_part,
                                            unsigned tag_out) {
  constexpr int D = 64;
  const StreamArgs& a = sh.args;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = a.c, splits = sh.splits;
  const int pos = sh.pos[b], nkeys = pos + 1;
  int k0 = 0, k1 = nkeys;
  if (splits > 1) {
    const int per = (nkeys + splits - 1) / splits;
    k0 = min(sp * per, nkeys);
    k1 = min(k0 + per, nkeys);
  }
  const bool owns_new = k0 <= pos && pos < k1;
  const int* table = sh.table[b];
  float* pool = a.kv_pool + (long long)l * a.kv_stride;
  const int pt = a.kv.page_tokens, psh = 31 - __clz(pt);
  const int vofs4 = (a.kv.n_head * pt * D) >> 2;  // from a key row to the value row of the same position, in float4
  const int part = lane & 3, kslot = lane >> 2;
  auto row_of = [&](int key) {
    const int page = table[key >> psh], off = key & (pt - 1);
    return reinterpret_cast<float4*>(pool + (((size_t)page * 2 * a.kv.n_head + h) * pt + off) * D);
  };

  // ---- early requests: this lane's first cached key and value
  float4 kreg[4], vreg[4];
  int key = k0 + warp * 8 + kslot;
  if (key < k1 && key != pos) {
    const float4* kr = row_of(key);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      kreg[i] = ldg_nc4(kr + i * 4 + part);
      vreg[i] = ldg_nc4(kr + vofs4 + i * 4 + part);
    }
  }

  // ---- q, and the new token's k and v, from the QKV phase
  if (warp < 3 && (warp == 0 || owns_new)) {
    const float4 t = ll_poll4(a.ll_qkv + (size_t)b * 3 * c + warp * c + h * D + lane, 32, 2, tag_qkv, 45);
    float* dst = warp == 0 ? sh.qs : warp == 1 ? sh.kn : sh.vn;
    dst[lane] = t.x;
    dst[lane + 32] = t.y;
  }
  compute_sync();
  if (owns_new && tid < 32) {  // append K, V of the new position
    const int which = tid >> 4, j = tid & 15;
    row_of(pos)[which * vofs4 + j] = reinterpret_cast<const float4*>(which ? sh.vn : sh.kn)[j];
  }
  float4 q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = reinterpret_cast<const float4*>(sh.qs)[i * 4 + part];
  const float scale = 0.125f;  // 1 / sqrt(64)
  float m_run = -INFINITY, l_run = 0.f;
  float4 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  bool first = true;
#pragma unroll 1
  for (int kw = k0 + warp * 8; kw < k1; kw += 8 * ST_WARPS) {
    key = kw + kslot;
    const bool valid = key < k1;
    if (valid) {
      if (key == pos) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kreg[i] = reinterpret_cast<const float4*>(sh.kn)[i * 4 + part];
          vreg[i] = reinterpret_cast<const float4*>(sh.vn)[i * 4 + part];
        }
      } else if (!first) {
        const float4* kr = row_of(key);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kreg[i] = ldg_nc4(kr + i * 4 + part);
          vreg[i] = ldg_nc4(kr + vofs4 + i * 4 + part);
        }
      }
    }
    first = false;
    float s = 0.f;
    if (valid) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s = dot4(q[i], kreg[i], s);
    }
    s += __shfl_xor_sync(FULL, s, 1);
    s += __shfl_xor_sync(FULL, s, 2);
    s = valid ? s * scale : -INFINITY;
    float m_new = s;
    m_new = fmaxf(m_new, __shfl_xor_sync(FULL, m_new, 4));
    m_new = fmaxf(m_new, __shfl_xor_sync(FULL, m_new, 8));
    m_new = fmaxf(m_new, __shfl_xor_sync(FULL, m_new, 16));
    m_new = fmaxf(m_new, m_run);  // finite: the warp's first key of the round is valid
    const float corr = __expf(m_run - m_new);
    const float p = valid ? __expf(s - m_new) : 0.f;
    l_run = l_run * corr + p;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 vv = valid ? vreg[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      acc[i].x = fmaf(p, vv.x, acc[i].x * corr);
      acc[i].y = fmaf(p, vv.y, acc[i].y * corr);
      acc[i].z = fmaf(p, vv.z, acc[i].z * corr);
      acc[i].w = fmaf(p, vv.w, acc[i].w * corr);
    }
    m_run = m_new;
  }
  // ---- the warp's eight key slots into one: lanes 0..3 end with the totals of their parts
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l_run += __shfl_xor_sync(FULL, l_run, o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[i].x += __shfl_xor_sync(FULL, acc[i].x, o);
      acc[i].y += __shfl_xor_sync(FULL, acc[i].y, o);
      acc[i].z += __shfl_xor_sync(FULL, acc[i].z, o);
      acc[i].w += __shfl_xor_sync(FULL, acc[i].w, o);
    }
  }
  if (lane < 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(&sh.att[warp][4])[i * 4 + part] = acc[i];
    if (lane == 0) {
      sh.att[warp][0] = m_run;
      sh.att[warp][1] = l_run;
    }
  }
  compute_sync();
  // ---- merge the warps (in warp order), then the splits (in split order)
  if (tid < D) {
    const int nw = min(ST_WARPS, (k1 - k0 + 7) >> 3);  // warps that had keys
    float mx = -INFINITY;
#pragma unroll 1
    for (int w = 0; w < nw; ++w) mx = fmaxf(mx, sh.att[w][0]);
    float lt = 0.f, o = 0.f;
    if (mx > -INFINITY) {
#pragma unroll 1
      for (int w = 0; w < nw; ++w) {
        const float sc = __expf(sh.att[w][0] - mx);  // exp(-inf) = 0 for a warp without keys
        lt = fmaf(sh.att[w][1], sc, lt);
        o = fmaf(sh.att[w][4 + tid], sc, o);
      }
    }
    u64* out = a.ll_attn + (size_t)b * c + h * D;
    if (splits == 1) {
      ll_st(out + tid, __fdividef(o, lt), tag_out);
    } else {
      const int pair = b * a.kv.n_head + h;
      u64* base = a.ll_part + (size_t)pair * ST_MAX_SPLITS * ST_PART_WORDS;
      u64* mine = base + sp * ST_PART_WORDS;
      ll_st(mine + 2 + tid, o, tag_part);
      if (tid == 0) {
        ll_st(mine, mx, tag_part);
        ll_st(mine + 1, lt, tag_part);
      }
      if (sp == 0) {  // the first split's CTA adds the partials in split order
        float m2 = -INFINITY;
#pragma unroll 1
        for (int s = 0; s < splits; s += 4)
          m2 = fmaxf(m2, [&] {
            const float4 t = ll_poll4(base + s * ST_PART_WORDS, ST_PART_WORDS, min(4, splits - s), tag_part, 46);
            // splits not asked for read as 0, which must not win the maximum
            return fmaxf(fmaxf(t.x, s + 1 < splits ? t.y : -INFINITY),
                         fmaxf(s + 2 < splits ? t.z : -INFINITY, s + 3 < splits ? t.w : -INFINITY));
          }());
        float l2 = 0.f, acc2 = 0.f;
#pragma unroll 1
        for (int s = 0; s < splits; ++s) {
          const float pm = ll_poll4(base + s * ST_PART_WORDS, 1, 1, tag_part, 46).x;
          const float pl = ll_poll4(base + s * ST_PART_WORDS + 1, 1, 1, tag_part, 46).x;
          const float pa = ll_poll4(base + s * ST_PART_WORDS + 2 + tid, 1, 1, tag_part, 46).x;
          const float sc = (pm == -INFINITY) ? 0.f : __expf(pm - m2);
          l2 = fmaf(pl, sc, l2);
          acc2 = fmaf(pa, sc, acc2);
        }
        ll_st(out + tid, __fdividef(acc2, l2), tag_out);
      }
    }
  }
  compute_sync();  // sh.att, sh.qs are reused by the next item
}

// ------------------------------------------------------------------ the kernel
template <int MT, int WT>
__global__ void __launch_bounds__(ST_THREADS, 1) decode_stream_kernel(const __grid_constant__ StreamArgs a, int ns,
                                                                      int block_stages) {
  constexpr int EB = Elem<WT>::BYTES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  if (tid < (int)(sizeof(StreamArgs) / sizeof(int)))
    reinterpret_cast<int*>(&sh.args)[tid] = reinterpret_cast<const int*>(&a)[tid];
  const int c = a.c, f = a.f, kx = max(c, f), L = a.n_layer;
  unsigned char* ring = st_smem;
  float* xs = reinterpret_cast<float*>(st_smem + ((size_t)ns << ST_STAGE_SHIFT));
  float* part = xs + (size_t)MT * kx;
  float* xkeep = part + 2 * ST_WARPS * 4 * MT;
  float* gb = xkeep + MT * ST_KEEP;  // LayerNorm scale and shift of the coming phase

  if (tid == 0) {
    for (int i = 0; i < ns; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&sh.full[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&sh.empty[i])) : "memory");
    }
    sh.failed = 0;
    sh.limit = a.spin_limit ? a.spin_limit : (1u << 22);
    sh.inv_c = 1.0f / (float)c;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid >= 32 && tid < 37) {  // this CTA's share of each kind of linear
    const int kind = tid - 32;
    const int n = kind == LIN_QKV ? 3 * c : kind == LIN_FC ? f : kind == LIN_HEAD ? a.v : c;
    const int k = kind == LIN_PROJ2 ? f : c;
    // which CTAs get the one extra row differs from kind to kind, so that the byte totals even out
    const int ci = (cta + kind * 31) % G;
    LinInfo li;
    li.r0 = (int)(((long long)ci * n) / G);
    li.nrows = (int)(((long long)(ci + 1) * n) / G) - li.r0;
    li.n = n;
    li.k4 = k >> 2;
    li.row_bytes = k * EB;
    li.rb = rows_per_block(k, EB, block_stages);
    li.ls = 31 - __clz(((k >> 2) + 31) >> 5);
    sh.lin[kind] = li;
  }
  if (tid >= 64 && tid < 72) {
    const int b = tid - 64;
    sh.pos[b] = b < a.m ? a.pos[b] : 0;
    sh.ids[b] = b < a.m ? a.ids[b] : 0;
  }
  if (tid == 96) {
    int nk_max = 1;
    for (int b = 0; b < a.m; ++b) nk_max = max(nk_max, a.pos[b] + 1);
    const int items0 = a.m * a.kv.n_head;
    int splits = a.attn_splits > 0 ? a.attn_splits : min(max(1, G / items0), (nk_max + 119) / 120);
    sh.splits = max(1, min(splits, ST_MAX_SPLITS));
  }
  for (int i = tid; i < a.m * ST_MAX_PAGES; i += ST_THREADS) {
    const int b = i / ST_MAX_PAGES, p = i - b * ST_MAX_PAGES;
    sh.table[b][p] = p < a.kv.pages_per_seq ? a.page_table[(size_t)b * a.kv.pages_per_seq + p] : 0;
  }
  const unsigned base = *a.epoch;  // tags of this launch start after the last launch's
  __syncthreads();
  if (warp == ST_WARPS) {  // the producer warp: one lane streams this CTA's weights, start to end of the step
    if (lane == 0) producer_run(ring, ns);
    return;
  }

  // tag of what (layer, kind of linear) hands on; the attention partials and outputs have their own
  enum { T_PART = 5, T_ATTN = 6 };
  auto tag_of = [&](int layer, int what) { return base + 1u + (unsigned)(layer * 8 + what); };
  RingPos rp{0, 0};
  float best_v = -INFINITY;
  int best_i = INT_MAX;
  const float4* xs4 = reinterpret_cast<const float4*>(xs);
#pragma unroll 1
  for (int lin = 0; lin <= 4 * L; ++lin) {
    const int kind = lin == 4 * L ? LIN_HEAD : (lin & 3), l = lin >> 2;
    const long long po = (long long)l * a.p_stride;
    ST_TRACE(l, 2 * kind);
    const EpiPre pre = epilogue_prefetch<MT, WT>(kind, l);
    if (kind == LIN_PROJ || kind == LIN_PROJ2) {
      if (kind == LIN_PROJ) {  // attention over the cache (+ append of the new K, V), then its output as input
        const int splits = sh.splits, items = a.m * a.kv.n_head * splits;
        int it = cta - (l * 13) % G;  // the CTAs that do attention differ from layer to layer
        if (it < 0) it += G;
#pragma unroll 1
        for (; it < items; it += G) {
          const int pair = it / splits, sp = it - pair * splits;
          const int b = pair / a.kv.n_head;
          attention_item(l, b, pair - b * a.kv.n_head, sp, tag_of(l, LIN_QKV), tag_of(l, T_PART), tag_of(l, T_ATTN));
        }
      }
      stage_input<MT>(kind == LIN_PROJ ? a.ll_attn : a.ll_h, kind == LIN_PROJ ? tag_of(l, T_ATTN) : tag_of(l, LIN_FC),
                      kind == LIN_PROJ ? c : f, false, xs);
    } else {  // LayerNorm of the residual stream: ln_1, ln_2 or ln_f
      const float* g = kind == LIN_HEAD ? a.lnf_g : a.ln_g[kind == LIN_FC] + po;
      const float* bt = kind == LIN_HEAD ? a.lnf_b : a.ln_b[kind == LIN_FC] + po;
      ln_params_prefetch(g, bt, gb);
      const unsigned tag = kind == LIN_FC ? (tag_of(l, LIN_PROJ) ^ a.poison) : tag_of(l - 1, LIN_PROJ2);
      stage_input<MT>(a.ll_x, tag, c, lin == 0, xs);
      const int next_resid = kind == LIN_QKV ? LIN_PROJ : LIN_PROJ2;
      ln_in_place<MT>(gb, sh.lin[next_resid].r0, kind == LIN_HEAD ? 0 : sh.lin[next_resid].nrows, xkeep, xs);
    }
    ST_TRACE(l, 2 * kind + 1);
    if (sh.failed) break;
    u64* out = kind == LIN_QKV ? a.ll_qkv : kind == LIN_FC ? a.ll_h : a.ll_x;
    if (!linear_phase<MT, WT>(ring, ns, rp, kind, l, pre, xs4, xkeep, part, out, tag_of(l, kind), best_v, best_i)) break;
  }
  ST_TRACE(L, 15);
  // ---- arg-max of the logits (generation.rs:269-279): per CTA, then CTA 0 over all CTAs
  if (!sh.failed) {
    const unsigned tag_best = tag_of(L, 7);
    if (tid < ST_BLOCK_ROWS * MT) {
      sh.best_v[tid] = best_v;
      sh.best_i[tid] = best_i;
    }
    compute_sync();
    if (tid < MT && tid < a.m) {
      float bv = -INFINITY;
      int bi = INT_MAX;
      for (int r = 0; r < ST_BLOCK_ROWS; ++r) {
        const float v = sh.best_v[r * MT + tid];
        const int i = sh.best_i[r * MT + tid];
        if (v > bv || (v == bv && i < bi)) {
          bv = v;
          bi = i;
        }
      }
      u64* dst = a.ll_best + ((size_t)tid * G + cta) * 2;
      ll_st(dst, bv, tag_best);
      ll_st(dst + 1, __int_as_float(bi), tag_best);
    }
    // ---- end of step: CTA 0, warp b finishes sequence b
    if (cta == 0 && warp < a.m) {
      float bv = -INFINITY;
      int bi = INT_MAX;
      for (int p = lane; p < G; p += 32) {
        const float4 t = ll_poll4(a.ll_best + ((size_t)warp * G + p) * 2, 1, 2, tag_best, 47);
        const int i = __float_as_int(t.y);
        if (t.x > bv || (t.x == bv && i < bi)) {
          bv = t.x;
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
      if (lane == 0 && !*(volatile int*)&sh.failed) {
        const int tok = (bi == INT_MAX) ? 0 : bi;
        a.argmax[warp] = tok;
        a.ids[warp] = tok;
        const int np = sh.pos[warp] + 1;
        a.pos[warp] = np;
        if (np < a.n_positions) a.token_log[(size_t)warp * a.n_positions + np] = tok;
      }
    }
  }
  // tags of the next launch start where these ended; written once every result of this launch is in
  // (CTA 0's last act is to read every CTA's last hand-over)
  compute_sync();
  if (cta == 0 && tid == 0 && !sh.failed) *a.epoch = base + 1u + (unsigned)((L + 1) * 8);
}

template <int MT, int WT>
cudaError_t launch_one(const StreamArgs& a, int grid, size_t smem, int ns, int block_stages, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(ST_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // the runtime checks that the whole grid is co-resident
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_stream_kernel<MT, WT>, a, ns, block_stages);
}

constexpr size_t ST_DYN_SMEM_MAX = 216 * 1024;  // leaves room for the static part (Shared)

inline int mt_of(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8; }
inline size_t fixed_smem(int mt, int c, int f) {  // xs, part, xkeep, gb
  return ((size_t)mt * std::max(c, f) + 2 * ST_WARPS * 4 * mt + (size_t)mt * ST_KEEP + 2 * (size_t)c) * sizeof(float);
}

template <int MT, int WT>
int max_grid(int num_sms) {
  int per_sm = 0;
  if (cudaFuncSetAttribute(decode_stream_kernel<MT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)ST_DYN_SMEM_MAX) != cudaSuccess)
    return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stream_kernel<MT, WT>, ST_THREADS, ST_DYN_SMEM_MAX) !=
      cudaSuccess)
    return 0;
  return per_sm >= 1 ? num_sms : 0;
}

template <int WT>
int max_grid_wt(int num_sms) {
  int g = max_grid<1, WT>(num_sms);
  g = std::min(g, max_grid<2, WT>(num_sms));
  g = std::min(g, max_grid<4, WT>(num_sms));
  g = std::min(g, max_grid<8, WT>(num_sms));
  return g;
}

}  // namespace

int decode_stream_elem_bytes(int weight_type) { return weight_type == WT_F32 ? 4 : weight_type == WT_BF16 ? 2 : 1; }

// Ring slots that fit beside the activations of `m` sequences, and the slots one block of rows may take.
static bool stream_geometry(int m, int c, int f, int weight_type, int* ns_out, int* block_stages_out) {
  const size_t fixed = fixed_smem(mt_of(m), c, f);
  if (fixed + 3 * (size_t)ST_STAGE > ST_DYN_SMEM_MAX) return false;
  int ns = (int)((ST_DYN_SMEM_MAX - fixed) / ST_STAGE);
  ns = std::min(ns, ST_MAX_STAGES);
  // Rows of a CTA's share are handed over in blocks of at most four ring slots and 16 rows; with narrow rows
  // (at most 3 KB: GPT-2 small in FP32, wider models with packed weights) and one or two sequences, blocks of up to
  // six slots (half the ring) and 32 rows, which take the CTA's rows of every layer linear of GPT-2 small in one round and halve the
  // rounds of the lm_head (one sequence: 283 against 293 us per token; GPT-2 medium and four sequences lose 1%)
  const bool wide_blocks = mt_of(m) <= 2 && (size_t)c * decode_stream_elem_bytes(weight_type) <= 3072 && ns >= 10;
  const int bs = std::max(1, std::min(wide_blocks ? 6 : 4, ns / 2));
  const int eb = decode_stream_elem_bytes(weight_type);
  if (rows_per_block(c, eb, bs) < 1 || rows_per_block(f, eb, bs) < 1) return false;
  *ns_out = ns;
  *block_stages_out = bs;
  return true;
}

bool decode_stream_supported(int m, int c, int f, int v, int head_dim, int n_positions, int page_tokens, int weight_type,
                             int grid) {
  int ns, bs;
  // every CTA must own at least one row of every linear
  return m >= 1 && m <= 8 && head_dim == 64 && c % 4 == 0 && f % 4 == 0 && c <= 2048 && grid > 0 && c >= grid && v >= grid &&
         n_positions <= ST_MAX_PAGES * page_tokens && stream_geometry(m, c, f, weight_type, &ns, &bs);
}

int decode_stream_grid(int num_sms) {
  int g = max_grid_wt<WT_F32>(num_sms);
  g = std::min(g, max_grid_wt<WT_BF16>(num_sms));
  g = std::min(g, max_grid_wt<WT_I8>(num_sms));
  return g;
}

cudaError_t launch_decode_stream(const StreamArgs& a, int weight_type, int grid, cudaStream_t s) {
  int ns = 0, bs = 0;
  if (!decode_stream_supported(a.m, a.c, a.f, a.v, a.kv.head_dim, a.n_positions, a.kv.page_tokens, weight_type, grid) ||
      !stream_geometry(a.m, a.c, a.f, weight_type, &ns, &bs))
    return cudaErrorInvalidValue;
  const size_t smem = ((size_t)ns << ST_STAGE_SHIFT) + fixed_smem(mt_of(a.m), a.c, a.f);
#define PG_ST_LAUNCH(MT)                                                        \
  (weight_type == WT_F32    ? launch_one<MT, WT_F32>(a, grid, smem, ns, bs, s)  \
   : weight_type == WT_BF16 ? launch_one<MT, WT_BF16>(a, grid, smem, ns, bs, s) \
                            : launch_one<MT, WT_I8>(a, grid, smem, ns, bs, s))
  switch (mt_of(a.m)) {
    case 1: return PG_ST_LAUNCH(1);
    case 2: return PG_ST_LAUNCH(2);
    case 4: return PG_ST_LAUNCH(4);
    default: return PG_ST_LAUNCH(8);
  }
#undef PG_ST_LAUNCH
}

}  // namespace pg
