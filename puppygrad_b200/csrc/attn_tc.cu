// Prefill attention on the tensor cores (sm_100a), TF32 inputs with FP32 accumulation: the variant
// of causal_self_attention (src/models/gpt2/rust.rs:1580-1659) used by the single-pass TF32
// prefill mode, whose stated bound already allows 10-bit mantissas. head_dim 64.
//
// CTA = 128 queries of one (sequence, head); keys / values in tiles of 128; two CTAs per SM, so
// that the softmax of one overlaps the MMAs of the other.
//   warp 0      TMA producer: Q once, then per tile K and V (rows of the [rows, 3c] QKV matrix),
//               each into its own buffer as soon as the previous tile has released it.
//   warp 1      MMA issuer: S = Q K^T with Q read from tensor memory (TS form) and K from shared
//               memory, then O += P V with P read from tensor memory and V^T from shared memory.
//               tcgen05 takes TF32 operands K-major only, so V cannot be used as it lies in
//               memory: the softmax warps write a transposed, swizzled copy.
//   warps 2-5   one thread per query row: at the start it moves its row of Q into tensor memory;
//               per tile it reads its 128 scores into registers in one go, takes the row maximum,
//               writes P = 2^x (cut to TF32) over S, keeps the running sum, rescales O only when
//               the maximum moved by more than 2^8, and transposes the V tile (one key each: its
//               64 values go to 64 rows of V^T, which consecutive lanes hit in consecutive words,
//               without bank conflicts).
// Every mbarrier wait is bounded; on expiry the error word is raised and all roles fall through.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace pg {
namespace {

constexpr int AT_Q = 128, AT_K = 128, AT_D = 64;
constexpr int AT_TILE_BYTES = AT_K * AT_D * 4;  // 32 KB: two boxes of [128 rows][32 floats]
// K tile, V tile (Q passes through it on its way to tensor memory), V^T, slack for the 1024-byte
// alignment. 97 KB: two CTAs per SM.
constexpr size_t AT_TC_SMEM = (size_t)AT_TILE_BYTES * 3 + 1024;
// P overwrites S in place (each thread rewrites its own row); O and Q follow: all 256 allocated columns.
constexpr uint32_t AT_S_COL = 0, AT_O_COL = 128, AT_Q_COL = 192, AT_TMEM_COLS = 256;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Every lane waits (bounded); the verdict is uniform over the warp.
__device__ __forceinline__ bool warp_wait_all(uint64_t* bar, uint32_t parity, volatile int* failed, int* err, int code) {
  const bool ok = mbar_wait(bar, parity, failed, err, code);
  return __all_sync(0xffffffffu, ok);
}

// 32 columns of this thread's row into r[OFF .. OFF + 31], without waiting for the data.
template <int OFF>
__device__ __forceinline__ void at_ld32(uint32_t taddr, uint32_t (&r)[128]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[OFF + 0]), "=r"(r[OFF + 1]), "=r"(r[OFF + 2]), "=r"(r[OFF + 3]), "=r"(r[OFF + 4]), "=r"(r[OFF + 5]),
        "=r"(r[OFF + 6]), "=r"(r[OFF + 7]), "=r"(r[OFF + 8]), "=r"(r[OFF + 9]), "=r"(r[OFF + 10]), "=r"(r[OFF + 11]),
        "=r"(r[OFF + 12]), "=r"(r[OFF + 13]), "=r"(r[OFF + 14]), "=r"(r[OFF + 15]), "=r"(r[OFF + 16]),
        "=r"(r[OFF + 17]), "=r"(r[OFF + 18]), "=r"(r[OFF + 19]), "=r"(r[OFF + 20]), "=r"(r[OFF + 21]),
        "=r"(r[OFF + 22]), "=r"(r[OFF + 23]), "=r"(r[OFF + 24]), "=r"(r[OFF + 25]), "=r"(r[OFF + 26]),
        "=r"(r[OFF + 27]), "=r"(r[OFF + 28]), "=r"(r[OFF + 29]), "=r"(r[OFF + 30]), "=r"(r[OFF + 31])
      : "r"(taddr + (uint32_t)OFF)
      : "memory");
}
template <int OFF>
__device__ __forceinline__ void at_st32(uint32_t taddr, const uint32_t (&r)[128]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr + (uint32_t)OFF),
      "r"(r[OFF + 0]), "r"(r[OFF + 1]), "r"(r[OFF + 2]), "r"(r[OFF + 3]), "r"(r[OFF + 4]), "r"(r[OFF + 5]),
      "r"(r[OFF + 6]), "r"(r[OFF + 7]), "r"(r[OFF + 8]), "r"(r[OFF + 9]), "r"(r[OFF + 10]), "r"(r[OFF + 11]),
      "r"(r[OFF + 12]), "r"(r[OFF + 13]), "r"(r[OFF + 14]), "r"(r[OFF + 15]), "r"(r[OFF + 16]), "r"(r[OFF + 17]),
      "r"(r[OFF + 18]), "r"(r[OFF + 19]), "r"(r[OFF + 20]), "r"(r[OFF + 21]), "r"(r[OFF + 22]), "r"(r[OFF + 23]),
      "r"(r[OFF + 24]), "r"(r[OFF + 25]), "r"(r[OFF + 26]), "r"(r[OFF + 27]), "r"(r[OFF + 28]), "r"(r[OFF + 29]),
      "r"(r[OFF + 30]), "r"(r[OFF + 31])
      : "memory");
}
__device__ __forceinline__ void at_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Row maximum of the 128 raw scores in s; MASK: keys after the query do not count.
template <bool MASK>
__device__ __forceinline__ float at_row_max(const uint32_t (&s)[128], int kt, int qpos) {
  float tmax = -INFINITY;
#pragma unroll
  for (int j = 0; j < AT_K; ++j)
    if (!MASK || kt + j <= qpos) tmax = fmaxf(tmax, __uint_as_float(s[j]));
  return tmax;
}

// s <- P = 2^(s * sl2 - mn), cut to TF32 (the bits the MMA reads) so that the returned sum is the
// sum the MMA sees.
template <bool MASK>
__device__ __forceinline__ float at_exp_rows(uint32_t (&s)[128], int kt, int qpos, float sl2, float mn) {
  float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
  for (int j = 0; j < AT_K; j += 2) {
    uint32_t b0 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(s[j]), sl2, -mn))) & 0xFFFFE000u;
    uint32_t b1 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(s[j + 1]), sl2, -mn))) & 0xFFFFE000u;
    if (MASK && kt + j > qpos) b0 = 0u;
    if (MASK && kt + j + 1 > qpos) b1 = 0u;
    ps0 += __uint_as_float(b0);
    ps1 += __uint_as_float(b1);
    s[j] = b0;
    s[j + 1] = b1;
  }
  return ps0 + ps1;
}

__global__ void __launch_bounds__(192, 2)
    prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_qkv, PrefillAttnArgs a, int* error_flag) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // query tiles with the most keys are scheduled first (z is the slowest grid dimension)
  const int h = blockIdx.x, b = blockIdx.y, qb = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int c = a.n_head * AT_D;
  const int r0 = a.seq_start[b], len = a.seq_start[b + 1] - r0;
  const int q0 = qb * AT_Q;
  if (q0 >= len) return;  // the whole CTA: nothing allocated yet
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* k_s = smem;
  uint8_t* v_s = smem + AT_TILE_BYTES;               // Q first, then the V tiles
  uint8_t* vt_s = smem + 2 * (size_t)AT_TILE_BYTES;  // V^T: [4 key blocks][64 rows d][32 keys]
  __shared__ uint64_t bars[8];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed_word;
  uint64_t* q_full = &bars[0];
  uint64_t* q_ready = &bars[1];  // Q is in tensor memory
  uint64_t* k_full = &bars[2];
  uint64_t* v_full = &bars[3];
  uint64_t* v_free = &bars[4];   // the V buffer has been read (Q moved, or a V tile transposed)
  uint64_t* s_full = &bars[5];   // S is in tensor memory; the K tile is no longer read
  uint64_t* p_ready = &bars[6];
  uint64_t* pv_done = &bars[7];
  volatile int* failed = &failed_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kend = min(len, q0 + AT_Q);
  const int ntiles = (kend + AT_K - 1) / AT_K;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_ready, 4);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(v_free, 4);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    failed_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, AT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_qkv) : "memory");
      mbar_expect_tx(q_full, AT_TILE_BYTES);
      tma_load_2d(v_s, &map_qkv, h * AT_D, r0 + q0, q_full);
      tma_load_2d(v_s + AT_TILE_BYTES / 2, &map_qkv, h * AT_D + 32, r0 + q0, q_full);
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int row = r0 + i * AT_K;
        if (i > 0) ok = mbar_wait(s_full, (i - 1) & 1, failed, error_flag, 40);  // the S MMAs have read K
        if (!ok) break;
        mbar_expect_tx(k_full, AT_TILE_BYTES);
        tma_load_2d(k_s, &map_qkv, c + h * AT_D, row, k_full);
        tma_load_2d(k_s + AT_TILE_BYTES / 2, &map_qkv, c + h * AT_D + 32, row, k_full);
        ok = mbar_wait(v_free, i & 1, failed, error_flag, 41);  // Q moved (i = 0) / V of tile i - 1 transposed
        if (!ok) break;
        mbar_expect_tx(v_full, AT_TILE_BYTES);
        tma_load_2d(v_s, &map_qkv, 2 * c + h * AT_D, row, v_full);
        tma_load_2d(v_s + AT_TILE_BYTES / 2, &map_qkv, 2 * c + h * AT_D + 32, row, v_full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_tf32(128, AT_K), idesc_o = umma_idesc_tf32(128, AT_D);
      bool ok = mbar_wait(q_ready, 0, failed, error_flag, 42);
      for (int i = 0; i < ntiles && ok; ++i) {
        // ---- S = Q K^T: eight k steps over the head dimension. S shares its columns with P of the
        // previous tile, which the MMAs issued before these have read.
        ok = mbar_wait(k_full, i & 1, failed, error_flag, 43);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t dk = umma_desc_sw128(k_s + kb * (AT_TILE_BYTES / 2));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_tf32_ts(tmem_base + AT_S_COL, tmem_base + AT_Q_COL + kb * 32 + k * 8, dk + (uint64_t)(k * 2), idesc_s,
                         (kb | k) != 0);
        }
        umma_commit(s_full);
        // ---- O += P V once P and V^T of this tile are in place
        ok = mbar_wait(p_ready, i & 1, failed, error_flag, 44);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < AT_K / 8; ++j) {
          const uint64_t dv = umma_desc_sw128(vt_s + (j >> 2) * 8192) + (uint64_t)((j & 3) * 2);
          umma_tf32_ts(tmem_base + AT_O_COL, tmem_base + AT_S_COL + j * 8, dv, idesc_o, (i | j) != 0);
        }
        umma_commit(pv_done);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;  // query row of the tile == tensor-memory lane == key handled in the transposition
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t s_addr = tmem_base + AT_S_COL + lane_addr, o_addr = tmem_base + AT_O_COL + lane_addr;
    const int qpos = q0 + r;
    const float sl2 = 0.125f * 1.4426950408889634f;  // 1 / sqrt(64), in powers of two
    float m = -INFINITY, l = 0.f;                    // running maximum (log2 units) and sum
    // row r of a [128][64] tile that TMA wrote as two boxes of [128][32] with the 128-byte swizzle:
    // logical 16-byte chunk jj of the row sits at chunk jj ^ (r & 7)
    const float4* row_lo = reinterpret_cast<const float4*>(v_s + (size_t)r * 128);
    const float4* row_hi = reinterpret_cast<const float4*>(v_s + AT_TILE_BYTES / 2 + (size_t)r * 128);
    bool ok = warp_wait_all(q_full, 0, failed, error_flag, 45);
    if (ok) {  // Q: shared memory -> tensor memory
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float4* src = half ? row_hi : row_lo;
        uint32_t w[32];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const float4 x = src[jj ^ (r & 7)];
          w[4 * jj + 0] = __float_as_uint(x.x);
          w[4 * jj + 1] = __float_as_uint(x.y);
          w[4 * jj + 2] = __float_as_uint(x.z);
          w[4 * jj + 3] = __float_as_uint(x.w);
        }
        tmem_st32(tmem_base + AT_Q_COL + lane_addr + (uint32_t)(half * 32), w);
      }
      tmem_wait_st();
      tc_fence_before();
    }
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(q_ready);
      mbar_arrive(v_free);
    }
    for (int i = 0; i < ntiles; ++i) {
      const int kt = i * AT_K;
      const bool diag = kt + AT_K - 1 > q0;  // some key of the tile lies after some query: mask
      if (ok) ok = warp_wait_all(s_full, i & 1, failed, error_flag, 46);
      if (ok) {
        tc_fence_after();
        uint32_t s[128];
        at_ld32<0>(s_addr, s);
        at_ld32<32>(s_addr, s);
        at_ld32<64>(s_addr, s);
        at_ld32<96>(s_addr, s);
        at_wait_ld();
        const float tmax = (diag ? at_row_max<true>(s, kt, qpos) : at_row_max<false>(s, kt, qpos)) * sl2;
        // The maximum is only moved (and O rescaled) when some row of the warp outgrew it by 2^8;
        // until then P simply runs up to 256, harmless in FP32 accumulators. Key kt is visible to
        // every row of the tile, so the first tile sets a finite maximum.
        const bool move = __any_sync(0xffffffffu, tmax > m + 8.0f);
        float corr = 1.0f;
        if (move) {
          const float mn = fmaxf(m, tmax);
          corr = ex2_approx(m - mn);  // 0 on the first tile (l is 0 and O not yet written)
          l *= corr;
          m = mn;
        }
        l += diag ? at_exp_rows<true>(s, kt, qpos, sl2, m) : at_exp_rows<false>(s, kt, qpos, sl2, m);
        // the PV MMAs of the previous tile read P and V^T and write O: wait for them
        if (i > 0) ok = warp_wait_all(pv_done, (i - 1) & 1, failed, error_flag, 47);
        if (ok) {
          tc_fence_after();
          at_st32<0>(s_addr, s);
          at_st32<32>(s_addr, s);
          at_st32<64>(s_addr, s);
          at_st32<96>(s_addr, s);
          if (move && i > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < AT_D; c0 += 32) {
              float v[32];
              uint32_t w[32];
              tmem_ld32(o_addr + (uint32_t)c0, v);
#pragma unroll
              for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(v[j] * corr);
              tmem_st32(o_addr + (uint32_t)c0, w);
            }
          }
          // V^T: this thread moves key r of the tile
          ok = warp_wait_all(v_full, i & 1, failed, error_flag, 48);
        }
        if (ok) {
          float* vt = reinterpret_cast<float*>(vt_s + (r >> 5) * 8192);
          const int kc = (r & 31) >> 2, kw = r & 3;  // 16-byte chunk and word of this key inside a V^T row
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const float4* src = half ? row_hi : row_lo;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const float4 x = src[jj ^ (r & 7)];
              const int d = half * 32 + jj * 4;
              vt[(d + 0) * 32 + ((kc ^ ((d + 0) & 7)) << 2) + kw] = x.x;
              vt[(d + 1) * 32 + ((kc ^ ((d + 1) & 7)) << 2) + kw] = x.y;
              vt[(d + 2) * 32 + ((kc ^ ((d + 2) & 7)) << 2) + kw] = x.z;
              vt[(d + 3) * 32 + ((kc ^ ((d + 3) & 7)) << 2) + kw] = x.w;
            }
          }
          tmem_wait_st();
          tc_fence_before();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // V^T is read by the tensor core
        }
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(v_free);
        mbar_arrive(p_ready);
      }
    }
    // ---- result: O / l
    if (ok) ok = warp_wait_all(pv_done, (ntiles - 1) & 1, failed, error_flag, 49);
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      float* orow = a.out + (size_t)(r0 + qpos) * c + h * AT_D;
#pragma unroll 1
      for (int c0 = 0; c0 < AT_D; c0 += 32) {
        float v[32];
        tmem_ld32(o_addr + (uint32_t)c0, v);
        if (qpos < len) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(orow + c0 + j) = make_float4(v[j] * inv, v[j + 1] * inv, v[j + 2] * inv, v[j + 3] * inv);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, AT_TMEM_COLS);
}


// ------------------------------------------------------------------ FP32-grade variant (three TF32 products)
// The same attention for the FP32-parity modes: every product is x.y + x_lo.y + x.y_lo with lo = v - hi(v),
// hi = the upper 19 bits the tensor core reads, so the scores and the weighted values are FP32-grade
// (causal_self_attention, src/models/gpt2/rust.rs:1580-1659, within the FP32 tolerance of the logits).
// The lo parts never come from memory: the softmax warps form Q_lo on the way into tensor memory, K_lo
// (same swizzled layout as the K tile) while the P.V MMAs of the previous tile run, P_lo next to P in
// tensor memory and V_lo^T while they transpose V. P keeps its full FP32 value in registers, 2^x is the
// hardware approximation (2 ulp). The hi.hi products of P.V and its two small terms have an accumulator
// each (the tensor core adds with truncation; the bias grows with the MMAs per accumulator). All 512
// tensor-memory columns: one CTA per SM, so nothing overlaps the softmax of a tile but the work of its
// own warps: EIGHT softmax warps, two per quarter of the tensor-memory lanes (a warp reaches the lanes
// 32 * (warp % 4) ..), each with half of the tile's 128 key columns, half of a row of Q, K, V in the
// conversions and transposition, and O or O_small when the maximum moves. The two threads of a row
// exchange their partial row maxima through shared memory at a 64-thread named barrier per tile.
constexpr size_t AT_X3_SMEM = (size_t)AT_TILE_BYTES * 5 + 1024;
constexpr uint32_t X3_S_COL = 0, X3_PLO_COL = 128, X3_O_COL = 256, X3_OS_COL = 320, X3_Q_COL = 384, X3_QLO_COL = 448,
                   X3_TMEM_COLS = 512;
constexpr int X3_THREADS = 320, X3_HC = AT_K / 2;  // threads per CTA; key columns per softmax thread

__device__ __forceinline__ uint32_t lo_bits(uint32_t v) {
  return __float_as_uint(__uint_as_float(v) - __uint_as_float(v & 0xFFFFE000u));
}

__device__ __forceinline__ void x3_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Row maximum of this thread's X3_HC raw scores (keys kt + cb ..); MASK: keys after the query do not count.
template <bool MASK>
__device__ __forceinline__ float x3_row_max(const uint32_t (&s)[X3_HC], int k0, int qpos) {
  float tmax = -INFINITY;
#pragma unroll
  for (int j = 0; j < X3_HC; ++j)
    if (!MASK || k0 + j <= qpos) tmax = fmaxf(tmax, __uint_as_float(s[j]));
  return tmax;
}

// s <- P = 2^(s * sl2 - mn) at full FP32 precision; returns the sum of the thread's columns
template <bool MASK>
__device__ __forceinline__ float x3_exp_rows(uint32_t (&s)[X3_HC], int k0, int qpos, float sl2, float mn) {
  float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
  for (int j = 0; j < X3_HC; j += 2) {
    float p0 = ex2_approx(fmaf(__uint_as_float(s[j]), sl2, -mn));
    float p1 = ex2_approx(fmaf(__uint_as_float(s[j + 1]), sl2, -mn));
    if (MASK && k0 + j > qpos) p0 = 0.f;
    if (MASK && k0 + j + 1 > qpos) p1 = 0.f;
    ps0 += p0;
    ps1 += p1;
    s[j] = __float_as_uint(p0);
    s[j + 1] = __float_as_uint(p1);
  }
  return ps0 + ps1;
}

__global__ void __launch_bounds__(X3_THREADS, 1)
    prefill_attention_x3_kernel(const __grid_constant__ CUtensorMap map_qkv, PrefillAttnArgs a, int* error_flag) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int h = blockIdx.x, b = blockIdx.y, qb = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int c = a.n_head * AT_D;
  const int r0 = a.seq_start[b], len = a.seq_start[b + 1] - r0;
  const int q0 = qb * AT_Q;
  if (q0 >= len) return;  // the whole CTA: nothing allocated yet
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* k_s = smem;
  uint8_t* klo_s = smem + AT_TILE_BYTES;
  uint8_t* v_s = smem + 2 * (size_t)AT_TILE_BYTES;     // Q first, then the V tiles
  uint8_t* vt_s = smem + 3 * (size_t)AT_TILE_BYTES;    // V^T: [4 key blocks][64 rows d][32 keys]
  uint8_t* vtlo_s = smem + 4 * (size_t)AT_TILE_BYTES;  // lo parts of V^T, same layout
  __shared__ uint64_t bars[9];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed_word;
  __shared__ float xmax[2][2][AT_Q];  // [tile parity][column half][row]: partial row maxima; at the end the partial sums
  uint64_t* q_full = &bars[0];
  uint64_t* q_ready = &bars[1];    // Q and Q_lo are in tensor memory
  uint64_t* k_full = &bars[2];
  uint64_t* v_full = &bars[3];
  uint64_t* v_free = &bars[4];     // the V buffer has been read (Q moved, or a V tile transposed)
  uint64_t* s_full = &bars[5];     // S is in tensor memory; the K and K_lo tiles are no longer read
  uint64_t* p_ready = &bars[6];
  uint64_t* pv_done = &bars[7];
  uint64_t* klo_ready = &bars[8];  // K_lo of the tile is in shared memory
  volatile int* failed = &failed_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kend = min(len, q0 + AT_Q);
  const int ntiles = (kend + AT_K - 1) / AT_K;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_ready, 8);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(v_free, 8);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 8);
    mbar_init(pv_done, 1);
    mbar_init(klo_ready, 8);
    failed_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, X3_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_qkv) : "memory");
      mbar_expect_tx(q_full, AT_TILE_BYTES);
      tma_load_2d(v_s, &map_qkv, h * AT_D, r0 + q0, q_full);
      tma_load_2d(v_s + AT_TILE_BYTES / 2, &map_qkv, h * AT_D + 32, r0 + q0, q_full);
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int row = r0 + i * AT_K;
        if (i > 0) ok = mbar_wait(s_full, (i - 1) & 1, failed, error_flag, 50);  // the S MMAs have read K and K_lo
        if (!ok) break;
        mbar_expect_tx(k_full, AT_TILE_BYTES);
        tma_load_2d(k_s, &map_qkv, c + h * AT_D, row, k_full);
        tma_load_2d(k_s + AT_TILE_BYTES / 2, &map_qkv, c + h * AT_D + 32, row, k_full);
        ok = mbar_wait(v_free, i & 1, failed, error_flag, 51);  // Q moved (i = 0) / V of tile i - 1 transposed
        if (!ok) break;
        mbar_expect_tx(v_full, AT_TILE_BYTES);
        tma_load_2d(v_s, &map_qkv, 2 * c + h * AT_D, row, v_full);
        tma_load_2d(v_s + AT_TILE_BYTES / 2, &map_qkv, 2 * c + h * AT_D + 32, row, v_full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_tf32(128, AT_K), idesc_o = umma_idesc_tf32(128, AT_D);
      bool ok = mbar_wait(q_ready, 0, failed, error_flag, 52);
      for (int i = 0; i < ntiles && ok; ++i) {
        // ---- S = Q K^T + Q_lo K^T + Q K_lo^T: eight k steps over the head dimension, three MMAs each
        ok = mbar_wait(k_full, i & 1, failed, error_flag, 53);
        if (ok) ok = mbar_wait(klo_ready, i & 1, failed, error_flag, 54);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t dk = umma_desc_sw128(k_s + kb * (AT_TILE_BYTES / 2));
          const uint64_t dkl = umma_desc_sw128(klo_s + kb * (AT_TILE_BYTES / 2));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t qa = tmem_base + X3_Q_COL + kb * 32 + k * 8, ql = tmem_base + X3_QLO_COL + kb * 32 + k * 8;
            umma_tf32_ts(tmem_base + X3_S_COL, ql, dk + (uint64_t)(k * 2), idesc_s, (kb | k) != 0);
            umma_tf32_ts(tmem_base + X3_S_COL, qa, dkl + (uint64_t)(k * 2), idesc_s, 1);
            umma_tf32_ts(tmem_base + X3_S_COL, qa, dk + (uint64_t)(k * 2), idesc_s, 1);
          }
        }
        umma_commit(s_full);
        // ---- O += P V, O_small += P_lo V + P V_lo once P, P_lo, V^T and V_lo^T of this tile are in place
        ok = mbar_wait(p_ready, i & 1, failed, error_flag, 55);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < AT_K / 8; ++j) {
          const uint64_t off = (uint64_t)((j & 3) * 2);
          const uint64_t dv = umma_desc_sw128(vt_s + (j >> 2) * 8192) + off;
          const uint64_t dvl = umma_desc_sw128(vtlo_s + (j >> 2) * 8192) + off;
          umma_tf32_ts(tmem_base + X3_OS_COL, tmem_base + X3_PLO_COL + j * 8, dv, idesc_o, (i | j) != 0);
          umma_tf32_ts(tmem_base + X3_OS_COL, tmem_base + X3_S_COL + j * 8, dvl, idesc_o, 1);
          umma_tf32_ts(tmem_base + X3_O_COL, tmem_base + X3_S_COL + j * 8, dv, idesc_o, (i | j) != 0);
        }
        umma_commit(pv_done);
      }
    }
  } else {
    const int q = warp & 3;          // quarter of the tensor-memory lanes this warp reaches
    const int hf = (warp - 2) >> 2;  // which half of the key columns / of a row of Q, K, V this thread handles
    const int r = q * 32 + lane;     // query row of the tile == tensor-memory lane == key handled in the transposition
    const int cb = hf * X3_HC;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t s_addr = tmem_base + X3_S_COL + lane_addr + (uint32_t)cb;
    const uint32_t plo_addr = tmem_base + X3_PLO_COL + lane_addr + (uint32_t)cb;
    const uint32_t o_addr = tmem_base + (hf ? X3_OS_COL : X3_O_COL) + lane_addr;  // rescaled by this thread when the maximum moves
    const int qpos = q0 + r;
    const float sl2 = 0.125f * 1.4426950408889634f;  // 1 / sqrt(64), in powers of two
    float m = -INFINITY, l = 0.f;                    // running maximum (log2 units) and this thread's part of the sum
    // this thread's half (32 floats = 128 bytes, one swizzle row) of row r of the Q / V tile and of the K tile
    const float4* vrow = reinterpret_cast<const float4*>(v_s + hf * (AT_TILE_BYTES / 2) + (size_t)r * 128);
    const float4* krow = reinterpret_cast<const float4*>(k_s + hf * (AT_TILE_BYTES / 2) + (size_t)r * 128);
    float4* klrow = reinterpret_cast<float4*>(klo_s + hf * (AT_TILE_BYTES / 2) + (size_t)r * 128);
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory"); };
    // K_lo of the tile in k_s: element by element at the same (swizzled) place
    auto make_klo = [&]() {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int cidx = jj ^ (r & 7);
        const float4 x = krow[cidx];
        klrow[cidx] = make_float4(__uint_as_float(lo_bits(__float_as_uint(x.x))), __uint_as_float(lo_bits(__float_as_uint(x.y))),
                                  __uint_as_float(lo_bits(__float_as_uint(x.z))), __uint_as_float(lo_bits(__float_as_uint(x.w))));
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // K_lo is read by the tensor core
    };
    bool ok = warp_wait_all(q_full, 0, failed, error_flag, 56);
    if (ok) {  // Q: shared memory -> tensor memory, as it is (the MMA reads its hi part) and its lo part
      uint32_t w[32];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float4 x = vrow[jj ^ (r & 7)];
        w[4 * jj + 0] = __float_as_uint(x.x);
        w[4 * jj + 1] = __float_as_uint(x.y);
        w[4 * jj + 2] = __float_as_uint(x.z);
        w[4 * jj + 3] = __float_as_uint(x.w);
      }
      tmem_st32(tmem_base + X3_Q_COL + lane_addr + (uint32_t)(hf * 32), w);
#pragma unroll
      for (int j = 0; j < 32; ++j) w[j] = lo_bits(w[j]);
      tmem_st32(tmem_base + X3_QLO_COL + lane_addr + (uint32_t)(hf * 32), w);
      tmem_wait_st();
      tc_fence_before();
    }
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(q_ready);
      mbar_arrive(v_free);
    }
    if (ok) ok = warp_wait_all(k_full, 0, failed, error_flag, 57);
    if (ok) make_klo();
    __syncwarp();
    if (lane == 0) mbar_arrive(klo_ready);
    for (int i = 0; i < ntiles; ++i) {
      const int kt = i * AT_K;
      const bool diag = kt + AT_K - 1 > q0;  // some key of the tile lies after some query: mask
      uint32_t s[X3_HC];
      float part_max = -INFINITY;
      if (ok) ok = warp_wait_all(s_full, i & 1, failed, error_flag, 58);
      if (ok) {
        tc_fence_after();
        x3_ld32(s_addr, s);
        x3_ld32(s_addr + 32u, s + 32);
        at_wait_ld();
        part_max = diag ? x3_row_max<true>(s, kt + cb, qpos) : x3_row_max<false>(s, kt + cb, qpos);
      }
      // the row maximum is over both halves: every softmax thread comes here once per tile, whatever `ok` says
      xmax[i & 1][hf][r] = part_max;
      pair_sync();
      if (ok) {
        const float tmax = fmaxf(part_max, xmax[i & 1][hf ^ 1][r]) * sl2;
        // The maximum is only moved (and O rescaled) when some row of the warp outgrew it by 2^8 (the same
        // decision in both warps of the pair: they hold the same rows); key kt is visible to every row of
        // the tile, so the first tile sets a finite maximum.
        const bool move = __any_sync(0xffffffffu, tmax > m + 8.0f);
        float corr = 1.0f;
        if (move) {
          const float mn = fmaxf(m, tmax);
          corr = ex2_approx(m - mn);  // 0 on the first tile (l is 0 and O not yet written)
          l *= corr;
          m = mn;
        }
        l += diag ? x3_exp_rows<true>(s, kt + cb, qpos, sl2, m) : x3_exp_rows<false>(s, kt + cb, qpos, sl2, m);
        // the PV MMAs of the previous tile read P, P_lo, V^T, V_lo^T and write O: wait for them
        if (i > 0) ok = warp_wait_all(pv_done, (i - 1) & 1, failed, error_flag, 59);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < X3_HC; c0 += 32) {
            uint32_t w[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = s[c0 + j] & 0xFFFFE000u;
            tmem_st32(s_addr + (uint32_t)c0, w);
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = lo_bits(s[c0 + j]);
            tmem_st32(plo_addr + (uint32_t)c0, w);
          }
          if (move && i > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < AT_D; c0 += 32) {  // column half 0 rescales O, half 1 O_small
              float v[32];
              uint32_t w[32];
              tmem_ld32(o_addr + (uint32_t)c0, v);
#pragma unroll
              for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(v[j] * corr);
              tmem_st32(o_addr + (uint32_t)c0, w);
            }
          }
          // V^T and V_lo^T: this thread moves 32 of the 64 values of key r
          ok = warp_wait_all(v_full, i & 1, failed, error_flag, 60);
        }
        if (ok) {
          float* vt = reinterpret_cast<float*>(vt_s + (r >> 5) * 8192);
          float* vtl = reinterpret_cast<float*>(vtlo_s + (r >> 5) * 8192);
          const int kc = (r & 31) >> 2, kw = r & 3;  // 16-byte chunk and word of this key inside a V^T row
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const float4 x = vrow[jj ^ (r & 7)];
            const float xs[4] = {x.x, x.y, x.z, x.w};
            const int d = hf * 32 + jj * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int o = (d + e) * 32 + ((kc ^ ((d + e) & 7)) << 2) + kw;
              vt[o] = xs[e];
              vtl[o] = __uint_as_float(lo_bits(__float_as_uint(xs[e])));
            }
          }
          tmem_wait_st();
          tc_fence_before();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // V^T and V_lo^T are read by the tensor core
        }
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(v_free);
        mbar_arrive(p_ready);
      }
      // K_lo of the next tile while the P.V MMAs of this one run (S of tile i has been read: K_lo is free)
      if (i + 1 < ntiles) {
        if (ok) ok = warp_wait_all(k_full, (i + 1) & 1, failed, error_flag, 61);
        if (ok) make_klo();
        __syncwarp();
        if (lane == 0) mbar_arrive(klo_ready);
      }
    }
    // ---- result: (O + O_small) / l, l = the sum over both column halves; each thread writes 32 of the 64 values
    xmax[ntiles & 1][hf][r] = l;
    pair_sync();
    l += xmax[ntiles & 1][hf ^ 1][r];
    if (ok) ok = warp_wait_all(pv_done, (ntiles - 1) & 1, failed, error_flag, 62);
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      const int c0 = hf * 32;
      float* orow = a.out + (size_t)(r0 + qpos) * c + h * AT_D + c0;
      float* lrow = a.out_lo ? a.out_lo + (size_t)(r0 + qpos) * c + h * AT_D + c0 : nullptr;
      float v[32], v2[32];
      tmem_ld32(tmem_base + X3_O_COL + lane_addr + (uint32_t)c0, v);
      tmem_ld32(tmem_base + X3_OS_COL + lane_addr + (uint32_t)c0, v2);
      if (qpos < len) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float y0 = (v[j] + v2[j]) * inv, y1 = (v[j + 1] + v2[j + 1]) * inv, y2 = (v[j + 2] + v2[j + 2]) * inv,
                      y3 = (v[j + 3] + v2[j + 3]) * inv;
          *reinterpret_cast<float4*>(orow + j) = make_float4(y0, y1, y2, y3);
          if (lrow)
            *reinterpret_cast<float4*>(lrow + j) =
                make_float4(y0 - tf32_hi(y0), y1 - tf32_hi(y1), y2 - tf32_hi(y2), y3 - tf32_hi(y3));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, X3_TMEM_COLS);
}

}  // namespace

bool prefill_attention_tc_supported(const PrefillAttnArgs& a) { return a.head_dim == 64 && encode_fn() != nullptr; }

cudaError_t init_attn_tc_attributes() {
  cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_TC_SMEM);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(prefill_attention_x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_X3_SMEM);
}

// qkv: [rows, 3c]; rows = total prompt rows of the batch
cudaError_t launch_prefill_attention_tc(const PrefillAttnArgs& a, int rows, int* error_flag, cudaStream_t s) {
  if (!prefill_attention_tc_supported(a)) return cudaErrorInvalidValue;
  const int c = a.n_head * 64;
  CUtensorMap map;
  if (!make_map(&map, a.qkv, (uint64_t)rows, (uint64_t)3 * c, 128)) return cudaErrorInvalidValue;
  dim3 grid(a.n_head, a.batch, (a.max_len + AT_Q - 1) / AT_Q);
  prefill_attention_tc_kernel<<<grid, 192, AT_TC_SMEM, s>>>(map, a, error_flag);
  return cudaGetLastError();
}

// FP32-grade variant; a.out_lo (optional) receives out - hi(out)
cudaError_t launch_prefill_attention_x3(const PrefillAttnArgs& a, int rows, int* error_flag, cudaStream_t s) {
  if (!prefill_attention_tc_supported(a)) return cudaErrorInvalidValue;
  const int c = a.n_head * 64;
  CUtensorMap map;
  if (!make_map(&map, a.qkv, (uint64_t)rows, (uint64_t)3 * c, 128)) return cudaErrorInvalidValue;
  dim3 grid(a.n_head, a.batch, (a.max_len + AT_Q - 1) / AT_Q);
  prefill_attention_x3_kernel<<<grid, X3_THREADS, AT_X3_SMEM, s>>>(map, a, error_flag);
  return cudaGetLastError();
}

}  // namespace pg
