// Tensor-core GEMMs for sm_100a: tcgen05.mma with accumulators in tensor memory, operands staged
// by TMA (plain per-CTA tiled loads, 128-byte swizzle), mbarrier pipelines, warp-specialised roles.
//
//   tc_gemm_ss_kernel   out[m, n] = x[m, k] . w[n, k]^T, single TF32 pass, both operands from
//                       shared memory. Prefill shapes (m = thousands of prompt rows).
//   tc_gemm_x3_kernel   the same product to FP32 accuracy from three TF32 products
//                       (hi*hi + hi*lo + lo*hi). The weight tile is the 128-row MMA operand: its
//                       raw FP32 tile is split into hi/lo by the epilogue warps and placed in tensor
//                       memory (tcgen05.st), so the MMA reads it from there; the few activation rows
//                       arrive pre-split (x_hi, x_lo) and are the N operand. Decode shapes
//                       (m <= 256 tokens), optional split-K with a fixed-order reduction.
//
// Every wait on an mbarrier is bounded: on expiry the kernel raises an error flag in global
// memory, stops issuing work, still frees its tensor memory and returns.
#include <algorithm>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace pg {
namespace {


// tanh-GELU with the hardware tanh approximation (relative error about 2^-11): only for the single
// TF32 pass of the prefill, whose products already carry 10-bit mantissas.
__device__ __forceinline__ float gelu_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978846f * (x + 0.044715f * x * x * x)));
  return 0.5f * x * (1.0f + t);
}

// ------------------------------------------------------------------ single-pass TF32, SS
// grid (ceil(n / BN), ceil(m / 128)); 192 threads: warp 0 TMA producer, warp 1 MMA issuer and
// tensor-memory owner, warps 2..5 epilogue (warp w reads TMEM lanes 32 * (w % 4) ...).
template <int BN>
struct SsSmem {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = TILE_M * BK * 4, B_BYTES = BN * BK * 4;
  static constexpr int EPI_BYTES = 4 * 32 * 33 * 4;  // one padded 32x32 transpose tile per epilogue warp
  static constexpr size_t BYTES = (size_t)STAGES * (A_BYTES + B_BYTES) + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
    tc_gemm_ss_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                      TcGemmArgs a) {
  using S = SsSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = base;
  uint8_t* smem_b = base + (size_t)S::STAGES * S::A_BYTES;
  float* epi_tiles = reinterpret_cast<float*>(smem_b + (size_t)S::STAGES * S::B_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(epi_tiles) + S::EPI_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* d_full = empty + S::STAGES;   // [2]: accumulator buffer holds a finished tile
  uint64_t* d_empty = d_full + 2;         // [2]: the epilogue warps have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // Persistent over output tiles (tile = blockIdx.x, + gridDim.x, ...; column tiles of one row panel
  // are neighbours, so the activation panel is reused from L2). Two accumulators in tensor memory:
  // while the epilogue warps drain one tile, the MMAs of the next one already run.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (a.n + BN - 1) / BN, tiles = tiles_n * ((a.m + TILE_M - 1) / TILE_M);
  const int nkb = a.k / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&d_full[i], 1);
      mbar_init(&d_empty[i], 4);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;  // stage counter over all tiles of this CTA
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int n0 = (tile % tiles_n) * BN, m0 = (tile / tiles_n) * TILE_M;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % S::STAGES;
          if (it >= S::STAGES) ok = mbar_wait(&empty[s], ((it / S::STAGES) - 1) & 1, failed, a.error_flag, 1);
          if (!ok) break;
          mbar_expect_tx(&full[s], S::A_BYTES + S::B_BYTES);
          tma_load_2d(smem_a + (size_t)s * S::A_BYTES, &map_x, kb * BK, m0, &full[s]);
          tma_load_2d(smem_b + (size_t)s * S::B_BYTES, &map_w, kb * BK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(TILE_M, BN);
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++ti) {
        const uint32_t buf = ti & 1;
        if (ti >= 2) ok = mbar_wait(&d_empty[buf], ((ti >> 1) - 1) & 1, failed, a.error_flag, 4);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
          const uint32_t s = it % S::STAGES;
          ok = mbar_wait(&full[s], (it / S::STAGES) & 1, failed, a.error_flag, 2);
          if (!ok) break;
          tc_fence_after();
          const uint64_t da = umma_desc_sw128(smem_a + (size_t)s * S::A_BYTES);
          const uint64_t db = umma_desc_sw128(smem_b + (size_t)s * S::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 8; ++k)
            umma_tf32_ss(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&d_full[buf]);
      }
    }
  } else {
    // TMEM lane = output row, but a row-per-thread store touches 32 cache lines per instruction:
    // every 32x32 block goes through a padded shared-memory tile and leaves column-per-lane, so
    // that residual loads and output stores are 128-byte coalesced.
    const int q = warp & 3;
    float* tile = epi_tiles + q * (32 * 33);
    uint32_t ti = 0;
    bool ok = true;
    for (int tile_id = blockIdx.x; tile_id < tiles && ok; tile_id += gridDim.x, ++ti) {
      const int n0 = (tile_id % tiles_n) * BN, m0 = (tile_id / tiles_n) * TILE_M;
      const uint32_t buf = ti & 1;
      const uint32_t tmem_d = tmem_base + buf * BN;
      ok = mbar_wait(&d_full[buf], (ti >> 1) & 1, failed, a.error_flag, 3);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col = n0 + c0 + lane;
        // the block's 32 residual values of this lane's column go out first: they do not depend on
        // the accumulator, and asked for one by one between the stores (which may alias them:
        // the residual is updated in place) they would each cost a full memory round trip
        float rv[32];
        if (a.epilogue == EPI_RESID && col < a.n) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) {
            const int row = m0 + q * 32 + rr;
            rv[rr] = row < a.m ? a.resid[(size_t)row * a.n + col] : 0.f;
          }
        }
        float v[32];
        tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) tile[lane * 33 + j] = v[j];
        __syncwarp();
        const float bias = (a.bias && col < a.n) ? a.bias[col] : 0.f;
        if (col < a.n) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) {
            const int row = m0 + q * 32 + rr;
            if (row < a.m) {
              float r = tile[rr * 33 + lane];
              if (a.bias) r = bias + r;
              if (a.epilogue == EPI_GELU) r = gelu_fast(r);
              if (a.epilogue == EPI_RESID) r = rv[rr] + r;
              a.out[(size_t)row * a.n + col] = r;
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&d_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ------------------------------------------------------------------ 3xTF32, both operands from shared memory
struct Ss3Smem {
  static constexpr int BN = 128;
  static constexpr int STAGES = 3;
  static constexpr int A_BYTES = TILE_M * BK * 4, B_BYTES = BN * BK * 4;
  static constexpr int EPI_BYTES = 4 * 32 * 33 * 4;  // one padded 32x32 transpose tile per epilogue warp
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;  // x, x_lo, w, w_lo tiles of one k block
  static constexpr size_t BYTES = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

// out[m, n] = x[m, k] . w[n, k]^T at FP32 grade on the tensor cores: the tensor core reads the upper 19 bits of
// every FP32 operand (its TF32 "hi" part), so with lo = v - hi(v) kept in a second array the product is
// x.w + x.w_lo + x_lo.w, three TF32 MMAs per k step accumulated in FP32 (the lo.lo term is below FP32 rounding).
// Same structure as tc_gemm_ss_kernel: TMA producer warp, one MMA-issuing thread, four epilogue warps, persistent
// over 128 x 128 output tiles with two accumulator pairs in tensor memory. Prefill GEMMs of the FP32-parity modes.
__global__ void __launch_bounds__(192, 1)
    tc_gemm_ss3_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_xlo,
                       const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_wlo,
                       TcGemmArgs a) {
  using S = Ss3Smem;
  constexpr int BN = S::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = base;  // per stage: x tile, x_lo tile, w tile, w_lo tile
  float* epi_tiles = reinterpret_cast<float*>(base + (size_t)S::STAGES * S::STAGE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(epi_tiles) + S::EPI_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* d_full = empty + S::STAGES;   // [2]: accumulator buffer holds a finished tile
  uint64_t* d_empty = d_full + 2;         // [2]: the epilogue warps have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // Persistent over output tiles (tile = blockIdx.x, + gridDim.x, ...; column tiles of one row panel
  // are neighbours, so the activation panel is reused from L2). Two accumulators in tensor memory:
  // while the epilogue warps drain one tile, the MMAs of the next one already run.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (a.n + BN - 1) / BN, tiles = tiles_n * ((a.m + TILE_M - 1) / TILE_M);
  const int nkb = a.k / BK;
  // Long reductions are cut into chunks of at most 56 k blocks, each accumulated in tensor memory on its own and
  // added to the result by the epilogue warps in FP32 (round to nearest): the accumulate inside the tensor core
  // truncates, and its bias grows with the length of one accumulation. Not with GELU (not additive; its GEMM
  // has k = n_embd, short enough).
  const int nchunk = (a.epilogue == EPI_GELU) ? 1 : (nkb + 55) / 56;
  const int kc = (nkb + nchunk - 1) / nchunk;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&d_full[i], 1);
      mbar_init(&d_empty[i], 4);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 4 * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;  // stage counter over all tiles of this CTA
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int n0 = (tile % tiles_n) * BN, m0 = (tile / tiles_n) * TILE_M;
        for (int kb = 0; kb < nkb; ++kb, ++it) {  // chunk boundaries do not matter to the operand stream
          const uint32_t s = it % S::STAGES;
          if (it >= S::STAGES) ok = mbar_wait(&empty[s], ((it / S::STAGES) - 1) & 1, failed, a.error_flag, 1);
          if (!ok) break;
          uint8_t* st = stages + (size_t)s * S::STAGE_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          tma_load_2d(st, &map_x, kb * BK, m0, &full[s]);
          tma_load_2d(st + S::A_BYTES, &map_xlo, kb * BK, m0, &full[s]);
          tma_load_2d(st + 2 * S::A_BYTES, &map_w, kb * BK, n0, &full[s]);
          tma_load_2d(st + 2 * S::A_BYTES + S::B_BYTES, &map_wlo, kb * BK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(TILE_M, BN);
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x)
      for (int kb0 = 0; kb0 < nkb && ok; kb0 += kc, ++ti) {
        const int kb1 = min(nkb, kb0 + kc);
        const uint32_t buf = ti & 1;
        if (ti >= 2) ok = mbar_wait(&d_empty[buf], ((ti >> 1) - 1) & 1, failed, a.error_flag, 4);
        if (!ok) break;
        tc_fence_after();
        // The tensor core adds into the accumulator with truncation, a bias that grows with the number of
        // MMAs into one accumulator: the hi . hi products get an accumulator of their own and the two small
        // terms share a second one (their magnitude, hence their bias, is 2^-11 of the first).
        const uint32_t tmem_d = tmem_base + buf * (2 * BN), tmem_s = tmem_d + BN;
        for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
          const uint32_t s = it % S::STAGES;
          ok = mbar_wait(&full[s], (it / S::STAGES) & 1, failed, a.error_flag, 2);
          if (!ok) break;
          tc_fence_after();
          uint8_t* st = stages + (size_t)s * S::STAGE_BYTES;
          const uint64_t da = umma_desc_sw128(st), dal = umma_desc_sw128(st + S::A_BYTES);
          const uint64_t db = umma_desc_sw128(st + 2 * S::A_BYTES), dbl = umma_desc_sw128(st + 2 * S::A_BYTES + S::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 8; ++k)
            umma_tf32_ss(tmem_s, dal + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb != kb0) || k != 0);
#pragma unroll
          for (int k = 0; k < BK / 8; ++k) umma_tf32_ss(tmem_s, da + (uint64_t)(k * 2), dbl + (uint64_t)(k * 2), idesc, 1);
#pragma unroll
          for (int k = 0; k < BK / 8; ++k)
            umma_tf32_ss(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb != kb0) || k != 0);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&d_full[buf]);
      }
    }
  } else {
    // TMEM lane = output row, but a row-per-thread store touches 32 cache lines per instruction:
    // every 32x32 block goes through a padded shared-memory tile and leaves column-per-lane, so
    // that residual loads and output stores are 128-byte coalesced.
    const int q = warp & 3;
    float* tile = epi_tiles + q * (32 * 33);
    uint32_t ti = 0;
    bool ok = true;
    for (int tile_id = blockIdx.x; tile_id < tiles && ok; tile_id += gridDim.x)
    for (int ch = 0; ch < nchunk && ok; ++ch, ++ti) {
      const bool first = ch == 0, last = ch == nchunk - 1;
      const int n0 = (tile_id % tiles_n) * BN, m0 = (tile_id / tiles_n) * TILE_M;
      const uint32_t buf = ti & 1;
      const uint32_t tmem_d = tmem_base + buf * (2 * BN);
      ok = mbar_wait(&d_full[buf], (ti >> 1) & 1, failed, a.error_flag, 3);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col = n0 + c0 + lane;
        // the block's 32 residual values of this lane's column go out first: they do not depend on
        // the accumulator, and asked for one by one between the stores (which may alias them:
        // the residual is updated in place) they would each cost a full memory round trip
        // (a later chunk of a long reduction adds to what the chunks before it left in `out`)
        float rv[32];
        const float* prev = first ? (a.epilogue == EPI_RESID ? a.resid : nullptr) : a.out;
        if (prev && col < a.n) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) {
            const int row = m0 + q * 32 + rr;
            rv[rr] = row < a.m ? prev[(size_t)row * a.n + col] : 0.f;
          }
        }
        float v[32], v2[32];
        tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(BN + c0), v2);
#pragma unroll
        for (int j = 0; j < 32; ++j) tile[lane * 33 + j] = v[j] + v2[j];
        __syncwarp();
        const float bias = (a.bias && col < a.n) ? a.bias[col] : 0.f;
        if (col < a.n) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) {
            const int row = m0 + q * 32 + rr;
            if (row < a.m) {
              float r = tile[rr * 33 + lane];
              if (a.bias && first) r = bias + r;
              if (a.epilogue == EPI_GELU) r = gelu_ref(r);
              if (prev) r = rv[rr] + r;
              a.out[(size_t)row * a.n + col] = r;
              if (a.out_lo && last) a.out_lo[(size_t)row * a.n + col] = r - tf32_hi(r);  // lo part for the GEMM that reads `out`
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&d_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 4 * BN);
}

// ------------------------------------------------------------------ 3xTF32, weights via TMEM
// grid (ceil(n / 128), splits) with thread-block clusters of (1, splits, 1): the CTAs of one
// cluster share a 128-row weight tile and each covers 1/splits of k. 192 threads per CTA.
// A shared-memory stage holds the raw FP32 weight tile (128 rows x 32 k) and the pre-split
// activation tiles x_hi, x_lo (BN rows x 32 k). The four epilogue warps turn each weight tile
// into hi/lo in tensor memory; the MMA warp then issues, per 8-wide k step, hi*hi, hi*lo and
// lo*hi into the same accumulator. Split-K partials are exchanged through distributed shared
// memory and added in split order, so the result does not depend on scheduling.
template <int BN>
struct X3 {
  static constexpr int STAGES = (BN == 64) ? 6 : (BN == 32) ? 8 : 10;  // shared-memory stages (TMA depth)
  static constexpr int TSTAGES = 6;  // tensor-memory stages of the split weight tile
  static constexpr int A_BYTES = TILE_M * BK * 4, B_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = A_BYTES + 2 * B_BYTES;
  static constexpr int D_BYTES = TILE_M * BN * 4;  // receive buffer of the split-K exchange (never aliased:
                                                   // peers write it while this CTA may still be in its main loop)
  static constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;
  static constexpr size_t BYTES = (size_t)PIPE_BYTES + D_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;  // BN accumulator columns, then TSTAGES * 64 from column 64
  static constexpr int A_COL0 = 128;     // accumulator: columns [0, BN) hi*hi + lo*hi, [BN, 2 BN) hi*lo
};

__device__ __forceinline__ void trace_mark(const TcGemmArgs& a, int slot) {
  if (a.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    a.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 16 + slot] = t;
  }
}

__device__ __forceinline__ void trace_add(const TcGemmArgs& a, int slot, long long cycles) {
  if (a.trace) a.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 16 + slot] = (unsigned long long)cycles;
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `local_addr` (a shared::cta address of this kernel's layout) inside CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_dsmem(uint32_t remote_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_addr), "f"(v) : "memory");
}


template <int BN, int SPLITS>
__global__ void __launch_bounds__(192, 1)
    tc_gemm_x3_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_xhi,
                      const __grid_constant__ CUtensorMap map_xlo, TcGemmArgs a) {
  using S = X3<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* recv = reinterpret_cast<float*>(base + (size_t)S::PIPE_BYTES);  // [split][token][row of my slice]
  uint64_t* full = reinterpret_cast<uint64_t*>(base + (size_t)S::PIPE_BYTES + S::D_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* a_ready = empty + S::STAGES;
  uint64_t* a_free = a_ready + S::TSTAGES;
  uint64_t* d_full = a_free + S::TSTAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TILE_M;  // first weight row (output feature) of this tile
  constexpr int splits = SPLITS;          // == gridDim.y == cluster size
  const int split = (int)cluster_rank();  // == blockIdx.y: the cluster spans the whole y extent
  const int nkb_total = a.k / BK;
  const int kb_per = (nkb_total + splits - 1) / splits;
  const int kb0 = min(split * kb_per, nkb_total), kb1 = min(kb0 + kb_per, nkb_total);
  const int nkb = kb1 - kb0;

  pdl_launch();
  if (threadIdx.x == 0) trace_mark(a, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < S::TSTAGES; ++s) {
      mbar_init(&a_ready[s], 128);
      mbar_init(&a_free[s], 1);
    }
    mbar_init(d_full, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) trace_mark(a, 1);

  auto stage_a = [&](int s) { return base + (size_t)s * S::STAGE_BYTES; };
  auto stage_bhi = [&](int s) { return base + (size_t)s * S::STAGE_BYTES + S::A_BYTES; };
  auto stage_blo = [&](int s) { return base + (size_t)s * S::STAGE_BYTES + S::A_BYTES + S::B_BYTES; };

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xhi) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xlo) : "memory");
      // weights do not depend on the previous kernel: start streaming them before the wait
      const int pre = min(nkb, S::STAGES);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], S::STAGE_BYTES);
        tma_load_2d(stage_a(i), &map_w, 0, (blockIdx.x * nkb_total + kb0 + i) * TILE_M, &full[i]);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) {
        tma_load_2d(stage_bhi(i), &map_xhi, (kb0 + i) * BK, 0, &full[i]);
        tma_load_2d(stage_blo(i), &map_xlo, (kb0 + i) * BK, 0, &full[i]);
      }
      for (int i = pre; i < nkb; ++i) {
        const int s = i % S::STAGES;
        if (!mbar_wait(&empty[s], ((i / S::STAGES) - 1) & 1, failed, a.error_flag, 11)) break;
        mbar_expect_tx(&full[s], S::STAGE_BYTES);
        tma_load_2d(stage_a(s), &map_w, 0, (blockIdx.x * nkb_total + kb0 + i) * TILE_M, &full[s]);
        tma_load_2d(stage_bhi(s), &map_xhi, (kb0 + i) * BK, 0, &full[s]);
        tma_load_2d(stage_blo(s), &map_xlo, (kb0 + i) * BK, 0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // x_hi and x_lo tiles are adjacent in a stage: one MMA over both (N = 2 BN) yields hi*hi and
      // hi*lo side by side, a second one (N = BN) adds lo*hi onto the first half. Two MMAs per k step
      // instead of three: the issue cost of these small MMAs does not depend on N.
      const uint32_t idesc = umma_idesc_tf32(TILE_M, BN), idesc2 = umma_idesc_tf32(TILE_M, 2 * BN);
      long long m_wait = 0, m_issue = 0;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % S::STAGES, ts = i % S::TSTAGES;
        long long c0 = clock64();
        if (!mbar_wait(&full[s], (i / S::STAGES) & 1, failed, a.error_flag, 12)) break;
        if (!mbar_wait(&a_ready[ts], (i / S::TSTAGES) & 1, failed, a.error_flag, 13)) break;
        long long c1 = clock64();
        m_wait += c1 - c0;
        tc_fence_after();
        long long f1 = clock64();
        const uint64_t dhi = umma_desc_sw128(stage_bhi(s));  // spans x_hi then x_lo
        const uint32_t ahi = tmem_base + S::A_COL0 + ts * 64, alo = ahi + 32;
#pragma unroll
        for (int k = 0; k < BK / 8; ++k) {
          umma_tf32_ts(tmem_base, ahi + k * 8, dhi + (uint64_t)(k * 2), idesc2, (i | k) != 0);
          umma_tf32_ts(tmem_base, alo + k * 8, dhi + (uint64_t)(k * 2), idesc, 1);
        }
        long long f2 = clock64();
        // one commit per block: it releases the shared-memory stage to the producer and, for the
        // splitters, the tensor-memory stage this block used
        umma_commit(&empty[s]);
        if (i == 5) {
          trace_add(a, 13, f1 - c1);
          trace_add(a, 14, f2 - f1);
          trace_add(a, 15, clock64() - f2);
        }
        m_issue += clock64() - c1;
      }
      umma_commit(d_full);
      trace_add(a, 11, m_wait);
      trace_add(a, 12, m_issue);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;  // row of the weight tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    long long t_wait = 0, t_ld = 0, t_st = 0;
    for (int i = 0; i < nkb && ok; ++i) {
      const int s = i % S::STAGES, ts = i % S::TSTAGES;
      long long c0 = clock64();
      ok = mbar_wait(&full[s], (i / S::STAGES) & 1, failed, a.error_flag, 14);
      if (ok && i >= S::TSTAGES) {  // block i - TSTAGES used this tensor-memory stage: wait for its MMAs
        const int ip = i - S::TSTAGES;
        ok = mbar_wait(&empty[ip % S::STAGES], (ip / S::STAGES) & 1, failed, a.error_flag, 15);
      }
      if (!ok) break;
      long long c1 = clock64();
      t_wait += c1 - c0;
      if (i == 0 && threadIdx.x == 64) trace_mark(a, 2);
      tc_fence_after();
      const float4* rowp = reinterpret_cast<const float4*>(stage_a(s) + (size_t)r * 128);
      uint32_t hi[32], lo[32];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 v = rowp[j ^ (r & 7)];  // undo the 128-byte swizzle: conflict-free per quarter warp
        const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float h = tf32_hi(f[e]);
          hi[j * 4 + e] = __float_as_uint(h);
          lo[j * 4 + e] = __float_as_uint(f[e] - h);
        }
      }
      const uint32_t col = tmem_base + S::A_COL0 + ts * 64 + lane_addr;
      long long c2 = clock64();
      t_ld += c2 - c1;
      tmem_st32(col, hi);
      tmem_st32(col + 32, lo);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&a_ready[ts]);
      t_st += clock64() - c2;
    }
    if (threadIdx.x == 64) {
      trace_add(a, 8, t_wait);
      trace_add(a, 9, t_ld);
      trace_add(a, 10, t_st);
    }
    // Split-K exchange, push model: row r of the tile is finished by CTA r / ROWS_PER of the
    // cluster, so this thread sends its partial sums of row r straight from registers into that
    // CTA's receive buffer (distributed shared memory).
    if (ok && mbar_wait(d_full, 0, failed, a.error_flag, 16)) {
      tc_fence_after();
      if (threadIdx.x == 64) trace_mark(a, 3);
      constexpr int RP = TILE_M / SPLITS;
      const uint32_t dst = dsmem_addr(smem_u32(recv), (uint32_t)(r / RP)) +
                           (uint32_t)((split * BN) * RP + (r % RP)) * 4u;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16], v2[16];
        tmem_ld16(tmem_base + lane_addr + (uint32_t)c0, v);
        tmem_ld16(tmem_base + lane_addr + (uint32_t)(BN + c0), v2);
#pragma unroll
        for (int j = 0; j < 16; ++j) st_dsmem(dst + (uint32_t)((c0 + j) * RP) * 4u, (nkb > 0) ? v[j] + v2[j] : 0.f);
      }
    }
  }
  // every thread of every CTA of the cluster passes the cluster barrier exactly once
  tc_fence_before();
  __syncthreads();
  // this CTA finishes rows [split * 128 / SPLITS, ...) of the tile: thread -> (row, token group)
  constexpr int ROWS_PER = TILE_M / SPLITS, OUTS = BN / SPLITS;
  const int t = (int)threadIdx.x - 64;
  const int rl = t >= 0 ? t % ROWS_PER : 0, tg = t >= 0 ? t / ROWS_PER : 0;
  const int row = split * ROWS_PER + rl;
  const int feat = n0 + row;
  const bool active = warp >= 2 && feat < a.n;
  float bias_v = 0.f, resid_v[OUTS];
  if (warp >= 2) pdl_wait();  // resid may come from the previous kernel; out must not be written before it ended
  if (active) {
    // loads that do not depend on the peers go out before the cluster barrier
    if (a.bias) bias_v = a.bias[feat];
#pragma unroll
    for (int o = 0; o < OUTS; ++o) {
      const int j = tg + o * SPLITS;
      resid_v[o] = (a.epilogue == EPI_RESID && j < a.m) ? a.resid[(size_t)j * a.n + feat] : 0.f;
    }
  }
  if (threadIdx.x == 64) trace_mark(a, 4);
  // release / acquire: every peer's pushes into this CTA's buffer are complete and visible after
  // the barrier, and no peer touches this CTA's shared memory after it, so the CTA may then exit
  cluster_sync_all();
  if (threadIdx.x == 64) trace_mark(a, 5);
  if (active && !*failed) {
#pragma unroll
    for (int o = 0; o < OUTS; ++o) {
      const int j = tg + o * SPLITS;
      float acc = 0.f;
#pragma unroll
      for (int sp = 0; sp < SPLITS; ++sp) acc += recv[(size_t)(sp * BN + j) * ROWS_PER + rl];  // split order
      if (j < a.m) {
        float v = a.bias ? bias_v + acc : acc;
        if (a.epilogue == EPI_GELU) v = gelu_ref(v);
        if (a.epilogue == EPI_RESID) v = resid_v[o] + v;
        if (a.out) a.out[(size_t)j * a.n + feat] = v;
        if (a.out_hi) {
          const float h = tf32_hi(v);
          a.out_hi[(size_t)j * a.n + feat] = h;
          a.out_lo[(size_t)j * a.n + feat] = v - h;
        }
      }
    }
  }
  if (threadIdx.x == 64) {
    trace_mark(a, 6);
    trace_mark(a, 7);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, S::TMEM_COLS);
}

// ------------------------------------------------------------------ host side

template <typename K>
cudaError_t launch_ex(K kernel, dim3 grid, size_t smem, cudaStream_t s, bool pdl, void** params, int cluster_y = 1) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_y > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = (unsigned)cluster_y;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(kernel), params);
}

}  // namespace

namespace {
// dst[((r / 128) * (k / 32) + c / 32) * 4096 + (r % 128) * 32 + c % 32] = src[r * k + c]; rows past n are zero
__global__ void tile_weights_kernel(const float* __restrict__ src, float* __restrict__ dst, int n, int k) {
  const int nkb = k / BK;
  const size_t total = (size_t)((n + TILE_M - 1) / TILE_M) * nkb * TILE_M * BK;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c_in = (int)(i % BK);
    const int r_in = (int)((i / BK) % TILE_M);
    const size_t tile = i / (BK * TILE_M);
    const int kb = (int)(tile % nkb);
    const int r = (int)(tile / nkb) * TILE_M + r_in;
    dst[i] = r < n ? src[(size_t)r * k + kb * BK + c_in] : 0.f;
  }
}
}  // namespace

size_t tc_tiled_weight_floats(int n, int k) { return (size_t)((n + TILE_M - 1) / TILE_M) * TILE_M * (size_t)k; }

cudaError_t launch_tile_weights(const float* src, float* dst, int n, int k, cudaStream_t s) {
  if (k % BK != 0) return cudaErrorInvalidValue;
  tile_weights_kernel<<<1184, 256, 0, s>>>(src, dst, n, k);
  return cudaGetLastError();
}

// lo[i] = x[i] - hi(x[i]) with hi = the upper 19 bits the tensor core reads
__global__ void __launch_bounds__(256) tf32_lo_kernel(const float4* __restrict__ x, float4* __restrict__ lo, size_t n4) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = x[i];
    lo[i] = make_float4(v.x - tf32_hi(v.x), v.y - tf32_hi(v.y), v.z - tf32_hi(v.z), v.w - tf32_hi(v.w));
  }
}

cudaError_t launch_tf32_lo(const float* x, float* lo, size_t n, cudaStream_t s) {
  if (n % 4 != 0) return cudaErrorInvalidValue;
  const size_t n4 = n / 4;
  const int blocks = (int)std::min<size_t>((n4 + 255) / 256, 148 * 8);
  tf32_lo_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(lo), n4);
  return cudaGetLastError();
}

static bool g_cluster16_ok = false;  // set by init_tc_kernel_attributes

bool tc_gemm_supported(int m, int n, int k) {
  (void)m;
  (void)n;
  return k % BK == 0 && k >= BK && encode_fn() != nullptr;
}

cudaError_t init_tc_kernel_attributes() {
  cudaError_t e;
  e = cudaFuncSetAttribute(tc_gemm_ss_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SsSmem<128>::BYTES);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(tc_gemm_ss_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SsSmem<256>::BYTES);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(tc_gemm_ss3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Ss3Smem::BYTES);
  if (e != cudaSuccess) return e;
#define PG_X3_ATTR(BN_, SP_)                                                                                  \
  e = cudaFuncSetAttribute(tc_gemm_x3_kernel<BN_, SP_>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                           (int)X3<BN_>::BYTES);                                                              \
  if (e != cudaSuccess) return e;
  PG_X3_ATTR(64, 1) PG_X3_ATTR(64, 2) PG_X3_ATTR(64, 4) PG_X3_ATTR(64, 8) PG_X3_ATTR(64, 16)
  // clusters of 16 CTAs are beyond the portable size of 8: opt in, and use them only if the device
  // can actually place one (a GPC with 16 free SMs)
  if (cudaFuncSetAttribute(tc_gemm_x3_kernel<64, 16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 16);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = X3<64>::BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = 16;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, tc_gemm_x3_kernel<64, 16>, &cfg) == cudaSuccess && clusters >= 8)
      g_cluster16_ok = true;
    cudaGetLastError();
  }
  PG_X3_ATTR(32, 1) PG_X3_ATTR(32, 2) PG_X3_ATTR(32, 4) PG_X3_ATTR(32, 8)
  PG_X3_ATTR(16, 1) PG_X3_ATTR(16, 2) PG_X3_ATTR(16, 4) PG_X3_ATTR(16, 8)
#undef PG_X3_ATTR
  return cudaSuccess;
}

cudaError_t launch_tc_gemm_tf32(const TcGemmArgs& a, cudaStream_t s) {
  if (!tc_gemm_supported(a.m, a.n, a.k)) return cudaErrorInvalidValue;
  CUtensorMap mx, mw;
  const int bn = (a.n >= 256 && a.m >= 2048) ? 256 : 128;
  if (!make_map(&mx, a.x, a.m, a.k, TILE_M) || !make_map(&mw, a.w, a.n, a.k, bn)) return cudaErrorInvalidValue;
  TcGemmArgs args = a;
  void* params[3] = {&mx, &mw, &args};
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const int tiles = ((a.n + bn - 1) / bn) * ((a.m + TILE_M - 1) / TILE_M);
  dim3 grid((unsigned)std::min(tiles, sms));
  if (bn == 256) return launch_ex(tc_gemm_ss_kernel<256>, grid, SsSmem<256>::BYTES, s, false, params);
  return launch_ex(tc_gemm_ss_kernel<128>, grid, SsSmem<128>::BYTES, s, false, params);
}

cudaError_t launch_tc_gemm_tf32x3_rows(const TcGemmArgs& a, cudaStream_t s) {
  if (!tc_gemm_supported(a.m, a.n, a.k) || !a.x || !a.x_lo || !a.w || !a.w_lo) return cudaErrorInvalidValue;
  CUtensorMap mx, mxl, mw, mwl;
  if (!make_map(&mx, a.x, a.m, a.k, TILE_M) || !make_map(&mxl, a.x_lo, a.m, a.k, TILE_M) ||
      !make_map(&mw, a.w, a.n, a.k, Ss3Smem::BN) || !make_map(&mwl, a.w_lo, a.n, a.k, Ss3Smem::BN))
    return cudaErrorInvalidValue;
  TcGemmArgs args = a;
  void* params[5] = {&mx, &mxl, &mw, &mwl, &args};
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const int tiles = ((a.n + Ss3Smem::BN - 1) / Ss3Smem::BN) * ((a.m + TILE_M - 1) / TILE_M);
  dim3 grid((unsigned)std::min(tiles, sms));
  return launch_ex(tc_gemm_ss3_kernel, grid, Ss3Smem::BYTES, s, false, params);
}

int tc_gemm_x3_splits(int n, int k, int num_sms) {
  const int tiles = (n + TILE_M - 1) / TILE_M;
  const int nkb = k / BK;
  int splits = 1;
  // spread small matrices over the SMs, one CTA per SM at most so that the next kernel of a
  // programmatic-launch chain finds room to prefetch its weights; keep at least 4 k-blocks
  // (64 KB of weights) per CTA; 8 is the portable cluster size, 16 is used where the device allows
  const int max_splits = g_cluster16_ok ? 16 : 8;
  while (tiles * splits * 2 <= num_sms && nkb / (splits * 2) >= 4 && splits < max_splits) splits *= 2;
  return splits;
}

cudaError_t launch_tc_gemm_x3(const TcGemmArgs& a, int splits, bool pdl, cudaStream_t s) {
  if (!tc_gemm_supported(a.m, a.n, a.k) || a.m > 64 || !a.x || !a.x_lo) return cudaErrorInvalidValue;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return cudaErrorInvalidValue;
  const int bn = a.m <= 16 ? 16 : a.m <= 32 ? 32 : 64;
  CUtensorMap mw, mhi, mlo;
  // weights in the tiled layout: a [tiles * 128, 32] matrix whose 128-row boxes are contiguous 16 KB
  const uint64_t tiled_rows = (uint64_t)((a.n + TILE_M - 1) / TILE_M) * (a.k / BK) * TILE_M;
  if (!make_map(&mw, a.w, tiled_rows, BK, TILE_M) || !make_map(&mhi, a.x, a.m, a.k, bn) ||
      !make_map(&mlo, a.x_lo, a.m, a.k, bn))
    return cudaErrorInvalidValue;
  TcGemmArgs args = a;
  void* params[4] = {&mw, &mhi, &mlo, &args};
  dim3 grid((a.n + TILE_M - 1) / TILE_M, splits);
#define PG_X3_CASE(BN_, SP_) \
  if (bn == BN_ && splits == SP_) return launch_ex(tc_gemm_x3_kernel<BN_, SP_>, grid, X3<BN_>::BYTES, s, pdl, params, splits);
  PG_X3_CASE(64, 1) PG_X3_CASE(64, 2) PG_X3_CASE(64, 4) PG_X3_CASE(64, 8) PG_X3_CASE(64, 16)
  PG_X3_CASE(32, 1) PG_X3_CASE(32, 2) PG_X3_CASE(32, 4) PG_X3_CASE(32, 8)
  PG_X3_CASE(16, 1) PG_X3_CASE(16, 2) PG_X3_CASE(16, 4) PG_X3_CASE(16, 8)
#undef PG_X3_CASE
  return cudaErrorInvalidValue;
}

}  // namespace pg
