// Prefill attention on the tensor cores (sm_100a), TF32 inputs with FP32 accumulation: the variant
// of causal_self_attention (src/models/gpt2/rust.rs:1580-1659) used by the single-pass TF32
// prefill mode, whose stated bound already allows 10-bit mantissas. head_dim 64.
//
// CTA = 128 queries of one (sequence, head); keys / values in tiles of 128; two CTAs per SM, so
// that the softmax of one overlaps the MMAs of the other.
//   warp 0      TMA producer: Q once, then per tile K and, once S has been computed, V of the same
//               keys into the same buffer (rows of the [rows, 3c] QKV matrix).
//   warp 1      MMA issuer: S = Q K^T (both operands in shared memory, accumulator in tensor
//               memory), then O += P V with P read from tensor memory (TS form) and V^T from
//               shared memory. tcgen05 takes TF32 operands K-major only, so V cannot be used as
//               it lies in memory: the softmax warps write a transposed, swizzled copy.
//   warps 2-5   one thread per query row: row maximum, 2^x, P (cut to TF32) stored over S in tensor
//               memory, running sum, rescaling of O only when the maximum moved by more than 2^8;
//               the same 128 threads transpose the V tile (one key each: its 64 values go to 64
//               rows of V^T, which consecutive lanes hit in consecutive words, without bank
//               conflicts).
// Every mbarrier wait is bounded; on expiry the error word is raised and all roles fall through.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace pg {
namespace {

constexpr int AT_Q = 128, AT_K = 128, AT_D = 64;
constexpr int AT_TILE_BYTES = AT_K * AT_D * 4;  // 32 KB: two boxes of [128 rows][32 floats]
// Q, one buffer that holds the K tile and then the V tile of the same keys, V^T, barriers (+ slack for
// the 1024-byte alignment). 97 KB: two CTAs per SM, so that one CTA's softmax overlaps the other's MMAs.
constexpr size_t AT_TC_SMEM = (size_t)AT_TILE_BYTES * 3 + 1024;
// P overwrites S in place (each thread rewrites its own row), O follows: 192 of 256 allocated columns.
constexpr uint32_t AT_S_COL = 0, AT_O_COL = 128, AT_TMEM_COLS = 256;

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

// Row maximum of this thread's 128 raw scores; MASK: keys after the query do not count.
template <bool MASK>
__device__ __forceinline__ float at_row_max(uint32_t s_addr, int kt, int qpos) {
  float tmax = -INFINITY;
#pragma unroll 1
  for (int c0 = 0; c0 < AT_K; c0 += 32) {
    float v[32];
    tmem_ld32(s_addr + (uint32_t)c0, v);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (!MASK || kt + c0 + j <= qpos) tmax = fmaxf(tmax, v[j]);
  }
  return tmax;
}

// P = 2^(s * sl2 - mn), cut to TF32 (the bits the MMA reads) so that the returned sum is the sum the
// MMA sees; written over S.
template <bool MASK>
__device__ __forceinline__ float at_exp_rows(uint32_t s_addr, int kt, int qpos, float sl2, float mn) {
  float ps = 0.f;
#pragma unroll 1
  for (int c0 = 0; c0 < AT_K; c0 += 32) {
    float v[32];
    uint32_t w[32];
    tmem_ld32(s_addr + (uint32_t)c0, v);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      uint32_t bits = __float_as_uint(ex2_approx(fmaf(v[j], sl2, -mn))) & 0xFFFFE000u;
      if (MASK && kt + c0 + j > qpos) bits = 0u;
      ps += __uint_as_float(bits);
      w[j] = bits;
    }
    tmem_st32(s_addr + (uint32_t)c0, w);
  }
  return ps;
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
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + AT_TILE_BYTES;                // K tile, then the V tile of the same keys
  uint8_t* vt_s = smem + 2 * (size_t)AT_TILE_BYTES;    // V^T: [4 key blocks][64 rows d][32 keys]
  __shared__ uint64_t bars[7];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed_word;
  uint64_t* q_full = &bars[0];
  uint64_t* k_full = &bars[1];
  uint64_t* v_full = &bars[2];
  uint64_t* kv_free = &bars[3];   // the V tile has been transposed: the buffer may take the next K tile
  uint64_t* s_full = &bars[4];    // S is in tensor memory; the K tile is no longer read
  uint64_t* p_ready = &bars[5];
  uint64_t* pv_done = &bars[6];
  volatile int* failed = &failed_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kend = min(len, q0 + AT_Q);
  const int ntiles = (kend + AT_K - 1) / AT_K;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(kv_free, 4);
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
      tma_load_2d(q_s, &map_qkv, h * AT_D, r0 + q0, q_full);
      tma_load_2d(q_s + AT_TILE_BYTES / 2, &map_qkv, h * AT_D + 32, r0 + q0, q_full);
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int row = r0 + i * AT_K;
        if (i > 0) ok = mbar_wait(kv_free, (i - 1) & 1, failed, error_flag, 41);
        if (!ok) break;
        mbar_expect_tx(k_full, AT_TILE_BYTES);
        tma_load_2d(kv_s, &map_qkv, c + h * AT_D, row, k_full);
        tma_load_2d(kv_s + AT_TILE_BYTES / 2, &map_qkv, c + h * AT_D + 32, row, k_full);
        ok = mbar_wait(s_full, i & 1, failed, error_flag, 40);  // the S MMAs have read K
        if (!ok) break;
        mbar_expect_tx(v_full, AT_TILE_BYTES);
        tma_load_2d(kv_s, &map_qkv, 2 * c + h * AT_D, row, v_full);
        tma_load_2d(kv_s + AT_TILE_BYTES / 2, &map_qkv, 2 * c + h * AT_D + 32, row, v_full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_tf32(128, AT_K), idesc_o = umma_idesc_tf32(128, AT_D);
      bool ok = mbar_wait(q_full, 0, failed, error_flag, 42);
      for (int i = 0; i < ntiles && ok; ++i) {
        // ---- S = Q K^T: two 32-wide blocks of the head dimension, four k steps each. S shares its
        // columns with P of the previous tile, which the MMAs issued before these have read.
        ok = mbar_wait(k_full, i & 1, failed, error_flag, 43);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t dq = umma_desc_sw128(q_s + kb * (AT_TILE_BYTES / 2));
          const uint64_t dk = umma_desc_sw128(kv_s + kb * (AT_TILE_BYTES / 2));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_tf32_ss(tmem_base + AT_S_COL, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, (kb | k) != 0);
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
    bool ok = true;
    for (int i = 0; i < ntiles; ++i) {
      const int kt = i * AT_K;
      const bool diag = kt + AT_K - 1 > q0;  // some key of the tile lies after some query: mask
      if (ok) ok = warp_wait_all(s_full, i & 1, failed, error_flag, 46);
      float tmax = 0.f;
      if (ok) {
        tc_fence_after();
        tmax = (diag ? at_row_max<true>(s_addr, kt, qpos) : at_row_max<false>(s_addr, kt, qpos)) * sl2;
        // the PV MMAs of the previous tile read P and V^T and write O: wait for them
        if (i > 0) ok = warp_wait_all(pv_done, (i - 1) & 1, failed, error_flag, 47);
      }
      if (ok) {
        tc_fence_after();
        // The maximum is only moved (and O rescaled) when some row of the warp outgrew it by 2^8;
        // until then P simply runs up to 256, harmless in FP32 accumulators. Key kt is visible to
        // every row of the tile, so the first tile sets a finite maximum.
        if (__any_sync(0xffffffffu, tmax > m + 8.0f)) {
          const float mn = fmaxf(m, tmax);
          const float corr = ex2_approx(m - mn);  // 0 on the first tile (l is 0 and O not yet written)
          l *= corr;
          m = mn;
          if (i > 0) {
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
        }
        l += diag ? at_exp_rows<true>(s_addr, kt, qpos, sl2, m) : at_exp_rows<false>(s_addr, kt, qpos, sl2, m);
        // V^T: this thread moves key r of the tile
        ok = warp_wait_all(v_full, i & 1, failed, error_flag, 48);
        if (ok) {
          float* vt = reinterpret_cast<float*>(vt_s + (r >> 5) * 8192);
          const int kc = (r & 31) >> 2, kw = r & 3;  // 16-byte chunk and word of this key inside a V^T row
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const float4* src = reinterpret_cast<const float4*>(kv_s + half * (AT_TILE_BYTES / 2) + (size_t)r * 128);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const float4 x = src[jj ^ (r & 7)];  // logical chunk jj of row r (undo the 128-byte swizzle)
              const int d = half * 32 + jj * 4;
              vt[(d + 0) * 32 + ((kc ^ ((d + 0) & 7)) << 2) + kw] = x.x;
              vt[(d + 1) * 32 + ((kc ^ ((d + 1) & 7)) << 2) + kw] = x.y;
              vt[(d + 2) * 32 + ((kc ^ ((d + 2) & 7)) << 2) + kw] = x.z;
              vt[(d + 3) * 32 + ((kc ^ ((d + 3) & 7)) << 2) + kw] = x.w;
            }
          }
        }
        tmem_wait_st();
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // V^T is read by the tensor core
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(kv_free);
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

}  // namespace

bool prefill_attention_tc_supported(const PrefillAttnArgs& a) { return a.head_dim == 64 && encode_fn() != nullptr; }

cudaError_t init_attn_tc_attributes() {
  return cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_TC_SMEM);
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

}  // namespace pg
