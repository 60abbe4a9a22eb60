// Row-wise symmetric int8 weights of the reference (QuantizedRows, src/models/cpu.rs:26-56) and the
// decode-sized projection over them (quantized_transposed_dense_projection_into + quantized_dot,
// cpu.rs:99-117, 173-184), as single operators behind the C ABI. HBM-bound integer/byte work: one
// byte per weight is streamed once, 16 bytes per lane per load, nothing is reshaped for tensor cores.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <string>

#include "common.h"
#include "kernels.cuh"

namespace pg {
int ensure_device(int device);  // model.cu

namespace {

// ------------------------------------------------------------------ QuantizedRows::from_f32
// One block per row: scale = max|w| / 127 (1 for an all-zero row; NaN does not take part in the
// maximum, as with f32::max), q = clamp(round-half-away(w / scale), -127, 127); NaN becomes 0 like
// Rust's saturating `as i8`. IEEE division and roundf: the bytes equal the reference's.
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float* __restrict__ w, int8_t* __restrict__ q,
                                                            float* __restrict__ scales, int cols) {
  __shared__ float red[8];
  const size_t r = blockIdx.x;
  const float* src = w + r * cols;
  float mx = 0.f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, fabsf(src[i]));  // fmaxf drops NaN
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  const float scale = mx == 0.f ? 1.f : __fdiv_rn(mx, 127.f);
  if (threadIdx.x == 0) scales[r] = scale;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const float t = roundf(__fdiv_rn(src[i], scale));
    // NaN first: fminf / fmaxf would replace it by the bound, f32::clamp keeps it and `as i8` makes it 0
    q[r * cols + i] = (t != t) ? (int8_t)0 : (int8_t)fminf(fmaxf(t, -127.f), 127.f);
  }
}

// w[r][i] = (q as f32) * scale[r]: the factor quantized_dot multiplies every activation by (cpu.rs:173-184)
__global__ void __launch_bounds__(256) dequantize_rows_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                                                              float* __restrict__ w, int cols) {
  const size_t r = blockIdx.x;
  const float scale = scales[r];
  for (int i = threadIdx.x; i < cols; i += blockDim.x) w[r * cols + i] = (float)q[r * cols + i] * scale;
}

// BF16 (round to nearest even; NaN stays NaN) of every value, packed, and written back as FP32
__global__ void __launch_bounds__(256) round_bf16_kernel(float* __restrict__ w, size_t n, uint16_t* __restrict__ packed) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t u = __float_as_uint(w[i]);
    uint32_t hi;
    if ((u & 0x7fffffffu) > 0x7f800000u) hi = (u >> 16) | 0x40u;  // quiet NaN
    else hi = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
    packed[i] = (uint16_t)hi;
    w[i] = __uint_as_float(hi << 16);
  }
}

// ------------------------------------------------------------------ projection, at most 8 activation rows
// int8 -> float without the quarter-rate conversion unit: with the sign bit flipped a byte is q + 128,
// placed in the mantissa of 2^23 it reads 8388608 + q + 128, and one subtraction leaves q exactly.
__device__ __forceinline__ float q8_to_float(uint32_t flipped_word, int byte) {
  const uint32_t bits = __byte_perm(flipped_word, 0x4B000000u, 0x7650u | (uint32_t)byte);
  return __uint_as_float(bits) - 8388736.0f;
}

// acc[r] += sum over the 16 weights of one load of x[r][i * 16 ..] * q
template <int MT>
__device__ __forceinline__ void q8_accumulate(const int4& pk, const float* __restrict__ x, int k, int i, int m,
                                              float (&acc)[MT]) {
  const uint32_t wd[4] = {(uint32_t)pk.x ^ 0x80808080u, (uint32_t)pk.y ^ 0x80808080u, (uint32_t)pk.z ^ 0x80808080u,
                          (uint32_t)pk.w ^ 0x80808080u};
  float wf[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) wf[j] = q8_to_float(wd[j >> 2], j & 3);
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    if (r < m) {
      const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * k + (size_t)i * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 xv = __ldg(xr + j);
        acc[r] = fmaf(xv.x, wf[4 * j + 0], acc[r]);
        acc[r] = fmaf(xv.y, wf[4 * j + 1], acc[r]);
        acc[r] = fmaf(xv.z, wf[4 * j + 2], acc[r]);
        acc[r] = fmaf(xv.w, wf[4 * j + 3], acc[r]);
      }
    }
  }
}

// One warp per output row o: out[r][o] = bias[o] + scale[o] * sum_i x[r][i] * q[o][i]. The reference
// scales every weight before the product (x * (q * scale)); taking the scale out of the sum changes
// the rounding of the partial sums only (the operator is checked at FP32 tolerance, not bit for bit).
// k is a multiple of 16: a lane reads 16 weights per load, a warp 512 contiguous bytes, and four
// loads per lane are in flight before the first is used (the activations come from L1 / L2).
template <int MT>
__global__ void __launch_bounds__(256, 4) linear_q8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                                                        const float* __restrict__ bias, const float* __restrict__ x,
                                                        float* __restrict__ out, int m, int n, int k) {
  constexpr int U = 4;
  const int lane = threadIdx.x & 31;
  const int warps = (int)(gridDim.x * blockDim.x) >> 5;
  const int k16 = k >> 4;
  for (int o = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5); o < n; o += warps) {
    const int4* wrow = reinterpret_cast<const int4*>(q + (size_t)o * k);
    float acc[MT];
#pragma unroll
    for (int r = 0; r < MT; ++r) acc[r] = 0.f;
    for (int i0 = lane; i0 < k16; i0 += 32 * U) {
      int4 pk[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + 32 * u < k16) pk[u] = __ldcs(wrow + i0 + 32 * u);  // streamed once: not kept in L1 / L2
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + 32 * u < k16) q8_accumulate<MT>(pk[u], x, k, i0 + 32 * u, m, acc);
    }
#pragma unroll
    for (int r = 0; r < MT; ++r) {
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], s);
    }
    if (lane == 0) {
      const float scale = scales[o], b = bias ? bias[o] : 0.f;
#pragma unroll
      for (int r = 0; r < MT; ++r)
        if (r < m) out[(size_t)r * n + o] = b + acc[r] * scale;
    }
  }
}

// The same projection with the activations held in shared memory (the default; the kernel above is
// the fallback when [MT][k] floats do not fit): read from L1 they cost 4 x MT 16-byte loads per lane
// for every 16 weights and bound the kernel. One block of
// 32 warps per SM stages x once ([MT][k] floats, at most 227 KB) and then walks its rows. Lane i reads
// the four 16-byte units 4 i .. 4 i + 3 of a row; unit (i, j) is stored at 4 i + (j ^ ((i >> 1) & 3)),
// so that the eight lanes of a quarter warp hit eight different bank groups.
template <int MT>
__global__ void __launch_bounds__(1024, 1) linear_q8_smem_kernel(const int8_t* __restrict__ q,
                                                                 const float* __restrict__ scales,
                                                                 const float* __restrict__ bias,
                                                                 const float* __restrict__ x, float* __restrict__ out,
                                                                 int m, int n, int k) {
  extern __shared__ float4 xs[];
  constexpr int U = 2;  // loads in flight per lane and row
  const int lane = threadIdx.x & 31;
  const int k4 = k >> 2, k16 = k >> 4;
  for (int idx = threadIdx.x; idx < MT * k4; idx += blockDim.x) {
    const int r = idx / k4, u = idx - r * k4;
    const int i = u >> 2, j = u & 3;
    const float4 v = r < m ? __ldg(reinterpret_cast<const float4*>(x) + (size_t)r * k4 + u) : make_float4(0.f, 0.f, 0.f, 0.f);
    xs[r * k4 + 4 * i + (j ^ ((i >> 1) & 3))] = v;
  }
  __syncthreads();
  // A warp walks two neighbouring output rows at a time: every activation read from shared memory
  // then serves eight weights instead of four.
  constexpr int R = 2;
  const int warps = (int)(gridDim.x * blockDim.x) >> 5;
  for (int o = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * R; o < n; o += warps * R) {
    const int4* wrow = reinterpret_cast<const int4*>(q + (size_t)o * k);
    const bool two = o + 1 < n;
    float acc[R][MT];
#pragma unroll
    for (int rr = 0; rr < R; ++rr)
#pragma unroll
      for (int r = 0; r < MT; ++r) acc[rr][r] = 0.f;
    for (int i0 = lane; i0 < k16; i0 += 32 * U) {
      int4 pk[R][U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + 32 * u;
        if (i < k16) {
          pk[0][u] = __ldcs(wrow + i);
          pk[1][u] = two ? __ldcs(wrow + k16 + i) : make_int4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + 32 * u;
        if (i < k16) {
          const int sw = (i >> 1) & 3;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float w[R][4];
#pragma unroll
            for (int rr = 0; rr < R; ++rr) {
              const int word = j == 0 ? pk[rr][u].x : j == 1 ? pk[rr][u].y : j == 2 ? pk[rr][u].z : pk[rr][u].w;
              const uint32_t wd = (uint32_t)word ^ 0x80808080u;
#pragma unroll
              for (int e = 0; e < 4; ++e) w[rr][e] = q8_to_float(wd, e);
            }
#pragma unroll
            for (int r = 0; r < MT; ++r) {
              const float4 xv = xs[r * k4 + 4 * i + (j ^ sw)];
#pragma unroll
              for (int rr = 0; rr < R; ++rr) {
                acc[rr][r] = fmaf(xv.x, w[rr][0], acc[rr][r]);
                acc[rr][r] = fmaf(xv.y, w[rr][1], acc[rr][r]);
                acc[rr][r] = fmaf(xv.z, w[rr][2], acc[rr][r]);
                acc[rr][r] = fmaf(xv.w, w[rr][3], acc[rr][r]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int rr = 0; rr < R; ++rr)
#pragma unroll
      for (int r = 0; r < MT; ++r) {
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc[rr][r] += __shfl_xor_sync(0xffffffffu, acc[rr][r], s);
      }
    if (lane == 0) {
#pragma unroll
      for (int rr = 0; rr < R; ++rr) {
        if (o + rr < n) {
          const float scale = scales[o + rr], b = bias ? bias[o + rr] : 0.f;
#pragma unroll
          for (int r = 0; r < MT; ++r)
            if (r < m) out[(size_t)r * n + o + rr] = b + acc[rr][r] * scale;
        }
      }
    }
  }
}

constexpr size_t Q8_MAX_SMEM = 227 * 1024;

template <int MT>
cudaError_t launch_q8_smem(const int8_t* q, const float* scales, const float* bias, const float* x, float* out, int m,
                           int n, int k, int sms, cudaStream_t s) {
  const size_t smem = (size_t)MT * k * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(linear_q8_smem_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int blocks = std::max(1, std::min((n + 63) / 64, sms));  // 32 warps of two rows each
  linear_q8_smem_kernel<MT><<<blocks, 1024, smem, s>>>(q, scales, bias, x, out, m, n, k);
  return cudaGetLastError();
}

cudaError_t launch_linear_q8(const int8_t* q, const float* scales, const float* bias, const float* x, float* out, int m,
                             int n, int k, int sms, cudaStream_t s) {
  const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8;
  if ((size_t)mt * k * sizeof(float) <= Q8_MAX_SMEM) {
    if (mt == 1) return launch_q8_smem<1>(q, scales, bias, x, out, m, n, k, sms, s);
    if (mt == 2) return launch_q8_smem<2>(q, scales, bias, x, out, m, n, k, sms, s);
    if (mt == 4) return launch_q8_smem<4>(q, scales, bias, x, out, m, n, k, sms, s);
    return launch_q8_smem<8>(q, scales, bias, x, out, m, n, k, sms, s);
  }
  const int blocks = std::max(1, std::min((n + 7) / 8, sms * 4));  // four resident blocks per SM: one wave
  if (mt == 1) linear_q8_kernel<1><<<blocks, 256, 0, s>>>(q, scales, bias, x, out, m, n, k);
  else if (mt == 2) linear_q8_kernel<2><<<blocks, 256, 0, s>>>(q, scales, bias, x, out, m, n, k);
  else if (mt == 4) linear_q8_kernel<4><<<blocks, 256, 0, s>>>(q, scales, bias, x, out, m, n, k);
  else linear_q8_kernel<8><<<blocks, 256, 0, s>>>(q, scales, bias, x, out, m, n, k);
  return cudaGetLastError();
}

struct Buf {
  void* p = nullptr;
  ~Buf() {
    if (p) cudaFree(p);
  }
};
constexpr size_t Q8_FLUSH_BYTES = 256u << 20;  // larger than the 126 MB L2

}  // namespace

cudaError_t launch_quantize_rows(const float* w, int rows, int cols, int8_t* q, float* scales, cudaStream_t s) {
  quantize_rows_kernel<<<rows, 256, 0, s>>>(w, q, scales, cols);
  return cudaGetLastError();
}
cudaError_t launch_dequantize_rows(const int8_t* q, const float* scales, int rows, int cols, float* w, cudaStream_t s) {
  dequantize_rows_kernel<<<rows, 256, 0, s>>>(q, scales, w, cols);
  return cudaGetLastError();
}
cudaError_t launch_round_bf16(float* w, size_t n, uint16_t* packed, cudaStream_t s) {
  const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 16);
  round_bf16_kernel<<<blocks, 256, 0, s>>>(w, n, packed);
  return cudaGetLastError();
}

}  // namespace pg

using namespace pg;

#define PG_Q_TRY(expr)                                                                                \
  do {                                                                                                \
    cudaError_t _e = (expr);                                                                          \
    if (_e != cudaSuccess) {                                                                          \
      rc = set_error(PG_CUDA, std::string("CUDA error: ") + cudaGetErrorString(_e) + " (" #expr ")"); \
      goto done;                                                                                      \
    }                                                                                                 \
  } while (0)

extern "C" int pg_op_quantize_rows(const float* w, int32_t rows, int32_t cols, int32_t device, int8_t* q_out,
                                   float* scales_out) {
  if (!w || !q_out || !scales_out) return set_error(PG_INVALID_INPUT, "null argument");
  if (rows <= 0 || cols <= 0) return set_error(PG_INVALID_INPUT, "rows and cols must be > 0");
  if (int r = ensure_device(device)) return r;
  int rc = PG_OK;
  const size_t total = (size_t)rows * cols;
  Buf dw, dq, ds;
  PG_Q_TRY(cudaMalloc(&dw.p, total * sizeof(float)));
  PG_Q_TRY(cudaMalloc(&dq.p, total));
  PG_Q_TRY(cudaMalloc(&ds.p, (size_t)rows * sizeof(float)));
  PG_Q_TRY(cudaMemcpy(dw.p, w, total * sizeof(float), cudaMemcpyHostToDevice));
  quantize_rows_kernel<<<rows, 256>>>(static_cast<const float*>(dw.p), static_cast<int8_t*>(dq.p),
                                      static_cast<float*>(ds.p), cols);
  PG_Q_TRY(cudaGetLastError());
  PG_Q_TRY(cudaMemcpy(q_out, dq.p, total, cudaMemcpyDeviceToHost));
  PG_Q_TRY(cudaMemcpy(scales_out, ds.p, (size_t)rows * sizeof(float), cudaMemcpyDeviceToHost));
done:
  return rc;
}

extern "C" int pg_op_linear_q8(const float* x, const int8_t* q, const float* scales, const float* bias, int32_t m,
                               int32_t n, int32_t k, int32_t device, int32_t reps, float* out,
                               double* seconds_per_launch) {
  if (!x || !q || !scales || !out) return set_error(PG_INVALID_INPUT, "null argument");
  if (m <= 0 || n <= 0 || k <= 0) return set_error(PG_INVALID_INPUT, "m, n, k must be > 0");
  if (m > 8) return set_error(PG_INVALID_INPUT, "the int8 projection is the decode path: m <= 8");
  if (k % 16 != 0) return set_error(PG_INVALID_INPUT, "the int8 projection needs k to be a multiple of 16");
  if (int r = ensure_device(device)) return r;
  int rc = PG_OK;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  Buf dx, dq, ds, db, dout, dflush;
  cudaStream_t s = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  PG_Q_TRY(cudaStreamCreate(&s));
  PG_Q_TRY(cudaMalloc(&dx.p, (size_t)m * k * sizeof(float)));
  PG_Q_TRY(cudaMalloc(&dq.p, (size_t)n * k));
  PG_Q_TRY(cudaMalloc(&ds.p, (size_t)n * sizeof(float)));
  PG_Q_TRY(cudaMalloc(&dout.p, (size_t)m * n * sizeof(float)));
  PG_Q_TRY(cudaMemcpyAsync(dx.p, x, (size_t)m * k * sizeof(float), cudaMemcpyHostToDevice, s));
  PG_Q_TRY(cudaMemcpyAsync(dq.p, q, (size_t)n * k, cudaMemcpyHostToDevice, s));
  PG_Q_TRY(cudaMemcpyAsync(ds.p, scales, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, s));
  if (bias) {
    PG_Q_TRY(cudaMalloc(&db.p, (size_t)n * sizeof(float)));
    PG_Q_TRY(cudaMemcpyAsync(db.p, bias, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, s));
  }
#define PG_Q_LAUNCH                                                                                               \
  launch_linear_q8(static_cast<const int8_t*>(dq.p), static_cast<const float*>(ds.p), static_cast<const float*>(db.p), \
                   static_cast<const float*>(dx.p), static_cast<float*>(dout.p), m, n, k, sms, s)
  PG_Q_TRY(PG_Q_LAUNCH);
  PG_Q_TRY(cudaMemcpyAsync(out, dout.p, (size_t)m * n * sizeof(float), cudaMemcpyDeviceToHost, s));
  PG_Q_TRY(cudaStreamSynchronize(s));
  if (reps > 0 && seconds_per_launch) {
    PG_Q_TRY(cudaMalloc(&dflush.p, Q8_FLUSH_BYTES));
    PG_Q_TRY(cudaEventCreate(&e0));
    PG_Q_TRY(cudaEventCreate(&e1));
    double total = 0.0;
    for (int i = 0; i < reps + 3; ++i) {
      PG_Q_TRY(cudaMemsetAsync(dflush.p, i, Q8_FLUSH_BYTES, s));
      PG_Q_TRY(cudaEventRecord(e0, s));
      PG_Q_TRY(PG_Q_LAUNCH);
      PG_Q_TRY(cudaEventRecord(e1, s));
      PG_Q_TRY(cudaEventSynchronize(e1));
      float ms = 0.f;
      PG_Q_TRY(cudaEventElapsedTime(&ms, e0, e1));
      if (i >= 3) total += ms * 1e-3;
    }
    *seconds_per_launch = total / reps;
  }
#undef PG_Q_LAUNCH
done:
  if (s) cudaStreamSynchronize(s);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (s) cudaStreamDestroy(s);
  return rc;
}
