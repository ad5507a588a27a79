// Shared helpers of libao_b200_lm (sm_100a): storage-type dispatch, fp32 loads / stores, block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../../include/ao_b200_lm.h"

#define LM_CHECK_ARG(cond)                        \
  do {                                            \
    if (!(cond)) return AO_B200_ERR_INVALID_ARG;  \
  } while (0)

// runs `...` with T = the storage type that `dt` names
#define LM_DISPATCH(dt, ...)              \
  do {                                    \
    if ((dt) == AO_LM_BF16) {             \
      using T = __nv_bfloat16;            \
      __VA_ARGS__;                        \
    } else if ((dt) == AO_LM_F32) {       \
      using T = float;                    \
      __VA_ARGS__;                        \
    } else {                              \
      return AO_B200_ERR_INVALID_ARG;     \
    }                                     \
  } while (0)

// the CUDA error behind the last AO_B200_ERR_CUDA that this library returned (0 = none); ao_lm_last_cuda_error reads it
extern int g_lm_last_cuda_error;
static inline int lm_launch_status() {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return AO_B200_OK;
  g_lm_last_cuda_error = (int)e;
  return AO_B200_ERR_CUDA;
}
static inline cudaStream_t lm_stream(void* s) { return static_cast<cudaStream_t>(s); }

namespace lm {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// sum over the block (any multiple of 32 threads up to 1024); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats of shared memory */) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();                        // scratch may still be read from an earlier call
  if (lane == 0) scratch[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// sum_k w[k] * xs[k] over one warp; w in global memory (row of K elements), xs fp32 in shared memory.
// 16-byte loads when the row allows it (K a multiple of the vector length keeps every row aligned).
__device__ __forceinline__ float warp_dot(const __nv_bfloat16* w, const float* xs, int64_t K, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {
    const uint4* w4 = reinterpret_cast<const uint4*>(w);
    const int64_t nv = K / 8;
    auto use = [&](const uint4& v, int64_t i) {
      const uint32_t r[4] = {v.x, v.y, v.z, v.w};
      const float* x = xs + i * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc = fmaf(__uint_as_float(r[j] << 16), x[2 * j], acc);
        acc = fmaf(__uint_as_float(r[j] & 0xFFFF0000u), x[2 * j + 1], acc);
      }
    };
    int64_t i = lane;
    for (; i + 96 < nv; i += 128) {   // four 16-byte loads of the row in flight per lane before the first is used
      const uint4 v0 = __ldg(w4 + i), v1 = __ldg(w4 + i + 32), v2 = __ldg(w4 + i + 64), v3 = __ldg(w4 + i + 96);
      use(v0, i);
      use(v1, i + 32);
      use(v2, i + 64);
      use(v3, i + 96);
    }
    for (; i < nv; i += 32) use(__ldg(w4 + i), i);
  } else {
    for (int64_t i = lane; i < K; i += 32) acc = fmaf(__bfloat162float(w[i]), xs[i], acc);
  }
  return warp_sum(acc);
}
__device__ __forceinline__ float warp_dot(const float* w, const float* xs, int64_t K, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (int64_t i = lane; i < K / 4; i += 32) {
      const float4 v = __ldg(w4 + i);
      const float* x = xs + i * 4;
      acc = fmaf(v.x, x[0], acc);
      acc = fmaf(v.y, x[1], acc);
      acc = fmaf(v.z, x[2], acc);
      acc = fmaf(v.w, x[3], acc);
    }
  } else {
    for (int64_t i = lane; i < K; i += 32) acc = fmaf(w[i], xs[i], acc);
  }
  return warp_sum(acc);
}
// NR dot products of one warp at once: out[r] = sum_k rows[r][k] * xs[r][k] for r < nr (<= NR), bf16 rows of K elements
// (K a multiple of 8, rows 16-byte aligned).  The loads of all rows, U vectors each, are issued before any is used: a
// matrix-vector kernel is a chain of DRAM round trips per warp, and this makes the chain NR * U times shorter.
template <int NR, int U>
__device__ __forceinline__ void warp_dot_rows(const __nv_bfloat16* const (&rows)[NR], const float* const (&xs)[NR], int nr,
                                              int64_t K, int lane, float (&out)[NR]) {
  const int64_t nv = K / 8;
  float acc[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) acc[r] = 0.f;
  for (int64_t i0 = lane; i0 < nv; i0 += 32 * U) {
    uint4 v[NR][U];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + 32 * u;
        v[r][u] = make_uint4(0, 0, 0, 0);
        if (r < nr && i < nv) v[r][u] = __ldg(reinterpret_cast<const uint4*>(rows[r]) + i);
      }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + 32 * u;
        if (r < nr && i < nv) {
          const uint32_t w[4] = {v[r][u].x, v[r][u].y, v[r][u].z, v[r][u].w};
          const float* x = xs[r] + i * 8;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[r] = fmaf(__uint_as_float(w[j] << 16), x[2 * j], acc[r]);
            acc[r] = fmaf(__uint_as_float(w[j] & 0xFFFF0000u), x[2 * j + 1], acc[r]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) out[r] = warp_sum(acc[r]);
}

// 16 bytes of storage type -> fp32
__device__ __forceinline__ void unpack16(const uint4& u, float* dst, const __nv_bfloat16*) {
  const uint32_t r[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dst[2 * i] = __uint_as_float(r[i] << 16);
    dst[2 * i + 1] = __uint_as_float(r[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void unpack16(const uint4& u, float* dst, const float*) {
  dst[0] = __uint_as_float(u.x), dst[1] = __uint_as_float(u.y), dst[2] = __uint_as_float(u.z), dst[3] = __uint_as_float(u.w);
}
// dst[0..count) (fp32, shared memory) = src[0..count) by the whole block: 16-byte loads, four in flight per thread, when
// the source is aligned; a matrix-vector kernel's activation row must not arrive one dependent load at a time
template <typename T>
__device__ __forceinline__ void stage_f32(const T* __restrict__ src, float* dst, int64_t count) {
  constexpr int kPer = 16 / (int)sizeof(T);
  int64_t done = 0;
  if (reinterpret_cast<uintptr_t>(src) % 16 == 0) {
    const int64_t nv = count / kPer, step = blockDim.x;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    int64_t i = threadIdx.x;
    for (; i + 3 * step < nv; i += 4 * step) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __ldg(s4 + i + j * step);
#pragma unroll
      for (int j = 0; j < 4; ++j) unpack16(v[j], dst + (i + j * step) * kPer, src);
    }
    for (; i < nv; i += step) unpack16(__ldg(s4 + i), dst + i * kPer, src);
    done = nv * kPer;
  }
  for (int64_t i = done + threadIdx.x; i < count; i += blockDim.x) dst[i] = ldf(src + i);
}

template <typename T>
__host__ __device__ __forceinline__ bool rows_vectorizable(const void* base, int64_t K) {
  return (K % (16 / (int)sizeof(T)) == 0) && (reinterpret_cast<uintptr_t>(base) % 16 == 0);
}

}  // namespace lm
