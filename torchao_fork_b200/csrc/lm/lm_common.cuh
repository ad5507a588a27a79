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

static inline int lm_launch_status() { return cudaGetLastError() == cudaSuccess ? AO_B200_OK : AO_B200_ERR_CUDA; }
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
    for (int64_t i = lane; i < K / 8; i += 32) {
      const uint4 v = __ldg(w4 + i);
      const uint32_t r[4] = {v.x, v.y, v.z, v.w};
      const float* x = xs + i * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc = fmaf(__uint_as_float(r[j] << 16), x[2 * j], acc);
        acc = fmaf(__uint_as_float(r[j] & 0xFFFF0000u), x[2 * j + 1], acc);
      }
    }
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
template <typename T>
__host__ __device__ __forceinline__ bool rows_vectorizable(const void* base, int64_t K) {
  return (K % (16 / (int)sizeof(T)) == 0) && (reinterpret_cast<uintptr_t>(base) % 16 == 0);
}

}  // namespace lm
