// Row-wise kernels of a residual that is kept as several fp32 streams per token (hyper-connections; one stream is the
// ordinary residual): embedding gather with a scale and sinusoidal positions, read-out of the streams into a
// per-coordinate-weighted RMS norm, write-back of a sublayer's result through a mixing matrix, and the tanh-GELU gated
// product of a dense feed-forward.  One CTA per token row; everything is computed in fp32.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kMaxStreams = 8;
constexpr int kMaxTaps = 8;

inline unsigned row_threads(int64_t rows, int64_t width) {
  unsigned t = 256;
  if (rows >= 128) return t;
  while (t < 1024 && (int64_t)t * 4 < width) t *= 2;
  return t;
}

template <typename T>
__global__ void __launch_bounds__(1024) embed_sinusoid_kernel(const T* __restrict__ table, const int64_t* __restrict__ tok,
                                      const int32_t* __restrict__ pos, int64_t W, float scale,
                                      const double* __restrict__ freq, int S, float* __restrict__ x) {
  const int64_t t = blockIdx.x;
  const T* row = table + tok[t] * W;
  const double p = (double)pos[t];
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    // the angle in double, reduced to [-pi, pi] before the fp32 sine: positions in the thousands keep all their bits
    const double a = p * freq[w >> 1];
    const double k = rint(a * 0.15915494309189535);
    const float r = (float)fma(-k, 6.283185307179586, a);
    const float v = fmaf(ldf(row + w), scale, (w & 1) ? cosf(r) : sinf(r));
    for (int s = 0; s < S; ++s) x[(t * S + s) * W + w] = v;
  }
}

// u = sum_s cin[s] x_s (cin == null: every coefficient 1);  out = u / sqrt(mean(u^2) + eps) * (offset + weight)
template <typename T>
__global__ void __launch_bounds__(1024) streams_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, int S, int64_t W,
                                    const T* __restrict__ cin, const T* __restrict__ weight, float offset, float eps,
                                    float* __restrict__ out_f32, T* __restrict__ out) {
  extern __shared__ float u[];          // [W]
  __shared__ float scratch[33];
  const int64_t i = blockIdx.x;
  const float* xr = x + (rows ? (int64_t)rows[i] : i) * S * W;
  float c[kMaxStreams];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) c[s] = s < S ? (cin ? ldf(cin + s) : 1.f) : 0.f;
  float ss = 0.f;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    float a = c[0] * xr[w];
#pragma unroll
    for (int s = 1; s < kMaxStreams; ++s)
      if (s < S) a = fmaf(c[s], xr[s * W + w], a);
    u[w] = a;
    ss = fmaf(a, a, ss);
  }
  ss = block_sum(ss, scratch);
  const float k = 1.f / sqrtf(ss / (float)W + eps);
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    const float v = u[w] * k * (offset + ldf(weight + w));
    if (out_f32) out_f32[i * W + w] = v;
    if (out) stf(out + i * W + w, v);
  }
}

// x_t <- sum_s mix[s][t] x_s + cout[t] * y, all streams from the old ones (mix == null: identity, cout == null: ones).
// The last row of every sequence in the step (ahead == 0) also shifts the rows of conv_in into the sequence's
// convolution memory: state[slot][k] = input at position p - (taps - 2 - k).
template <typename T, typename TY>
__global__ void __launch_bounds__(1024) streams_update_kernel(float* __restrict__ x, const TY* __restrict__ y, int S, int64_t W,
                                      const T* __restrict__ mix, const T* __restrict__ cout, const float* __restrict__ conv_in,
                                      float* __restrict__ conv_state, int taps, const int32_t* __restrict__ slot,
                                      const int32_t* __restrict__ back, const int32_t* __restrict__ ahead) {
  __shared__ float m[kMaxStreams * kMaxStreams], co[kMaxStreams];
  const int64_t t = blockIdx.x;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) m[i] = mix ? ldf(mix + i) : ((i / S) == (i % S) ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) co[i] = cout ? ldf(cout + i) : 1.f;
  __syncthreads();
  float* xr = x + t * S * W;
  const TY* yr = y + t * W;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    float xs[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) xs[s] = s < S ? xr[s * W + w] : 0.f;
    const float yv = ldf(yr + w);
#pragma unroll
    for (int d = 0; d < kMaxStreams; ++d) {
      if (d < S) {
        float a = co[d] * yv;
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < S) a = fmaf(m[s * S + d], xs[s], a);
        xr[d * W + w] = a;
      }
    }
  }
  if (conv_state && ahead[t] == 0) {
    const int b = back[t];
    float* st = conv_state + (int64_t)slot[t] * (taps - 1) * W;
    for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
      float v[kMaxTaps];
#pragma unroll
      for (int k = 0; k < kMaxTaps - 1; ++k) {
        if (k < taps - 1) {
          const int delta = taps - 2 - k;
          v[k] = delta <= b ? conv_in[(t - delta) * W + w] : st[(int64_t)(b - delta + taps - 1) * W + w];
        }
      }
#pragma unroll
      for (int k = 0; k < kMaxTaps - 1; ++k)
        if (k < taps - 1) st[(int64_t)k * W + w] = v[k];
    }
  }
}


// ---- the same two kernels for widths that are multiples of 4: 16-byte loads and stores, the stream count a
// compile-time constant (no predicated loops)
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xFFFF0000u));
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float4& v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename T, int S>
__global__ void __launch_bounds__(512) streams_norm_vec_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                                                int64_t W, const T* __restrict__ cin, const T* __restrict__ weight,
                                                                float offset, float eps, float* __restrict__ out_f32,
                                                                T* __restrict__ out) {
  extern __shared__ __align__(16) float u[];   // [W]
  __shared__ float scratch[33];
  const int64_t i = blockIdx.x;
  const float* xr = x + (rows ? (int64_t)rows[i] : i) * S * W;
  float c[S];
#pragma unroll
  for (int s = 0; s < S; ++s) c[s] = cin ? ldf(cin + s) : 1.f;
  float ss = 0.f;
  for (int64_t w = (int64_t)threadIdx.x * 4; w < W; w += (int64_t)blockDim.x * 4) {
    float4 v[S];
#pragma unroll
    for (int s = 0; s < S; ++s) v[s] = ld4(xr + s * W + w);
    float4 a = make_float4(c[0] * v[0].x, c[0] * v[0].y, c[0] * v[0].z, c[0] * v[0].w);
#pragma unroll
    for (int s = 1; s < S; ++s) {
      a.x = fmaf(c[s], v[s].x, a.x), a.y = fmaf(c[s], v[s].y, a.y), a.z = fmaf(c[s], v[s].z, a.z), a.w = fmaf(c[s], v[s].w, a.w);
    }
    st4(u + w, a);
    ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss))));
  }
  ss = block_sum(ss, scratch);
  const float k = 1.f / sqrtf(ss / (float)W + eps);
  for (int64_t w = (int64_t)threadIdx.x * 4; w < W; w += (int64_t)blockDim.x * 4) {
    const float4 a = ld4(u + w), g = ld4(weight + w);
    const float4 v = make_float4(a.x * k * (offset + g.x), a.y * k * (offset + g.y), a.z * k * (offset + g.z), a.w * k * (offset + g.w));
    if (out_f32) st4(out_f32 + i * W + w, v);
    if (out) st4(out + i * W + w, v);
  }
}

template <typename T, typename TY, int S>
__global__ void __launch_bounds__(512) streams_update_vec_kernel(float* __restrict__ x, const TY* __restrict__ y, int64_t W,
                                                                  const T* __restrict__ mix, const T* __restrict__ cout) {
  float m[S][S], co[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    co[s] = cout ? ldf(cout + s) : 1.f;
#pragma unroll
    for (int d = 0; d < S; ++d) m[s][d] = mix ? ldf(mix + s * S + d) : (s == d ? 1.f : 0.f);
  }
  const int64_t t = blockIdx.x;
  float* xr = x + t * S * W;
  const TY* yr = y + t * W;
  for (int64_t w = (int64_t)threadIdx.x * 4; w < W; w += (int64_t)blockDim.x * 4) {
    float4 v[S];
#pragma unroll
    for (int s = 0; s < S; ++s) v[s] = ld4(xr + s * W + w);
    const float4 yv = ld4(yr + w);
#pragma unroll
    for (int d = 0; d < S; ++d) {
      float4 a = make_float4(co[d] * yv.x, co[d] * yv.y, co[d] * yv.z, co[d] * yv.w);
#pragma unroll
      for (int s = 0; s < S; ++s) {
        a.x = fmaf(m[s][d], v[s].x, a.x), a.y = fmaf(m[s][d], v[s].y, a.y), a.z = fmaf(m[s][d], v[s].z, a.z),
        a.w = fmaf(m[s][d], v[s].w, a.w);
      }
      st4(xr + d * W + w, a);
    }
  }
}

// the convolution memory alone (what streams_update_kernel does for rows with ahead == 0), for the vector path
__global__ void conv_memory_kernel(const float* __restrict__ conv_in, float* __restrict__ conv_state, int64_t W, int taps,
                                   const int32_t* __restrict__ slot, const int32_t* __restrict__ back,
                                   const int32_t* __restrict__ ahead) {
  const int64_t t = blockIdx.x;
  if (ahead[t] != 0) return;
  const int b = back[t];
  float* st = conv_state + (int64_t)slot[t] * (taps - 1) * W;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    float v[kMaxTaps];
#pragma unroll
    for (int k = 0; k < kMaxTaps - 1; ++k) {
      if (k < taps - 1) {
        const int delta = taps - 2 - k;
        v[k] = delta <= b ? conv_in[(t - delta) * W + w] : st[(int64_t)(b - delta + taps - 1) * W + w];
      }
    }
#pragma unroll
    for (int k = 0; k < kMaxTaps - 1; ++k)
      if (k < taps - 1) st[(int64_t)k * W + w] = v[k];
  }
}

inline unsigned vec_threads(int64_t rows, int64_t width) {
  unsigned t = 128;
  const unsigned cap = rows >= 128 ? 256 : 512;
  while (t < cap && (int64_t)t * 4 < width) t *= 2;
  return t;
}

#define LM_STREAMS_SWITCH(S_, ...)          \
  switch (S_) {                             \
    case 1: { constexpr int S = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int S = 2; __VA_ARGS__; } break; \
    case 3: { constexpr int S = 3; __VA_ARGS__; } break; \
    case 4: { constexpr int S = 4; __VA_ARGS__; } break; \
    case 5: { constexpr int S = 5; __VA_ARGS__; } break; \
    case 6: { constexpr int S = 6; __VA_ARGS__; } break; \
    case 7: { constexpr int S = 7; __VA_ARGS__; } break; \
    default: { constexpr int S = 8; __VA_ARGS__; } break; \
  }

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void gelu_glu_kernel(const T* __restrict__ gu, int64_t n, int64_t ff, T* __restrict__ y) {
  const int64_t total = n * ff;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / ff, c = i - t * ff;
    stf(y + i, gelu_tanh(ldf(gu + t * 2 * ff + c)) * ldf(gu + t * 2 * ff + ff + c));
  }
}

}  // namespace

extern "C" int ao_lm_embed_sinusoid(const void* table, int dt, const int64_t* tok, const int32_t* pos, int64_t n,
                                    int64_t width, float scale, const double* freq, int n_streams, float* x, void* stream) {
  LM_CHECK_ARG(table && tok && pos && freq && x && n > 0 && width > 0 && n_streams >= 1);
  LM_DISPATCH(dt, embed_sinusoid_kernel<T><<<(unsigned)n, row_threads(n, width), 0, lm_stream(stream)>>>(
                      static_cast<const T*>(table), tok, pos, width, scale, freq, n_streams, x));
  return lm_launch_status();
}

extern "C" int ao_lm_streams_norm(const float* x, const int32_t* rows, int64_t m, int n_streams, int64_t width,
                                  const void* coef_in, const void* weight, int dt, float weight_offset, float eps,
                                  float* out_f32, void* out, void* stream) {
  LM_CHECK_ARG(x && weight && (out_f32 || out) && m > 0 && width > 0 && n_streams >= 1 && n_streams <= kMaxStreams);
  LM_CHECK_ARG(width * 4 <= 160 * 1024);
  const size_t smem = (size_t)width * 4;
  const bool vec = width % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(weight) % 8 == 0 &&
                   reinterpret_cast<uintptr_t>(out_f32) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0 && smem <= 40 * 1024;
  if (vec) {
    LM_DISPATCH(dt, LM_STREAMS_SWITCH(n_streams, streams_norm_vec_kernel<T, S><<<(unsigned)m, vec_threads(m, width), smem, lm_stream(stream)>>>(
                        x, rows, width, static_cast<const T*>(coef_in), static_cast<const T*>(weight), weight_offset, eps, out_f32,
                        static_cast<T*>(out))));
    return lm_launch_status();
  }
  LM_DISPATCH(dt, {
    auto kern = streams_norm_kernel<T>;
    if (smem > 40 * 1024) {
      static bool set = false;
      if (!set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
        set = true;
      }
    }
    kern<<<(unsigned)m, row_threads(m, width), smem, lm_stream(stream)>>>(
        x, rows, n_streams, width, static_cast<const T*>(coef_in), static_cast<const T*>(weight), weight_offset, eps, out_f32,
        static_cast<T*>(out));
  });
  return lm_launch_status();
}

extern "C" int ao_lm_streams_update(float* x, const void* y, int y_dt, int64_t n, int n_streams, int64_t width,
                                    const void* mix, const void* coef_out, int dt, const float* conv_in, float* conv_state,
                                    int taps, const int32_t* slot, const int32_t* back, const int32_t* ahead, void* stream) {
  LM_CHECK_ARG(x && y && n > 0 && width > 0 && n_streams >= 1 && n_streams <= kMaxStreams);
  LM_CHECK_ARG(!conv_state || (conv_in && slot && back && ahead && taps >= 2 && taps <= kMaxTaps));
  const cudaStream_t st = lm_stream(stream);
  const unsigned th = row_threads(n, width);
  if (width % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0 &&
      (y_dt == AO_LM_F32 || dt == AO_LM_BF16)) {
    const unsigned vt = vec_threads(n, width);
    if (y_dt == AO_LM_F32) {
      LM_DISPATCH(dt, LM_STREAMS_SWITCH(n_streams, streams_update_vec_kernel<T, float, S><<<(unsigned)n, vt, 0, st>>>(
                          x, static_cast<const float*>(y), width, static_cast<const T*>(mix), static_cast<const T*>(coef_out))));
    } else {
      using T = __nv_bfloat16;
      LM_STREAMS_SWITCH(n_streams, streams_update_vec_kernel<T, T, S><<<(unsigned)n, vt, 0, st>>>(
                            x, static_cast<const T*>(y), width, static_cast<const T*>(mix), static_cast<const T*>(coef_out)));
    }
    if (conv_state) conv_memory_kernel<<<(unsigned)n, 256, 0, st>>>(conv_in, conv_state, width, taps, slot, back, ahead);
    return lm_launch_status();
  }
  if (y_dt == AO_LM_F32) {
    LM_DISPATCH(dt, streams_update_kernel<T, float><<<(unsigned)n, th, 0, st>>>(
                        x, static_cast<const float*>(y), n_streams, width, static_cast<const T*>(mix),
                        static_cast<const T*>(coef_out), conv_in, conv_state, taps, slot, back, ahead));
  } else {
    LM_CHECK_ARG(y_dt == AO_LM_BF16 && dt == AO_LM_BF16);
    using T = __nv_bfloat16;
    streams_update_kernel<T, T><<<(unsigned)n, th, 0, st>>>(x, static_cast<const T*>(y), n_streams, width,
                                                            static_cast<const T*>(mix), static_cast<const T*>(coef_out),
                                                            conv_in, conv_state, taps, slot, back, ahead);
  }
  return lm_launch_status();
}

extern "C" int ao_lm_gelu_glu(const void* gu, int dt, int64_t n, int64_t ff, void* y, void* stream) {
  LM_CHECK_ARG(gu && y && n > 0 && ff > 0);
  const int64_t total = n * ff;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  LM_DISPATCH(dt, gelu_glu_kernel<T><<<blocks, 256, 0, lm_stream(stream)>>>(static_cast<const T*>(gu), n, ff, static_cast<T*>(y)));
  return lm_launch_status();
}
