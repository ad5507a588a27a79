// Recurrent mechanisms with per-sequence state in numbered slots: a short causal convolution over time per channel,
// and two gated linear recurrences S_t = a_t S_(t-1) + b_t per channel (the minimal GRU whose gates read only the
// current token, and the real-gated linear recurrent unit with block-diagonal gates).  State, gates, decays and the
// recurrence itself are fp32; only the result that feeds the next matrix product is written in the storage type.
//
// A step's rows are runs ("segments") of consecutive positions of one sequence.  back[t] = rows of the same segment in
// front of row t, ahead[t] = rows behind it.  A recurrence over a long segment runs in three launches: every tile of
// rows reduces to (product of a, local end state), a pass over the tiles of each segment turns those into the state
// at each tile's start, and the tiles run again from there and write their rows.  Segments of one tile take one launch.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kMaxTaps = 8;
constexpr int kScanThreads = 128;

// y[t][c] = (residual ? v(t) : 0) + out_bias[c] + sum_j kern[c][j] * v(t - (taps - 1 - j)),  v(row) = x[row][c] + in_bias[c];
// rows in front of the step come from state[slot][k][c] (k-th oldest of the taps - 1 kept inputs, bias included), rows
// in front of position 0 are zero.
constexpr int kConvRows = 8;   // rows of one CTA: taps, metadata and the rows' inputs are loaded once, all up front
template <typename T>
__global__ void causal_conv_kernel(const float* __restrict__ x, int64_t ldx, const T* __restrict__ in_bias, int64_t n, int64_t C,
                                   int taps, const T* __restrict__ kern, const T* __restrict__ out_bias, int residual,
                                   const float* __restrict__ state, const int32_t* __restrict__ slot,
                                   const int32_t* __restrict__ pos, const int32_t* __restrict__ back,
                                   float* __restrict__ out_f32, T* __restrict__ out) {
  const int64_t c = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int64_t t0 = (int64_t)blockIdx.x * kConvRows;
  // xin[i] = input row t0 - (kMaxTaps - 1) + i, whichever sequence it belongs to (the rows decide below what they use)
  float xin[kConvRows + kMaxTaps - 1];
#pragma unroll
  for (int i = 0; i < kConvRows + kMaxTaps - 1; ++i) {
    const int64_t r = t0 - (kMaxTaps - 1) + i;
    xin[i] = (r >= 0 && r < n && i >= kMaxTaps - taps) ? x[r * ldx + c] : 0.f;
  }
  int pb[kConvRows], pp[kConvRows], ps[kConvRows];
#pragma unroll
  for (int k = 0; k < kConvRows; ++k) {
    const bool in = t0 + k < n;
    pb[k] = in ? back[t0 + k] : 0, pp[k] = in ? pos[t0 + k] : 0, ps[k] = in ? slot[t0 + k] : 0;
  }
  const float ib = in_bias ? ldf(in_bias + c) : 0.f, ob = out_bias ? ldf(out_bias + c) : 0.f;
  float wr[kMaxTaps];           // wr[delta] = the tap that meets the input delta rows back
#pragma unroll
  for (int dl = 0; dl < kMaxTaps; ++dl) wr[dl] = dl < taps ? ldf(kern + c * taps + (taps - 1 - dl)) : 0.f;
  // a tile whose rows all have taps - 1 rows of their own segment in front of them needs neither memory nor zeros
  bool interior = t0 + kConvRows <= n;
#pragma unroll
  for (int k = 0; k < kConvRows; ++k) interior = interior && pb[k] >= taps - 1;
  if (interior) {   // uniform over the CTA
#pragma unroll
    for (int k = 0; k < kConvRows; ++k) {
      const float cur = xin[k + kMaxTaps - 1] + ib;
      float acc = fmaf(wr[0], cur, ob);
#pragma unroll
      for (int dl = 1; dl < kMaxTaps; ++dl) acc = fmaf(wr[dl], xin[k + kMaxTaps - 1 - dl] + ib, acc);   // wr = 0 past the taps
      if (residual) acc += cur;
      if (out_f32) out_f32[(t0 + k) * C + c] = acc;
      if (out) stf(out + (t0 + k) * C + c, acc);
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < kConvRows; ++k) {
    const int64_t t = t0 + k;
    if (t >= n) break;
    const float cur = xin[k + kMaxTaps - 1] + ib;
    float acc = fmaf(wr[0], cur, ob);
#pragma unroll
    for (int dl = 1; dl < kMaxTaps; ++dl) {
      if (dl < taps) {
        float v;
        if (dl <= pb[k]) v = xin[k + kMaxTaps - 1 - dl] + ib;
        else if (pp[k] - dl >= 0) v = state[((int64_t)ps[k] * (taps - 1) + (pb[k] - dl + taps - 1)) * C + c];
        else v = 0.f;
        acc = fmaf(wr[dl], v, acc);
      }
    }
    if (residual) acc += cur;
    if (out_f32) out_f32[t * C + c] = acc;
    if (out) stf(out + t * C + c, acc);
  }
}

// ---------------------------------------------------------------------------------------------- gated recurrences
// kFast (bf16 storage): one hardware exponential and an approximate reciprocal per function, errors of a few 1e-7 —
// three orders of magnitude below what bf16 operands leave in the inputs.  fp32 storage keeps the library functions.
template <bool kFast>
__device__ __forceinline__ float sigmoid_(float v) {
  return kFast ? __fdividef(1.f, 1.f + __expf(-v)) : 1.f / (1.f + expf(-v));
}
template <bool kFast>
__device__ __forceinline__ float gelu_tanh_(float z) {
  const float x = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  const float th = kFast ? 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f) : tanhf(x);
  return 0.5f * z * (1.f + th);
}
template <typename T>
struct FastMath { static constexpr bool value = true; };
template <>
struct FastMath<float> { static constexpr bool value = false; };

// minimal GRU: z = sigmoid(zp + zb), u = xp + xb, candidate = u + 1/2 (u >= 0) | sigmoid(u);  a = 1 - z, b = z * candidate;
// row result = S * silu(gp) * out_scale
template <typename T>
struct MinGru {
  const float *zp, *xp, *gp;   // columns of one projection row, fp32
  int64_t ld;
  const T *zb, *xb;
  float out_scale;
  T* out;
  int64_t ld_out;
  static constexpr bool kFast = FastMath<T>::value;
  struct Chan { float zb, xb; };
  struct Raw { float z, x, g; };
  __device__ Chan channel(int64_t c) const { return {zb ? ldf(zb + c) : 0.f, xb ? ldf(xb + c) : 0.f}; }
  __device__ void load(const Chan&, int64_t t, int64_t c, bool rows, Raw& r) const {
    r.z = zp[t * ld + c], r.x = xp[t * ld + c];
    if (rows) r.g = gp[t * ld + c];
  }
  __device__ void gates(const Chan& ch, const Raw& r, float& a, float& b) const {
    const float z = sigmoid_<kFast>(r.z + ch.zb), u = r.x + ch.xb;
    const float cand = u >= 0.f ? u + 0.5f : sigmoid_<kFast>(u);
    a = 1.f - z;
    b = z * cand;
  }
  __device__ void emit(const Chan&, const Raw& r, int64_t t, int64_t c, float S) const {
    stf(out + t * ld_out + c, S * r.g * sigmoid_<kFast>(r.g) * out_scale);
  }
};

// real-gated linear recurrent unit: r = sigmoid(rp + rb), i = sigmoid(ip + ib) from block-diagonal products
// gates[block][t][2 bw] = (r | i) of the block's channels;  log a = -decay * r * softplus(lam), a = exp(log a),
// b = sqrt(1 - a^2) * i * u;  row result = S * gelu(yp + yb)
template <typename T>
struct RgLru {
  const float* pre;
  int64_t n;
  int bw;
  const T *rb, *ib, *lam;
  float decay;
  const float* u;      // [n][Rw]
  const float* yp;
  int64_t ldy;
  const T* yb;
  T* out;
  int64_t Rw;
  static constexpr bool kFast = FastMath<T>::value;
  struct Chan { float rb, ib, sp, yb; int64_t goff; };
  __device__ Chan channel(int64_t c) const {
    const float l = ldf(lam + c);
    const float sp = l > 20.f ? l : log1pf(expf(l));
    const int64_t blk = c / bw, o = c - blk * bw;
    return {ldf(rb + c), ldf(ib + c), sp, yb ? ldf(yb + c) : 0.f, blk * n * 2 * bw + o};
  }
  struct Raw { float r, i, u, y; };
  __device__ void load(const Chan& ch, int64_t t, int64_t c, bool rows, Raw& v) const {
    const float* g = pre + ch.goff + t * 2 * bw;
    v.r = g[0], v.i = g[bw], v.u = u[t * Rw + c];
    if (rows) v.y = yp[t * ldy + c];
  }
  __device__ void gates(const Chan& ch, const Raw& v, float& a, float& b) const {
    const float r = sigmoid_<kFast>(v.r + ch.rb), i = sigmoid_<kFast>(v.i + ch.ib);
    const float la = -decay * r * ch.sp;
    if (kFast) {
      a = __expf(la);
      b = sqrtf(fmaxf(1.f - a * a, 0.f)) * i * v.u;
    } else {
      a = expf(la);
      b = sqrtf(-expm1f(2.f * la)) * i * v.u;
    }
  }
  __device__ void emit(const Chan& ch, const Raw& v, int64_t t, int64_t c, float S) const {
    stf(out + t * Rw + c, S * gelu_tanh_<kFast>(v.y + ch.yb));
  }
};

// what a scan launch knows about the step besides the recurrence itself
struct ScanMeta {
  const int32_t *slot, *pos, *back;
  const int32_t *tile_first, *tile_count;   // runs of rows of one segment
  float* state;                             // [slots][Rw]
  // convolution memory kept beside the recurrence (optional): the last taps - 1 inputs of the convolution in front of it
  const float* conv_x;
  int64_t conv_ld;
  const void* conv_bias;
  float* conv_state;
  int taps;
};

template <typename T>
__device__ __forceinline__ void save_conv_rows(const ScanMeta& m, int64_t last, int64_t c, int64_t Rw) {
  // `last` = the segment's last row: state[k] = input at position p - (taps - 2 - k)
  const int b = m.back[last], taps = m.taps;
  float* st = m.conv_state + (int64_t)m.slot[last] * (taps - 1) * Rw;
  const float ib = m.conv_bias ? ldf(static_cast<const T*>(m.conv_bias) + c) : 0.f;
  float v[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps - 1; ++k) {
    if (k < taps - 1) {
      const int delta = taps - 2 - k;
      v[k] = delta <= b ? m.conv_x[(last - delta) * m.conv_ld + c] + ib : st[(int64_t)(b - delta + taps - 1) * Rw + c];
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxTaps - 1; ++k)
    if (k < taps - 1) st[(int64_t)k * Rw + c] = v[k];
}

// rows [first, first + count) of one channel: the raw inputs of kScanAhead rows are loaded before any is used (the
// recurrence itself is a dependent chain; its loads are not)
constexpr int kScanAhead = 4;
template <bool kRows, typename F, typename Step>
__device__ __forceinline__ void scan_rows(const F& f, const typename F::Chan& ch, int64_t first, int64_t count, int64_t c, Step step) {
  for (int64_t t0 = first; t0 < first + count; t0 += kScanAhead) {
    typename F::Raw raw[kScanAhead];
#pragma unroll
    for (int j = 0; j < kScanAhead; ++j)
      if (t0 + j < first + count) f.load(ch, t0 + j, c, kRows, raw[j]);
#pragma unroll
    for (int j = 0; j < kScanAhead; ++j) {
      if (t0 + j < first + count) {
        float a, b;
        f.gates(ch, raw[j], a, b);
        step(t0 + j, raw[j], a, b);
      }
    }
  }
}

// one launch: every tile is a whole segment.  grid (tiles, channel blocks)
template <typename T, typename F>
__global__ void __launch_bounds__(kScanThreads) scan_direct_kernel(F f, ScanMeta m, int64_t Rw) {
  const int64_t c = (int64_t)blockIdx.y * kScanThreads + threadIdx.x;
  if (c >= Rw) return;
  const int64_t first = m.tile_first[blockIdx.x], count = m.tile_count[blockIdx.x];
  float* st = m.state + (int64_t)m.slot[first] * Rw + c;
  float S = m.pos[first] > 0 ? *st : 0.f;
  const auto ch = f.channel(c);
  scan_rows<true>(f, ch, first, count, c, [&](int64_t t, const typename F::Raw& raw, float a, float b) {
    S = fmaf(a, S, b);
    f.emit(ch, raw, t, c, S);
  });
  *st = S;
  if (m.conv_state) save_conv_rows<T>(m, first + count - 1, c, Rw);
}

// phase 1: tile -> (A = product of a, B = end state from zero)
template <typename T, typename F>
__global__ void __launch_bounds__(kScanThreads) scan_reduce_kernel(F f, ScanMeta m, int64_t Rw, float* __restrict__ tA,
                                                                   float* __restrict__ tB) {
  const int64_t c = (int64_t)blockIdx.y * kScanThreads + threadIdx.x;
  if (c >= Rw) return;
  const int64_t first = m.tile_first[blockIdx.x], count = m.tile_count[blockIdx.x];
  const auto ch = f.channel(c);
  float A = 1.f, B = 0.f;
  scan_rows<false>(f, ch, first, count, c, [&](int64_t, const typename F::Raw&, float a, float b) {
    A *= a;
    B = fmaf(a, B, b);
  });
  tA[(int64_t)blockIdx.x * Rw + c] = A;
  tB[(int64_t)blockIdx.x * Rw + c] = B;
}

// phase 2: per segment (seg_tile0, seg_tiles), over its tiles in order: tB[tile] <- state at the tile's start
template <typename T>
__global__ void __launch_bounds__(kScanThreads) scan_carry_kernel(ScanMeta m, int64_t Rw, const int32_t* __restrict__ seg_tile0,
                                                                  const int32_t* __restrict__ seg_tiles,
                                                                  const float* __restrict__ tA, float* __restrict__ tB) {
  const int64_t c = (int64_t)blockIdx.y * kScanThreads + threadIdx.x;
  if (c >= Rw) return;
  const int t0 = seg_tile0[blockIdx.x], nt = seg_tiles[blockIdx.x];
  const int64_t first = m.tile_first[t0];
  float* st = m.state + (int64_t)m.slot[first] * Rw + c;
  float S = m.pos[first] > 0 ? *st : 0.f;
  for (int i0 = t0; i0 < t0 + nt; i0 += 16) {   // sixteen tiles' summaries in flight
    float A[16], B[16];
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (i0 + j < t0 + nt) A[j] = tA[(int64_t)(i0 + j) * Rw + c], B[j] = tB[(int64_t)(i0 + j) * Rw + c];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (i0 + j < t0 + nt) {
        tB[(int64_t)(i0 + j) * Rw + c] = S;
        S = fmaf(A[j], S, B[j]);
      }
    }
  }
  *st = S;
  if (m.conv_state) {
    const int64_t last = m.tile_first[t0 + nt - 1] + m.tile_count[t0 + nt - 1] - 1;
    save_conv_rows<T>(m, last, c, Rw);
  }
}

// phase 3: the tile again from the state at its start, rows written
template <typename T, typename F>
__global__ void __launch_bounds__(kScanThreads) scan_apply_kernel(F f, ScanMeta m, int64_t Rw, const float* __restrict__ tS) {
  const int64_t c = (int64_t)blockIdx.y * kScanThreads + threadIdx.x;
  if (c >= Rw) return;
  const int64_t first = m.tile_first[blockIdx.x], count = m.tile_count[blockIdx.x];
  const auto ch = f.channel(c);
  float S = tS[(int64_t)blockIdx.x * Rw + c];
  scan_rows<true>(f, ch, first, count, c, [&](int64_t t, const typename F::Raw& raw, float a, float b) {
    S = fmaf(a, S, b);
    f.emit(ch, raw, t, c, S);
  });
}

template <typename T, typename F>
int run_scan(const F& f, const ScanMeta& m, int64_t Rw, int n_tiles, const int32_t* seg_tile0, const int32_t* seg_tiles,
             int n_segments, float* workspace, cudaStream_t st) {
  const unsigned cb = (unsigned)((Rw + kScanThreads - 1) / kScanThreads);
  if (!seg_tile0) {   // every tile is a whole segment
    scan_direct_kernel<T, F><<<dim3((unsigned)n_tiles, cb), kScanThreads, 0, st>>>(f, m, Rw);
    return lm_launch_status();
  }
  float *tA = workspace, *tB = workspace + (int64_t)n_tiles * Rw;
  scan_reduce_kernel<T, F><<<dim3((unsigned)n_tiles, cb), kScanThreads, 0, st>>>(f, m, Rw, tA, tB);
  scan_carry_kernel<T><<<dim3((unsigned)n_segments, cb), kScanThreads, 0, st>>>(m, Rw, seg_tile0, seg_tiles, tA, tB);
  scan_apply_kernel<T, F><<<dim3((unsigned)n_tiles, cb), kScanThreads, 0, st>>>(f, m, Rw, tB);
  return lm_launch_status();
}

}  // namespace

extern "C" int ao_lm_causal_conv(const float* x, int64_t ldx, const void* in_bias, int64_t n, int64_t channels, int taps,
                                 const void* kernel, const void* out_bias, int dt, int residual, const float* state,
                                 const int32_t* slot, const int32_t* pos, const int32_t* back, float* out_f32, void* out,
                                 void* stream) {
  LM_CHECK_ARG(x && kernel && state && slot && pos && back && (out_f32 || out));
  LM_CHECK_ARG(n > 0 && channels > 0 && taps >= 1 && taps <= kMaxTaps && ldx >= channels);
  const unsigned cb = (unsigned)((channels + 127) / 128);
  LM_DISPATCH(dt, causal_conv_kernel<T><<<dim3((unsigned)((n + kConvRows - 1) / kConvRows), cb), 128, 0, lm_stream(stream)>>>(
                      x, ldx, static_cast<const T*>(in_bias), n, channels, taps, static_cast<const T*>(kernel),
                      static_cast<const T*>(out_bias), residual, state, slot, pos, back, out_f32, static_cast<T*>(out)));
  return lm_launch_status();
}

extern "C" int64_t ao_lm_scan_workspace_bytes(int n_tiles, int64_t channels) { return (int64_t)n_tiles * channels * 2 * 4; }

extern "C" int ao_lm_mingru_scan(const float* proj, int64_t ld, int64_t z_off, int64_t x_off, int64_t g_off, const void* z_bias,
                                 const void* x_bias, int dt, int64_t channels, float* state, const int32_t* slot,
                                 const int32_t* pos, const int32_t* back, const int32_t* tile_first, const int32_t* tile_count,
                                 int n_tiles, const int32_t* seg_tile0, const int32_t* seg_tiles, int n_segments,
                                 float* workspace, float out_scale, void* out, int64_t ld_out, void* stream) {
  LM_CHECK_ARG(proj && state && slot && pos && back && tile_first && tile_count && out && n_tiles > 0 && channels > 0);
  LM_CHECK_ARG(!seg_tile0 || (seg_tiles && n_segments > 0 && workspace));
  ScanMeta m{slot, pos, back, tile_first, tile_count, state, nullptr, 0, nullptr, nullptr, 0};
  LM_DISPATCH(dt, {
    MinGru<T> f{proj + z_off, proj + x_off, proj + g_off, ld, static_cast<const T*>(z_bias), static_cast<const T*>(x_bias),
                out_scale, static_cast<T*>(out), ld_out};
    return run_scan<T>(f, m, channels, n_tiles, seg_tile0, seg_tiles, n_segments, workspace, lm_stream(stream));
  });
  return AO_B200_OK;
}

extern "C" int ao_lm_rglru_scan(const float* gates, int64_t n, int block_width, const void* r_bias, const void* i_bias,
                                const void* lam, float decay, const float* u, const float* y_pre, int64_t ld_y,
                                const void* y_bias, int dt, int64_t channels, float* state, const float* conv_x,
                                int64_t conv_ld, const void* conv_in_bias, float* conv_state, int taps, const int32_t* slot,
                                const int32_t* pos, const int32_t* back, const int32_t* tile_first, const int32_t* tile_count,
                                int n_tiles, const int32_t* seg_tile0, const int32_t* seg_tiles, int n_segments,
                                float* workspace, void* out, void* stream) {
  LM_CHECK_ARG(gates && r_bias && i_bias && lam && u && y_pre && state && slot && pos && back && tile_first && tile_count && out);
  LM_CHECK_ARG(n > 0 && n_tiles > 0 && channels > 0 && block_width > 0 && channels % block_width == 0);
  LM_CHECK_ARG(!seg_tile0 || (seg_tiles && n_segments > 0 && workspace));
  LM_CHECK_ARG(!conv_state || (conv_x && taps >= 2 && taps <= kMaxTaps));
  ScanMeta m{slot, pos, back, tile_first, tile_count, state, conv_x, conv_ld, conv_in_bias, conv_state, taps};
  LM_DISPATCH(dt, {
    RgLru<T> f{gates, n, block_width, static_cast<const T*>(r_bias), static_cast<const T*>(i_bias), static_cast<const T*>(lam),
               decay, u, y_pre, ld_y, static_cast<const T*>(y_bias), static_cast<T*>(out), channels};
    return run_scan<T>(f, m, channels, n_tiles, seg_tile0, seg_tiles, n_segments, workspace, lm_stream(stream));
  });
  return AO_B200_OK;
}
