// Latent attention over the cached compressed keys: every head of a token scores the SAME cached rows (latent c_j of R
// numbers + rotated key part kr_j of dr numbers), with the key up-projection folded into the query beforehand, so the
// kernel is multi-query attention with key size R + dr and value = the latent itself.  Scores, softmax (with a sink
// term in the denominator) and the weighted sum are fp32 on the CUDA cores for both storage types.
//
// One warp owns one token and four heads (the cached row is loaded from shared memory once for four score rows); the
// eight warps of a CTA are TQ consecutive tokens of one sequence x HQ head quads and share every 32-key tile staged
// in shared memory.  grid = (token tiles, head-quad groups, key splits).  Within its key range a warp keeps a running
// maximum / denominator / unnormalised output (lane l owns latent coordinates l, l + 32, ...); with one split it
// finishes the row itself, otherwise the splits' partial results are merged by a second kernel.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kWarps = 8;
constexpr int kKeys = 32;   // keys per tile = one per lane

__host__ __device__ inline int head_quads_per_cta(int H) {
  const int q = (H + 3) / 4;
  return q >= 8 ? 8 : q >= 4 ? 4 : q >= 2 ? 2 : 1;
}

template <typename T, int RPL>
__global__ void __launch_bounds__(kWarps * 32)
latent_attn_kernel(const float* __restrict__ qa, const float* __restrict__ qr, const T* __restrict__ c_cache,
                   const T* __restrict__ kr_cache, int64_t S, const int32_t* __restrict__ slot,
                   const int32_t* __restrict__ pos, const int32_t* __restrict__ tile_first,
                   const int32_t* __restrict__ tile_count, int64_t n, int H, int R, int dr, float scale, int HQ,
                   int tiles_per_split, int n_split, const T* __restrict__ sink, const float* __restrict__ gate,
                   T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml) {
  extern __shared__ float smem[];
  const int D = R + dr, DP = D + 1;
  float* qs = smem;                         // [kWarps][D][4]
  float* ks = smem + (size_t)kWarps * D * 4;  // [kKeys][DP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TQ = kWarps / HQ;
  const int tq = warp / HQ, hq = warp - tq * HQ;
  const int first = tile_first[blockIdx.x], count = tile_count[blockIdx.x];
  const bool tok_ok = tq < count;
  const int64_t t = first + (tok_ok ? tq : 0);
  const int head0 = (blockIdx.y * HQ + hq) * 4;
  const bool active = tok_ok && head0 < H;
  const int my_pos = pos[t];
  const int64_t seq = slot[first];
  int max_pos = 0;
  for (int i = 0; i < count && i < TQ; ++i) max_pos = max(max_pos, pos[first + i]);
  const int k_lo = blockIdx.z * tiles_per_split * kKeys;
  const int k_hi = min(k_lo + tiles_per_split * kKeys, max_pos + 1);
  if (k_lo >= k_hi) return;   // uniform over the CTA: nothing of this split is visible to any of its tokens

  // the warp's four query rows, interleaved so that one 16-byte broadcast load feeds four score rows
  float* myq = qs + (size_t)warp * D * 4;
  if (active) {
    for (int d = lane; d < D; d += 32) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int h = head0 + r;
        float v = 0.f;
        if (h < H) v = d < R ? qa[((int64_t)h * n + t) * R + d] : qr[(t * H + h) * dr + (d - R)];
        myq[d * 4 + r] = v;
      }
    }
  }
  float m[4], l[4], o[4][RPL];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < RPL; ++i) o[r][i] = 0.f;
  }
  const T* cbase = c_cache + seq * S * R;
  const T* kbase = kr_cache + seq * S * dr;
  for (int k0 = k_lo; k0 < k_hi; k0 += kKeys) {
    __syncthreads();   // the previous tile is consumed (and myq is written, first time round)
    for (int j = warp; j < kKeys; j += kWarps) {
      const int key = k0 + j;
      float* dst = ks + (size_t)j * DP;
      if (key < k_hi) {
        const T* c = cbase + (int64_t)key * R;
        const T* kr = kbase + (int64_t)key * dr;
        for (int d = lane; d < R; d += 32) dst[d] = ldf(c + d);
        for (int d = lane; d < dr; d += 32) dst[R + d] = ldf(kr + d);
      } else {
        for (int d = lane; d < D; d += 32) dst[d] = 0.f;
      }
    }
    __syncthreads();
    if (!active || k0 > my_pos) continue;   // uniform over the warp
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kk = ks + (size_t)lane * DP;
    const float4* q4 = reinterpret_cast<const float4*>(myq);
#pragma unroll 4
    for (int d = 0; d < D; ++d) {
      const float kv = kk[d];
      const float4 q = q4[d];
      s[0] = fmaf(q.x, kv, s[0]);
      s[1] = fmaf(q.y, kv, s[1]);
      s[2] = fmaf(q.z, kv, s[2]);
      s[3] = fmaf(q.w, kv, s[3]);
    }
    const int key = k0 + lane;
    const bool seen = key < k_hi && key <= my_pos;
    float p[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float sc = seen ? s[r] * scale : -INFINITY;
      const float mn = fmaxf(m[r], warp_max(sc));   // finite: key k0 <= my_pos is seen
      const float corr = __expf(m[r] - mn);         // exp(-inf) = 0 on the first tile
      p[r] = seen ? __expf(sc - mn) : 0.f;
      m[r] = mn;
      l[r] = fmaf(l[r], corr, p[r]);
#pragma unroll
      for (int i = 0; i < RPL; ++i) o[r][i] *= corr;
    }
    const int jn = min(kKeys, min(k_hi, my_pos + 1) - k0);
    for (int j = 0; j < jn; ++j) {
      const float p0 = __shfl_sync(0xffffffffu, p[0], j), p1 = __shfl_sync(0xffffffffu, p[1], j);
      const float p2 = __shfl_sync(0xffffffffu, p[2], j), p3 = __shfl_sync(0xffffffffu, p[3], j);
      const float* c = ks + (size_t)j * DP;
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        const int d = lane + 32 * i;
        const float cv = d < R ? c[d] : 0.f;
        o[0][i] = fmaf(p0, cv, o[0][i]);
        o[1][i] = fmaf(p1, cv, o[1][i]);
        o[2][i] = fmaf(p2, cv, o[2][i]);
        o[3][i] = fmaf(p3, cv, o[3][i]);
      }
    }
  }
  if (!active) return;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int h = head0 + r;
    if (h >= H) break;
    const float lsum = warp_sum(l[r]);
    if (n_split == 1) {
      const float sk = ldf(sink + h);
      const float top = fmaxf(m[r], sk);
      const float e = __expf(m[r] - top);
      const float k = gate[t * H + h] * e / (lsum * e + __expf(sk - top));
      T* dst = out + (t * H + h) * R;
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        const int d = lane + 32 * i;
        if (d < R) stf(dst + d, o[r][i] * k);
      }
    } else {
      const int64_t at = (t * H + h) * n_split + blockIdx.z;
      float* dst = part_o + at * R;
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        const int d = lane + 32 * i;
        if (d < R) dst[d] = o[r][i];
      }
      if (lane == 0) part_ml[at * 2] = m[r], part_ml[at * 2 + 1] = lsum;
    }
  }
}

// one CTA per (token, head): merges the key splits that hold keys this token sees, then sink, gate, normalisation
template <typename T>
__global__ void latent_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int32_t* __restrict__ pos, int H, int R, int tiles_per_split, int n_split,
                                         const T* __restrict__ sink, const float* __restrict__ gate, T* __restrict__ out) {
  const int64_t row = blockIdx.x;
  const int64_t t = row / H;
  const int h = (int)(row - t * H);
  const int ns = min(n_split, pos[t] / (tiles_per_split * kKeys) + 1);
  const float sk = ldf(sink + h);
  float top = sk;
  for (int s = 0; s < ns; ++s) top = fmaxf(top, part_ml[(row * n_split + s) * 2]);
  float den = __expf(sk - top);
  for (int s = 0; s < ns; ++s) den = fmaf(part_ml[(row * n_split + s) * 2 + 1], __expf(part_ml[(row * n_split + s) * 2] - top), den);
  const float k = gate[row] / den;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < ns; ++s) acc = fmaf(part_o[(row * n_split + s) * R + d], __expf(part_ml[(row * n_split + s) * 2] - top), acc);
    stf(out + row * R + d, acc * k);
  }
}

template <typename T, int RPL>
int launch(const float* qa, const float* qr, const void* c_cache, const void* kr_cache, int64_t S, const int32_t* slot,
           const int32_t* pos, const int32_t* tile_first, const int32_t* tile_count, int n_tiles, int64_t n, int H, int R,
           int dr, float scale, const void* sink, const float* gate, int max_pos, int n_split, float* part_o,
           float* part_ml, void* out, cudaStream_t st) {
  const int HQ = head_quads_per_cta(H);
  const int D = R + dr;
  const size_t smem = ((size_t)kWarps * D * 4 + (size_t)kKeys * (D + 1)) * sizeof(float);
  if (smem > 220 * 1024) return AO_B200_ERR_UNSUPPORTED;
  auto kern = latent_attn_kernel<T, RPL>;
  if (smem > 48 * 1024) {
    static bool set = false;   // per instantiation
    if (!set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
      set = true;
    }
  }
  const int tiles = (max_pos + kKeys) / kKeys;                 // 32-key tiles that hold keys 0 .. max_pos
  const int tps = (tiles + n_split - 1) / n_split;
  const int quads = (H + 3) / 4;
  dim3 grid((unsigned)n_tiles, (unsigned)((quads + HQ - 1) / HQ), (unsigned)n_split);
  kern<<<grid, kWarps * 32, smem, st>>>(qa, qr, static_cast<const T*>(c_cache), static_cast<const T*>(kr_cache), S, slot, pos,
                                        tile_first, tile_count, n, H, R, dr, scale, HQ, tps, n_split,
                                        static_cast<const T*>(sink), gate, static_cast<T*>(out), part_o, part_ml);
  if (n_split > 1)
    latent_attn_merge_kernel<T><<<(unsigned)(n * H), 128, 0, st>>>(part_o, part_ml, pos, H, R, tps, n_split,
                                                                  static_cast<const T*>(sink), gate, static_cast<T*>(out));
  return lm_launch_status();
}

}  // namespace

extern "C" int ao_lm_latent_attention_plan(int H, int* tile_tokens) {
  LM_CHECK_ARG(H > 0 && tile_tokens);
  *tile_tokens = kWarps / head_quads_per_cta(H);
  return AO_B200_OK;
}

extern "C" int64_t ao_lm_latent_attention_workspace_bytes(int64_t n, int H, int R, int n_split) {
  if (n_split <= 1) return 0;
  return n * H * n_split * (int64_t)(R + 2) * 4;
}

extern "C" int ao_lm_latent_attention(const float* qa, const float* qr, const void* c_cache, const void* kr_cache, int dt,
                                      int64_t S, const int32_t* slot, const int32_t* pos, const int32_t* tile_first,
                                      const int32_t* tile_count, int n_tiles, int64_t n, int H, int R, int dr, float scale,
                                      const void* sink, const float* gate, int max_pos, int n_split, void* workspace,
                                      int64_t workspace_bytes, void* out, void* stream) {
  LM_CHECK_ARG(qa && qr && c_cache && kr_cache && slot && pos && tile_first && tile_count && sink && gate && out);
  LM_CHECK_ARG(n > 0 && n_tiles > 0 && H > 0 && R > 0 && dr >= 0 && S > 0 && max_pos >= 0 && max_pos < S && n_split >= 1);
  if (R > 512) return AO_B200_ERR_UNSUPPORTED;
  float *part_o = nullptr, *part_ml = nullptr;
  if (n_split > 1) {
    if (!workspace || workspace_bytes < ao_lm_latent_attention_workspace_bytes(n, H, R, n_split)) return AO_B200_ERR_WORKSPACE;
    part_o = static_cast<float*>(workspace);
    part_ml = part_o + n * H * n_split * (int64_t)R;
  }
  const cudaStream_t st = lm_stream(stream);
#define LM_ATTN(RPL)                                                                                                        \
  LM_DISPATCH(dt, return (launch<T, RPL>(qa, qr, c_cache, kr_cache, S, slot, pos, tile_first, tile_count, n_tiles, n, H, R, dr, \
                                         scale, sink, gate, max_pos, n_split, part_o, part_ml, out, st)))
  if (R <= 32) LM_ATTN(1);
  else if (R <= 64) LM_ATTN(2);
  else if (R <= 128) LM_ATTN(4);
  else if (R <= 256) LM_ATTN(8);
  else LM_ATTN(16);
#undef LM_ATTN
  return AO_B200_OK;
}
