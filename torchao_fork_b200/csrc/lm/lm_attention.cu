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

constexpr int kPrefetch = 10;   // 16-byte chunks per thread held in registers for the next key tile

// a 16-byte load that stays where it is written: the compiler may not sink it towards its first use
__device__ __forceinline__ uint4 ld16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

// chunk `ch` of the cached row `key`: the first cr chunks are the latent, the rest the rotated key part
template <typename T>
__device__ __forceinline__ const T* chunk_src(const T* cbase, const T* kbase, int key, int ch, int cr, int R, int dr) {
  constexpr int kPer = 16 / (int)sizeof(T);
  return ch < cr ? cbase + (int64_t)key * R + ch * kPer : kbase + (int64_t)key * dr + (ch - cr) * kPer;
}
// 16 bytes of a cached row -> fp32 in shared memory
template <typename T>
__device__ __forceinline__ void store_chunk(const uint4& u, float* dst);
template <>
__device__ __forceinline__ void store_chunk<__nv_bfloat16>(const uint4& u, float* dst) {
  const uint32_t r[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dst[2 * i] = __uint_as_float(r[i] << 16);
    dst[2 * i + 1] = __uint_as_float(r[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void store_chunk<float>(const uint4& u, float* dst) {
  dst[0] = __uint_as_float(u.x), dst[1] = __uint_as_float(u.y), dst[2] = __uint_as_float(u.z), dst[3] = __uint_as_float(u.w);
}
// all of a thread's loads for the tile that starts at key k0 are issued before any is used
template <typename T>
__device__ __forceinline__ void fetch_tile(uint4 (&pf)[kPrefetch], const T* cbase, const T* kbase, int k0, int k_hi, int cpk,
                                           int cr, int R, int dr, int total_chunks) {
  (void)cpk;
#pragma unroll
  for (int b = 0; b < kPrefetch; ++b) {
    const int i = threadIdx.x + b * kWarps * 32;
    pf[b] = make_uint4(0, 0, 0, 0);
    if (i < total_chunks) {
      const int j = i & (kKeys - 1), ch = i / kKeys;   // consecutive lanes: consecutive keys (odd row pitch: no bank conflicts)
      if (k0 + j < k_hi) pf[b] = ld16(chunk_src(cbase, kbase, k0 + j, ch, cr, R, dr));
    }
  }
}
template <typename T>
__device__ __forceinline__ void store_tile(const uint4 (&pf)[kPrefetch], float* ks, int DP, int total_chunks) {
  constexpr int kPer = 16 / (int)sizeof(T);
#pragma unroll
  for (int b = 0; b < kPrefetch; ++b) {
    const int i = threadIdx.x + b * kWarps * 32;
    if (i < total_chunks) {
      const int j = i & (kKeys - 1), ch = i / kKeys;
      store_chunk<T>(pf[b], ks + (size_t)j * DP + ch * kPer);
    }
  }
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
    const bool qvec = R % 4 == 0 && dr % 4 == 0 && reinterpret_cast<uintptr_t>(qa) % 16 == 0 && reinterpret_cast<uintptr_t>(qr) % 16 == 0;
    if (qvec) {
      // 16-byte loads, the four heads' chunks of one coordinate group in flight together
      for (int ch = lane; ch < D / 4; ch += 32) {
        const int d = ch * 4;
        uint4 v[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int h = head0 + r;
          v[r] = make_uint4(0, 0, 0, 0);
          if (h < H) v[r] = ld16(d < R ? qa + ((int64_t)h * n + t) * R + d : qr + (t * H + h) * dr + (d - R));
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          myq[(d + 0) * 4 + r] = __uint_as_float(v[r].x);
          myq[(d + 1) * 4 + r] = __uint_as_float(v[r].y);
          myq[(d + 2) * 4 + r] = __uint_as_float(v[r].z);
          myq[(d + 3) * 4 + r] = __uint_as_float(v[r].w);
        }
      }
    } else {
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
  constexpr int kVecElems = 16 / (int)sizeof(T);
  const bool vec = R % kVecElems == 0 && dr % kVecElems == 0 && reinterpret_cast<uintptr_t>(c_cache) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(kr_cache) % 16 == 0;
  const int cr = R / kVecElems, cpk = cr + dr / kVecElems, total_chunks = kKeys * cpk;   // 16-byte chunks per row / tile
  uint4 pf[kPrefetch];
  if (vec) fetch_tile<T>(pf, cbase, kbase, k_lo, k_hi, cpk, cr, R, dr, total_chunks);
  for (int k0 = k_lo; k0 < k_hi; k0 += kKeys) {
    __syncthreads();   // the previous tile is consumed (and myq is written, first time round)
    if (vec) {
      store_tile<T>(pf, ks, DP, total_chunks);
      if (total_chunks > kPrefetch * kWarps * 32) {   // rows too long for the register stage: the rest directly
        for (int i = threadIdx.x + kPrefetch * kWarps * 32; i < total_chunks; i += kWarps * 32) {
          const int j = i & (kKeys - 1), ch = i / kKeys;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (k0 + j < k_hi) v = ld16(chunk_src(cbase, kbase, k0 + j, ch, cr, R, dr));
          store_chunk<T>(v, ks + (size_t)j * DP + ch * kVecElems);
        }
      }
    } else {
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
    }
    __syncthreads();
    // the next tile's rows travel while this one is computed (registers are the second buffer)
    if (vec && k0 + kKeys < k_hi) fetch_tile<T>(pf, cbase, kbase, k0 + kKeys, k_hi, cpk, cr, R, dr, total_chunks);
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

// ---- bf16 storage, tensor cores -------------------------------------------------------------------------------------
// The cached rows are bf16, hence exact as TF32.  Queries and softmax weights are fp32: each is split into a TF32 high
// part and a TF32 low part (x = hi + lo to 2^-21), and every product with the cached rows is two m16n8k8 TF32 MMAs with
// fp32 accumulation — the fp32 result without rounding a score or a weight to 16 bits.
// One CTA = one m16 tile of (token, head) rows: HB = min(H, 16) heads of 16 / HB consecutive tokens.  Per 32-key tile
// the score tile [16][32] is split over the 8 warps (4 key octets x 2 halves of the R + dr key coordinates) and summed
// through shared memory; then every warp redoes the row statistics (cheap) and accumulates ITS R / 8 output columns.
constexpr int kMmaRows = 16;

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NT>   // n-tiles (8 output columns each) per warp: R = 64 * NT
__global__ void __launch_bounds__(kWarps * 32, 1)
latent_attn_mma_kernel(const float* __restrict__ qa, const float* __restrict__ qr, const __nv_bfloat16* __restrict__ c_cache,
                       const __nv_bfloat16* __restrict__ kr_cache, int64_t S, const int32_t* __restrict__ slot,
                       const int32_t* __restrict__ pos, const int32_t* __restrict__ tile_first,
                       const int32_t* __restrict__ tile_count, int64_t n, int H, int dr, float scale, int HB,
                       int tiles_per_split, int n_split, const __nv_bfloat16* __restrict__ sink,
                       const float* __restrict__ gate, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                       float* __restrict__ part_ml) {
  using T = __nv_bfloat16;
  constexpr int R = 64 * NT;
  extern __shared__ float smem[];
  const int D = R + dr, DP = D + 4;            // pitch = 4 or 20 mod 32: fragment loads along rows hit 32 banks
  float* qhi = smem;                           // [16][DP]
  float* qlo = qhi + kMmaRows * DP;            // [16][DP]
  float* ks = qlo + kMmaRows * DP;             // [32][DP]
  float* sp = ks + kKeys * DP;                 // [2][16][33] partial scores of the two coordinate halves
  __shared__ int row_pos[kMmaRows];            // position of the row's token, -1 for a row that does not exist
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq4 = lane & 3;
  const int TQ = kMmaRows / HB;
  const int first = tile_first[blockIdx.x], count = min(tile_count[blockIdx.x], TQ);
  const int head_base = blockIdx.y * HB;
  const int64_t seq = slot[first];
  int max_pos = 0;
  for (int i = 0; i < count; ++i) max_pos = max(max_pos, pos[first + i]);
  const int k_lo = blockIdx.z * tiles_per_split * kKeys;
  const int k_hi = min(k_lo + tiles_per_split * kKeys, max_pos + 1);
  if (k_lo >= k_hi) return;
  if (threadIdx.x < kMmaRows) {
    const int r = threadIdx.x, tq = r / HB, hh = r - tq * HB;
    row_pos[r] = (tq < count && head_base + hh < H) ? pos[first + tq] : -1;
  }
  const T* cbase = c_cache + seq * S * R;
  const T* kbase = kr_cache + seq * S * dr;
  const int cr = R / 8, cpk = cr + dr / 8, total_chunks = kKeys * cpk;
  uint4 pf[kPrefetch];
  fetch_tile<T>(pf, cbase, kbase, k_lo, k_hi, cpk, cr, R, dr, total_chunks);
  // queries of the 16 rows, split into TF32 high and low parts; 16-byte loads, four in flight per thread
  {
    const int cq = D / 4, total_q = kMmaRows * cq;
    for (int base = threadIdx.x; base < total_q; base += 4 * kWarps * 32) {
      uint4 v[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int i = base + b * kWarps * 32;
        v[b] = make_uint4(0, 0, 0, 0);
        if (i < total_q) {
          const int r = i / cq, d = (i - r * cq) * 4, tq = r / HB, hh = r - tq * HB, h = head_base + hh;
          if (tq < count && h < H) {
            const int64_t t = first + tq;
            v[b] = ld16(d < R ? qa + ((int64_t)h * n + t) * R + d : qr + (t * H + h) * dr + (d - R));
          }
        }
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int i = base + b * kWarps * 32;
        if (i < total_q) {
          const int r = i / cq, d = (i - r * cq) * 4;
          const uint32_t w[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x = __uint_as_float(w[e]);
            const uint32_t hi = to_tf32(x);
            qhi[r * DP + d + e] = __uint_as_float(hi);
            qlo[r * DP + d + e] = __uint_as_float(to_tf32(x - __uint_as_float(hi)));
          }
        }
      }
    }
  }
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8 (l: this thread's share)
  const int nt_s = warp & 3, kh = warp >> 2;                  // this warp's share of the score tile
  const int ksteps = D / 8, kbeg = kh * (ksteps / 2), kend = kh ? ksteps : ksteps / 2;
  const int col0 = warp * NT * 8;
  for (int k0 = k_lo; k0 < k_hi; k0 += kKeys) {
    __syncthreads();
    store_tile<T>(pf, ks, DP, total_chunks);
    for (int i = threadIdx.x + kPrefetch * kWarps * 32; i < total_chunks; i += kWarps * 32) {
      const int j = i & (kKeys - 1), ch = i / kKeys;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (k0 + j < k_hi) v = ld16(chunk_src(cbase, kbase, k0 + j, ch, cr, R, dr));
      store_chunk<T>(v, ks + (size_t)j * DP + ch * 8);
    }
    __syncthreads();
    if (k0 + kKeys < k_hi) fetch_tile<T>(pf, cbase, kbase, k0 + kKeys, k_hi, cpk, cr, R, dr, total_chunks);
    {   // scores: rows 16 x keys [8 nt_s, +8) over coordinates [8 kbeg, 8 kend)
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const float* kb = ks + (size_t)(nt_s * 8 + g) * DP + tq4;
      const float* ah = qhi + g * DP + tq4;
      const float* al = qlo + g * DP + tq4;
#pragma unroll 2
      for (int kk = kbeg; kk < kend; ++kk) {
        const int d = kk * 8;
        const uint32_t b0 = __float_as_uint(kb[d]), b1 = __float_as_uint(kb[d + 4]);
        uint32_t a[4] = {__float_as_uint(ah[d]), __float_as_uint(ah[8 * DP + d]), __float_as_uint(ah[d + 4]),
                         __float_as_uint(ah[8 * DP + d + 4])};
        mma_tf32(acc, a, b0, b1);
        uint32_t a2[4] = {__float_as_uint(al[d]), __float_as_uint(al[8 * DP + d]), __float_as_uint(al[d + 4]),
                          __float_as_uint(al[8 * DP + d + 4])};
        mma_tf32(acc, a2, b0, b1);
      }
      float* dst = sp + kh * (kMmaRows * 33);
      dst[g * 33 + nt_s * 8 + 2 * tq4] = acc[0];
      dst[g * 33 + nt_s * 8 + 2 * tq4 + 1] = acc[1];
      dst[(g + 8) * 33 + nt_s * 8 + 2 * tq4] = acc[2];
      dst[(g + 8) * 33 + nt_s * 8 + 2 * tq4 + 1] = acc[3];
    }
    __syncthreads();
    // every warp: weights of all 16 rows for this tile, in the A-fragment layout of the second product
    const int p0 = row_pos[g], p1 = row_pos[g + 8];
    float s0[8], s1[8];   // rows g / g + 8, keys 8 ks + tq4 (+ 4)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int kc = (i >> 1) * 8 + tq4 + (i & 1) * 4, key = k0 + kc;
      const float v0 = (sp[g * 33 + kc] + sp[kMmaRows * 33 + g * 33 + kc]) * scale;
      const float v1 = (sp[(g + 8) * 33 + kc] + sp[kMmaRows * 33 + (g + 8) * 33 + kc]) * scale;
      s0[i] = (key < k_hi && key <= p0) ? v0 : -INFINITY;
      s1[i] = (key < k_hi && key <= p1) ? v1 : -INFINITY;
      mx0 = fmaxf(mx0, s0[i]);
      mx1 = fmaxf(mx1, s1[i]);
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float c0 = n0 == -INFINITY ? 1.f : __expf(m0 - n0), c1 = n1 == -INFINITY ? 1.f : __expf(m1 - n1);
    m0 = n0, m1 = n1;
    l0 *= c0, l1 *= c1;
    uint32_t phi[4][4], plo[4][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float e0 = n0 == -INFINITY ? 0.f : __expf(s0[i] - n0), e1 = n1 == -INFINITY ? 0.f : __expf(s1[i] - n1);
      l0 += e0, l1 += e1;
      const int kstep = i >> 1, half = i & 1;    // a0 = (g, t), a1 = (g + 8, t), a2 = (g, t + 4), a3 = (g + 8, t + 4)
      const uint32_t h0 = to_tf32(e0), h1 = to_tf32(e1);
      phi[kstep][2 * half] = h0;
      phi[kstep][2 * half + 1] = h1;
      plo[kstep][2 * half] = to_tf32(e0 - __uint_as_float(h0));
      plo[kstep][2 * half + 1] = to_tf32(e1 - __uint_as_float(h1));
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= c0, o[i][1] *= c0, o[i][2] *= c1, o[i][3] *= c1;
    }
#pragma unroll
    for (int kstep = 0; kstep < 4; ++kstep) {
      const float* vb = ks + (size_t)(kstep * 8 + tq4) * DP + col0 + g;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const uint32_t b0 = __float_as_uint(vb[i * 8]), b1 = __float_as_uint(vb[4 * DP + i * 8]);
        mma_tf32(o[i], phi[kstep], b0, b1);
        mma_tf32(o[i], plo[kstep], b0, b1);
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + 8 * half, tq = r / HB, hh = r - tq * HB, h = head_base + hh;
    if (tq >= count || h >= H) continue;
    const int64_t t = first + tq;
    const float mr = half ? m1 : m0, lr = half ? l1 : l0;
    if (n_split == 1) {
      const float sk = __bfloat162float(sink[h]);
      const float top = fmaxf(mr, sk);
      const float e = __expf(mr - top);
      const float k = gate[t * H + h] * e / (lr * e + __expf(sk - top));
      T* dst = out + (t * H + h) * R + col0 + 2 * tq4;
#pragma unroll
      for (int i = 0; i < NT; ++i)
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * half] * k, o[i][2 * half + 1] * k);
    } else {
      const int64_t at = (t * H + h) * n_split + blockIdx.z;
      float* dst = part_o + at * R + col0 + 2 * tq4;
#pragma unroll
      for (int i = 0; i < NT; ++i) dst[i * 8] = o[i][2 * half], dst[i * 8 + 1] = o[i][2 * half + 1];
      if (warp == 0 && tq4 == 0) part_ml[at * 2] = mr, part_ml[at * 2 + 1] = lr;
    }
  }
}

__host__ __device__ inline bool mma_path(int dt, int H, int R, int dr) {
  (void)H;
  return dt == AO_LM_BF16 && R % 64 == 0 && R <= 512 && dr % 16 == 0;
}

// one CTA per (token, head): merges the key splits that hold keys this token sees, then sink, gate, normalisation
template <typename T>
__global__ void latent_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int32_t* __restrict__ pos, int H, int R, int tiles_per_split, int n_split,
                                         const T* __restrict__ sink, const float* __restrict__ gate, T* __restrict__ out) {
  __shared__ float wsplit[64];   // n_split <= 64: exp(m_s - top) / denominator, gate folded in
  __shared__ float red[2];
  const int64_t row = blockIdx.x;
  const int64_t t = row / H;
  const int h = (int)(row - t * H);
  const int ns = min(n_split, pos[t] / (tiles_per_split * kKeys) + 1);
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const float sk = ldf(sink + h);
    float m_a = lane < ns ? part_ml[(row * n_split + lane) * 2] : -INFINITY;
    float m_b = lane + 32 < ns ? part_ml[(row * n_split + lane + 32) * 2] : -INFINITY;
    const float top = fmaxf(warp_max(fmaxf(m_a, m_b)), sk);
    const float e_a = lane < ns ? __expf(m_a - top) : 0.f, e_b = lane + 32 < ns ? __expf(m_b - top) : 0.f;
    float den = (lane < ns ? part_ml[(row * n_split + lane) * 2 + 1] * e_a : 0.f) +
                (lane + 32 < ns ? part_ml[(row * n_split + lane + 32) * 2 + 1] * e_b : 0.f);
    den = warp_sum(den) + __expf(sk - top);
    const float k = gate[row] / den;
    wsplit[lane] = e_a * k;
    wsplit[lane + 32] = e_b * k;
    (void)red;
  }
  __syncthreads();
  // blockIdx.y: which 128 output coordinates (one per thread), so that a decoded token's few rows still fill many SMs
  const int d = blockIdx.y * blockDim.x + threadIdx.x;
  if (d < R) {
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < ns; ++s) acc = fmaf(part_o[(row * n_split + s) * R + d], wsplit[s], acc);
    stf(out + row * R + d, acc);
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
    latent_attn_merge_kernel<T><<<dim3((unsigned)(n * H), (unsigned)((R + 127) / 128)), 128, 0, st>>>(part_o, part_ml, pos, H, R, tps, n_split,
                                                                  static_cast<const T*>(sink), gate, static_cast<T*>(out));
  return lm_launch_status();
}

template <int NT>
int launch_mma(const float* qa, const float* qr, const void* c_cache, const void* kr_cache, int64_t S, const int32_t* slot,
               const int32_t* pos, const int32_t* tile_first, const int32_t* tile_count, int n_tiles, int64_t n, int H, int dr,
               float scale, const void* sink, const float* gate, int max_pos, int n_split, float* part_o, float* part_ml,
               void* out, cudaStream_t st) {
  using T = __nv_bfloat16;
  constexpr int R = 64 * NT;
  const int DP = R + dr + 4;
  const size_t smem = ((size_t)(2 * kMmaRows + kKeys) * DP + 2 * kMmaRows * 33) * sizeof(float);
  if (smem > 220 * 1024) return AO_B200_ERR_UNSUPPORTED;
  auto kern = latent_attn_mma_kernel<NT>;
  if (smem > 48 * 1024) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
      set = true;
    }
  }
  const int HB = H < kMmaRows ? H : kMmaRows;
  const int tiles = (max_pos + kKeys) / kKeys;
  const int tps = (tiles + n_split - 1) / n_split;
  dim3 grid((unsigned)n_tiles, (unsigned)((H + HB - 1) / HB), (unsigned)n_split);
  kern<<<grid, kWarps * 32, smem, st>>>(qa, qr, static_cast<const T*>(c_cache), static_cast<const T*>(kr_cache), S, slot, pos,
                                        tile_first, tile_count, n, H, dr, scale, HB, tps, n_split, static_cast<const T*>(sink),
                                        gate, static_cast<T*>(out), part_o, part_ml);
  if (n_split > 1)
    latent_attn_merge_kernel<T><<<dim3((unsigned)(n * H), (unsigned)((R + 127) / 128)), 128, 0, st>>>(part_o, part_ml, pos, H, R, tps, n_split,
                                                                  static_cast<const T*>(sink), gate, static_cast<T*>(out));
  return lm_launch_status();
}

}  // namespace

extern "C" int ao_lm_latent_attention_plan(int dt, int H, int R, int dr, int* tile_tokens) {
  LM_CHECK_ARG(H > 0 && R > 0 && dr >= 0 && tile_tokens);
  *tile_tokens = mma_path(dt, H, R, dr) ? kMmaRows / (H < kMmaRows ? H : kMmaRows) : kWarps / head_quads_per_cta(H);
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
  LM_CHECK_ARG(n > 0 && n_tiles > 0 && H > 0 && R > 0 && dr >= 0 && S > 0 && max_pos >= 0 && max_pos < S && n_split >= 1 && n_split <= 64);
  if (R > 512) return AO_B200_ERR_UNSUPPORTED;
  float *part_o = nullptr, *part_ml = nullptr;
  if (n_split > 1) {
    if (!workspace || workspace_bytes < ao_lm_latent_attention_workspace_bytes(n, H, R, n_split)) return AO_B200_ERR_WORKSPACE;
    part_o = static_cast<float*>(workspace);
    part_ml = part_o + n * H * n_split * (int64_t)R;
  }
  const cudaStream_t st = lm_stream(stream);
  if (mma_path(dt, H, R, dr)) {
#define LM_MMA(NT)                                                                                                            \
  case NT:                                                                                                                    \
    return launch_mma<NT>(qa, qr, c_cache, kr_cache, S, slot, pos, tile_first, tile_count, n_tiles, n, H, dr, scale, sink, gate, \
                          max_pos, n_split, part_o, part_ml, out, st);
    switch (R / 64) {
      LM_MMA(1) LM_MMA(2) LM_MMA(3) LM_MMA(4) LM_MMA(5) LM_MMA(6) LM_MMA(7) LM_MMA(8)
    }
#undef LM_MMA
  }
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
