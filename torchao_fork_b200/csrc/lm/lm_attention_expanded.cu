// Latent attention for prompt portions, in the expanded form: the caller up-projects the cached latents of a sequence
// into per-head keys and values once per step (two library GEMMs), and this kernel runs causal attention of a tile of
// consecutive tokens of ONE head over them.  Per (query, key) pair that is (dn + dr) + dv multiply-adds instead of the
// (R + dr) + R of the folded form that the decode kernel uses, and a 64-key tile is shared by 64 query rows.
//
// bf16 storage, mma.sync m16n8k16 with fp32 accumulators.  What the design computes in 32 bits stays in 32 bits:
//   scores   bf16 x bf16 products accumulated in fp32; the rotated query part (an fp32 rotation result) enters as TWO
//            bf16 parts (q = hi + lo to 2^-17), the cached keys are bf16 as stored;
//   weights  exp(s - max) in fp32, multiplied into the values as THREE bf16 parts (p = p1 + p2 + p3 exactly, 24 bits),
//            the denominator summed in fp32 from the unsplit weights;
//   sink, gate, normalisation in fp32.
// One CTA = 64 consecutive tokens of one sequence x one head (4 warps x 16 rows).  K and V tiles arrive by cp.async in
// separate groups: the next keys load while the weights meet the values, the next values during the score product.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kPM = 64;      // query rows per CTA
constexpr int kPN = 64;      // keys per tile
constexpr int kPWarps = 4;
constexpr int kPad = 8;      // bf16 elements added to every shared-memory row: 16-byte rows land on distinct banks

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// x -> (bf16 part, what is left of x); the remainder is exact in fp32
__device__ __forceinline__ float split_bf16(float& x) {
  const float h = __bfloat162float(__float2bfloat16_rn(x));
  x -= h;
  return h;
}

template <int NV>   // value size = 16 NV
__global__ void __launch_bounds__(kPWarps * 32)
latent_attn_expanded_kernel(const __nv_bfloat16* __restrict__ qn, const float* __restrict__ qr,
                            const __nv_bfloat16* __restrict__ kx, const __nv_bfloat16* __restrict__ vx,
                            const __nv_bfloat16* __restrict__ kr_cache, int64_t S, const int32_t* __restrict__ slot,
                            const int32_t* __restrict__ pos, const int32_t* __restrict__ tile_first,
                            const int32_t* __restrict__ tile_count, const int32_t* __restrict__ tile_kv_row, int64_t n, int H,
                            int dn, int dr, float scale, const __nv_bfloat16* __restrict__ sink,
                            const float* __restrict__ gate, __nv_bfloat16* __restrict__ out) {
  using T = __nv_bfloat16;
  constexpr int DV = 16 * NV;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int DK = dn + dr, QP = DK + dr + kPad, KP = DK + kPad, VP = DV + kPad;
  T* Qs = reinterpret_cast<T*>(smem_raw);   // [kPM][QP]: unrotated | rotated, high part | rotated, low part
  T* Ks = Qs + (size_t)kPM * QP;            // [kPN][KP]: unrotated key of this head | rotated key part of the row
  T* Vs = Ks + (size_t)kPN * KP;            // [kPN][VP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int h = blockIdx.y;
  const int tile = gridDim.x - 1 - blockIdx.x;   // a prompt's last tiles see the most keys: they start first
  const int first = tile_first[tile], count = min(tile_count[tile], kPM);
  const int64_t seq = slot[first];
  const int64_t row0 = tile_kv_row[tile];
  const int pos0 = pos[first];
  const int k_hi = pos[first + count - 1] + 1;   // keys 0 .. the last row's position
  const T* kbase = kx + row0 * (int64_t)H * dn + (int64_t)h * dn;
  const T* vbase = vx + row0 * (int64_t)H * DV + (int64_t)h * DV;
  const T* rbase = kr_cache + seq * S * dr;
  const int kc_n = dn / 8, kc = kc_n + dr / 8;   // 16-byte chunks of a key row
  constexpr int vc = DV / 8;

  auto load_k = [&](int k0) {
    for (int i = threadIdx.x; i < kPN * kc; i += kPWarps * 32) {
      const int j = i / kc, c = i - j * kc, key = k0 + j;
      T* dst = Ks + (size_t)j * KP + c * 8;
      if (key < k_hi)
        cp_async16(dst, c < kc_n ? kbase + (int64_t)key * H * dn + c * 8 : rbase + (int64_t)key * dr + (c - kc_n) * 8);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  };
  auto load_v = [&](int k0) {
    for (int i = threadIdx.x; i < kPN * vc; i += kPWarps * 32) {
      const int j = i / vc, c = i - j * vc, key = k0 + j;
      T* dst = Vs + (size_t)j * VP + c * 8;
      if (key < k_hi)
        cp_async16(dst, vbase + (int64_t)key * H * DV + c * 8);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  };
  load_k(0);
  cp_async_commit();
  load_v(0);
  cp_async_commit();
  // the query tile (rows past the run are zero)
  for (int i = threadIdx.x; i < kPM * kc_n; i += kPWarps * 32) {
    const int r = i / kc_n, c = i - r * kc_n;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < count) v = *reinterpret_cast<const uint4*>(qn + ((int64_t)h * n + first + r) * dn + c * 8);
    *reinterpret_cast<uint4*>(Qs + (size_t)r * QP + c * 8) = v;
  }
  for (int i = threadIdx.x; i < kPM * (dr / 4); i += kPWarps * 32) {
    const int r = i / (dr / 4), d = (i - r * (dr / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < count) v = *reinterpret_cast<const float4*>(qr + ((int64_t)(first + r) * H + h) * dr + d);
    float x[4] = {v.x, v.y, v.z, v.w}, hi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) hi[e] = split_bf16(x[e]);
    T* qh = Qs + (size_t)r * QP + dn + d;
    *reinterpret_cast<uint2*>(qh) = make_uint2(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]));
    *reinterpret_cast<uint2*>(qh + dr) = make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
  }
  float o[2 * NV][4];
#pragma unroll
  for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows 16 warp + g and + 8 (l: this thread's share)
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  const int p0 = r0 < count ? pos0 + r0 : -1, p1 = r1 < count ? pos0 + r1 : -1;
  // ldmatrix row addresses of this lane: A (queries), B (keys), B transposed (values)
  const T* qa_ptr = Qs + (size_t)(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QP + (lane >> 4) * 8;
  const T* kb_ptr = Ks + (size_t)((lane & 7) + (lane >> 4) * 8) * KP + ((lane >> 3) & 1) * 8;
  const T* vb_ptr = Vs + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * VP + (lane >> 4) * 8;
  const int ks_main = DK / 16, ks_lo = dr / 16, ks_n = dn / 16;
  // a warp whose rows all come before a key tile skips the tile (its weights there are all zero)
  const int warp_last = min(count, warp * 16 + 16) - 1;             // < warp * 16: the warp has no rows
  const int warp_hi = warp_last >= warp * 16 ? pos0 + warp_last + 1 : 0;

  for (int k0 = 0; k0 < k_hi; k0 += kPN) {
    cp_async_wait<1>();
    __syncthreads();   // keys of this tile (and, the first time, the queries) are in shared memory
    float s[kPN / 8][4];
#pragma unroll
    for (int i = 0; i < kPN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const bool live = k0 < warp_hi;
    if (live) {
      for (int kk = 0; kk < ks_main + ks_lo; ++kk) {
        uint32_t a[4];
        ldsm_x4(a, qa_ptr + kk * 16);
        const int kcol = (kk < ks_main ? kk : ks_n + (kk - ks_main)) * 16;   // the low query part meets the rotated keys again
#pragma unroll
        for (int j = 0; j < kPN / 16; ++j) {
          uint32_t b[4];
          ldsm_x4(b, kb_ptr + (size_t)j * 16 * KP + kcol);
          mma_bf16(s[2 * j], a, b[0], b[1]);
          mma_bf16(s[2 * j + 1], a, b[2], b[3]);
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPN / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = k0 + i * 8 + 2 * t4 + e;
        s[i][e] = key <= p0 ? s[i][e] * scale : -INFINITY;
        s[i][2 + e] = key <= p1 ? s[i][2 + e] * scale : -INFINITY;
        mx0 = fmaxf(mx0, s[i][e]);
        mx1 = fmaxf(mx1, s[i][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float c0 = n0 == -INFINITY ? 1.f : __expf(m0 - n0), c1 = n1 == -INFINITY ? 1.f : __expf(m1 - n1);
    m0 = n0, m1 = n1;
    l0 *= c0, l1 *= c1;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) o[i][0] *= c0, o[i][1] *= c0, o[i][2] *= c1, o[i][3] *= c1;
#pragma unroll
    for (int i = 0; i < kPN / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        s[i][e] = n0 == -INFINITY ? 0.f : __expf(s[i][e] - n0);
        s[i][2 + e] = n1 == -INFINITY ? 0.f : __expf(s[i][2 + e] - n1);
        l0 += s[i][e];
        l1 += s[i][2 + e];
      }
    }
    cp_async_wait<0>();
    __syncthreads();   // values of this tile are in shared memory, and every warp is done with its keys
    const bool more = k0 + kPN < k_hi;
    if (more) load_k(k0 + kPN);   // lands while the weights meet the values
    cp_async_commit();
    if (live) {
      // the three bf16 parts of the weights as A fragments; every value fragment is loaded once and meets all three
      uint32_t pa[3][kPN / 16][4];
#pragma unroll
      for (int part = 0; part < 3; ++part) {
#pragma unroll
        for (int j = 0; j < kPN / 16; ++j) {
          const float h00 = split_bf16(s[2 * j][0]), h01 = split_bf16(s[2 * j][1]);
          const float h10 = split_bf16(s[2 * j][2]), h11 = split_bf16(s[2 * j][3]);
          const float h20 = split_bf16(s[2 * j + 1][0]), h21 = split_bf16(s[2 * j + 1][1]);
          const float h30 = split_bf16(s[2 * j + 1][2]), h31 = split_bf16(s[2 * j + 1][3]);
          pa[part][j][0] = pack_bf16(h00, h01);
          pa[part][j][1] = pack_bf16(h10, h11);
          pa[part][j][2] = pack_bf16(h20, h21);
          pa[part][j][3] = pack_bf16(h30, h31);
        }
      }
#pragma unroll
      for (int j = 0; j < kPN / 16; ++j) {
#pragma unroll
        for (int v0 = 0; v0 < NV; v0 += 4) {   // four fragments at a time: eight accumulators between two uses of one
          uint32_t b[4][4];
#pragma unroll
          for (int vv = 0; vv < 4; ++vv)
            if (v0 + vv < NV) ldsm_x4_trans(b[vv], vb_ptr + (size_t)j * 16 * VP + (v0 + vv) * 16);
#pragma unroll
          for (int part = 0; part < 3; ++part) {
#pragma unroll
            for (int vv = 0; vv < 4; ++vv) {
              if (v0 + vv < NV) {
                mma_bf16(o[2 * (v0 + vv)], pa[part][j], b[vv][0], b[vv][1]);
                mma_bf16(o[2 * (v0 + vv) + 1], pa[part][j], b[vv][2], b[vv][3]);
              }
            }
          }
        }
      }
    }
    __syncthreads();   // every warp is done with this tile's values
    if (more) load_v(k0 + kPN);   // lands during the next tile's score product
    cp_async_commit();
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float sk = __bfloat162float(sink[h]);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r1 : r0;
    if (r >= count) continue;
    const int64_t t = first + r;
    const float mr = half ? m1 : m0, lr = half ? l1 : l0;
    const float top = fmaxf(mr, sk);
    const float e = __expf(mr - top);
    const float k = gate[t * H + h] * e / (lr * e + __expf(sk - top));
    T* dst = out + (t * H + h) * DV + 2 * t4;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i)
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * half] * k, o[i][2 * half + 1] * k);
  }
}

inline bool expanded_ok(int dt, int dn, int dr, int dv) {
  if (dt != AO_LM_BF16 || dn <= 0 || dn % 16 || dr % 16 || dv % 16 || dv < 16 || dv > 128) return false;
  const size_t smem = ((size_t)kPM * (dn + 2 * dr + kPad) + (size_t)kPN * (dn + dr + kPad) + (size_t)kPN * (dv + kPad)) * 2;
  return smem <= 200 * 1024;
}

template <int NV>
int launch_expanded(const void* qn, const float* qr, const void* kx, const void* vx, const void* kr_cache, int64_t S,
                    const int32_t* slot, const int32_t* pos, const int32_t* tile_first, const int32_t* tile_count,
                    const int32_t* tile_kv_row, int n_tiles, int64_t n, int H, int dn, int dr, float scale, const void* sink,
                    const float* gate, void* out, cudaStream_t st) {
  using T = __nv_bfloat16;
  const size_t smem = ((size_t)kPM * (dn + 2 * dr + kPad) + (size_t)kPN * (dn + dr + kPad) + (size_t)kPN * (16 * NV + kPad)) * 2;
  auto kern = latent_attn_expanded_kernel<NV>;
  if (smem > 48 * 1024) {
    static bool set = false;   // per instantiation
    if (!set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
      set = true;
    }
  }
  dim3 grid((unsigned)n_tiles, (unsigned)H);
  kern<<<grid, kPWarps * 32, smem, st>>>(static_cast<const T*>(qn), qr, static_cast<const T*>(kx), static_cast<const T*>(vx),
                                         static_cast<const T*>(kr_cache), S, slot, pos, tile_first, tile_count, tile_kv_row, n, H,
                                         dn, dr, scale, static_cast<const T*>(sink), gate, static_cast<T*>(out));
  return lm_launch_status();
}

}  // namespace

extern "C" int ao_lm_latent_attention_expanded_plan(int dt, int dn, int dr, int dv, int* tile_tokens) {
  LM_CHECK_ARG(tile_tokens);
  *tile_tokens = expanded_ok(dt, dn, dr, dv) ? kPM : 0;
  return AO_B200_OK;
}

extern "C" int ao_lm_latent_attention_expanded(const void* qn, const float* qr, const void* kx, const void* vx,
                                               const void* kr_cache, int dt, int64_t S, const int32_t* slot,
                                               const int32_t* pos, const int32_t* tile_first, const int32_t* tile_count,
                                               const int32_t* tile_kv_row, int n_tiles, int64_t n, int H, int dn, int dr, int dv,
                                               float scale, const void* sink, const float* gate, void* out, void* stream) {
  LM_CHECK_ARG(qn && kx && vx && slot && pos && tile_first && tile_count && tile_kv_row && sink && gate && out);
  LM_CHECK_ARG((qr && kr_cache) || dr == 0);
  LM_CHECK_ARG(n > 0 && n_tiles > 0 && H > 0 && H <= 65535 && S > 0);
  if (!expanded_ok(dt, dn, dr, dv)) return AO_B200_ERR_UNSUPPORTED;
  const cudaStream_t st = lm_stream(stream);
#define LM_XP(NV)                                                                                                          \
  case NV:                                                                                                                 \
    return launch_expanded<NV>(qn, qr, kx, vx, kr_cache, S, slot, pos, tile_first, tile_count, tile_kv_row, n_tiles, n, H, dn, \
                               dr, scale, sink, gate, out, st);
  switch (dv / 16) { LM_XP(1) LM_XP(2) LM_XP(3) LM_XP(4) LM_XP(5) LM_XP(6) LM_XP(7) LM_XP(8) }
#undef LM_XP
  return AO_B200_ERR_UNSUPPORTED;
}
