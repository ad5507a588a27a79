/*
 * ao_b200_lm.h — C ABI of libao_b200_lm.so: B200 (sm_100a) kernels of the sequence-model mechanisms that are not
 * weight-only linears: fp32 residual stream with scalar-weight RMS norms, token shift, depth-weighted averaging of
 * layer results, latent (compressed key/value) attention with a softmax sink and an output gate, clipped-GLU experts
 * with a softmax top-k router.  Every constant of a mechanism is a parameter.
 *
 * Same boundary rules as ao_b200.h: device pointers + sizes + cudaStream_t as void*; nothing is allocated, freed,
 * synchronised or retained; every entry point can be captured into a CUDA graph; 0 = ok, else an AO_B200_ERR_* code.
 *
 * `dt` selects the storage type of weights, activations and caches: AO_LM_BF16 or AO_LM_F32.  The residual stream,
 * norm statistics, rotary angles, attention scores / weights and router scores are fp32 in both modes.
 * Per-token metadata lives in device memory: slot[t] = which sequence state the token belongs to, pos[t] = its
 * position in that sequence.  Tokens of one sequence are contiguous and in order.
 */
#ifndef AO_B200_LM_H_
#define AO_B200_LM_H_

#include "ao_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { AO_LM_BF16 = 0, AO_LM_F32 = 1 };

AO_B200_API int ao_lm_abi_version(void);

/* x[t][:] = table[tok[t]][:]  (fp32 out) */
AO_B200_API int ao_lm_embed(const void* table, int dt, const int64_t* tok, int64_t n, int64_t width, float* x, void* stream);

/* h[t] = x[t] + (prev - x[t]) * mu, prev = x[t-1] if that row is the same sequence's previous position, the saved row
 * state[slot[t]] if the sequence continues from an earlier step, zeros at position 0.  h is written in `dt`. */
AO_B200_API int ao_lm_token_shift(const float* x, const void* mu, int dt, const float* state, const int32_t* slot,
                                  const int32_t* pos, int64_t n, int64_t width, void* h, void* stream);

/* x_out = x_in + mult * g * y / sqrt(mean(y^2) + eps)   (g: ONE number, stored in `dt`; y in `y_dt`).
 * Optional, each skipped when its pointer is null:
 *   state:   the last row of every sequence in the batch saves x_in into state[slot] (the token-shift memory);
 *   streams: avg = sum_{j < n_streams} coef[j] * streams[j * stream_stride + ...] + coef[n_streams] * x_out  -> avg_out;
 *   cast_out: the last value computed (avg if streams, else x_out) in `dt`. */
AO_B200_API int ao_lm_residual_norm(const float* x_in, const void* y, int y_dt, const void* g, int dt, float mult, float eps,
                                    int64_t n, int64_t width, float* x_out, float* state, const int32_t* slot,
                                    const float* streams, int n_streams, int64_t stream_stride, const void* coef,
                                    float* avg_out, void* cast_out, void* stream);

/* out[i] = g * x[rows[i]] / sqrt(mean(x[rows[i]]^2) + eps) in `dt`; rows == null: all m rows in order. */
AO_B200_API int ao_lm_scalar_norm_rows(const float* x, const int32_t* rows, int64_t m, int64_t width, const void* g, int dt,
                                       float eps, void* out, void* stream);

/* Splits one projection row [q (H heads x (dn | dr)) at q_off | latent (R | dr) at kv_off, -1 = none | H gate logits
 * at g_off] of proj[n][ld]:
 *   qn[h][t][dn]  unrotated query parts, head-major, in `dt`;      qr[t][h][dr] rotated parts, fp32;
 *   gate[t][h] = sigmoid(logit), fp32;
 *   c_cache[slot][pos][R] = RMS norm (weight c_norm, eps) of the latent;  kr_cache[slot][pos][dr] = rotated shared key part.
 * Rotation: pairs (2i, 2i+1), i < rot_dims / 2, angle pos * inv_freq[i]; coordinates >= rot_dims pass through. */
AO_B200_API int ao_lm_latent_prep(const void* proj, int dt, int64_t ld, int64_t n, int H, int dn, int dr, int R, int64_t q_off,
                                  int64_t kv_off, int64_t g_off, const void* c_norm, float eps, int rot_dims,
                                  const float* inv_freq, const int32_t* slot, const int32_t* pos, void* c_cache,
                                  void* kr_cache, int64_t S, void* qn, float* qr, float* gate, void* stream);

/* Attention of (token, head) rows over the cached latents of their sequence, keys 0 .. pos[t]:
 *   score_j = scale * (qa[h][t] . c_j + qr[t][h] . kr_j);  weights = softmax with exp(sink[h]) added to the denominator;
 *   out[t][h][:] = gate[t][h] * sum_j weight_j * c_j      (R numbers, in `dt`).
 * tile_first / tile_count [n_tiles]: runs of <= tile_tokens consecutive rows of ONE sequence (ao_lm_latent_attention_plan
 * gives tile_tokens for a storage type and shape).  1 < n_split <= 64 splits the keys over CTAs (max_pos + 1 keys are
 * covered; workspace from ao_lm_latent_attention_workspace_bytes).
 * bf16 storage with R a multiple of 64 (<= 512) and dr a multiple of 16 runs on the tensor cores: queries and weights stay
 * fp32, split into two TF32 parts each, against the cached rows (exact in TF32); every other case is fp32 FMA code. */
AO_B200_API int ao_lm_latent_attention_plan(int dt, int H, int R, int dr, int* tile_tokens);
AO_B200_API int64_t ao_lm_latent_attention_workspace_bytes(int64_t n, int H, int R, int n_split);
AO_B200_API int ao_lm_latent_attention(const float* qa, const float* qr, const void* c_cache, const void* kr_cache, int dt,
                                       int64_t S, const int32_t* slot, const int32_t* pos, const int32_t* tile_first,
                                       const int32_t* tile_count, int n_tiles, int64_t n, int H, int R, int dr, float scale,
                                       const void* sink, const float* gate, int max_pos, int n_split, void* workspace,
                                       int64_t workspace_bytes, void* out, void* stream);

/* The same attention for prompt portions, in the expanded form (bf16 storage; tensor cores): the caller has up-projected
 * the cached latents of every sequence in the step into keys kx[row][h][dn] and values vx[row][h][dv], the rows of one
 * sequence contiguous from key 0;
 *   score_j = scale * (qn[h][t] . kx_j[h] + qr[t][h] . kr_j);  the same sink, gate and causal mask;  out[t][h][dv] in bf16.
 * tile_first / tile_count [n_tiles]: runs of <= tile_tokens consecutive rows of ONE sequence at consecutive positions;
 * tile_kv_row[tile]: the row of kx / vx that holds key 0 of the tile's sequence.  The plan call gives tile_tokens, or 0
 * when the shape is not covered (dn, dr, dv multiples of 16, dv up to 128): use ao_lm_latent_attention then.
 * Scores accumulate in fp32 (the fp32 rotated query part as two bf16 parts); the fp32 weights enter the value product
 * as three bf16 parts, i.e. exactly. */
AO_B200_API int ao_lm_latent_attention_expanded_plan(int dt, int dn, int dr, int dv, int* tile_tokens);
AO_B200_API int ao_lm_latent_attention_expanded(const void* qn, const float* qr, const void* kx, const void* vx,
                                                const void* kr_cache, int dt, int64_t S, const int32_t* slot,
                                                const int32_t* pos, const int32_t* tile_first, const int32_t* tile_count,
                                                const int32_t* tile_kv_row, int n_tiles, int64_t n, int H, int dn, int dr,
                                                int dv, float scale, const void* sink, const float* gate, void* out,
                                                void* stream);

/* Router: scores = softmax over all E logits (fp32 accumulation of h . w_router[e]); the `top` largest (ties: lowest
 * index) -> idx[t][top], weight[t][top] = their scores, not renormalised. */
AO_B200_API int ao_lm_router_topk(const void* h, const void* w_router, int dt, int64_t n, int64_t width, int E, int top,
                                  int32_t* idx, float* weight, void* stream);
/* The same choice from fp32 logits[n][E] that a GEMM has made (prompt portions). */
AO_B200_API int ao_lm_router_topk_logits(const float* logits, int64_t n, int E, int top, int32_t* idx, float* weight,
                                         void* stream);

/* Clipped GLU: g = min(a, limit), u = clamp(b, -limit, limit), y = g * sigmoid(alpha * g) * (u + 1).
 *   ao_lm_glu_act: gu[n][2 ff] = (a | b) -> y[n][ff].
 *   ao_lm_expert_gate_up: per (token, choice) pair p (t = p / top, expert = idx ? idx[p] : 0): a = w_gate[e] h[t],
 *       b = w_up[e] h[t] -> y[p][ff]        (w_gate / w_up: expert e's [ff][width] block starts expert_stride elements
 *       after expert e-1's, so one [E][2 ff][width] tensor can hold both).
 *   ao_lm_expert_down: out[t] (fp32) = (accumulate ? out[t] : 0) + sum_k weight[t][k] * w_down[e_k] y[t][k]
 *       (w_down: [E][width][ff]; weight == null: 1). */
AO_B200_API int ao_lm_glu_act(const void* gu, int dt, int64_t n, int64_t ff, float limit, float alpha, void* y, void* stream);
AO_B200_API int ao_lm_expert_gate_up(const void* h, const void* w_gate, const void* w_up, int dt, const int32_t* idx, int64_t n,
                                     int top, int64_t width, int64_t ff, int64_t expert_stride, float limit, float alpha,
                                     void* y, void* stream);
AO_B200_API int ao_lm_expert_down(const void* y, const void* w_down, int dt, const int32_t* idx, const float* weight, int64_t n,
                                  int top, int64_t width, int64_t ff, int accumulate, float* out, void* stream);

/* Prompt-sized mixtures: rows sorted by expert.  gather: xs[i] = h[src[i] / top]; scatter: out[src[i] / top] +=
 * weight[src[i]] * y[i] (fp32 atomics; out must hold the shared expert's output or zeros before). */
AO_B200_API int ao_lm_gather_rows(const void* h, int dt, const int64_t* src, int top, int64_t m, int64_t width, void* xs,
                                  void* stream);
AO_B200_API int ao_lm_scatter_add_rows(const void* y, int dt, const int64_t* src, const float* weight, int top, int64_t m,
                                       int64_t width, float* out, void* stream);

/* out[t][:] (fp32) = a[t][:] (fp32) + b[t][:] (dt) */
AO_B200_API int ao_lm_add_cast(const void* b, int dt, int64_t count, float* a_inout, void* stream);

/* greedy choice: out[b] = index of the largest of logits[b][0..V) (first one on ties) */
AO_B200_API int ao_lm_argmax(const float* logits, int64_t ld, int64_t B, int64_t V, int64_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif
