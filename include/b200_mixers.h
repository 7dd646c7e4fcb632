/*
 * b200_mixers.h — C ABI of the ragged-batch sequence mixers and feed-forward pieces (libb200_mixers.so, sm_100a).
 *
 * Same conventions as b200_kv.h: extern "C", device pointers owned by the caller, work queued on `stream`
 * (a cudaStream_t passed as void*), nothing allocates or synchronises, 0 on success, negative B200_E* or a positive
 * cudaError_t otherwise with the text in b200_mixers_last_error().  `dtype` is the storage type T of activations,
 * weights and pools (0 = float16, 1 = float32, 2 = bfloat16).  The residual stream, norm statistics, attention
 * scores and weights, recurrence gates and state are fp32 for every T.
 *
 * A step's tokens are PACKED: row n of every activation is one token; the tokens of a sequence are consecutive and
 * in order.  tok_pos[n] is the token's position in its sequence.
 */
#ifndef B200_MIXERS_H_
#define B200_MIXERS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_MIXERS_ABI_VERSION 1

int b200_mixers_abi_version(void);
const char* b200_mixers_last_error(void);

/* out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * (1 + weight);  x fp32 [rows, width], out T [rows, width]. */
int b200_offset_rmsnorm(void* out, const float* x, const void* weight, float eps, int rows, int width, int dtype,
                        void* stream);

/* x[r] += mult * offset_norm(y[r]; w_post) in fp32 (x is updated in place); when w_next is given, out_next[r] =
 * offset_norm(x[r]; w_next) in T — the next sublayer's input.  y is T, or fp32 when y_is_f32. */
int b200_postnorm_residual(float* x, const void* y, int64_t y_stride, int y_is_f32, const void* w_post, float mult,
                           const void* w_next, void* out_next, float eps, int rows, int width, int dtype, void* stream);

/* Per token and kv head: v <- v / rms(v) (eps inside the root); with v_prev [n_tok, G*dv]: v <- (1 - lam) v + lam
 * v_prev.  The result (rounded to T) is scattered with k through slot_mapping (slot = block * block_size + offset,
 * negative = skip) into k_pool [max_blocks, G, block_size, dk] and v_pool [max_blocks, G, block_size, dv], and
 * copied to v_keep [n_tok, G*dv] when given. */
int b200_value_prep_append(const void* k, int64_t k_stride, const void* v, int64_t v_stride, const void* v_prev,
                           void* v_keep, float lam, float eps, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                           int n_tok, int G, int dk, int dv, int block_size, int64_t max_blocks, int dtype, void* stream);

/* Tokens of one sequence that a CTA of b200_biased_paged_attn serves at most (cut portions into tiles of this). */
int b200_biased_attn_tile_tokens(int n_tokens_in_portion, int H, int G);

/* Causal attention of packed query rows over the paged cache (which already holds this step's keys and values).
 *   score(i, j) = (q_i . k_j) * scale * (1 + temp_coef * ln(floor((i + 1) / temp_every) + 1)) + bias_lut[h][min(i - j, lut_len - 1)]
 *   out[n, h, :] = sigmoid(gate[n, h]) * softmax_j(score) . v_j          (gate may be NULL)
 * tiles: int32 [n_tiles, 3] = (first packed row, token count <= max_tile_tokens, block-table row); a tile's tokens
 * belong to one sequence.  bias_lut: fp32 [H, lut_len].  q: T rows of H*dk with row stride q_stride; out: T
 * [n_tok, H*dv] contiguous. */
int b200_biased_paged_attn(void* out, const void* q, int64_t q_stride, const void* gate, int64_t gate_stride,
                           const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                           const int32_t* tiles, int n_tiles, int max_tile_tokens, const int32_t* tok_pos,
                           const float* bias_lut, int lut_len, float scale, float temp_coef, int temp_every, int H, int G,
                           int dk, int dv, int block_size, int dtype, void* stream);

/* The same attention on the tensor cores (16-bit dtypes; dk a multiple of 16 up to 256, dv a multiple of 8 up to
 * 128 — b200_biased_prompt_attn_supported says whether a layer qualifies).  A CTA serves 64 rows = the tokens of a tile
 * times the query heads of one kv head, so tiles hold up to b200_biased_prompt_attn_tile_tokens(H, G) = 64 / (H / G)
 * tokens; a tile's tokens have consecutive positions.  Prompt portions and single decoded tokens alike: when no tile
 * has more than max_tile_tokens tokens and that many tokens are at most 16 rows, the warps of a CTA split the keys
 * instead of the rows (pass 0 when unknown).  Scores, bias and softmax are fp32; the softmax
 * weights are rounded to the storage type only as the operand of the P.V product.  Rows written: the tiles' tokens. */
int b200_biased_prompt_attn_supported(int dk, int dv, int dtype);
int b200_biased_prompt_attn_tile_tokens(int H, int G);
int b200_biased_prompt_attn(void* out, const void* q, int64_t q_stride, const void* gate, int64_t gate_stride,
                            const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                            const int32_t* tiles, int n_tiles, int max_tile_tokens, const int32_t* tok_pos,
                            const float* bias_lut, int lut_len, float scale, float temp_coef, int temp_every, int H, int G,
                            int dk, int dv, int block_size, int dtype, void* stream);

/* Gated linear recurrence per (sequence, head) over the sequence's tokens of this step, in order:
 *   q = silu(zq), f = lower + (1 - lower) * sigmoid(zf + f_bias), S <- diag(f) S + (1 - f) v^T, o = S^T q.
 * state: fp32 [slots, H, dk, dv]; seqs: int32 [n_seqs, 4] = (first packed row, token count, state slot, fresh);
 * fresh != 0 starts from a zero state.  The final state is written back.  o_raw: fp32 [n_tok, H, dv].  max_count: the
 * largest token count among seqs (a hint: portions of 8 tokens or more and key sizes up to 128 take the kernel that
 * keeps the state in registers, steps of single tokens the one that keeps it in shared memory). */
int b200_gated_scan(float* o_raw, const void* zq, const void* zf, const void* v, int64_t in_stride, const void* f_bias,
                    const void* lower, float* state, const int32_t* seqs, int n_seqs, int max_count, int H, int dk, int dv,
                    int dtype, void* stream);

/* out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * weight;  x fp32 [rows, dv], weight T [dv], out T. */
int b200_head_rmsnorm(void* out, const float* x, const void* weight, float eps, int64_t rows, int dv, int dtype,
                      void* stream);

/* out[r] = a N(z) + b N(z^2) + c N(z^3) + e with N(u) = u * rsqrt(mean(u^2) + eps) over the row; coef = (a, b, c, e). */
int b200_polynorm(void* out, const void* z, int64_t z_stride, const void* coef, float eps, int rows, int ff, int dtype,
                  void* stream);

/* The `top` largest of E fp32 logits per token (ties: lowest index); weights = sigmoid(logit). */
int b200_sigmoid_topk(int32_t* ids, float* weights, const float* logits, int n_tok, int E, int top, void* stream);

/* xs[r] = T(weights[src[r]] * h[src[r] / top]): the expert-sorted, input-scaled rows. */
int b200_scaled_gather(void* xs, const void* h, const float* weights, const int64_t* src, int64_t n_rows, int top,
                       int width, int dtype, void* stream);

/* Grouped linear over expert-sorted rows (16-bit dtypes, K a multiple of 8): out[r] = xs[r] . w[e]^T for
 * offsets[e] <= r < offsets[e + 1].  xs T [rows, K], w T [E, N, K], offsets int32 [E + 1] ON THE DEVICE, out T [rows, N].
 * max_rows: a bound on the rows of any one expert (the total row count will do); it sizes the grid only. */
int b200_grouped_linear_supported(int K, int dtype);
int b200_grouped_linear(void* out, const void* xs, const void* w, const int32_t* offsets, int64_t max_rows, int E, int N,
                        int K, int dtype, void* stream);

/* y = g' * sigmoid(alpha * g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit); gu rows = g | u. */
int b200_clamped_glu(void* y, const void* gu, int64_t rows, int ff, float limit, float alpha, int dtype, void* stream);

/* out[n] = sum over k (ascending) of ys[where[n * top + k]], fp32. */
int b200_expert_combine(float* out, const void* ys, const int64_t* where, int64_t n_tok, int top, int width, int dtype,
                        void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MIXERS_H_ */
