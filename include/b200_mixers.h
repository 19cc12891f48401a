/* C ABI of libb200mixers.so: sequence-mixing and normalisation kernels for decoder layers that are not plain softmax
 * attention -- Dynamic-Tanh normalisation fused with the residual update, sliding-window attention with sigmoid weights,
 * short causal convolutions, the gated delta rule, gated linear attention and RWKV-style recurrences, token shift, layer norm
 * fused with the residual update, PolyNorm, gated RMS output norm, soft-capped logits, softmax attention over strided or latent
 * caches (capped scores, sinks), routers and experts of mixtures of experts.  All pointers are device pointers; every function enqueues on `stream` and returns 0 or a cudaError_t.
 *
 * dtype: 0 = float, 1 = bfloat16, 2 = half: the type of activations AND of parameters (a model lives in one type).
 * Whatever the dtype, the residual stream, attention scores and weights, every normalisation and everything inside a
 * recurrence (state, decays, gates, unit vectors) are 32-bit floats.
 *
 * Batches: a row holds S new tokens that follow the tokens of earlier calls; `slot0` numbers the first new token's slot
 * (the same for all rows) and `pad[b]` is row b's left padding: its token in slot c has position c - pad[b] and does not
 * exist when that is negative. */
#ifndef B200_MIXERS_H
#define B200_MIXERS_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct CUstream_st* mixers_stream_t;

/* x[n, :] = float(table[ids[n], :]) */
int mixers_embed_rows(int dtype, const void* table, const int64_t* ids, long n_rows, int width, float* x, mixers_stream_t stream);

/* x += tanh(post_alpha * y) * post_w + post_b   (if y);   x += add (if add);   out = tanh(pre_alpha * x) * pre_w + pre_b (if out).
 * x: float [n_rows, width], updated in place; y, out: dtype [n_rows, width]; vectors [width]; alphas: one element each. */
int mixers_dyt_residual_norm(int dtype, float* x, long n_rows, int width, const void* y, const void* post_w, const void* post_b,
                             const void* post_alpha, const void* add, const void* pre_w, const void* pre_b, const void* pre_alpha,
                             void* out, mixers_stream_t stream);

/* Queries, keys and values of new tokens taken from the columns of one projection output `proj` [B, S, ld]: per-head RMS norm
 * (weights q_w / k_w [dim]), rotation of the pairs (2i, 2i+1), i < rot_dims / 2, by position * inv_freq[i] (doubles: the angle is formed and its sine / cosine taken in double precision); queries go to
 * q_out float [B, S, heads, dim], keys and values into the caches k_store [B, kv_heads, cap, dim] / v_store [.., vdim] at
 * storage index held + t.  The token at storage index j sits in slot j + shift.  dyn (may be null): a device word that holds
 * `held` instead of the argument, for a step that is replayed from a CUDA graph while the cache grows. */
int mixers_window_qk_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads,
                             int kv_heads, int dim, int vdim, const void* q_w, const void* k_w, float eps, const double* inv_freq,
                             int rot_dims, float* q_out, void* k_store, void* v_store, int cap, int held, int shift,
                             const int32_t* pad, const int32_t* dyn, mixers_stream_t stream);

/* out[b, t, out_col + h * vdim + :] = out_scale * sum_j sigmoid(q . k_j * scale + head_bias[h]) v_j over the keys j of the same
 * row with 0 <= c - j < window (c = held + t the query's own storage index) that are not padding.  out: dtype [B * S, ld_out]. */
int mixers_sigmoid_window_attention(int dtype, const float* q, const void* k_store, const void* v_store, int B, int S, int heads,
                                    int kv_heads, int dim, int vdim, int cap, int held, int shift, const int32_t* pad, int window,
                                    float scale, const void* head_bias, void* out, int ld_out, int out_col, float out_scale,
                                    const int32_t* dyn, mixers_stream_t stream);

/* y[b, t, c] = silu(sum_j w[c, j] * in(t - taps + 1 + j)): in(t') = proj[b, t', off + c] for a new token, tail[b, taps-1+t', c]
 * for t' < 0, zero for padding.  tail_next receives the last taps-1 inputs (for S == 1 it may be `tail` itself: a thread
 * then owns its channel's whole tail).  w: [C, taps]; tails: [B, max(taps-1,1), C].  In this and the two recurrences `pad` may
 * be null: none of the new tokens is padding (true for every call but a batch's first). */
int mixers_short_conv_silu(int dtype, const void* proj, int B, int S, int ld, int off, int C, int taps, const void* w,
                           const void* tail, void* tail_next, int slot0, const int32_t* pad, void* y, mixers_stream_t stream);
/* the same taps with a bias per channel (may be null) and flags: bit 0 = silu on the result, bit 1 = the token's own input is
 * added to the result, y = in(t) + conv (a convolution that refines what a mixer reads instead of replacing it) */
int mixers_short_conv(int dtype, const void* proj, int B, int S, int ld, int off, int C, int taps, const void* w, const void* bias,
                      int flags, const void* tail, void* tail_next, int slot0, const int32_t* pad, void* y, mixers_stream_t stream);

/* Gated delta rule.  conv [B, S, C]: q | k (kv_heads x dim each) | v (heads x vdim) after the short convolution; q and k are
 * made unit vectors here (q also times dim^-1/2).  beta = sigmoid(proj[.., off_b + h]), decay = exp(-exp(A_log[h]) *
 * softplus(proj[.., off_a + h] + dt_bias[h])).  Per head:  M <- decay M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q.
 * state: float [B, heads, dim, vdim], updated in place; o: float [B, S, heads, vdim]. */
int mixers_gated_delta_rule(int dtype, const void* conv, int B, int S, int kv_heads, int heads, int dim, int vdim,
                            const void* proj, int ld, int off_b, int off_a, const void* A_log, const void* dt_bias, float* state,
                            int slot0, const int32_t* pad, float* o, mixers_stream_t stream);

/* Delta rule whose state decays per key channel.  conv as above; beta = sigmoid(proj[.., off_b + h]); z [B, S, heads * dim]: decay
 * logits, a = exp(-exp(A_log[h]) * softplus(z + dt_bias)) with dt_bias [heads * dim].  Per head:  M <- diag(a) M;
 * u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q (q, k unit vectors, q times dim^-1/2). */
int mixers_channel_delta_rule(int dtype, const void* conv, int B, int S, int kv_heads, int heads, int dim, int vdim, const void* proj,
                              int ld, int off_b, const void* z, const void* A_log, const void* dt_bias, float* state, int slot0,
                              const int32_t* pad, float* o, mixers_stream_t stream);

/* State-space scan with a scalar decay per head.  conv [B, S, C]: x (heads x vdim) | B (groups x n_state) | C (groups x n_state)
 * after the short convolution; dt = softplus(proj[.., off_dt + h] + dt_bias[h]).  Per head (its group's B and C):
 * M <- exp(-exp(A_log[h]) dt) M + dt B x^T;  o = M^T C + skip[h] x.  state: float [B, heads, n_state, vdim]. */
int mixers_state_space_scan(int dtype, const void* conv, int B, int S, int groups, int heads, int n_state, int vdim, const void* proj,
                            int ld, int off_dt, const void* A_log, const void* dt_bias, const void* skip, float* state, int slot0,
                            const int32_t* pad, float* o, mixers_stream_t stream);

/* Gated linear attention.  proj [B, S, ld]: q | k (heads x dim each) | v (heads x vdim) from column 0; z [B, S, heads * dim]:
 * decay logits, alpha = sigmoid(z)^(1/tau).  Per head:  M <- diag(alpha) M + k v^T;  o = M^T (q dim^-1/2). */
int mixers_gated_linear_attention(int dtype, const void* proj, int B, int S, int ld, int heads, int dim, int vdim, const void* z,
                                  float tau, float* state, int slot0, const int32_t* pad, float* o, mixers_stream_t stream);

/* out[n, out_col + h * vdim + c] = out_scale * o[n, h, c] / rms(o[n, h, :]) * w[h * w_head_stride + c] * silu(gate[n, off_g + h * vdim + c])
 * (w_head_stride 0: one weight vector [vdim] for every head; vdim: a vector per head, [heads * vdim]).  gate_mode bit 0: the gate
 * is sigmoid(.) instead of silu(.); bit 1: the gate multiplies before the norm, i.e. rms is taken of o * gate. */
int mixers_gated_rms_norm(int dtype, const float* o, long n_rows, int heads, int vdim, const void* gate, int ld_gate, int off_g,
                          const void* w, int w_head_stride, float eps, void* out, int ld_out, int out_col, float out_scale,
                          int gate_mode, mixers_stream_t stream);

/* o[n, c] *= sigmoid(gate[n, off_g + c / per_gate]) in place, o dtype [n_rows, cols] */
int mixers_sigmoid_gate(int dtype, void* o, long n_rows, int cols, const void* gate, int ld_gate, int off_g, int per_gate,
                        mixers_stream_t stream);

/* out float [n_rows, width] = scale * (a / rms(a) * w_a + b / rms(b) * w_b): two branch outputs meet as normalised vectors */
int mixers_rms_pair_sum(int dtype, const void* a, const void* b, const void* w_a, const void* w_b, float eps, float scale, long n_rows,
                        int width, float* out, mixers_stream_t stream);

/* The boundary between layers whose mixer and feed-forward read two scalar-gain RMS norms of the same stream x (float
 * [n_rows, width], in place):  x += y_a + y_c + y_b + y_d (dtype, dtype, float, float; each may be null);  with pre_gain:
 * x <- x / rms(x) * pre_gain[0] (the norm behind an embedding);  with stack (float [streams, n_rows, width]): the new x is kept
 * as stream `index` and, with coef (dtype [index + 1]), replaced by sum_j coef[j] * stack[j];  h1 = x / rms(x) * gain1[0],
 * h2 = x / rms(x) * gain2[0] in dtype (either may be null). */
int mixers_sum_residual_norms(int dtype, float* x, long n_rows, int width, const void* y_a, const void* y_c, const float* y_b,
                              const float* y_d, const void* pre_gain, float eps, float* stack, long stack_stride, int index,
                              const void* coef, const void* gain1, const void* gain2, void* h1, void* h2, mixers_stream_t stream);

/* out = exact (erf) gelu of in, n elements */
int mixers_gelu_erf(int dtype, const void* in, long n, void* out, mixers_stream_t stream);

/* Token shift.  out[m, n, c] = h[n, c] + (h[n - 1, c] - h[n, c]) * mu[m, c], m < n_mix: h dtype [B, S, C], mu [n_mix, C], out
 * [n_mix, B * S, C].  The token before a call's first one is tail [B, 1, C] (zeros before a sequence's first token); padding
 * slots count as zeros and give zeros.  tail_next receives the last token's h (for S == 1 it may be `tail` itself).  pad may be
 * null as in the recurrences. */
int mixers_token_shift_mix(int dtype, const void* h, int B, int S, int C, const void* mu, int n_mix, const void* tail, void* tail_next,
                           int slot0, const int32_t* pad, void* out, mixers_stream_t stream);

/* RWKV-style recurrence with a decay per key channel and a bonus for the current token.  r, k, v: dtype, row n of each at
 * ptr + n * ld, heads x dim channels (three tensors, or three column ranges of one); z [B, S, heads * dim]: decay logits, w =
 * exp(-exp(z + w0)), w0 and u [heads * dim].  Per head:  o = (M + diag(u) k v^T)^T r;  M <- diag(w) M + k v^T.
 * state: float [B, heads, dim, dim], updated in place; o: float [B, S, heads, dim]. */
int mixers_wkv(int dtype, const void* r, const void* k, const void* v, int B, int S, int ld, int heads, int dim, const void* z,
               const void* w0, const void* u, float* state, int slot0, const int32_t* pad, float* o, mixers_stream_t stream);

/* x += y_a + y_b (y_a dtype, y_b float; either may be null), then out = (x - mean) / sqrt(var + eps) * w over each row (out, w
 * dtype; out may be null: only the update).  x: float [n_rows, width], updated in place. */
int mixers_layer_norm_residual(int dtype, float* x, long n_rows, int width, const void* y_a, const float* y_b, const void* w, float eps,
                               void* out, mixers_stream_t stream);

/* out = a N(z) + b N(z^2) + c N(z^3) + e, N(v) = v / rms(v) over a row; coef = {a, b, c, e} */
int mixers_poly_norm(int dtype, const void* z, long n_rows, int width, const void* coef, float eps, void* out, mixers_stream_t stream);

/* out = cap * tanh(x / cap) as floats (cap <= 0: a plain conversion) */
int mixers_soft_cap(int dtype, const void* x, long n, float cap, float* out, mixers_stream_t stream);

/* ---- designs that normalise a sublayer's OUTPUT, cache a key/value latent and route tokens to experts ---- */

/* x[n, :] = table[ids[n], :] * scale + pair[row(n), :] as floats (x_copy, if given, gets the same; h, if given, the same in
 * dtype).  row(n) = (previous id * mul_prev + ids[n] * mul_cur) mod buckets; `buckets` itself for a sequence's first token
 * (position 0); the token before a call's first token is prev[b].  pair may be null (no second table).  ids: [B, S]; padding
 * slots (position < 0) give zeros.  pad may be null when slot0 > 0 (no new token is padding or a first token then): a step that
 * is replayed from a CUDA graph has no current slot0 to give. */
int mixers_embed_pair(int dtype, const void* table, float scale, const void* pair, long buckets, long mul_prev, long mul_cur,
                      const int64_t* ids, const int64_t* prev, int B, int S, int width, int slot0, const int32_t* pad, float* x,
                      float* x_copy, void* h, mixers_stream_t stream);

/* x += y / rms(y) * gain[0] * vec[:]  (gain, vec: dtype, either may be null; y: dtype, or float if y_is_float; rms over a row
 * with eps inside the root).  With `stack` (float [streams, n_rows, width], stack_stride = n_rows * width) the new x is stored
 * as stream `index`, and with `coef` (dtype [index + 1]) x becomes sum_{j <= index} coef[j] * stack[j].  h (may be null): x in dtype. */
int mixers_rms_residual(int dtype, float* x, long n_rows, int width, const void* y, int y_is_float, const void* gain, const void* vec,
                        float eps, float* stack, long stack_stride, int index, const void* coef, void* h, mixers_stream_t stream);

/* out = x / rms(x) * gain[0] * vec[:]   (x float, out dtype; gain, vec may be null) */
int mixers_rms_norm_rows(int dtype, const float* x, long n_rows, int width, const void* gain, const void* vec, float eps, void* out,
                         mixers_stream_t stream);

/* xIELU with pq = {p, q}; with a = softplus(p) and c = 1/2 + softplus(q): f(z) = a z^2 + z/2 where z is positive, c (expm1(z) - z) + z/2 elsewhere */
int mixers_xielu(int dtype, const void* z, long n, const void* pq, void* out, mixers_stream_t stream);

/* out[n, c] = silu(in[n, off_gate + c]) * in[n, off_up + c], c < cols; in: [n_rows, ld] */
int mixers_silu_mul(int dtype, const void* in, long n_rows, int ld, int off_gate, int off_up, int cols, void* out, mixers_stream_t stream);

/* out[n, c] = g' sigmoid(1.702 g') (u' + 1) with g' = min(in[n, off_gate + c], limit), u' = clamp(in[n, off_up + c], -limit, limit) */
int mixers_clamped_glu(int dtype, const void* in, long n_rows, int ld, int off_gate, int off_up, int cols, float limit, void* out,
                       mixers_stream_t stream);

/* out[n, c] = gelu_tanh(g[n, c]) * table[ids[n], col0 + c], c < cols */
int mixers_gelu_table_mul(int dtype, const void* g, long n_rows, int cols, const void* table, int ld_table, int col0, const int64_t* ids,
                          void* out, mixers_stream_t stream);

/* RMS norms (plain weights q_w [q_rank], c_w [kv_rank]) of two column ranges of proj [B, S, ld]: columns off_q.. -> cq_out
 * [B * S, q_rank]; columns off_c.. -> store [B, cap, kv_rank] at storage index held + t (zeros for padding).  dyn as above. */
int mixers_latent_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int q_rank, const void* q_w, int off_c,
                          int kv_rank, const void* c_w, float eps, void* cq_out, void* store, int cap, int held, int shift,
                          const int32_t* pad, const int32_t* dyn, mixers_stream_t stream);

/* Queries, keys and values of new tokens from the columns of one projection output `proj` [B, S, ld], for attention that
 * normalises a token's WHOLE query projection (heads * dim channels) and whole key projection (kv_heads * dim channels) at
 * once: RMS norm with one weight per channel (q_w [heads * dim], k_w [kv_heads * dim]).  Queries go to q_out dtype
 * [B * S, heads * dim]; keys and values into k_store [B, kv_heads, cap, dim] / v_store [.., vdim] at storage index held + t.
 * With v_other (row n at v_other + n * ld_other, kv_heads * vdim channels: another layer's values of the same tokens) the
 * stored value is (1 - blend[0]) v + blend[0] v_other.  Padding slots store zeros.  shift, dyn as above. */
int mixers_wide_qkv_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads,
                            int dim, int vdim, const void* q_w, const void* k_w, float eps, const void* v_other, long ld_other,
                            const void* blend, void* q_out, void* k_store, void* v_store, int cap, int held, int shift,
                            const int32_t* pad, const int32_t* dyn, mixers_stream_t stream);

/* Rotary positions and cache write for the new tokens' queries and keys (columns of proj [B, S, ld]): `heads` query heads of q_dim
 * channels from off_q, `kv_heads` key heads of k_dim channels from off_k and, if vdim > 0, `kv_heads` value heads from off_v.
 * Inside a head channel rot_off + i pairs with rot_off + i + rot_dims / 2: (u, v) -> (u cos a - v sin a, v cos a + u sin a) * amp,
 * a = position * inv_freq[i] (doubles; angle, sine and cosine in double precision).  k_norm_w (may be null): the first
 * k_norm_cols channels of a key head are divided by their root mean square (eps) and multiplied by k_norm_w first.  q_out dtype
 * [B * S, heads * q_dim]; key of row b, storage index j, head g at k_store + b * k_bs + j * k_ps + g * k_hs (values alike);
 * the new tokens go to index held + t; padding slots store zeros.  dyn as in mixers_window_qk_prepare. */
int mixers_rope_qk_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads,
                           int q_dim, int k_dim, int vdim, int q_rot_off, int k_rot_off, int rot_dims, const double* inv_freq, float amp,
                           const void* k_norm_w, int k_norm_cols, float eps, void* q_out, void* k_store, long k_bs, long k_ps, long k_hs,
                           void* v_store, long v_bs, long v_ps, long v_hs, int held, int shift, const int32_t* pad, const int32_t* dyn,
                           mixers_stream_t stream);

/* Causal softmax attention of S new tokens per row.  q: head h of token n at q + n * q_ld + h * q_hs.  Key (value) of storage
 * index j, row b, kv head g at k + b * k_bs + j * k_ps + g * k_hs (strides in elements).  The query at storage index c = held
 * + t sees the keys j <= c of its row that are not padding (j + shift >= pad[b]) and, if window > 0, c - j < window, and, if
 * chunk > 0, only keys whose position p_j has floor(p_j / chunk) = floor(p_c / chunk) (positions count from the row's first token).  Scores
 * (q . k) * scale -- then softcap * tanh(score / softcap) if softcap > 0 -- and the softmax weights are 32-bit.  sink (dtype
 * [heads], may be null): the denominator of head h's softmax also holds exp(sink[h]), which has no key and no value.  out[n, out_col + h * vdim + :] in dtype (zeros for padding queries).
 * allow_tensor_cores: 16-bit models may take the tensor-core kernels: for S >= 16 one block per 64 tokens of a head (head sizes
 * multiples of 16, <= 256); for S <= 16 and at least 4 query heads per kv head one pass over the keys for all heads of a
 * group, the keys split over blocks (dim a multiple of 16, <= 512; vdim 128, 256 or 512), which needs `ws`:
 * mixers_softmax_attention_workspace(...) floats (0: these sizes never take that kernel).  dyn as above. */
int mixers_softmax_attention(int dtype, const void* q, long q_ld, long q_hs, const void* k, long k_bs, long k_ps, long k_hs, const void* v,
                             long v_bs, long v_ps, long v_hs, int B, int S, int heads, int kv_heads, int dim, int vdim, int held,
                             int shift, const int32_t* pad, int window, int chunk, float scale, float softcap, const void* sink, void* out,
                             long ld_out, int out_col, const int32_t* dyn, int allow_tensor_cores, float* ws, mixers_stream_t stream);
long mixers_softmax_attention_workspace(int dtype, int B, int S, int heads, int kv_heads, int dim, int vdim);

/* Router of a mixture of experts.  z = router h (32-bit; router [n_out, width], h [n_rows, width] in dtype); s = softmax(z) over
 * all n_out outputs (score_mode 0) or sigmoid(z) each (score_mode 1); choice = s + correction.  Outputs [g * n_out / groups,
 * (g + 1) * n_out / groups) are group g; groups are ranked by the sum of their group_top largest choice scores, the `keep` first
 * groups stay eligible (every other output is out of the running, whatever its sign), and the `top` eligible outputs of highest
 * choice win (the lower index on a tie); correction may be null (none).  idx_out int32 [n_rows, top] (n_out where nothing was left to choose); w_out float
 * [n_rows, top] = s of the chosen, divided by their sum + 1e-20 if renorm, times w_scale.  gate_row (dtype [width], may be null):
 * gate_out[n] = sigmoid(gate_row . h[n]), the gate of an expert that every token runs. */
int mixers_scored_router(int dtype, const void* h, long n_rows, int width, const void* router, const void* correction, int n_out,
                         int groups, int keep, int top, int score_mode, int group_top, int renorm, float w_scale, const void* gate_row,
                         float* gate_out, int32_t* idx_out, float* w_out, mixers_stream_t stream);
/* the same with softmax scores, groups ranked by their best member, plain scores as weights */
int mixers_grouped_router(int dtype, const void* h, long n_rows, int width, const void* router, const void* correction, int n_out,
                          int groups, int keep, int top, int32_t* idx_out, float* w_out, mixers_stream_t stream);

/* The chosen experts of a few tokens without host work.  gate_up[e] / down[e]: addresses of expert e's [2 ff_e, width] (gate rows,
 * then up rows) and [width, ff_e] matrices in dtype; ffs[e] = ff_e (null: `ff` for all; `ff` is the largest).  always_on != 0:
 * table entry n_experts is an expert that every token runs (a shared expert) with weight always_w[n] (null: 1).  act: scratch dtype
 * [n_rows, top + (always_on ? 1 : 0), ff].  The experts' activation A(g, u): act_kind 0 = silu(g) u; 1 = g' sigmoid(1.702 g')
 * (u' + 1) with g' = min(g, L), u' = clamp(u, -L, L), L = `limit` for chosen experts and `limit_always` for the always-on one;
 * 2 = no gate, the exact gelu of u, the first matrix being [ff_e, width].  weight_input != 0: a chosen expert's weight multiplies
 * its INPUT (w_k h rounded to dtype) instead of its output.
 * y float [n_rows, width] = sum_k w_k * down_e A(gate_e h, up_e h) for chosen e < n_experts, w_k * h for n_experts <= e < n_out,
 * + the always-on expert, + shared_out (dtype [n_rows, width], may be null). */
int mixers_moe_small(int dtype, const void* h, long n_rows, int width, int ff, int top, int n_experts, int n_out, const int32_t* idx,
                     const float* wgt, const int64_t* gate_up, const int64_t* down, const int32_t* ffs, int always_on,
                     const float* always_w, int act_kind, int weight_input, float limit, float limit_always, const void* shared_out,
                     void* act, float* y, mixers_stream_t stream);

/* Counting sort of n_pairs = n_rows * top (token, choice) pairs by chosen output idx[i] in [0, n_keys): counts[e] = pairs of e;
 * pos[i] = row of pair i among the sorted pairs; token_of[row] = i / top. */
int mixers_moe_sort(const int32_t* idx, long n_pairs, int top, int n_keys, int32_t* counts, int32_t* pos, int64_t* token_of,
                    mixers_stream_t stream);

/* y float [n_rows, width] = sum_k w[n, k] * rows[pos[n, k], :] for chosen e < n_experts, w * h[n, :] for identity experts,
 * + shared_w[n] * shared_out (shared_w null: 1); rows: dtype [*, width], the experts' outputs on rows sorted by expert; wgt null:
 * weights of 1 (experts that were fed their weighted input). */
int mixers_moe_combine(int dtype, const void* rows, const int32_t* pos, const int32_t* idx, const float* wgt, const void* h,
                       const void* shared_out, const float* shared_w, long n_rows, int width, int top, int n_experts, int n_out, float* y,
                       mixers_stream_t stream);

/* rows_in[pos[i], :] = h[i / top, :] * wgt[i] in dtype for every pair i with idx[i] < n_experts: the sorted input rows of experts
 * that are fed their weighted input */
int mixers_moe_scatter_scaled(int dtype, const void* h, const int32_t* pos, const int32_t* idx, const float* wgt, long n_pairs, int top,
                              int width, int n_experts, void* rows_in, mixers_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
