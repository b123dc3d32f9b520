/*
 * crabml_seqops.h -- sequence-mixing, routing and normalisation ops beyond the reference's `Tensor` trait.
 *
 * The reference's trait (crabml-core/src/tensor/api.rs:11-79) covers the llama family: rope, softmax attention over a growing
 * cache, a dense gated feed-forward.  The ops below are the building blocks of hybrid decoders (recurrent and windowed mixers,
 * routed feed-forwards, norms on the sublayer output).  Every constant of a mechanism is a parameter, so that any model built
 * from these mechanisms can use them; crabml_b200/csrc/host/zatorax_runner.cpp is the first user.
 *
 * Conventions are those of crabml_cuda.h: cc_view = buffer + shape + strides (contiguous views only here), all work on the
 * device's stream, status codes, nothing blocks.  Activations and all state are F32; everything a recurrence, a norm, a softmax
 * or a router computes is computed in 32-bit floats.  Weight matrices of the dense products may be F32 or BF16 (cc_matmul_vec:
 * BF16 weights round the activation to bfloat16 and accumulate in 32 bits).  These ops are eager-only: a lazy (graph /
 * megakernel) device refuses them with CC_ERR_UNSUPPORTED.
 */
#ifndef CRABML_SEQOPS_H
#define CRABML_SEQOPS_H

#include "crabml_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* CC_ACT_SWISH: z * sigmoid(alpha * z) with alpha given beside it (cc_glu_params); the others take no constant */
enum cc_activation { CC_ACT_NONE = 0, CC_ACT_SILU = 1, CC_ACT_GELU_TANH = 2, CC_ACT_SWISH = 3, CC_ACT_SIGMOID = 4 };

/* x (any shape) = 0 */
CC_API int cc_tensor_zero(cc_device* dev, const cc_view* x);

/* ---- norms ------------------------------------------------------------------------------------------------------------------ */
/* dst[r] = (accumulate ? dst[r] : 0) + y[r] / sqrt(mean(y[r]^2) + eps) * gain ; dst, y: [rows, cols]; gain: 1 element (one number
 * for all coordinates) or cols elements.  accumulate = 1 is the residual update of a block whose norm sits on the sublayer OUTPUT. */
CC_API int cc_rms_norm_gain(cc_device* dev, const cc_view* dst, const cc_view* y, const cc_view* gain, float eps, int32_t accumulate);
/* dst[r] = dst[r] + mult * (y[r] / sqrt(mean(y[r]^2) + eps) * gain): cc_rms_norm_gain with accumulate = 1 and a factor on the normed
 * sublayer output (a residual multiplier), applied after the gain. */
CC_API int cc_rms_norm_gain_mult(cc_device* dev, const cc_view* dst, const cc_view* y, const cc_view* gain, float eps, float mult);
/* x[r, h, :] = x[r, h, :] / sqrt(mean(x[r, h, :]^2) + eps) * w * act(gate[r, h, :]) ; x, gate: [rows, heads * head_size].  w: [head_size]
 * (one weight vector for all heads) or [heads * head_size] (a weight per column; x must then be 2-D) or NULL (1).  gate NULL: no gate
 * (the plain per-head norm of queries and keys). */
CC_API int cc_gated_head_rms_norm(cc_device* dev, const cc_view* x, const cc_view* gate, const cc_view* w, int32_t head_size, float eps,
                                  int32_t gate_act);
/* dst[r] = x[r] with every one of `groups` equal consecutive parts of the row divided by its own sqrt(mean(part^2) + eps), times w[:]
 * (w: cols numbers).  groups = 1 is the plain weighted RMS norm.  dst may be x. */
CC_API int cc_group_rms_norm(cc_device* dev, const cc_view* dst, const cc_view* x, const cc_view* w, int32_t groups, float eps);
/* Layer norm with weight and bias: dst[r] = (x[r] - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations from the
 * mean.  dst, x: [rows, cols]; w, b: [cols] (b NULL: no bias).  dst may be x. */
CC_API int cc_layer_norm(cc_device* dev, const cc_view* dst, const cc_view* x, const cc_view* w, const cc_view* b, float eps);
/* dst = x * act(gate) with every one of `groups` equal consecutive parts of the row then divided by its own root mean square, times w[:]:
 * the gate comes BEFORE the norm (cc_gated_head_rms_norm gates after it).  All [rows, cols]; w: [cols].  dst may be x. */
CC_API int cc_gated_group_rms_norm(cc_device* dev, const cc_view* dst, const cc_view* x, const cc_view* gate, const cc_view* w, int32_t groups, float eps,
                                   int32_t gate_act);
/* PolyNorm, in place on z [rows, cols]: z <- a N(z) + b N(z^2) + c N(z^3) + e with coef = {a, b, c, e}; powers are taken element by
 * element and N divides the row by its root mean square, N(y) = y / sqrt(mean(y^2) + eps). */
CC_API int cc_poly_norm(cc_device* dev, const cc_view* z, const cc_view* coef, float eps);
/* dst = (accumulate ? dst : 0) + y1 * sigmoid(g1 + b1) + y2 * sigmoid(g2 + b2) ; all [rows, cols] but the biases [cols].  g1 / g2 NULL:
 * that operand is not gated; y2 NULL: one operand.  The residual update of a block whose sublayers run side by side on one input. */
CC_API int cc_gated_sum(cc_device* dev, const cc_view* dst, int32_t accumulate, const cc_view* y1, const cc_view* g1, const cc_view* b1, const cc_view* y2,
                        const cc_view* g2, const cc_view* b2);
/* src [rows, cols] cut into n_parts (<= 16) blocks of neighbouring columns, widths[p] wide, each returned as a contiguous tensor
 * [rows, widths[p]] in outs[p].  For matrices that multiply the same input and are stacked one under the other: ONE product (one launch,
 * one conversion of the input), then this. */
CC_API int cc_split_cols(cc_device* dev, const cc_view* src, int32_t n_parts, const int32_t* widths, cc_buf** outs);
/* gate = act(gate) * up, elementwise (the inner step of a gated feed-forward, exact 32-bit activation) */
CC_API int cc_glu_inplace(cc_device* dev, const cc_view* gate, const cc_view* up, int32_t act);
/* The same step on ONE product of the stacked matrix [W_gate ; W_up]: src [rows, 2 * ff] holds gate | up side by side;
 * out[r, c] = act(src[r, c] + bias[c]) * (src[r, ff + c] + bias[ff + c]) ; bias: [2 * ff] or NULL.  out: [rows, ff]. */
CC_API int cc_glu_halves(cc_device* dev, const cc_view* src, const cc_view* bias, int32_t act, cc_buf** out);
/* x[r, c] += bias[c] ; x: [rows, cols], bias: [cols] (the bias of a projection, added to its product) */
CC_API int cc_add_row_bias(cc_device* dev, const cc_view* x, const cc_view* bias);
/* dst = sa * a + sb * b, elementwise (two branches that read one input, joined with fixed weights); dst may be a or b */
CC_API int cc_scaled_sum(cc_device* dev, const cc_view* dst, const cc_view* a, float sa, const cc_view* b, float sb);
/* dst += sa * a + sb * b + c, elementwise (c NULL: no third operand): two weighted branches and a third sublayer's result join the residual
 * stream in one pass. */
CC_API int cc_scaled_sum_accumulate(cc_device* dev, const cc_view* dst, const cc_view* a, float sa, const cc_view* b, float sb, const cc_view* c);
/* x[t, h, :] *= act(g[t, h]): ONE gate number per (row, head) on the head's whole output.  x: [rows, heads * head_size], g: [rows, heads]. */
CC_API int cc_head_gate(cc_device* dev, const cc_view* x, const cc_view* g, int32_t n_heads, int32_t act);
/* out = [a | b], row by row: a [rows, ca], b [rows, cb] -> out [rows, ca + cb] (two streams that enter one product side by side) */
CC_API int cc_concat_cols(cc_device* dev, const cc_view* a, const cc_view* b, cc_buf** out);

/* ---- a second embedding row chosen by a hash of the token pair ------------------------------------------------------------------ */
/* dst[t] += table[row_t], row_t = (prev_t * mul_prev + token_t * mul_cur) mod buckets, where prev_t is the token before token_t in the
 * sequence; a sequence's first token takes row `buckets` (table: [buckets + 1, cols]).  The n tokens come from the host (`tokens`) or,
 * when tokens is NULL, ONE token from device slot `slot` (cc_argmax_to_slot).  last: I32 [1], part of the sequence's state: 1 + the
 * sequence's last token so far (0: none yet); read for prev_0, then set to 1 + the last of these tokens. */
CC_API int cc_pair_hash_rows_add(cc_device* dev, const cc_view* dst, const cc_view* table, const int64_t* tokens, int32_t n, int32_t slot, const cc_view* last,
                                 int64_t mul_prev, int64_t mul_cur, int64_t buckets);

/* ---- short causal convolution over time (depthwise) --------------------------------------------------------------------------- */
/* x: [T, C] the new inputs of one sequence; w: [C, K] (the last column multiplies the current input); tail: [K-1, C], the K-1 inputs
 * that precede x (zeros at the start of a sequence) -- read, then replaced by the last K-1 inputs of tail ++ x.
 * out[t, c] = act(sum_j w[c, j] * in[t - (K-1) + j, c]).  unit_norm != 0: afterwards every run of head_size channels is divided by
 * sqrt(sum of its squares + unit_eps) and multiplied by unit_scale. */
CC_API int cc_short_conv(cc_device* dev, const cc_view* x, const cc_view* w, const cc_view* tail, int32_t act, int32_t head_size,
                         int32_t unit_norm, float unit_eps, float unit_scale, cc_buf** out);

/* cc_short_conv_bias with a bias on the INPUT as well (in_bias: [C] or NULL): the convolution runs over x + in_bias -- the bias of the projection
 * that made x -- while the positions before the sequence stay zero; the tail then holds inputs that carry the bias. */
CC_API int cc_short_conv_biases(cc_device* dev, const cc_view* x, const cc_view* w, const cc_view* in_bias, const cc_view* bias, const cc_view* tail, int32_t act,
                                cc_buf** out);
/* cc_short_conv with a bias per channel added to the sum before the activation (bias: [C] or NULL) */
CC_API int cc_short_conv_bias(cc_device* dev, const cc_view* x, const cc_view* w, const cc_view* bias, const cc_view* tail, int32_t act, cc_buf** out);

/* ---- gated delta rule ------------------------------------------------------------------------------------------------------ */
/* One sequence, T new tokens.  q, k: [T, n_kv * dk] (already normalised), v: [T, n_heads * dv]; a, b: [T, n_heads] raw projections;
 * a_log, dt_bias: [n_heads]; state: [n_heads, dk, dv] F32, carried between calls.  Head h reads q/k head h / (n_heads / n_kv).
 *   beta = sigmoid(b) ; decay = exp(-exp(a_log) * softplus(a + dt_bias))
 *   S = decay * S ; u = beta * (v - S^T k) ; S = S + k u^T ; out = S^T q      (in this order, per token)
 * out: [T, n_heads * dv]. */
CC_API int cc_gated_delta_rule(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* a, const cc_view* b,
                               const cc_view* a_log, const cc_view* dt_bias, const cc_view* state, int32_t n_heads, int32_t n_kv, int32_t dk,
                               int32_t dv, cc_buf** out);

/* ---- sliding-window attention over a ring cache ------------------------------------------------------------------------------ */
/* Append T tokens at positions pos0 .. pos0+T-1 to a ring of `ring` positions (position p lives in row p % ring):
 * kring: [ring, n_kv * dk], vring: [ring, n_kv * dv]; k: [T, n_kv * dk], v: [T, n_kv * dv].  k_norm_w ([dk], may be NULL): each key
 * head is RMS-normalised (eps) and multiplied by it before it is stored. */
CC_API int cc_kv_ring_append(cc_device* dev, const cc_view* kring, const cc_view* vring, const cc_view* k, const cc_view* v,
                             const cc_view* k_norm_w, float eps, int64_t pos0, int32_t n_kv, int32_t dk, int32_t dv);
/* q: [T, n_heads * dk] raw queries of positions pos0 .. ; q_norm_w ([dk], may be NULL): per-head RMS norm (eps) times weight, applied
 * to q IN PLACE (q is the caller's projection output; pass a copy to keep the raw values).
 * Position i attends to j with 0 <= i - j < window (window <= 0: no limit but j >= 0); the ring must still hold those rows.
 *   score = (q . k) * scale - r1[h] * ln(1 + r2[h] * (i - j))        (r1, r2: [n_heads], both NULL = no distance term)
 * then softmax over the visible keys and the weighted sum of values.  out: [T, n_heads * dv]. */
CC_API int cc_window_attention(cc_device* dev, const cc_view* q, const cc_view* q_norm_w, float eps, const cc_view* kring, const cc_view* vring,
                               int64_t pos0, int32_t n_heads, int32_t n_kv, int32_t dk, int32_t dv, int32_t window, float scale,
                               const cc_view* r1, const cc_view* r2, cc_buf** out);

/* cc_window_attention with two more options.  sink ([n_heads] or NULL): the softmax denominator also holds exp(sink[h]), a key that has
 * no value and whose score is sink[h] as it stands.  vring == NULL: a key row's first dv columns are its value (dv <= dk): a cache of
 * latent rows that serve as keys and as values. */
CC_API int cc_window_attention_sink(cc_device* dev, const cc_view* q, const cc_view* q_norm_w, float eps, const cc_view* kring, const cc_view* vring,
                                    int64_t pos0, int32_t n_heads, int32_t n_kv, int32_t dk, int32_t dv, int32_t window, float scale,
                                    const cc_view* r1, const cc_view* r2, const cc_view* sink, cc_buf** out);

/* cc_window_attention_sink with one more kind of mask.  block > 0: positions are cut into blocks of `block` counted from position 0 of the
 * sequence, and position i sees j <= i only inside its own block, floor(i / block) == floor(j / block).  window and block may both be
 * given (both limits hold); both <= 0: every j <= i. */
CC_API int cc_masked_attention(cc_device* dev, const cc_view* q, const cc_view* kring, const cc_view* vring, int64_t pos0, int32_t n_heads, int32_t n_kv, int32_t dk,
                               int32_t dv, int32_t window, int32_t block, float scale, const cc_view* sink, cc_buf** out);
/* cc_masked_attention with a cap on the scores: softcap > 0 turns score into softcap * tanh(score / softcap) (after the scale, before the
 * softmax); softcap <= 0: no cap. */
CC_API int cc_masked_attention_capped(cc_device* dev, const cc_view* q, const cc_view* kring, const cc_view* vring, int64_t pos0, int32_t n_heads, int32_t n_kv,
                                      int32_t dk, int32_t dv, int32_t window, int32_t block, float scale, float softcap, const cc_view* sink, cc_buf** out);

/* ---- linear recurrences over a matrix state -------------------------------------------------------------------------------------------
 * Three mixers share one form: per head a state S [dk, dv] (F32, carried between calls, zero at the start of a sequence) that every token
 * first shrinks and then adds an outer product to, and a read-out S^T q.  They differ in what shrinks S and what scales the outer product;
 * all of that is computed in 32-bit floats from raw projections, inside the op.  One sequence, T new tokens, in order. */
/* Matrix memory with exponential gates and a running maximum (the mLSTM of xLSTM).  q, k: [T, H * dk], v: [T, H * dv]; gi, gf: [T, H] raw
 * gate projections with biases bi, bf [H]; state: [H, dk, dv + 1], the matrix S and, as its last column, the normaliser n; mstate: [H],
 * the running maximum m, which starts at 0 like the rest.
 *   i = cap tanh((gi + bi) / cap) ; f = logsigmoid(cap tanh((gf + bf) / cap)) ; m' = max(f + m, i)
 *   S = exp(f + m - m') S + exp(i - m') k v^T ; n likewise with k alone ; out = S^T (q_scale q) / (max(|n . q_scale q|, exp(-m')) + 1e-6)
 * out: [T, H * dv]. */
CC_API int cc_matrix_memory(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* gi, const cc_view* gf, const cc_view* bi,
                            const cc_view* bf, float cap, float q_scale, const cc_view* state, const cc_view* mstate, int32_t n_heads, int32_t dk, int32_t dv,
                            cc_buf** out);
/* Linear attention with a decay per key channel (gated linear attention).  q, k, z: [T, H * dk], v: [T, H * dv]; zb: [H * dk] bias of z.
 *   alpha = sigmoid(z + zb)^(1 / tau) ; S = diag(alpha) S + k v^T ; out = S^T (q_scale q) */
CC_API int cc_decayed_linear_attention(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* z, const cc_view* zb, float tau,
                                       float q_scale, const cc_view* state, int32_t n_heads, int32_t dk, int32_t dv, cc_buf** out);
/* Selective state-space recurrence (the SSD form of Mamba-2).  xbc: [T, H * P + 2 * G * N], a row is x | B | C (the convolution's output);
 * dt: [T, H] raw; dt_bias, a_log, d_skip: [H]; state: [H, N, P].  Head h reads B and C of group h / (H / G).
 *   d = softplus(dt + dt_bias) ; S = exp(-exp(a_log) d) S + d B x^T ; out = S^T C + d_skip x
 * out: [T, H * P]. */
CC_API int cc_state_space_scan(cc_device* dev, const cc_view* xbc, const cc_view* dt, const cc_view* dt_bias, const cc_view* a_log, const cc_view* d_skip,
                               const cc_view* state, int32_t n_heads, int32_t n_groups, int32_t n_state, int32_t head_dim, cc_buf** out);
/* Retention: linear attention with one fixed decay per head, no softmax and no denominator.  q, k: [T, H * dk], v: [T, H * dv];
 * decay: [H]; state: [H, dk, dv].
 *   S = decay[h] S + (k_scale k) v^T ; out = S^T q */
CC_API int cc_retention(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* decay, float k_scale, const cc_view* state,
                        int32_t n_heads, int32_t dk, int32_t dv, cc_buf** out);

/* ---- gated diagonal recurrence ----------------------------------------------------------------------------------------------------------
 * The real-gated linear recurrent unit (RG-LRU of Griffin): a state of one number per channel, S [C] (F32, carried between calls, zero at
 * the start of a sequence).  u: [T, C] the recurrence's input; gates: [T, 2 C] raw gate projections laid out as n_blocks equal blocks of
 * channels, each block's recurrence gate followed by its input gate ([n_blocks][2][C / n_blocks], what one product per block of the stacked
 * matrices [W_r,b ; W_i,b] leaves); gate_bias: [2 C] in the same layout; lam: [C].
 *   r = sigmoid(gate_r + bias) ; i = sigmoid(gate_i + bias) ; log a = -c r softplus(lam)
 *   S = exp(log a) S + sqrt(1 - exp(2 log a)) (i u) ; out = S * act(y + y_bias)        (y: [T, C] or NULL: out = S; y_bias: [C] or NULL)
 * Everything is 32-bit; 1 - a^2 is taken as -expm1(2 log a).  out: [T, C]. */
CC_API int cc_gated_diagonal_recurrence(cc_device* dev, const cc_view* u, const cc_view* gates, const cc_view* gate_bias, const cc_view* lam, float c, int32_t n_blocks,
                                        const cc_view* y, const cc_view* y_bias, int32_t y_act, const cc_view* state, cc_buf** out);

/* ---- rotary positions from a frequency table ----------------------------------------------------------------------------------- */
/* x: [T, n_heads * head_size], rows are positions pos0 .. ; freq: [P] one frequency per pair.  In every head the columns
 * offset + 2i and offset + 2i + 1 (i < P) are rotated by the angle a = position * freq[i] (a 32-bit product):
 *   (u, v) <- ((u cos a - v sin a) * mag, (v cos a + u sin a) * mag) ; all other columns stay.  In place.
 * The table carries whatever scaling of the frequencies a model uses (crabml_b200/rotary.py builds plain and YaRN tables). */
CC_API int cc_rope_pairs(cc_device* dev, const cc_view* x, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag, int64_t pos0);
/* The same rotation with another pairing: with P = len(freq), column offset + i turns together with column offset + i + P (i < P), the
 * "two halves" layout; all other columns stay.  In place. */
CC_API int cc_rope_halves(cc_device* dev, const cc_view* x, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag, int64_t pos0);
/* cc_rope_halves on two tensors of one shape (the queries and keys of a mixer whose heads are equally many) in one pass */
CC_API int cc_rope_halves_two(cc_device* dev, const cc_view* x1, const cc_view* x2, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag,
                              int64_t pos0);

/* ---- queries and keys from projection to cache in one pass ------------------------------------------------------------------------ */
/* What lies between the projections and the attention, fused: q [T, n_heads * dk] and k [T, n_kv * dk] are normalised, rotated, q is
 * written back in place, k and v [T, n_kv * dv] go into the rings' rows of positions pos0 .. (cc_kv_ring_append's layout).
 *   qk_norm  CC_QK_NORM_NONE; CC_QK_NORM_HEAD: every head divided by sqrt(mean(head^2) + eps), times q_w / k_w [dk] (NULL: 1);
 *            CC_QK_NORM_ROW: the whole projection divided by sqrt(mean(row^2) + eps), times q_w [n_heads * dk] / k_w [n_kv * dk] (NULL: 1)
 *   freq     [P] or NULL: after the norm, P column pairs of every head starting at column `offset` turn by position * freq[i], times mag;
 *            pairing CC_ROPE_NEIGHBOURS: (offset + 2i, offset + 2i + 1), CC_ROPE_HALVES: (offset + i, offset + i + P)
 * The same arithmetic as cc_gated_head_rms_norm / cc_group_rms_norm, cc_rope_pairs / cc_rope_halves and cc_kv_ring_append one after the other. */
enum cc_qk_norm { CC_QK_NORM_NONE = 0, CC_QK_NORM_HEAD = 1, CC_QK_NORM_ROW = 2 };
enum cc_rope_pairing { CC_ROPE_NEIGHBOURS = 0, CC_ROPE_HALVES = 1 };
CC_API int cc_qk_prepare_append(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* kring, const cc_view* vring, int32_t qk_norm,
                                const cc_view* q_w, const cc_view* k_w, float eps, const cc_view* freq, int32_t pairing, int32_t offset, float mag, int64_t pos0,
                                int32_t n_heads, int32_t n_kv, int32_t dk, int32_t dv);

/* ---- latent key/value cache --------------------------------------------------------------------------------------------------- */
/* A cache row is [c | r]: c, `rank` numbers from which keys and values of all heads derive, and r, a rotated key part that all heads
 * share.  Appends T rows ckv [T, cols] at positions pos0 .. to ring [R, cols] (position p lives in row p % R): the first `rank` columns
 * are RMS-normalised (eps) and multiplied by norm_w ([rank], NULL = 1), the next 2 * P columns are rotated like cc_rope_pairs does
 * (freq [P], NULL = none), any further column is copied. */
CC_API int cc_latent_ring_append(cc_device* dev, const cc_view* ring, const cc_view* ckv, const cc_view* norm_w, float eps, int32_t rank, const cc_view* freq,
                                 float mag, int64_t pos0);
/* A product per head, with the columns behind a head's inputs carried along:
 *   out[t, h] = [ W_h x[t, h, :n_in] | x[t, h, n_in:] ]     x: [T, heads * (n_in + rest)], w: [heads * n_out, n_in] (W_h = rows h * n_out ..), F32
 * out: [T, heads * (n_out + rest)].  With W_h the TRANSPOSED key up-projection of head h (n_out = rank) it folds that projection into the
 * query, so that scores are taken against the latent rows themselves (q_h . (U_h c) = (U_h^T q_h) . c; the rotated part rides along as
 * `rest`); with W_h the value up-projection and rest = 0 it turns an attention result over latent rows into the head's values.
 * freq ([P], 2 P <= rest, or NULL): the first 2 P carried columns are rotated on the way like cc_rope_pairs does (rows are positions
 * pos0 ..), which saves the separate rotation of a query that is folded anyway. */
CC_API int cc_head_project(cc_device* dev, const cc_view* x, const cc_view* w, int32_t n_heads, int32_t rest, const cc_view* freq, float mag, int64_t pos0,
                           cc_buf** out);

/* out[j, h] = [ a[j, h] | shared[j, col0 : col0 + rest] ]: a: [rows, heads * dim]; shared: [>= rows, cols] (its first `rows` rows are used);
 * out: [rows, heads * (dim + rest)].  Builds per-head keys out of their own part and a part all heads share (a latent cache's rotated columns). */
CC_API int cc_head_concat_shared(cc_device* dev, const cc_view* a, const cc_view* shared, int32_t n_heads, int32_t col0, int32_t rest, cc_buf** out);

/* ---- routed feed-forward ---------------------------------------------------------------------------------------------------- */
/* x: [T, D]; router_w: [E, D] F32; correction: [E] or NULL.  s = softmax(router_w x) over all experts (32-bit).  Choice score =
 * s + correction.  Experts form n_groups equal groups of neighbours; a group's score is its largest choice score; only experts of the
 * keep_groups best groups can be chosen (n_groups <= 1: no limit).  The `top` experts with the largest choice scores are chosen; their
 * weights are s (without the correction), not renormalised unless renormalise != 0.
 * ids_out: I32 [T, top]; weights_out: F32 [T, top]. */
CC_API int cc_moe_route(cc_device* dev, const cc_view* x, const cc_view* router_w, const cc_view* correction, int32_t top, int32_t n_groups,
                        int32_t keep_groups, int32_t renormalise, cc_buf** ids_out, cc_buf** weights_out);
/* cc_moe_route with every constant of the choice as a parameter. */
enum cc_route_score { CC_ROUTE_SOFTMAX = 0, CC_ROUTE_SIGMOID = 1 };
typedef struct cc_route_params {
    int32_t score;               /* CC_ROUTE_SOFTMAX: s = softmax over all experts; CC_ROUTE_SIGMOID: s = sigmoid, expert by expert */
    int32_t top, n_groups, keep_groups;
    int32_t group_top;           /* a group's score is the sum of its group_top largest choice scores (1: its largest) */
    int32_t renormalise;         /* != 0: the chosen weights are divided by (their sum + renorm_eps) */
    float renorm_eps;
} cc_route_params;
CC_API int cc_moe_route_ex(cc_device* dev, const cc_view* x, const cc_view* router_w, const cc_view* correction, const cc_route_params* params,
                           cc_buf** ids_out, cc_buf** weights_out);
/* the gated unit of an expert: act(min(g, limit)) * (clamp(u, -limit, limit) + up_shift); limit <= 0: nothing is clamped */
typedef struct cc_glu_params {
    int32_t act;                 /* cc_activation */
    float alpha;                 /* CC_ACT_SWISH only */
    float limit, up_shift;
} cc_glu_params;
/* cc_moe_experts with the gated unit's constants as parameters (cc_moe_experts = {act, 1, 0, 0}) */
CC_API int cc_moe_experts_glu(cc_device* dev, const cc_view* x, const cc_view* ids, const cc_view* weights, const cc_view* w_gate, const cc_view* w_up,
                              const cc_view* w_down, int32_t n_experts, int32_t ff, const cc_glu_params* glu, cc_buf** out);
/* out[t] = sum_s weights[t, s] * W_down[ids[t, s]] (act(W_gate[ids[t, s]] x[t]) * (W_up[ids[t, s]] x[t]))
 * w_gate, w_up: [E * ff, D]; w_down: [E * D, ff] (expert-major stacks; F32 or BF16).  out: [T, D]. */
CC_API int cc_moe_experts(cc_device* dev, const cc_view* x, const cc_view* ids, const cc_view* weights, const cc_view* w_gate, const cc_view* w_up,
                          const cc_view* w_down, int32_t n_experts, int32_t ff, int32_t act, cc_buf** out);

#ifdef __cplusplus
}
#endif
#endif /* CRABML_SEQOPS_H */
