/*
 * crabml_vuzinex.h -- creation of the host driver of the Vuzinex decoder family (crabml_b200/csrc/host/vuzinex_runner.cpp); the runner it
 * returns is served through crabml_seqrunner.h (slots, step, greedy generation) like every multi-sequence runner.
 *
 * The stack: x = embed[token] (the table arrives already multiplied by the embedding scale) + a second row chosen by a hash of the
 * previous and the current token (cc_pair_hash_rows_add).  A layer normalises before AND after each sublayer,
 *   x += mult * norm_b(mixer(norm_a(x))) ; x += mult * norm_d(ff(norm_c(x)))           (RMS norms; the weights arrive as 1 + stored value)
 * and layers loop_start .. loop_stop-1 run loop_times times with the same weights, every run on a cache / state of its own.
 * Mixers:
 *   pair         softmax attention and a linear recurrence side by side on one input, joined as left_scale * left + right_scale * right.
 *                Left: grouped key/value heads, optional projection biases, optional per-head RMS norm of queries and keys (before the
 *                rotation), rotary positions on neighbouring coordinate pairs from a frequency table, a mask that is causal, a sliding
 *                window or blocks of positions (cc_masked_attention), an optional sink in the softmax, an optional sigmoid gate on the
 *                heads' output.  Right: the matrix memory with exponential gates (cc_matrix_memory; per-head unit RMS, a weight per
 *                column, sigmoid gate) or linear attention with a decay per key channel through a low-rank projection
 *                (cc_decayed_linear_attention; per-head RMS norm with one weight vector, silu gate).
 *   state space  one input projection cut into z | x B C | dt, a short causal convolution with bias and silu over x B C
 *                (cc_short_conv_bias), the selective scan (cc_state_space_scan), silu(z) gate BEFORE an RMS norm in groups
 *                (cc_gated_group_rms_norm), output projection.
 * Feed-forward: W_down (silu(W_gate h + b) * (W_up h + b)) + b, gate and up as one stacked product (cc_glu_halves), or none.
 * Output: the final norm, the embedding table (without its scale) as the head, logits times logit_scale.
 */
#ifndef CRABML_VUZINEX_H
#define CRABML_VUZINEX_H

#include "crabml_seqops.h"
#include "crabml_seqrunner.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CVR_MIXER_PAIR 0
#define CVR_MIXER_STATE_SPACE 1
#define CVR_RIGHT_MATRIX_MEMORY 0
#define CVR_RIGHT_DECAYED 1

typedef struct cvr_layer_config {
    int32_t mixer;                          /* CVR_MIXER_* */
    /* pair, left */
    int32_t heads, kv_heads, dim, vdim;
    int32_t window, block;                  /* position i sees j <= i with i - j < window (if > 0) and floor(i / block) == floor(j / block) (if > 0) */
    int32_t left_gate;                      /* != 0: the stack holds the left output gate behind the left values */
    float scale, rot_mag;                   /* score scale; factor on cos and sin */
    /* pair, right */
    int32_t right;                          /* CVR_RIGHT_* */
    int32_t r_heads, r_dim, r_vdim;
    int32_t r_rank;                         /* decayed: inner width of the decay's two projections */
    float gate_cap, tau, r_q_scale;         /* matrix memory: cap of the gates; decayed: root of the decay; factor on the right queries */
    float left_scale, right_scale;
    /* state space */
    int32_t s_heads, s_vdim, s_state, s_groups, s_conv, s_norm_groups;
    int32_t ff;                             /* hidden width of the feed-forward; 0: the layer is its mixer only */
} cvr_layer_config;

typedef struct cvr_config {
    int32_t n_layers, width, vocab;
    float norm_eps, residual_mult, logit_scale;
    int32_t loop_start, loop_stop, loop_times;      /* loop_times <= 1: every layer runs once */
    int64_t hash_buckets, hash_mul_prev, hash_mul_cur;      /* hash_buckets <= 0: no second embedding row */
    int32_t chunk;                          /* longest run of tokens one pass takes; sizes the caches.  <= 0: 256 */
    int32_t max_seq;                        /* rows of the cache of an attention without window or blocks.  <= 0: 4096 */
} cvr_config;

/* every pointer is a tensor uploaded by the caller; unused ones are NULL.  Matrices of dense products: F32 or BF16; everything else F32. */
typedef struct cvr_layer_weights {
    cc_buf *norm_a, *norm_b, *norm_c, *norm_d;      /* [width] each, 1 + the stored weight; c and d only with a feed-forward */
    /* pair: every matrix that multiplies the mixer's input, one under the other, so that it is ONE product -- left q [heads * dim], k
     * [kv_heads * dim], v [kv_heads * vdim], (left gate [heads * vdim]), right q, k [r_heads * r_dim], v, gate [r_heads * r_vdim], then
     * matrix memory: the two gate rows i, f [r_heads] each; decayed: the decay's first projection [r_rank].  h_bias: [rows of the stack],
     * the projections' biases (zero where a projection has none), or NULL */
    cc_buf *h_stack, *h_bias;
    cc_buf *q_norm, *k_norm;                        /* [dim] or NULL */
    cc_buf *sink, *rot_freq, *left_o;               /* [heads] or NULL, [P] frequencies of the rotated pairs or NULL, [width, heads * vdim] */
    cc_buf *right_norm, *right_o;                   /* matrix memory [r_heads * r_vdim], decayed [r_vdim]; [width, r_heads * r_vdim] */
    cc_buf *gate_bias_i, *gate_bias_f;              /* matrix memory: [r_heads] */
    cc_buf *decay_up, *decay_bias;                  /* decayed: [r_heads * r_dim, r_rank], [r_heads * r_dim] */
    /* state space */
    cc_buf *in, *conv, *conv_bias;                  /* [2 inner + 2 groups * state + heads, width], [inner + 2 groups * state, taps], [..] */
    cc_buf *dt_bias, *a_log, *d_skip, *s_norm, *s_o;        /* [heads] x 3, [inner], [width, inner] */
    /* feed-forward */
    cc_buf *gate_up, *gate_up_bias, *down, *down_bias;      /* [2 ff, width] (gate over up), [2 ff], [width, ff], [width] */
} cvr_layer_weights;

/* embed: [vocab, width] F32, times the embedding scale; pair_table: [hash_buckets + 1, width] F32 or NULL; head: [vocab, width] */
CC_API int cvr_runner_create(cc_device* dev, const cvr_config* conf, const cvr_layer_config* layers, const cvr_layer_weights* weights, cc_buf* embed,
                             cc_buf* pair_table, cc_buf* final_norm, cc_buf* head, csr_runner** out);

#ifdef __cplusplus
}
#endif
#endif
