/*
 * crabml_lifesun.h -- creation of the host driver of the Lifesun decoder family (crabml_b200/csrc/host/lifesun_runner.cpp); the runner it
 * returns is served through crabml_seqrunner.h (slots, step, greedy generation) like every multi-sequence runner.
 *
 * The stack: x = embed[token]; the looked-up rows are kept as x0.  A layer run reads ONE layer norm (mean and variance, weight and bias)
 * of the 32-bit residual stream and hands it to its mixer and its feed-forward side by side:
 *   h = LN(x) ; x += mixer(h) + ff(h)
 * Layers loop_start .. loop_stop-1 run loop_times times with the same weights, every run on a cache / state of its own; right before the
 * first layer of every repetition x = W_in [x | x0] (one product over the two streams side by side).
 * A mixer is a softmax attention and a recurrence side by side on h, joined as left_scale * left + right_scale * right.
 *   left    grouped key/value heads; queries and keys either scaled to unit RMS per head (no weights) or RMS-normalised over the whole
 *           projection with a weight per column; optional rotation of the column pairs (i, i + dims / 2) of every head; a mask of blocks
 *           of positions counted from 0 and / or a sliding window (cc_masked_attention_capped); optional tanh cap on the scores; an
 *           optional sink in the softmax denominator; an optional sigmoid gate of one number per head on the result.
 *   right   CLR_RIGHT_DIAGONAL: y = act(W_y h + b) beside u = conv(W_x h + b) (short causal convolution with bias), gates from one
 *           product per block of channels, the gated diagonal recurrence (cc_gated_diagonal_recurrence), W_o (S * y).
 *           CLR_RIGHT_RETENTION: rotated q and k, S = decay_h S + (dim^-1/2 k) v^T, read-out S^T q (cc_retention), unit RMS per head,
 *           silu gate, W_o.
 * Feed-forward: W_down (gelu_tanh(W_gate h) * (W_up h)), or none.  Every matrix that multiplies h is part of ONE stacked product.
 * Output: the final layer norm, the head, logits times logit_scale.
 */
#ifndef CRABML_LIFESUN_H
#define CRABML_LIFESUN_H

#include "crabml_seqops.h"
#include "crabml_seqrunner.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CLR_RIGHT_DIAGONAL 0
#define CLR_RIGHT_RETENTION 1
#define CLR_QK_NONE 0
#define CLR_QK_UNIT_PER_HEAD 1          /* every head of q and k divided by its root mean square, no weight */
#define CLR_QK_WHOLE_WEIGHTED 2         /* RMS norm over the whole projection, a weight per column (q_norm, k_norm) */

typedef struct clr_layer_config {
    /* left */
    int32_t heads, kv_heads, dim, vdim;
    int32_t window, block;                  /* position i sees j <= i with i - j < window (if > 0) and floor(i / block) == floor(j / block) (if > 0) */
    int32_t qk_norm;                        /* CLR_QK_* */
    int32_t left_gate;                      /* != 0: the stack holds one gate row per head behind the left values */
    float scale, softcap;                   /* score scale; cap of the scores (<= 0: none) */
    /* right */
    int32_t right;                          /* CLR_RIGHT_* */
    int32_t r_width, r_blocks, r_conv;      /* diagonal: channels, gate blocks, taps of the convolution */
    int32_t r_heads, r_dim, r_vdim;         /* retention */
    float r_rate;                           /* diagonal: the constant c of log a = -c r softplus(lam) */
    float left_scale, right_scale;
    int32_t ff;                             /* hidden width of the feed-forward; 0: the layer is its mixer only */
} clr_layer_config;

typedef struct clr_config {
    int32_t n_layers, width, vocab;
    float norm_eps, logit_scale;
    int32_t loop_start, loop_stop, loop_times;      /* loop_times < 1: no loop, and no product before a repetition */
    int32_t chunk;                          /* longest run of tokens one pass takes; sizes the caches.  <= 0: 256 */
    int32_t max_seq;                        /* rows of the cache of an attention without window or blocks.  <= 0: 4096 */
} clr_config;

/* every pointer is a tensor uploaded by the caller; unused ones are NULL.  Matrices of dense products: F32 or BF16; everything else F32. */
typedef struct clr_layer_weights {
    cc_buf *norm_w, *norm_b;                        /* [width] each */
    /* every matrix that multiplies the layer's normed input, one under the other -- left q [heads * dim], k [kv_heads * dim], v
     * [kv_heads * vdim], (left gate [heads]); diagonal: y, x [r_width] each; retention: q, k [r_heads * r_dim], v, gate [r_heads * r_vdim];
     * then, with a feed-forward, gate and up [ff] each */
    cc_buf* h_stack;
    cc_buf *q_norm, *k_norm;                        /* CLR_QK_WHOLE_WEIGHTED: [heads * dim], [kv_heads * dim] */
    cc_buf *sink, *rot_freq, *left_o;               /* [heads] or NULL; [P] frequencies of the rotated pairs or NULL; [width, heads * vdim] */
    cc_buf* right_o;                                /* [width, r_width] or [width, r_heads * r_vdim] */
    /* diagonal */
    cc_buf *x_bias, *y_bias;                        /* [r_width] or NULL each: the biases of the two branches' projections */
    cc_buf *conv, *conv_bias;                       /* [r_width, taps], [r_width] or NULL */
    cc_buf *gate_w, *gate_b, *lam;                  /* per block the recurrence gate's matrix over the input gate's: [r_blocks * 2 * bs, bs]; [2 r_width] likewise; [r_width] */
    /* retention */
    cc_buf *r_rot_freq, *decay;                     /* [P] or NULL; [r_heads] */
    cc_buf* down;                                   /* [width, ff] */
} clr_layer_weights;

/* embed: [vocab, width] F32; loop_in: [width, 2 width] (with a loop) or NULL; final_norm_w / _b: [width]; head: [vocab, width] */
CC_API int clr_runner_create(cc_device* dev, const clr_config* conf, const clr_layer_config* layers, const clr_layer_weights* weights, cc_buf* embed, cc_buf* loop_in,
                             cc_buf* final_norm_w, cc_buf* final_norm_b, cc_buf* head, csr_runner** out);

#ifdef __cplusplus
}
#endif
#endif
