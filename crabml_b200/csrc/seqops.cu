// seqops.cu -- sequence-mixing and normalisation ops of include/crabml_seqops.h: norms on the sublayer output, the short causal
// convolution, the gated delta rule, and sliding-window attention over a ring cache.  Everything here is computed in 32-bit floats
// (explicit fmaf; expf / logf / log1pf of the CUDA math library, not the fast intrinsics).
//
// One property every kernel keeps: the value computed for a token depends only on that token's inputs and on the state / cache
// contents, never on how many tokens the call carries or where the token sits in the call.  Sums run in a fixed order per output
// (a warp's lane-strided partial sums and the xor butterfly, or one thread's sequential loop), so prefill, chunked prefill and
// token-by-token decoding give the same bits for the recurrent layers and the same bits per (query, key set) for attention.
#include <cuda_bf16.h>

#include "../../include/crabml_seqops.h"
#include "capi_checks.cuh"

#define SEQ_ENTER(dev, what)                                                                                          \
    if (!(dev)) return CC_ERR_ARG;                                                                                    \
    CC_ENTER(dev);                                                                                                    \
    if (LAZY(dev)) return cc_fail((dev), CC_ERR_UNSUPPORTED, "%s: not available on a lazy (graph / megakernel) device", what)
#define SEQ_VIEW(dev, v, what)                                                                                        \
    do {                                                                                                              \
        if (!view_ok(v)) return cc_fail((dev), CC_ERR_ARG, "%s: bad tensor view", what);                              \
        if (!view_in_bounds(v)) return cc_fail((dev), CC_ERR_TENSOR, "%s: view addresses element %lld of a buffer of %lld", what, \
                                               (long long)view_max_offset(v), (long long)(v)->buf->nelems);           \
        CC_REQUIRE(dev, view_contiguous(v), "%s: not contiguous", what);                                              \
    } while (0)
#define SEQ_F32(dev, v, what)                \
    do {                                     \
        SEQ_VIEW(dev, v, what);              \
        REQUIRE_F32(dev, v, what);           \
    } while (0)
static inline float* fptr(const cc_view* v) { return (float*)v->buf->plane[0]; }

__device__ __forceinline__ float seq_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float seq_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float seq_softplus(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float seq_gelu_tanh(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
__device__ __forceinline__ float seq_act(float z, int act) {
    return act == CC_ACT_SILU ? seq_silu(z) : act == CC_ACT_GELU_TANH ? seq_gelu_tanh(z) : act == CC_ACT_SIGMOID ? seq_sigmoid(z) : z;
}

extern "C" CC_API int cc_tensor_zero(cc_device* dev, const cc_view* x) {
    SEQ_ENTER(dev, "tensor_zero");
    SEQ_VIEW(dev, x, "tensor_zero");
    const size_t esz = cc_block_bytes(x->buf->dtype);
    CC_REQUIRE(dev, !cc_is_quant(x->buf->dtype), "tensor_zero: plain types only");
    if (view_len(x)) CC_CUDA(dev, cudaMemsetAsync(x->buf->plane[0], 0, (size_t)view_len(x) * esz, dev->stream));
    return CC_OK;
}

// ---- norms --------------------------------------------------------------------------------------------------------------------
// one warp per row: lane-strided sum of squares, butterfly, then the scaled write
__global__ void rms_norm_gain_kernel(float* __restrict__ dst, const float* __restrict__ y, const float* __restrict__ gain, int gain_n, int rows, int cols,
                                     float eps, int accumulate, float mult) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    const float* yr = y + (int64_t)r * cols;
    float ss = 0.0f;
    for (int c = lane; c < cols; c += 32) ss = fmaf(yr[c], yr[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    float* dr = dst + (int64_t)r * cols;
    for (int c = lane; c < cols; c += 32) {
        const float v = yr[c] * inv * gain[gain_n == 1 ? 0 : c] * mult;
        dr[c] = accumulate ? dr[c] + v : v;
    }
}
static int rms_norm_gain_impl(cc_device* dev, const cc_view* dst, const cc_view* y, const cc_view* gain, float eps, int32_t accumulate, float mult) {
    SEQ_ENTER(dev, "rms_norm_gain");
    SEQ_F32(dev, dst, "rms_norm_gain dst"); SEQ_F32(dev, y, "rms_norm_gain y"); SEQ_F32(dev, gain, "rms_norm_gain gain");
    CC_REQUIRE(dev, dst->ndim == 2 && y->ndim == 2 && dst->shape[0] == y->shape[0] && dst->shape[1] == y->shape[1], "rms_norm_gain: dst and y must be [rows, cols]");
    const int64_t rows = y->shape[0], cols = y->shape[1], gn = view_len(gain);
    CC_REQUIRE(dev, gn == 1 || gn == cols, "rms_norm_gain: gain has %lld elements, need 1 or %lld", (long long)gn, (long long)cols);
    if (rows == 0) return CC_OK;
    rms_norm_gain_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, dev->stream>>>(fptr(dst), fptr(y), fptr(gain), (int)gn, (int)rows, (int)cols, eps, accumulate, mult);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
extern "C" CC_API int cc_rms_norm_gain(cc_device* dev, const cc_view* dst, const cc_view* y, const cc_view* gain, float eps, int32_t accumulate) {
    return rms_norm_gain_impl(dev, dst, y, gain, eps, accumulate, 1.0f);
}
extern "C" CC_API int cc_rms_norm_gain_mult(cc_device* dev, const cc_view* dst, const cc_view* y, const cc_view* gain, float eps, float mult) {
    return rms_norm_gain_impl(dev, dst, y, gain, eps, 1, mult);
}

// one warp per (row, head)
// w_heads: how many heads have weights of their own (1: one vector for all)
__global__ void gated_head_rms_norm_kernel(float* __restrict__ x, const float* __restrict__ gate, const float* __restrict__ w, int64_t n_units, int hs, float eps, int act,
                                           int w_heads) {
    const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (u >= n_units) return;
    float* xr = x + u * hs;
    const float* gr = gate ? gate + u * hs : nullptr;
    const float* wr = w ? w + (u % w_heads) * hs : nullptr;
    float ss = 0.0f;
    for (int c = lane; c < hs; c += 32) ss = fmaf(xr[c], xr[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hs + eps);
    for (int c = lane; c < hs; c += 32) {
        float v = xr[c] * inv;
        if (wr) v *= wr[c];
        if (gr) v *= seq_act(gr[c], act);
        xr[c] = v;
    }
}
extern "C" CC_API int cc_gated_head_rms_norm(cc_device* dev, const cc_view* x, const cc_view* gate, const cc_view* w, int32_t head_size, float eps, int32_t gate_act) {
    SEQ_ENTER(dev, "gated_head_rms_norm");
    SEQ_F32(dev, x, "gated_head_rms_norm x");
    if (gate) SEQ_F32(dev, gate, "gated_head_rms_norm gate");
    if (w) SEQ_F32(dev, w, "gated_head_rms_norm w");
    const int64_t n = view_len(x);
    CC_REQUIRE(dev, head_size > 0 && n % head_size == 0 && (!gate || view_len(gate) == n), "gated_head_rms_norm: shapes do not fit head_size %d", head_size);
    int w_heads = 1;
    if (w && view_len(w) != head_size) {
        CC_REQUIRE(dev, x->ndim == 2 && view_len(w) == x->shape[1], "gated_head_rms_norm: w must have head_size elements or one per column");
        w_heads = (int)(x->shape[1] / head_size);
    }
    const int64_t units = n / head_size;
    if (!units) return CC_OK;
    gated_head_rms_norm_kernel<<<(unsigned)((units + 7) / 8), 256, 0, dev->stream>>>(fptr(x), gate ? fptr(gate) : nullptr, w ? fptr(w) : nullptr, units, head_size, eps, gate_act,
                                                                                    w_heads);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

__global__ void glu_kernel(float* __restrict__ g, const float* __restrict__ u, int64_t n, int act) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) g[i] = seq_act(g[i], act) * u[i];
}
extern "C" CC_API int cc_glu_inplace(cc_device* dev, const cc_view* gate, const cc_view* up, int32_t act) {
    SEQ_ENTER(dev, "glu_inplace");
    SEQ_F32(dev, gate, "glu_inplace gate"); SEQ_F32(dev, up, "glu_inplace up");
    const int64_t n = view_len(gate);
    CC_REQUIRE(dev, view_len(up) == n, "glu_inplace: sizes differ");
    if (!n) return CC_OK;
    glu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(gate), fptr(up), n, act);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
// gate | up side by side in one product's rows
__global__ void glu_halves_kernel(const float* __restrict__ src, const float* __restrict__ bias, float* __restrict__ out, int64_t n, int ff, int act) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t r = i / ff;
    const int c = (int)(i - r * ff);
    float g = src[r * 2 * ff + c], u = src[r * 2 * ff + ff + c];
    if (bias) { g += bias[c]; u += bias[ff + c]; }
    out[i] = seq_act(g, act) * u;
}
extern "C" CC_API int cc_glu_halves(cc_device* dev, const cc_view* src, const cc_view* bias, int32_t act, cc_buf** out) {
    SEQ_ENTER(dev, "glu_halves");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "glu_halves: out is NULL");
    SEQ_F32(dev, src, "glu_halves src");
    CC_REQUIRE(dev, src->ndim == 2 && src->shape[1] % 2 == 0, "glu_halves: src must be [rows, 2 * ff]");
    const int64_t rows = src->shape[0], ff = src->shape[1] / 2;
    if (bias) { SEQ_F32(dev, bias, "glu_halves bias"); CC_REQUIRE(dev, view_len(bias) == 2 * ff, "glu_halves: the bias needs one number per column of src"); }
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, rows * ff, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    const int64_t n = rows * ff;
    if (!n) return CC_OK;
    glu_halves_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(src), bias ? fptr(bias) : nullptr, (float*)o->base, n, (int)ff, act);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
__global__ void add_row_bias_kernel(float* __restrict__ x, const float* __restrict__ b, int64_t n, int cols) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += b[i % cols];
}
extern "C" CC_API int cc_add_row_bias(cc_device* dev, const cc_view* x, const cc_view* bias) {
    SEQ_ENTER(dev, "add_row_bias");
    SEQ_F32(dev, x, "add_row_bias x"); SEQ_F32(dev, bias, "add_row_bias bias");
    CC_REQUIRE(dev, x->ndim == 2 && view_len(bias) == x->shape[1], "add_row_bias: x must be [rows, cols] and bias [cols]");
    const int64_t n = view_len(x);
    if (!n) return CC_OK;
    add_row_bias_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(x), fptr(bias), n, (int)x->shape[1]);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
__global__ void scaled_sum_kernel(float* __restrict__ dst, const float* __restrict__ a, float sa, const float* __restrict__ b, float sb, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = sa * a[i] + sb * b[i];
}
extern "C" CC_API int cc_scaled_sum(cc_device* dev, const cc_view* dst, const cc_view* a, float sa, const cc_view* b, float sb) {
    SEQ_ENTER(dev, "scaled_sum");
    SEQ_F32(dev, dst, "scaled_sum dst"); SEQ_F32(dev, a, "scaled_sum a"); SEQ_F32(dev, b, "scaled_sum b");
    const int64_t n = view_len(dst);
    CC_REQUIRE(dev, view_len(a) == n && view_len(b) == n, "scaled_sum: sizes differ");
    if (!n) return CC_OK;
    scaled_sum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(dst), fptr(a), sa, fptr(b), sb, n);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

__global__ void scaled_sum_accumulate_kernel(float* __restrict__ dst, const float* __restrict__ a, float sa, const float* __restrict__ b, float sb, const float* __restrict__ c,
                                             int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = sa * a[i] + sb * b[i];
    if (c) v += c[i];
    dst[i] += v;
}
extern "C" CC_API int cc_scaled_sum_accumulate(cc_device* dev, const cc_view* dst, const cc_view* a, float sa, const cc_view* b, float sb, const cc_view* c) {
    SEQ_ENTER(dev, "scaled_sum_accumulate");
    SEQ_F32(dev, dst, "scaled_sum_accumulate dst"); SEQ_F32(dev, a, "scaled_sum_accumulate a"); SEQ_F32(dev, b, "scaled_sum_accumulate b");
    if (c) SEQ_F32(dev, c, "scaled_sum_accumulate c");
    const int64_t n = view_len(dst);
    CC_REQUIRE(dev, view_len(a) == n && view_len(b) == n && (!c || view_len(c) == n), "scaled_sum_accumulate: sizes differ");
    if (!n) return CC_OK;
    scaled_sum_accumulate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(dst), fptr(a), sa, fptr(b), sb, c ? fptr(c) : nullptr, n);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
// one gate number per (row, head): one thread per element
__global__ void head_gate_kernel(float* __restrict__ x, const float* __restrict__ g, int64_t n, int hs, int act) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= seq_act(g[i / hs], act);
}
extern "C" CC_API int cc_head_gate(cc_device* dev, const cc_view* x, const cc_view* g, int32_t n_heads, int32_t act) {
    SEQ_ENTER(dev, "head_gate");
    SEQ_F32(dev, x, "head_gate x"); SEQ_F32(dev, g, "head_gate g");
    CC_REQUIRE(dev, x->ndim == 2 && n_heads > 0 && x->shape[1] % n_heads == 0 && view_len(g) == x->shape[0] * n_heads,
               "head_gate: x must be [rows, heads * head_size] and g [rows, heads]");
    const int64_t n = view_len(x);
    if (!n) return CC_OK;
    head_gate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(x), fptr(g), n, (int)(x->shape[1] / n_heads), act);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
// out = [a | b] row by row: one thread per element of out
__global__ void concat_cols_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int64_t n, int ca, int cb) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t r = i / (ca + cb);
    const int c = (int)(i - r * (ca + cb));
    out[i] = c < ca ? a[r * ca + c] : b[r * cb + (c - ca)];
}
extern "C" CC_API int cc_concat_cols(cc_device* dev, const cc_view* a, const cc_view* b, cc_buf** out) {
    SEQ_ENTER(dev, "concat_cols");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "concat_cols: out is NULL");
    SEQ_F32(dev, a, "concat_cols a"); SEQ_F32(dev, b, "concat_cols b");
    CC_REQUIRE(dev, a->ndim == 2 && b->ndim == 2 && a->shape[0] == b->shape[0], "concat_cols: a and b must be [rows, ca] and [rows, cb]");
    const int64_t rows = a->shape[0], ca = a->shape[1], cb = b->shape[1];
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, rows * (ca + cb), CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    const int64_t n = rows * (ca + cb);
    if (!n) return CC_OK;
    concat_cols_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(a), fptr(b), (float*)o->base, n, (int)ca, (int)cb);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- a second embedding row chosen by a hash of the token pair ------------------------------------------------------------------------
// one thread per (token, column); the hash is taken in 64-bit integers
__global__ void pair_hash_rows_add_kernel(float* __restrict__ dst, const float* __restrict__ table, const int64_t* __restrict__ tok, const int32_t* __restrict__ last, int64_t n,
                                          int cols, int64_t mul_prev, int64_t mul_cur, int64_t buckets) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / cols;
    const int c = (int)(i - t * cols);
    const int64_t prev = t > 0 ? tok[t - 1] : (int64_t)last[0] - 1;
    const int64_t row = prev < 0 ? buckets : (prev * mul_prev + tok[t] * mul_cur) % buckets;
    dst[i] += table[row * cols + c];
}
__global__ void pair_hash_last_kernel(const int64_t* __restrict__ tok, int32_t* __restrict__ last, int n) { last[0] = (int32_t)tok[n - 1] + 1; }
extern "C" CC_API int cc_pair_hash_rows_add(cc_device* dev, const cc_view* dst, const cc_view* table, const int64_t* tokens, int32_t n, int32_t slot, const cc_view* last,
                                            int64_t mul_prev, int64_t mul_cur, int64_t buckets) {
    SEQ_ENTER(dev, "pair_hash_rows_add");
    SEQ_F32(dev, dst, "pair_hash_rows_add dst"); SEQ_F32(dev, table, "pair_hash_rows_add table");
    SEQ_VIEW(dev, last, "pair_hash_rows_add last");
    CC_REQUIRE(dev, last->buf->dtype == CC_I32 && view_len(last) == 1, "pair_hash_rows_add: last must be I32 [1]");
    CC_REQUIRE(dev, dst->ndim == 2 && table->ndim == 2 && dst->shape[1] == table->shape[1] && buckets >= 1 && table->shape[0] == buckets + 1 && mul_prev >= 0 && mul_cur >= 0,
               "pair_hash_rows_add: dst must be [n, cols] and table [buckets + 1, cols]");
    CC_REQUIRE(dev, n >= 0 && dst->shape[0] == n && (tokens || (n == 1 && slot >= 0 && slot < CC_N_SLOTS)), "pair_hash_rows_add: %d tokens for %lld rows", n, (long long)dst->shape[0]);
    if (n == 0) return CC_OK;
    const int64_t* tok = nullptr;
    if (tokens) {
        for (int i = 0; i < n; i++) CC_REQUIRE(dev, tokens[i] >= 0 && tokens[i] < ((int64_t)1 << 31) - 1, "pair_hash_rows_add: token id %lld", (long long)tokens[i]);
        int rc = cc_ensure_dev_idx(dev, (size_t)n * 8);
        if (rc) return rc;
        CC_CUDA(dev, cudaMemcpyAsync(dev->dev_idx, tokens, (size_t)n * 8, cudaMemcpyHostToDevice, dev->stream));
        tok = (const int64_t*)dev->dev_idx;
    } else {
        int rc = cc_ensure_slots(dev);
        if (rc) return rc;
        tok = dev->slots + slot;
    }
    const int64_t total = (int64_t)n * dst->shape[1];
    int32_t* lp = (int32_t*)last->buf->plane[0];
    pair_hash_rows_add_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(fptr(dst), fptr(table), tok, lp, total, (int)dst->shape[1], mul_prev, mul_cur, buckets);
    dev->launches++;
    pair_hash_last_kernel<<<1, 1, 0, dev->stream>>>(tok, lp, n);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- short causal convolution ----------------------------------------------------------------------------------------------------
// one warp per (token, run of hs channels).  in[t'] for t' < 0 comes from the tail: tail row (K-1) + t'.
// in_bias (or NULL) is added to every input of x as it is read; the tail holds inputs that already carry it (or the zeros before a sequence)
__global__ void short_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ tail,
                                  float* __restrict__ y, int T, int C, int K, int hs, int act, int unit, float ueps, float uscale, const float* __restrict__ in_bias) {
    const int heads = C / hs;
    const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (u >= (int64_t)T * heads) return;
    const int t = (int)(u / heads), h = (int)(u % heads);
    float ss = 0.0f;
    for (int cc = lane; cc < hs; cc += 32) {
        const int c = h * hs + cc;
        float acc = bias ? bias[c] : 0.0f;
        for (int j = 0; j < K; j++) {
            const int ti = t - (K - 1) + j;
            const float v = ti >= 0 ? (in_bias ? x[(int64_t)ti * C + c] + in_bias[c] : x[(int64_t)ti * C + c]) : tail[(int64_t)(ti + K - 1) * C + c];
            acc = fmaf(w[(int64_t)c * K + j], v, acc);
        }
        acc = seq_act(acc, act);
        y[(int64_t)t * C + c] = acc;
        ss = fmaf(acc, acc, ss);
    }
    if (unit) {
        ss = warp_sum(ss);
        const float f = uscale / sqrtf(ss + ueps);
        for (int cc = lane; cc < hs; cc += 32) y[(int64_t)t * C + h * hs + cc] *= f;
    }
}
// tail <- the last K-1 rows of (tail ++ x); one thread per channel, ascending rows: row j is written after row T + j > j was read
__global__ void short_conv_tail_kernel(const float* __restrict__ x, float* __restrict__ tail, int T, int C, int K, const float* __restrict__ in_bias) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float ib = in_bias ? in_bias[c] : 0.0f;
    for (int j = 0; j < K - 1; j++) {
        const int ti = T + j - (K - 1);
        tail[(int64_t)j * C + c] = ti >= 0 ? (in_bias ? x[(int64_t)ti * C + c] + ib : x[(int64_t)ti * C + c]) : tail[(int64_t)(ti + K - 1) * C + c];
    }
}
static int short_conv_impl(cc_device* dev, const cc_view* x, const cc_view* w, const cc_view* bias, const cc_view* tail, int32_t act, int32_t head_size, int32_t unit_norm,
                           float unit_eps, float unit_scale, cc_buf** out, const cc_view* in_bias = nullptr) {
    SEQ_ENTER(dev, "short_conv");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "short_conv: out is NULL");
    SEQ_F32(dev, x, "short_conv x"); SEQ_F32(dev, w, "short_conv w");
    CC_REQUIRE(dev, x->ndim == 2 && w->ndim == 2 && w->shape[0] == x->shape[1], "short_conv: x must be [T, C] and w [C, K]");
    const int64_t T = x->shape[0], C = x->shape[1], K = w->shape[1];
    CC_REQUIRE(dev, K >= 1, "short_conv: no taps");
    if (K > 1) {
        SEQ_F32(dev, tail, "short_conv tail");
        CC_REQUIRE(dev, view_len(tail) == (K - 1) * C, "short_conv: tail must be [K-1, C]");
    }
    int hs = head_size > 0 ? head_size : (int)C;
    CC_REQUIRE(dev, C % hs == 0, "short_conv: head_size %d does not divide %lld channels", hs, (long long)C);
    if (!unit_norm) {            // nothing ties the channels of a head together: a warp takes the widest run of at most 32 channels that divides C
        hs = 32;
        while (C % hs) hs--;
    }
    if (bias) { SEQ_F32(dev, bias, "short_conv bias"); CC_REQUIRE(dev, view_len(bias) == C, "short_conv: the bias needs one number per channel"); }
    if (in_bias) { SEQ_F32(dev, in_bias, "short_conv in_bias"); CC_REQUIRE(dev, view_len(in_bias) == C, "short_conv: the input bias needs one number per channel"); }
    const float* ibp = in_bias ? fptr(in_bias) : nullptr;
    cc_buf* y = nullptr;
    int rc = cc_new_activation(dev, T * C, CC_F32, false, &y);
    if (rc) return rc;
    *out = y;
    if (T == 0) return CC_OK;
    const float* tp = K > 1 ? fptr(tail) : nullptr;
    const int64_t units = T * (C / hs);
    short_conv_kernel<<<(unsigned)((units + 7) / 8), 256, 0, dev->stream>>>(fptr(x), fptr(w), bias ? fptr(bias) : nullptr, tp, (float*)y->base, (int)T, (int)C, (int)K, hs, act, unit_norm,
                                                                        unit_eps, unit_scale, ibp);
    CC_LAUNCH_CHECK(dev);
    if (K > 1) {
        short_conv_tail_kernel<<<(unsigned)((C + 127) / 128), 128, 0, dev->stream>>>(fptr(x), fptr(tail), (int)T, (int)C, (int)K, ibp);
        CC_LAUNCH_CHECK(dev);
    }
    return CC_OK;
}

extern "C" CC_API int cc_short_conv(cc_device* dev, const cc_view* x, const cc_view* w, const cc_view* tail, int32_t act, int32_t head_size, int32_t unit_norm,
                                    float unit_eps, float unit_scale, cc_buf** out) {
    return short_conv_impl(dev, x, w, nullptr, tail, act, head_size, unit_norm, unit_eps, unit_scale, out);
}
extern "C" CC_API int cc_short_conv_biases(cc_device* dev, const cc_view* x, const cc_view* w, const cc_view* in_bias, const cc_view* bias, const cc_view* tail, int32_t act,
                                           cc_buf** out) {
    return short_conv_impl(dev, x, w, bias, tail, act, 0, 0, 0.0f, 1.0f, out, in_bias);
}
extern "C" CC_API int cc_short_conv_bias(cc_device* dev, const cc_view* x, const cc_view* w, const cc_view* bias, const cc_view* tail, int32_t act, cc_buf** out) {
    return short_conv_impl(dev, x, w, bias, tail, act, 0, 0, 0.0f, 1.0f, out);
}

// ---- gated delta rule -------------------------------------------------------------------------------------------------------------
// beta / decay of every (token, head): bd[(t * H + h) * 2] = {sigmoid(b), exp(-exp(a_log) * softplus(a + dt_bias))}
__global__ void delta_gates_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ bd, int64_t n, int H) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int h = (int)(i % H);
    bd[i * 2] = seq_sigmoid(b[i]);
    bd[i * 2 + 1] = expf(-expf(a_log[h]) * seq_softplus(a[i] + dt_bias[h]));
}
// grid (H, ceil(dv / columns per CTA)).  A column j of the head's state S[dk][dv] is owned for the whole call by SPLIT adjacent threads,
// each holding dk / SPLIT of its entries: DK > 0 keeps them in registers (SPLIT = 2 for dk = 128, so that 64 registers hold a thread's
// share), DK == 0 (any dk) in shared memory [dk][DR_THREADS].  Tokens run in order; per token two passes over dk:
//   acc = sum_i S[i] k[i]           (the decayed read-out is decay * acc)
//   u = beta * (v - decay * acc) ;  S[i] = decay * S[i] + k[i] * u ;  out = sum_i S[i] q[i]
// k, q, beta and decay of DR_TB tokens at a time are staged in shared memory and the thread's v values in registers (one trip to L2 per
// block of tokens instead of several per token).  Both dot products run as four interleaved partial sums per thread (i mod 4), added as
// (p0 + p1) + (p2 + p3), then the SPLIT shares are added by a shuffle: a fixed order, the same for any T.
#define DR_THREADS 64
#define DR_TB 16
__device__ __forceinline__ void dr_cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
// one staging buffer: k[DR_TB][dk4], q[DR_TB][dk4], bd[DR_TB][2], v[DR_TB][DR_THREADS] (a thread's own value column)
__device__ __forceinline__ int dr_stage_floats(int dk4) { return 2 * DR_TB * dk4 + 2 * DR_TB + DR_TB * DR_THREADS; }
template <int DK, int SPLIT>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                                const float* __restrict__ bd, float* __restrict__ state, float* __restrict__ o, int T, int H, int G,
                                                                int dk, int dv) {
    extern __shared__ __align__(16) float dr_sm[];            // two staging buffers, then (DK == 0) the state columns
    constexpr int DKP = DK > 0 ? DK / SPLIT : 1;
    constexpr int COLS = DR_THREADS / SPLIT;
    const int dk4 = (dk + 3) & ~3;
    const int stage_floats = dr_stage_floats(dk4);
    const int h = blockIdx.x, g = h / (H / G);
    const int part = threadIdx.x % SPLIT;
    const int j = blockIdx.y * COLS + threadIdx.x / SPLIT;
    const bool live = j < dv;
    const int jj = live ? j : dv - 1;                       // idle threads shadow the last column and never store
    float S[DKP];
    float* Ss = dr_sm + 2 * stage_floats + threadIdx.x;      // generic: S[i] at Ss[i * DR_THREADS]
    float* sp = state + ((int64_t)h * dk + part * DKP) * dv + jj;
    if (DK > 0) {
#pragma unroll
        for (int i = 0; i < DKP; i++) S[i] = sp[(int64_t)i * dv];
    } else {
        for (int i = 0; i < dk4; i++) Ss[i * DR_THREADS] = i < dk ? sp[(int64_t)i * dv] : 0.0f;
    }
    // the pad lanes dk .. dk4 of both buffers are zero for the whole call (the copies below never touch them)
    if (dk4 != dk)
        for (int idx = threadIdx.x; idx < 2 * 2 * DR_TB; idx += DR_THREADS)
            for (int i = dk; i < dk4; i++) dr_sm[(idx / (2 * DR_TB)) * stage_floats + (idx % (2 * DR_TB)) * dk4 + i] = 0.0f;
    // asynchronous copies (cp.async) of a block of tokens: issued one block ahead, so the trip to L2 overlaps the recurrence
    auto stage = [&](int buf, int tb) {
        float* base = dr_sm + buf * stage_floats;
        const int nt = min(DR_TB, T - tb);
        if ((dk & 3) == 0) {
            const int per = dk >> 2;
            for (int idx = threadIdx.x; idx < nt * per; idx += DR_THREADS) {
                const int tt = idx / per, c = (idx - tt * per) * 4;
                const int64_t src = ((int64_t)(tb + tt) * G + g) * dk + c;
                dr_cp_async16(base + tt * dk4 + c, k + src);
                dr_cp_async16(base + (DR_TB + tt) * dk4 + c, q + src);
            }
        } else {
            for (int idx = threadIdx.x; idx < nt * dk; idx += DR_THREADS) {
                const int tt = idx / dk, c = idx - tt * dk;
                const int64_t src = ((int64_t)(tb + tt) * G + g) * dk + c;
                dr_cp_async4(base + tt * dk4 + c, k + src);
                dr_cp_async4(base + (DR_TB + tt) * dk4 + c, q + src);
            }
        }
        float* sbd = base + 2 * DR_TB * dk4;
        for (int idx = threadIdx.x; idx < nt * 2; idx += DR_THREADS) dr_cp_async4(sbd + idx, bd + ((int64_t)(tb + (idx >> 1)) * H + h) * 2 + (idx & 1));
        float* sv = sbd + 2 * DR_TB + threadIdx.x;
        for (int tt = 0; tt < nt; tt++) dr_cp_async4(sv + tt * DR_THREADS, v + ((int64_t)(tb + tt) * H + h) * dv + jj);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (T > 0) stage(0, 0);
    int buf = 0;
    for (int tb = 0; tb < T; tb += DR_TB, buf ^= 1) {
        const int nt = min(DR_TB, T - tb);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                      // this block has landed for everyone, and everyone is done with the other buffer
        if (tb + DR_TB < T) stage(buf ^ 1, tb + DR_TB);
        const float* base = dr_sm + buf * stage_floats;
        const float* sbd = base + 2 * DR_TB * dk4;
        const float* sv = sbd + 2 * DR_TB + threadIdx.x;
#pragma unroll 1
        for (int tt = 0; tt < nt; tt++) {
            const int t = tb + tt;
            const float* kt = base + tt * dk4 + part * DKP;
            const float* qt = base + (DR_TB + tt) * dk4 + part * DKP;
            const float beta = sbd[tt * 2], dec = sbd[tt * 2 + 1];
            const float vj = sv[tt * DR_THREADS];
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f, o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
            if (DK > 0) {
#pragma unroll
                for (int i = 0; i < DKP; i += 4) {
                    const float4 kv = *(const float4*)(kt + i);
                    a0 = fmaf(S[i], kv.x, a0); a1 = fmaf(S[i + 1], kv.y, a1); a2 = fmaf(S[i + 2], kv.z, a2); a3 = fmaf(S[i + 3], kv.w, a3);
                }
                float acc = (a0 + a1) + (a2 + a3);
                if (SPLIT == 2) acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                const float u = beta * (vj - dec * acc);
#pragma unroll
                for (int i = 0; i < DKP; i += 4) {
                    const float4 kv = *(const float4*)(kt + i);
                    const float4 qv = *(const float4*)(qt + i);
                    S[i] = fmaf(kv.x, u, dec * S[i]); S[i + 1] = fmaf(kv.y, u, dec * S[i + 1]); S[i + 2] = fmaf(kv.z, u, dec * S[i + 2]); S[i + 3] = fmaf(kv.w, u, dec * S[i + 3]);
                    o0 = fmaf(S[i], qv.x, o0); o1 = fmaf(S[i + 1], qv.y, o1); o2 = fmaf(S[i + 2], qv.z, o2); o3 = fmaf(S[i + 3], qv.w, o3);
                }
            } else {
                for (int i = 0; i < dk4; i += 4) {
                    const float4 kv = *(const float4*)(kt + i);
                    a0 = fmaf(Ss[i * DR_THREADS], kv.x, a0); a1 = fmaf(Ss[(i + 1) * DR_THREADS], kv.y, a1);
                    a2 = fmaf(Ss[(i + 2) * DR_THREADS], kv.z, a2); a3 = fmaf(Ss[(i + 3) * DR_THREADS], kv.w, a3);
                }
                const float u = beta * (vj - dec * ((a0 + a1) + (a2 + a3)));
                for (int i = 0; i < dk4; i += 4) {
                    const float4 kv = *(const float4*)(kt + i);
                    const float4 qv = *(const float4*)(qt + i);
                    const float s0 = fmaf(kv.x, u, dec * Ss[i * DR_THREADS]), s1 = fmaf(kv.y, u, dec * Ss[(i + 1) * DR_THREADS]);
                    const float s2 = fmaf(kv.z, u, dec * Ss[(i + 2) * DR_THREADS]), s3 = fmaf(kv.w, u, dec * Ss[(i + 3) * DR_THREADS]);
                    Ss[i * DR_THREADS] = s0; Ss[(i + 1) * DR_THREADS] = s1; Ss[(i + 2) * DR_THREADS] = s2; Ss[(i + 3) * DR_THREADS] = s3;
                    o0 = fmaf(s0, qv.x, o0); o1 = fmaf(s1, qv.y, o1); o2 = fmaf(s2, qv.z, o2); o3 = fmaf(s3, qv.w, o3);
                }
            }
            float outv = (o0 + o1) + (o2 + o3);
            if (SPLIT == 2) outv += __shfl_xor_sync(0xffffffffu, outv, 1);
            if (live && part == 0) o[((int64_t)t * H + h) * dv + j] = outv;
        }
    }
    if (live) {
        if (DK > 0) {
#pragma unroll
            for (int i = 0; i < DKP; i++) sp[(int64_t)i * dv] = S[i];
        } else {
            for (int i = 0; i < dk; i++) sp[(int64_t)i * dv] = Ss[i * DR_THREADS];
        }
    }
}
extern "C" CC_API int cc_gated_delta_rule(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* a, const cc_view* b,
                                          const cc_view* a_log, const cc_view* dt_bias, const cc_view* state, int32_t H, int32_t G, int32_t dk, int32_t dv,
                                          cc_buf** out) {
    SEQ_ENTER(dev, "gated_delta_rule");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "gated_delta_rule: out is NULL");
    SEQ_F32(dev, q, "gated_delta_rule q"); SEQ_F32(dev, k, "gated_delta_rule k"); SEQ_F32(dev, v, "gated_delta_rule v");
    SEQ_F32(dev, a, "gated_delta_rule a"); SEQ_F32(dev, b, "gated_delta_rule b"); SEQ_F32(dev, a_log, "gated_delta_rule a_log");
    SEQ_F32(dev, dt_bias, "gated_delta_rule dt_bias"); SEQ_F32(dev, state, "gated_delta_rule state");
    CC_REQUIRE(dev, H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0, "gated_delta_rule: bad head counts / sizes");
    CC_REQUIRE(dev, q->ndim == 2, "gated_delta_rule: q must be [T, n_kv * dk]");
    const int64_t T = q->shape[0];
    CC_REQUIRE(dev, view_len(q) == T * G * dk && view_len(k) == T * G * dk && view_len(v) == T * H * dv && view_len(a) == T * H && view_len(b) == T * H &&
                        view_len(a_log) == H && view_len(dt_bias) == H && view_len(state) == (int64_t)H * dk * dv,
               "gated_delta_rule: operand sizes do not fit T=%lld heads=%d kv=%d dk=%d dv=%d", (long long)T, H, G, dk, dv);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * H * dv, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    void* bdp = nullptr; size_t cls = 0;
    rc = cc_pool_alloc(dev, (size_t)T * H * 2 * 4, &bdp, &cls);
    if (rc) return rc;
    delta_gates_kernel<<<(unsigned)((T * H + 255) / 256), 256, 0, dev->stream>>>(fptr(a), fptr(b), fptr(a_log), fptr(dt_bias), (float*)bdp, T * H, H);
    dev->launches++;
    const int cols = dk == 128 ? DR_THREADS / 2 : DR_THREADS;
    dim3 grid((unsigned)H, (unsigned)((dv + cols - 1) / cols));
#define DR_ARGS fptr(q), fptr(k), fptr(v), (const float*)bdp, fptr(state), (float*)o->base, (int)T, H, G, dk, dv
    const int dk4 = (dk + 3) & ~3;
    const size_t stage = (size_t)2 * ((size_t)2 * DR_TB * dk4 + 2 * DR_TB + DR_TB * DR_THREADS) * 4;      // two staging buffers
    if (stage > 48 * 1024 && (dk == 32 || dk == 64 || dk == 128)) {
        cudaError_t e = dk == 32 ? cudaFuncSetAttribute(delta_rule_kernel<32, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage)
                        : dk == 64 ? cudaFuncSetAttribute(delta_rule_kernel<64, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage)
                                   : cudaFuncSetAttribute(delta_rule_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage);
        if (e != cudaSuccess) { cc_pool_free(dev, bdp, cls); return cc_fail(dev, CC_ERR_CUDA, "gated_delta_rule: %s", cudaGetErrorString(e)); }
    }
    if (dk == 32) delta_rule_kernel<32, 1><<<grid, DR_THREADS, stage, dev->stream>>>(DR_ARGS);
    else if (dk == 64) delta_rule_kernel<64, 1><<<grid, DR_THREADS, stage, dev->stream>>>(DR_ARGS);
    else if (dk == 128) delta_rule_kernel<128, 2><<<grid, DR_THREADS, stage, dev->stream>>>(DR_ARGS);
    else {
        const size_t smem = stage + (size_t)dk4 * DR_THREADS * 4;
        if (smem > 200 * 1024) { cc_pool_free(dev, bdp, cls); return cc_fail(dev, CC_ERR_UNSUPPORTED, "gated_delta_rule: dk=%d is too large", dk); }
        if (smem > 48 * 1024) CC_CUDA(dev, cudaFuncSetAttribute(delta_rule_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        delta_rule_kernel<0, 1><<<grid, DR_THREADS, smem, dev->stream>>>(DR_ARGS);
    }
#undef DR_ARGS
    cc_pool_free(dev, bdp, cls);            // stream-ordered pool: the next user of this block runs after the kernels above
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- sliding-window attention over a ring cache ---------------------------------------------------------------------------------------
// one warp per (token, kv head)
__global__ void kv_ring_append_kernel(float* __restrict__ kring, float* __restrict__ vring, const float* __restrict__ k, const float* __restrict__ v,
                                      const float* __restrict__ knw, float eps, int64_t pos0, int ring, int T, int G, int dk, int dv) {
    const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (u >= (int64_t)T * G) return;
    const int t = (int)(u / G), g = (int)(u % G);
    const int64_t row = (pos0 + t) % ring;
    const float* kr = k + ((int64_t)t * G + g) * dk;
    float* kd = kring + (row * G + g) * dk;
    if (knw) {
        float ss = 0.0f;
        for (int c = lane; c < dk; c += 32) ss = fmaf(kr[c], kr[c], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dk + eps);
        for (int c = lane; c < dk; c += 32) kd[c] = kr[c] * inv * knw[c];
    } else {
        for (int c = lane; c < dk; c += 32) kd[c] = kr[c];
    }
    const float* vr = v + ((int64_t)t * G + g) * dv;
    float* vd = vring + (row * G + g) * dv;
    for (int c = lane; c < dv; c += 32) vd[c] = vr[c];
}
extern "C" CC_API int cc_kv_ring_append(cc_device* dev, const cc_view* kring, const cc_view* vring, const cc_view* k, const cc_view* v, const cc_view* knw,
                                        float eps, int64_t pos0, int32_t G, int32_t dk, int32_t dv) {
    SEQ_ENTER(dev, "kv_ring_append");
    SEQ_F32(dev, kring, "kv_ring_append kring"); SEQ_F32(dev, vring, "kv_ring_append vring"); SEQ_F32(dev, k, "kv_ring_append k"); SEQ_F32(dev, v, "kv_ring_append v");
    if (knw) { SEQ_F32(dev, knw, "kv_ring_append k_norm_w"); CC_REQUIRE(dev, view_len(knw) == dk, "kv_ring_append: k_norm_w must have dk elements"); }
    CC_REQUIRE(dev, G > 0 && dk > 0 && dv > 0 && kring->ndim == 2 && k->ndim == 2 && pos0 >= 0, "kv_ring_append: bad arguments");
    const int64_t ring = kring->shape[0], T = k->shape[0];
    CC_REQUIRE(dev, view_len(kring) == ring * G * dk && view_len(vring) == ring * G * dv && view_len(k) == T * G * dk && view_len(v) == T * G * dv,
               "kv_ring_append: operand sizes do not fit kv=%d dk=%d dv=%d", G, dk, dv);
    CC_REQUIRE(dev, T <= ring, "kv_ring_append: %lld tokens do not fit a ring of %lld", (long long)T, (long long)ring);
    if (T == 0) return CC_OK;
    kv_ring_append_kernel<<<(unsigned)((T * G + 7) / 8), 256, 0, dev->stream>>>(fptr(kring), fptr(vring), fptr(k), fptr(v), knw ? fptr(knw) : nullptr, eps, pos0, (int)ring,
                                                                             (int)T, G, dk, dv);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// Three kernels (plus the query norm), all plain 32-bit arithmetic, shaped as banded tile products so that keys and values are read once
// per TILE of queries and once for all query heads of a key/value head, not once per (query, head):
//   1. wa_scores_kernel : S[row][c] = (q_row . k_j) * scale - r1 ln(1 + r2 (i - j)) for the visible j = lo_i + c, a 64 x 64 tile product over dk
//   2. wa_softmax_kernel: one warp per row: max, exp, sum, normalise (in place)
//   3. wa_values_kernel : out[row][d] = sum_c S[row][c] v[lo_i + c][d], a 64 x 64 tile product over the keys of the tile's band
// A row is one (query, head); a tile's 64 rows are the R = n_heads / n_kv heads of one key/value head for 64 / R consecutive queries.
// Every dot product runs over its index in ascending order inside ONE thread, the softmax sums depend on the row alone, and the value sum
// has one order per kernel (ascending keys in the tile kernel, masked keys adding an exact 0; four ascending quarters in the row kernel that
// serves calls of few rows): a query's result does not depend on where the call starts or what else it carries, and differs between a
// prompt pass and a decoded token only by the rounding of that last sum.
#define WA_TILE 64
#define WA_K 16
#define WA_THREADS 256
struct WaGeom {
    int T, H, G, R, dk, dv, window, block, ring, QT, cap;      // QT queries per tile; cap = row stride of S; block > 0: a query sees only its own block of positions
    int krs, vrs, vhs;                                  // floats between two rows of the key / value ring (vhs: between two heads' values inside a row)
    float softcap;                                      // > 0: score <- softcap * tanh(score / softcap), after the scale
    int64_t pos0;
};
__host__ __device__ __forceinline__ int64_t wa_lo(const WaGeom& g, int64_t i) {
    int64_t lo = (g.window > 0 && i - g.window + 1 > 0) ? i - g.window + 1 : 0;
    if (g.block > 0) { const int64_t b = i - i % g.block; lo = b > lo ? b : lo; }
    return lo;
}

__global__ void head_rms_norm_kernel(float* __restrict__ x, const float* __restrict__ w, int64_t n_units, int hs, float eps) {
    const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (u >= n_units) return;
    float* xr = x + u * hs;
    float ss = 0.0f;
    for (int c = lane; c < hs; c += 32) ss = fmaf(xr[c], xr[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hs + eps);
    for (int c = lane; c < hs; c += 32) xr[c] = xr[c] * inv * w[c];
}

// grid (key tiles of the band, query tiles, G)
__global__ void __launch_bounds__(WA_THREADS) wa_scores_kernel(const float* __restrict__ q, const float* __restrict__ kring, float* __restrict__ S, WaGeom g, float scale,
                                                               const float* __restrict__ r1, const float* __restrict__ r2) {
    __shared__ float sq[WA_K][WA_TILE + 4];
    __shared__ float sk[WA_K][WA_TILE + 4];
    const int t0 = blockIdx.y * g.QT, kvh = blockIdx.z;
    const int tq_n = min(g.QT, g.T - t0);
    const int64_t i_first = g.pos0 + t0, i_last = i_first + tq_n - 1;
    const int64_t band_lo = wa_lo(g, i_first);
    const int64_t j0 = band_lo + (int64_t)blockIdx.x * WA_TILE;
    if (j0 > i_last) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.0f;
    // the next 16 coordinates of queries and keys are fetched into registers while the current ones are multiplied
    float pq[4], pk[4];
    auto fetch = [&](int d0) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = threadIdx.x + e * WA_THREADS;
            const int r = idx >> 4, dd = idx & 15;
            const int tq = r / g.R, hr = r - tq * g.R;
            const bool din = d0 + dd < g.dk;
            pq[e] = (din && tq < tq_n) ? q[((int64_t)(t0 + tq) * g.H + kvh * g.R + hr) * g.dk + d0 + dd] : 0.0f;
            const int64_t j = j0 + r;
            pk[e] = (din && j <= i_last) ? kring[(j % g.ring) * g.krs + kvh * g.dk + d0 + dd] : 0.0f;
        }
    };
    fetch(0);
    for (int d0 = 0; d0 < g.dk; d0 += WA_K) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = threadIdx.x + e * WA_THREADS;
            sq[idx & 15][idx >> 4] = pq[e];
            sk[idx & 15][idx >> 4] = pk[e];
        }
        __syncthreads();
        if (d0 + WA_K < g.dk) fetch(d0 + WA_K);
#pragma unroll
        for (int dd = 0; dd < WA_K; dd++) {
            const float4 qv = *(const float4*)&sq[dd][ty * 4];
            const float4 kv = *(const float4*)&sk[dd][tx * 4];
            const float qr[4] = {qv.x, qv.y, qv.z, qv.w}, kr[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++) acc[a][b] = fmaf(qr[a], kr[b], acc[a][b]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; a++) {
        const int r = ty * 4 + a;
        const int tq = r / g.R, hr = r - tq * g.R;
        if (tq >= tq_n) continue;
        const int h = kvh * g.R + hr;
        const int64_t i = i_first + tq, lo = wa_lo(g, i);
        float* Sr = S + ((int64_t)(t0 + tq) * g.H + h) * g.cap;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int64_t j = j0 + tx * 4 + b;
            if (j < lo || j > i) continue;
            float sc = acc[a][b] * scale;
            if (g.softcap > 0.0f) sc = g.softcap * tanhf(sc / g.softcap);
            if (r1) sc -= r1[h] * log1pf(r2[h] * (float)(i - j));
            Sr[j - lo] = sc;
        }
    }
}
// few rows (decoding): grid (ceil(keys / 8), T, G), 256 threads.  The CTA stages the R queries of (token, key/value head); a warp owns one
// visible key and takes its dot product with each of them: lane-strided partial sums, then the butterfly.  The key row is read once for all
// R heads, and the keys spread over the whole device however few rows the call has.
__global__ void __launch_bounds__(256) wa_scores_row_kernel(const float* __restrict__ q, const float* __restrict__ kring, float* __restrict__ S, WaGeom g, float scale,
                                                            const float* __restrict__ r1, const float* __restrict__ r2) {
    extern __shared__ float wsr_sm[];             // [R][dk]
    const int t = blockIdx.y, kvh = blockIdx.z;
    const int64_t i = g.pos0 + t, lo = wa_lo(g, i);
    for (int e = threadIdx.x; e < g.R * g.dk; e += 256) wsr_sm[e] = q[((int64_t)t * g.H + kvh * g.R) * g.dk + e];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t j = lo + (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (j > i) return;
    const float* kr = kring + (j % g.ring) * g.krs + kvh * g.dk;
    for (int hr = 0; hr < g.R; hr++) {
        const float* qh = wsr_sm + hr * g.dk;
        float acc = 0.0f;
        for (int d = lane; d < g.dk; d += 32) acc = fmaf(qh[d], kr[d], acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            const int h = kvh * g.R + hr;
            float sc = acc * scale;
            if (g.softcap > 0.0f) sc = g.softcap * tanhf(sc / g.softcap);
            if (r1) sc -= r1[h] * log1pf(r2[h] * (float)(i - j));
            S[((int64_t)t * g.H + h) * g.cap + (j - lo)] = sc;
        }
    }
}
// one warp per row
// sink != NULL: the denominator also holds exp(sink[head]), a key without a value whose score is sink[head] as it stands (no scale)
__global__ void wa_softmax_kernel(float* __restrict__ S, WaGeom g, const float* __restrict__ sink) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (int64_t)g.T * g.H) return;
    const int64_t i = g.pos0 + row / g.H;
    const int n = (int)(i - wa_lo(g, i) + 1);
    float* Sr = S + row * g.cap;
    float mx = -INFINITY;
    for (int c = lane; c < n; c += 32) mx = fmaxf(mx, Sr[c]);
    mx = warp_max(mx);
    const float sk = sink ? sink[row % g.H] : -INFINITY;
    mx = fmaxf(mx, sk);
    float sum = 0.0f;
    for (int c = lane; c < n; c += 32) { const float e = expf(Sr[c] - mx); Sr[c] = e; sum += e; }
    sum = warp_sum(sum);
    if (sink) sum += expf(sk - mx);
    const float inv = 1.0f / sum;
    for (int c = lane; c < n; c += 32) Sr[c] *= inv;
}
// few rows (decoding): grid (rows, ceil(dv / 32)); a CTA owns 32 output columns of one row = (query, head).  The row's probabilities go to
// shared memory; the visible keys are cut into four contiguous quarters, warp w adds quarter w in ascending order for its lane's column,
// and the quarters are added as (p0 + p1) + (p2 + p3).  The order depends on the row alone (its number of visible keys), not on T.
// S holds the raw scores: every CTA of a row redoes the row's softmax in shared memory (warp 0, the sums in wa_softmax_kernel's order, so the
// weights are the same bits), which saves a launch per layer in decoding.
__global__ void __launch_bounds__(128) wa_values_row_kernel(const float* __restrict__ S, const float* __restrict__ vring, float* __restrict__ out, WaGeom g,
                                                            const float* __restrict__ sink) {
    extern __shared__ float wr_sm[];
    __shared__ float part[4][32];
    const int64_t row = blockIdx.x;
    const int t = (int)(row / g.H), h = (int)(row % g.H), kvh = h / g.R;
    const int64_t i = g.pos0 + t, lo = wa_lo(g, i);
    const int n = (int)(i - lo + 1);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int c = threadIdx.x; c < n; c += 128) wr_sm[c] = S[row * g.cap + c];
    __syncthreads();
    if (w == 0) {
        float mx = -INFINITY;
        for (int c = lane; c < n; c += 32) mx = fmaxf(mx, wr_sm[c]);
        mx = warp_max(mx);
        const float sk = sink ? sink[h] : -INFINITY;
        mx = fmaxf(mx, sk);
        float sum = 0.0f;
        for (int c = lane; c < n; c += 32) { const float e = expf(wr_sm[c] - mx); wr_sm[c] = e; sum += e; }
        sum = warp_sum(sum);
        if (sink) sum += expf(sk - mx);
        const float inv = 1.0f / sum;
        for (int c = lane; c < n; c += 32) wr_sm[c] *= inv;
    }
    __syncthreads();
    const int d = blockIdx.y * 32 + lane;
    const int per = (n + 3) >> 2;
    const int c_begin = min(n, w * per), c_end = min(n, c_begin + per);
    const int r0 = (int)(lo % g.ring);
    const int64_t rs = g.vrs;
    float acc = 0.0f;
    if (d < g.dv) {
        const float* vb = vring + (int64_t)kvh * g.vhs + d;
        int r = r0 + c_begin;
        if (r >= g.ring) r -= g.ring;
#pragma unroll 8
        for (int c = c_begin; c < c_end; c++) {
            acc = fmaf(wr_sm[c], vb[r * rs], acc);
            if (++r == g.ring) r = 0;
        }
    }
    part[w][lane] = acc;
    __syncthreads();
    if (w == 0 && d < g.dv) out[row * g.dv + d] = (part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane]);
}
// few rows, R > 1 query heads per key/value head: grid (T * G, ceil(dv / 32)), 512 threads.  A CTA owns 32 value columns of ALL R heads of
// one (token, key/value head), so every value row is read once for the group instead of once per head.  Each head's softmax is redone
// in shared memory by one warp (wa_softmax_kernel's order); the visible keys are cut into 16 contiguous segments, warp w adds segment w in
// ascending order into R accumulators per lane, and the segments are added in ascending order.  The order depends on the row alone.
template <int R>
__global__ void __launch_bounds__(512) wa_values_group_kernel(const float* __restrict__ S, const float* __restrict__ vring, float* __restrict__ out, WaGeom g,
                                                              const float* __restrict__ sink) {
    extern __shared__ float wg_sm[];
    const int t = blockIdx.x / g.G, kvh = blockIdx.x % g.G;
    const int64_t i = g.pos0 + t, lo = wa_lo(g, i);
    const int n = (int)(i - lo + 1);
    float* pr = wg_sm;                            // [R][n]
    float* part = wg_sm + (size_t)R * n;          // [16][R][32]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int hr = w; hr < R; hr += 16) {
        const int h = kvh * R + hr;
        const float* Sr = S + ((int64_t)t * g.H + h) * g.cap;
        float* p = pr + (size_t)hr * n;
        float mx = -INFINITY;
        for (int c = lane; c < n; c += 32) { const float v = Sr[c]; p[c] = v; mx = fmaxf(mx, v); }
        mx = warp_max(mx);
        const float sk = sink ? sink[h] : -INFINITY;
        mx = fmaxf(mx, sk);
        float sum = 0.0f;
        for (int c = lane; c < n; c += 32) { const float e = expf(p[c] - mx); p[c] = e; sum += e; }
        sum = warp_sum(sum);
        if (sink) sum += expf(sk - mx);
        const float inv = 1.0f / sum;
        for (int c = lane; c < n; c += 32) p[c] *= inv;
    }
    __syncthreads();
    const int d = blockIdx.y * 32 + lane;
    const int per = (n + 15) >> 4;
    const int c_begin = min(n, w * per), c_end = min(n, c_begin + per);
    float acc[R];
#pragma unroll
    for (int hr = 0; hr < R; hr++) acc[hr] = 0.0f;
    if (d < g.dv) {
        const float* vb = vring + (int64_t)kvh * g.vhs + d;
        const int64_t rs = g.vrs;
        int r = (int)(lo % g.ring) + c_begin;
        if (r >= g.ring) r -= g.ring;
#pragma unroll 4
        for (int c = c_begin; c < c_end; c++) {
            const float v = vb[r * rs];
#pragma unroll
            for (int hr = 0; hr < R; hr++) acc[hr] = fmaf(pr[(size_t)hr * n + c], v, acc[hr]);
            if (++r == g.ring) r = 0;
        }
    }
#pragma unroll
    for (int hr = 0; hr < R; hr++) part[(w * R + hr) * 32 + lane] = acc[hr];
    __syncthreads();
    for (int idx = threadIdx.x; idx < R * 32; idx += 512) {
        const int hr = idx >> 5, l = idx & 31;
        float sum = 0.0f;
#pragma unroll
        for (int ww = 0; ww < 16; ww++) sum += part[(ww * R + hr) * 32 + l];
        const int col = blockIdx.y * 32 + l;
        if (col < g.dv) out[((int64_t)t * g.H + kvh * R + hr) * g.dv + col] = sum;
    }
}
template <int R>
static cudaError_t wa_launch_group(cc_device* dev, const float* S, const float* v, float* out, const WaGeom& g, const float* sink, size_t smem) {
    if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(wa_values_group_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
    wa_values_group_kernel<R><<<dim3((unsigned)(g.T * g.G), (unsigned)((g.dv + 31) / 32)), 512, smem, dev->stream>>>(S, v, out, g, sink);
    return cudaSuccess;
}
// grid (dv tiles, query tiles, G)
__global__ void __launch_bounds__(WA_THREADS) wa_values_kernel(const float* __restrict__ S, const float* __restrict__ vring, float* __restrict__ out, WaGeom g) {
    __shared__ float sp[WA_K][WA_TILE + 4];       // [key][row]
    __shared__ float sv[WA_K][WA_TILE + 4];       // [key][dv column]
    const int t0 = blockIdx.y * g.QT, kvh = blockIdx.z, c0 = blockIdx.x * WA_TILE;
    const int tq_n = min(g.QT, g.T - t0);
    const int64_t i_first = g.pos0 + t0, i_last = i_first + tq_n - 1;
    const int64_t band_lo = wa_lo(g, i_first);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.0f;
    // the next block of 16 keys (probabilities and values) is fetched into registers while the current one is multiplied: the loads' latency
    // hides behind the arithmetic of a CTA that often has its SM to itself
    float pp[4], pv[4];
    auto fetch = [&](int64_t j0) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = threadIdx.x + e * WA_THREADS;
            {   // probabilities: consecutive threads read consecutive keys of one row
                const int r = idx >> 4, kk = idx & 15;
                const int tq = r / g.R, hr = r - tq * g.R;
                float p = 0.0f;
                if (tq < tq_n) {
                    const int64_t i = i_first + tq, lo = wa_lo(g, i), j = j0 + kk;
                    if (j >= lo && j <= i) p = S[((int64_t)(t0 + tq) * g.H + kvh * g.R + hr) * g.cap + (j - lo)];
                }
                pp[e] = p;
            }
            {   // values: consecutive threads read consecutive columns of one key
                const int kk = idx >> 6, c = idx & 63;
                const int64_t j = j0 + kk;
                pv[e] = (j <= i_last && c0 + c < g.dv) ? vring[(j % g.ring) * g.vrs + kvh * g.vhs + c0 + c] : 0.0f;
            }
        }
    };
    fetch(band_lo);
    for (int64_t j0 = band_lo; j0 <= i_last; j0 += WA_K) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = threadIdx.x + e * WA_THREADS;
            sp[idx & 15][idx >> 4] = pp[e];
            sv[idx >> 6][idx & 63] = pv[e];
        }
        __syncthreads();
        if (j0 + WA_K <= i_last) fetch(j0 + WA_K);
#pragma unroll
        for (int kk = 0; kk < WA_K; kk++) {
            const float4 pv4 = *(const float4*)&sp[kk][ty * 4];
            const float4 vv = *(const float4*)&sv[kk][tx * 4];
            const float pr[4] = {pv4.x, pv4.y, pv4.z, pv4.w}, vr[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++) acc[a][b] = fmaf(pr[a], vr[b], acc[a][b]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; a++) {
        const int r = ty * 4 + a;
        const int tq = r / g.R, hr = r - tq * g.R;
        if (tq >= tq_n) continue;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int c = c0 + tx * 4 + b;
            if (c < g.dv) out[((int64_t)(t0 + tq) * g.H + kvh * g.R + hr) * g.dv + c] = acc[a][b];
        }
    }
}
static int masked_attention_impl(cc_device* dev, const cc_view* q, const cc_view* qnw, float eps, const cc_view* kring, const cc_view* vring, int64_t pos0, int32_t H, int32_t G,
                                 int32_t dk, int32_t dv, int32_t window, int32_t block, float scale, const cc_view* r1, const cc_view* r2, const cc_view* sink, cc_buf** out,
                                 float softcap = 0.0f) {
    SEQ_ENTER(dev, "window_attention");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "window_attention: out is NULL");
    SEQ_F32(dev, q, "window_attention q"); SEQ_F32(dev, kring, "window_attention kring");
    if (vring) SEQ_F32(dev, vring, "window_attention vring");
    if (sink) { SEQ_F32(dev, sink, "window_attention sink"); CC_REQUIRE(dev, view_len(sink) == H, "window_attention: sink must have one number per head"); }
    if (qnw) { SEQ_F32(dev, qnw, "window_attention q_norm_w"); CC_REQUIRE(dev, view_len(qnw) == dk, "window_attention: q_norm_w must have dk elements"); }
    CC_REQUIRE(dev, (r1 == nullptr) == (r2 == nullptr), "window_attention: r1 and r2 come together");
    if (r1) {
        SEQ_F32(dev, r1, "window_attention r1"); SEQ_F32(dev, r2, "window_attention r2");
        CC_REQUIRE(dev, view_len(r1) == H && view_len(r2) == H, "window_attention: r1 / r2 must have one number per head");
    }
    CC_REQUIRE(dev, H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && q->ndim == 2 && kring->ndim == 2 && pos0 >= 0, "window_attention: bad arguments");
    const int64_t T = q->shape[0], ring = kring->shape[0];
    CC_REQUIRE(dev, view_len(q) == T * H * dk && view_len(kring) == ring * G * dk && (vring ? view_len(vring) == ring * G * dv : dv <= dk),
               "window_attention: operand sizes do not fit heads=%d kv=%d dk=%d dv=%d", H, G, dk, dv);
    const float* vptr = vring ? fptr(vring) : fptr(kring);            // no value ring: a key row's first dv columns are its value
    // the oldest row the first query needs must not have been overwritten by the newest row of this call
    const int64_t last = pos0 + T - 1;
    WaGeom g;
    g.window = window; g.block = block; g.softcap = softcap;
    const int64_t oldest = wa_lo(g, pos0);
    CC_REQUIRE(dev, T == 0 || last - oldest + 1 <= ring, "window_attention: positions %lld..%lld with window %d, block %d need more than the ring's %lld rows",
               (long long)pos0, (long long)last, window, block, (long long)ring);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * H * dv, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    // the most keys one query can see
    int64_t reach = last + 1;
    if (window > 0 && window < reach) reach = window;
    if (block > 0 && block < reach) reach = block;
    const int64_t maxn = reach;
    const int R = H / G;
    CC_REQUIRE(dev, R <= WA_TILE, "window_attention: %d query heads per key/value head (at most %d)", R, WA_TILE);
    g.T = (int)T; g.H = H; g.G = G; g.R = R; g.dk = dk; g.dv = dv; g.ring = (int)ring; g.QT = WA_TILE / R; g.cap = (int)maxn; g.pos0 = pos0;
    g.krs = G * dk; g.vrs = vring ? G * dv : G * dk; g.vhs = vring ? dv : dk;
    float* qp = fptr(q);
    if (qnw) {             // the query norm, in place: q is this call's private projection output in every caller of the runner; a caller that
                           // needs its q untouched passes a copy
        head_rms_norm_kernel<<<(unsigned)((T * H + 7) / 8), 256, 0, dev->stream>>>(qp, fptr(qnw), T * H, dk, eps);
        dev->launches++;
    }
    void* Sp = nullptr; size_t cls = 0;
    rc = cc_pool_alloc(dev, (size_t)T * H * maxn * 4, &Sp, &cls);
    if (rc) return rc;
    const int q_tiles = (int)((T + g.QT - 1) / g.QT);
    const int64_t band = reach - 1 + g.QT;                                             // keys a query tile can see
    const int64_t band_max = band < last + 1 ? band : last + 1;
    const bool few_rows = T * H <= 64;
    if (few_rows && (size_t)R * dk * 4 <= 160 * 1024) {
        const size_t smem = (size_t)R * dk * 4;
        if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(wa_scores_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) { cc_pool_free(dev, Sp, cls); return cc_fail(dev, CC_ERR_CUDA, "window_attention: %s", cudaGetErrorString(e)); } }
        wa_scores_row_kernel<<<dim3((unsigned)((maxn + 7) / 8), (unsigned)T, (unsigned)G), 256, smem, dev->stream>>>(qp, fptr(kring), (float*)Sp, g, scale, r1 ? fptr(r1) : nullptr,
                                                                                                                      r2 ? fptr(r2) : nullptr);
    } else {
        dim3 g1((unsigned)((band_max + WA_TILE - 1) / WA_TILE), (unsigned)q_tiles, (unsigned)G);
        wa_scores_kernel<<<g1, WA_THREADS, 0, dev->stream>>>(qp, fptr(kring), (float*)Sp, g, scale, r1 ? fptr(r1) : nullptr, r2 ? fptr(r2) : nullptr);
    }
    dev->launches++;
    const size_t group_smem = ((size_t)R * maxn + 16 * (size_t)R * 32) * 4;
    const bool group_values = few_rows && (R == 2 || R == 4 || R == 8 || R == 16) && group_smem <= 160 * 1024;
    const bool row_values = group_values || (few_rows && (size_t)maxn * 4 <= 160 * 1024);
    if (!row_values) {
        wa_softmax_kernel<<<(unsigned)((T * H + 7) / 8), 256, 0, dev->stream>>>((float*)Sp, g, sink ? fptr(sink) : nullptr);
        dev->launches++;
    }
    if (group_values) {
        const float* sp = sink ? fptr(sink) : nullptr;
        cudaError_t e = R == 2 ? wa_launch_group<2>(dev, (const float*)Sp, vptr, (float*)o->base, g, sp, group_smem)
                      : R == 4 ? wa_launch_group<4>(dev, (const float*)Sp, vptr, (float*)o->base, g, sp, group_smem)
                      : R == 8 ? wa_launch_group<8>(dev, (const float*)Sp, vptr, (float*)o->base, g, sp, group_smem)
                               : wa_launch_group<16>(dev, (const float*)Sp, vptr, (float*)o->base, g, sp, group_smem);
        if (e != cudaSuccess) { cc_pool_free(dev, Sp, cls); return cc_fail(dev, CC_ERR_CUDA, "window_attention: %s", cudaGetErrorString(e)); }
    } else if (row_values) {
        const size_t smem = (size_t)maxn * 4;
        if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(wa_values_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) { cc_pool_free(dev, Sp, cls); return cc_fail(dev, CC_ERR_CUDA, "window_attention: %s", cudaGetErrorString(e)); } }
        wa_values_row_kernel<<<dim3((unsigned)(T * H), (unsigned)((dv + 31) / 32)), 128, smem, dev->stream>>>((const float*)Sp, vptr, (float*)o->base, g, sink ? fptr(sink) : nullptr);
    } else {
        dim3 g3((unsigned)((dv + WA_TILE - 1) / WA_TILE), (unsigned)q_tiles, (unsigned)G);
        wa_values_kernel<<<g3, WA_THREADS, 0, dev->stream>>>((const float*)Sp, vptr, (float*)o->base, g);
    }
    cc_pool_free(dev, Sp, cls);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
extern "C" CC_API int cc_window_attention_sink(cc_device* dev, const cc_view* q, const cc_view* qnw, float eps, const cc_view* kring, const cc_view* vring, int64_t pos0,
                                               int32_t H, int32_t G, int32_t dk, int32_t dv, int32_t window, float scale, const cc_view* r1, const cc_view* r2,
                                               const cc_view* sink, cc_buf** out) {
    return masked_attention_impl(dev, q, qnw, eps, kring, vring, pos0, H, G, dk, dv, window, 0, scale, r1, r2, sink, out);
}
extern "C" CC_API int cc_masked_attention(cc_device* dev, const cc_view* q, const cc_view* kring, const cc_view* vring, int64_t pos0, int32_t H, int32_t G, int32_t dk, int32_t dv,
                                          int32_t window, int32_t block, float scale, const cc_view* sink, cc_buf** out) {
    return masked_attention_impl(dev, q, nullptr, 0.0f, kring, vring, pos0, H, G, dk, dv, window, block, scale, nullptr, nullptr, sink, out);
}
extern "C" CC_API int cc_masked_attention_capped(cc_device* dev, const cc_view* q, const cc_view* kring, const cc_view* vring, int64_t pos0, int32_t H, int32_t G, int32_t dk,
                                                 int32_t dv, int32_t window, int32_t block, float scale, float softcap, const cc_view* sink, cc_buf** out) {
    return masked_attention_impl(dev, q, nullptr, 0.0f, kring, vring, pos0, H, G, dk, dv, window, block, scale, nullptr, nullptr, sink, out, softcap);
}
extern "C" CC_API int cc_window_attention(cc_device* dev, const cc_view* q, const cc_view* qnw, float eps, const cc_view* kring, const cc_view* vring, int64_t pos0,
                                          int32_t H, int32_t G, int32_t dk, int32_t dv, int32_t window, float scale, const cc_view* r1, const cc_view* r2,
                                          cc_buf** out) {
    if (dev && !vring) return cc_fail(dev, CC_ERR_ARG, "window_attention: vring is NULL");
    return cc_window_attention_sink(dev, q, qnw, eps, kring, vring, pos0, H, G, dk, dv, window, scale, r1, r2, nullptr, out);
}

// ---- RMS norm in groups ----------------------------------------------------------------------------------------------------------------
// one warp per (row, group): the units are consecutive in memory, unit u covers x[u * gs, (u + 1) * gs)
__global__ void group_rms_norm_kernel(float* __restrict__ dst, const float* __restrict__ x, const float* __restrict__ w, int64_t n_units, int groups, int gs, float eps) {
    const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (u >= n_units) return;
    const float* xr = x + u * gs;
    const float* wr = w + (u % groups) * gs;
    float ss = 0.0f;
    for (int c = lane; c < gs; c += 32) ss = fmaf(xr[c], xr[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
    float* dr = dst + u * gs;
    for (int c = lane; c < gs; c += 32) dr[c] = xr[c] * inv * wr[c];
}
extern "C" CC_API int cc_group_rms_norm(cc_device* dev, const cc_view* dst, const cc_view* x, const cc_view* w, int32_t groups, float eps) {
    SEQ_ENTER(dev, "group_rms_norm");
    SEQ_F32(dev, dst, "group_rms_norm dst"); SEQ_F32(dev, x, "group_rms_norm x"); SEQ_F32(dev, w, "group_rms_norm w");
    CC_REQUIRE(dev, x->ndim == 2 && dst->ndim == 2 && dst->shape[0] == x->shape[0] && dst->shape[1] == x->shape[1], "group_rms_norm: dst and x must be [rows, cols]");
    const int64_t rows = x->shape[0], cols = x->shape[1];
    CC_REQUIRE(dev, groups >= 1 && cols % groups == 0 && view_len(w) == cols, "group_rms_norm: %lld columns, %d groups, %lld weights", (long long)cols, groups, (long long)view_len(w));
    if (rows == 0) return CC_OK;
    const int64_t units = rows * groups;
    group_rms_norm_kernel<<<(unsigned)((units + 7) / 8), 256, 0, dev->stream>>>(fptr(dst), fptr(x), fptr(w), units, groups, (int)(cols / groups), eps);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- layer norm with weight and bias ------------------------------------------------------------------------------------------------------
// one CTA per row: a thread keeps its (up to LN_KEEP) elements of the row in registers, so the row is read once; the mean first
// (thread-strided partial sums, the butterfly, then the warps' sums in warp order), then the mean of the squared deviations from it in the same
// order, then the scaled write.  The order depends on the row's length alone.
#define LN_THREADS 256
#define LN_KEEP 8
__device__ __forceinline__ float ln_block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();                                         // red may still be read from the sum before
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < LN_THREADS / 32; w++) t += red[w];
    return t;
}
__global__ void __launch_bounds__(LN_THREADS) layer_norm_kernel(float* dst, const float* x, const float* __restrict__ w, const float* __restrict__ b, int cols, float eps) {
    __shared__ float red[LN_THREADS / 32];
    const float* xr = x + (int64_t)blockIdx.x * cols;
    float* dr = dst + (int64_t)blockIdx.x * cols;
    float keep[LN_KEEP];
    float s = 0.0f;
#pragma unroll
    for (int e = 0; e < LN_KEEP; e++) {
        const int c = threadIdx.x + e * LN_THREADS;
        keep[e] = c < cols ? xr[c] : 0.0f;
        s += keep[e];
    }
    for (int c = threadIdx.x + LN_KEEP * LN_THREADS; c < cols; c += LN_THREADS) s += xr[c];
    const float mean = ln_block_sum(s, red) / (float)cols;
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < LN_KEEP; e++) {
        const int c = threadIdx.x + e * LN_THREADS;
        const float d = keep[e] - mean;
        if (c < cols) ss = fmaf(d, d, ss);
    }
    for (int c = threadIdx.x + LN_KEEP * LN_THREADS; c < cols; c += LN_THREADS) { const float d = xr[c] - mean; ss = fmaf(d, d, ss); }
    const float inv = 1.0f / sqrtf(ln_block_sum(ss, red) / (float)cols + eps);
    // a row wider than the registers hold is read again here, before any of it is overwritten by another thread: dst may be x, and thread t only
    // ever touches columns t, t + 256, ...
#pragma unroll
    for (int e = 0; e < LN_KEEP; e++) {
        const int c = threadIdx.x + e * LN_THREADS;
        if (c < cols) { const float v = (keep[e] - mean) * inv * w[c]; dr[c] = b ? v + b[c] : v; }
    }
    for (int c = threadIdx.x + LN_KEEP * LN_THREADS; c < cols; c += LN_THREADS) { const float v = (xr[c] - mean) * inv * w[c]; dr[c] = b ? v + b[c] : v; }
}
extern "C" CC_API int cc_layer_norm(cc_device* dev, const cc_view* dst, const cc_view* x, const cc_view* w, const cc_view* b, float eps) {
    SEQ_ENTER(dev, "layer_norm");
    SEQ_F32(dev, dst, "layer_norm dst"); SEQ_F32(dev, x, "layer_norm x"); SEQ_F32(dev, w, "layer_norm w");
    if (b) SEQ_F32(dev, b, "layer_norm b");
    CC_REQUIRE(dev, x->ndim == 2 && dst->ndim == 2 && dst->shape[0] == x->shape[0] && dst->shape[1] == x->shape[1], "layer_norm: dst and x must be [rows, cols]");
    const int64_t rows = x->shape[0], cols = x->shape[1];
    CC_REQUIRE(dev, cols >= 1 && view_len(w) == cols && (!b || view_len(b) == cols), "layer_norm: %lld columns need as many weights (and biases)", (long long)cols);
    if (rows == 0) return CC_OK;
    layer_norm_kernel<<<(unsigned)rows, LN_THREADS, 0, dev->stream>>>(fptr(dst), fptr(x), fptr(w), b ? fptr(b) : nullptr, (int)cols, eps);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// the gate first, then the norm.  One warp per (row, group), or one CTA of GGN_THREADS threads when a group is wide (a single warp would walk
// it in many dependent trips to memory).  Either way the gated value is written once, its squares are summed in an order that depends on
// the group's size alone (lane- or thread-strided partial sums, the butterfly, then the warps' sums in warp order), and the value is scaled.
#define GGN_THREADS 256
__global__ void gated_group_rms_norm_kernel(float* dst, const float* x, const float* __restrict__ gate, const float* __restrict__ w, int64_t n_units,
                                            int groups, int gs, float eps, int act) {
    const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (u >= n_units) return;
    const float* xr = x + u * gs;
    const float* gr = gate + u * gs;
    const float* wr = w + (u % groups) * gs;
    float* dr = dst + u * gs;
    float ss = 0.0f;
    for (int c = lane; c < gs; c += 32) { const float v = xr[c] * seq_act(gr[c], act); dr[c] = v; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
    for (int c = lane; c < gs; c += 32) dr[c] = dr[c] * inv * wr[c];
}
__global__ void __launch_bounds__(GGN_THREADS) gated_group_rms_norm_wide_kernel(float* dst, const float* x, const float* __restrict__ gate,
                                                                                const float* __restrict__ w, int groups, int gs, float eps, int act) {
    __shared__ float red[GGN_THREADS / 32];
    const int64_t u = blockIdx.x;
    const float* xr = x + u * gs;
    const float* gr = gate + u * gs;
    const float* wr = w + (u % groups) * gs;
    float* dr = dst + u * gs;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < gs; c += GGN_THREADS) { const float v = xr[c] * seq_act(gr[c], act); dr[c] = v; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < GGN_THREADS / 32; i++) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)gs + eps);
    for (int c = threadIdx.x; c < gs; c += GGN_THREADS) dr[c] = dr[c] * inv * wr[c];
}
extern "C" CC_API int cc_gated_group_rms_norm(cc_device* dev, const cc_view* dst, const cc_view* x, const cc_view* gate, const cc_view* w, int32_t groups, float eps,
                                              int32_t gate_act) {
    SEQ_ENTER(dev, "gated_group_rms_norm");
    SEQ_F32(dev, dst, "gated_group_rms_norm dst"); SEQ_F32(dev, x, "gated_group_rms_norm x"); SEQ_F32(dev, gate, "gated_group_rms_norm gate"); SEQ_F32(dev, w, "gated_group_rms_norm w");
    CC_REQUIRE(dev, x->ndim == 2 && dst->ndim == 2 && dst->shape[0] == x->shape[0] && dst->shape[1] == x->shape[1] && view_len(gate) == view_len(x),
               "gated_group_rms_norm: dst, x and gate must be [rows, cols]");
    const int64_t rows = x->shape[0], cols = x->shape[1];
    CC_REQUIRE(dev, groups >= 1 && cols % groups == 0 && view_len(w) == cols, "gated_group_rms_norm: %lld columns, %d groups, %lld weights", (long long)cols, groups,
               (long long)view_len(w));
    if (rows == 0) return CC_OK;
    const int64_t units = rows * groups;
    const int gs = (int)(cols / groups);
    if (gs >= 512) gated_group_rms_norm_wide_kernel<<<(unsigned)units, GGN_THREADS, 0, dev->stream>>>(fptr(dst), fptr(x), fptr(gate), fptr(w), groups, gs, eps, gate_act);
    else gated_group_rms_norm_kernel<<<(unsigned)((units + 7) / 8), 256, 0, dev->stream>>>(fptr(dst), fptr(x), fptr(gate), fptr(w), units, groups, gs, eps, gate_act);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- rotary positions from a frequency table, neighbouring coordinates paired -------------------------------------------------------------
// the angle is the 32-bit product of the position and the pair's frequency; cosf / sinf are the accurate library functions
__device__ __forceinline__ void rotate_pair(float u, float v, float pos, float f, float mag, float& ou, float& ov) {
    const float a = pos * f;
    const float c = cosf(a) * mag, s = sinf(a) * mag;
    ou = u * c - v * s;
    ov = v * c + u * s;
}
// one thread per (token, head, pair)
// pair i of a head is the columns off + i * step and off + i * step + gap: (step, gap) = (2, 1) pairs neighbours, (1, half) pairs the two
// halves of the rotated columns
__global__ void rope_pairs_kernel(float* x, const float* __restrict__ freq, int64_t n, int heads, int hs, int off, int half, float mag, int64_t pos0, int step, int gap,
                                  float* x2) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (x2 ? 2 * n : n)) return;
    if (idx >= n) { idx -= n; x = x2; }                              // a second tensor of the same shape rides along
    const int i = (int)(idx % half);
    const int64_t th = idx / half;                                   // token * heads + head
    float* p = x + th * hs + off + step * i;
    float ou, ov;
    rotate_pair(p[0], p[gap], (float)(pos0 + th / heads), freq[i], mag, ou, ov);
    p[0] = ou; p[gap] = ov;
}
static int rope_table_impl(cc_device* dev, const cc_view* x, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag, int64_t pos0, bool halves,
                           const cc_view* x2 = nullptr);
extern "C" CC_API int cc_rope_pairs(cc_device* dev, const cc_view* x, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag, int64_t pos0) {
    return rope_table_impl(dev, x, n_heads, head_size, offset, freq, mag, pos0, false);
}
extern "C" CC_API int cc_rope_halves(cc_device* dev, const cc_view* x, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag, int64_t pos0) {
    return rope_table_impl(dev, x, n_heads, head_size, offset, freq, mag, pos0, true);
}
extern "C" CC_API int cc_rope_halves_two(cc_device* dev, const cc_view* x1, const cc_view* x2, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag,
                                         int64_t pos0) {
    if (dev && !x2) return cc_fail(dev, CC_ERR_ARG, "rope_halves_two: the second tensor is NULL");
    return rope_table_impl(dev, x1, n_heads, head_size, offset, freq, mag, pos0, true, x2);
}
static int rope_table_impl(cc_device* dev, const cc_view* x, int32_t n_heads, int32_t head_size, int32_t offset, const cc_view* freq, float mag, int64_t pos0, bool halves,
                           const cc_view* x2) {
    SEQ_ENTER(dev, "rope_pairs");
    if (x2) { SEQ_F32(dev, x2, "rope_pairs second tensor"); CC_REQUIRE(dev, x2->ndim == 2 && x->ndim == 2 && x2->shape[0] == x->shape[0] && x2->shape[1] == x->shape[1], "rope_pairs: the two tensors differ in shape"); }
    SEQ_F32(dev, x, "rope_pairs x"); SEQ_F32(dev, freq, "rope_pairs freq");
    const int64_t half = view_len(freq);
    CC_REQUIRE(dev, x->ndim == 2 && n_heads > 0 && head_size > 0 && x->shape[1] == (int64_t)n_heads * head_size && offset >= 0 && offset + 2 * half <= head_size && pos0 >= 0,
               "rope_pairs: %lld pairs at column %d do not fit heads of %d", (long long)half, offset, head_size);
    const int64_t n = x->shape[0] * n_heads * half;
    if (n == 0) return CC_OK;
    const int64_t items = x2 ? 2 * n : n;
    rope_pairs_kernel<<<(unsigned)((items + 255) / 256), 256, 0, dev->stream>>>(fptr(x), fptr(freq), n, n_heads, head_size, offset, (int)half, mag, pos0, halves ? 1 : 2,
                                                                                halves ? (int)half : 1, x2 ? fptr(x2) : nullptr);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- queries and keys from projection to cache in one pass ---------------------------------------------------------------------------------
struct QkPrepArgs {
    float *q, *kring, *vring;
    const float *k, *v, *qw, *kw, *freq;
    int H, G, dk, dv, ring, norm, half, step, gap, off;      // pair i of a head: columns off + i * step and off + i * step + gap
    float eps, mag;
    int64_t pos0;
};
#define QKP_THREADS 256
// one CTA per token.  First the inverse root mean squares -- one per head (a warp per head: lane-strided sum, butterfly) or one per projection
// (thread-strided sums, butterfly, the warps' sums in warp order) -- then every element once: a rotated pair by the thread of its first
// column, which reads both raw values and writes both results; all raw values were read for the sums before the barrier, so q may be
// overwritten in place.
__global__ void __launch_bounds__(QKP_THREADS) qk_prepare_kernel(QkPrepArgs a) {
    extern __shared__ float qkp_sm[];               // inv[H + G], red[8]
    float* inv = qkp_sm;
    float* red = qkp_sm + a.H + a.G;
    const int t = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float* qr = a.q + (int64_t)t * a.H * a.dk;
    const float* kr = a.k + (int64_t)t * a.G * a.dk;
    const int units = a.H + a.G;
    if (a.norm == CC_QK_NORM_HEAD) {
        for (int u = w; u < units; u += QKP_THREADS / 32) {
            const float* src = u < a.H ? qr + u * a.dk : kr + (u - a.H) * a.dk;
            float ss = 0.0f;
            for (int c = lane; c < a.dk; c += 32) ss = fmaf(src[c], src[c], ss);
            ss = warp_sum(ss);
            if (lane == 0) inv[u] = 1.0f / sqrtf(ss / (float)a.dk + a.eps);
        }
    } else if (a.norm == CC_QK_NORM_ROW) {
        for (int side = 0; side < 2; side++) {
            const float* src = side ? kr : qr;
            const int n = (side ? a.G : a.H) * a.dk;
            float ss = 0.0f;
            for (int c = threadIdx.x; c < n; c += QKP_THREADS) ss = fmaf(src[c], src[c], ss);
            ss = warp_sum(ss);
            __syncthreads();
            if (lane == 0) red[w] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < QKP_THREADS / 32; i++) tot += red[i];
            const float v = 1.0f / sqrtf(tot / (float)n + a.eps);
            for (int u = threadIdx.x; u < (side ? a.G : a.H); u += QKP_THREADS) inv[(side ? a.H : 0) + u] = v;
        }
    } else {
        for (int u = threadIdx.x; u < units; u += QKP_THREADS) inv[u] = 1.0f;
    }
    __syncthreads();
    const int64_t row = (a.pos0 + t) % a.ring;
    const float pos = (float)(a.pos0 + t);
    for (int idx = threadIdx.x; idx < units * a.dk; idx += QKP_THREADS) {
        const int u = idx / a.dk, c = idx - u * a.dk;
        const bool is_q = u < a.H;
        const int ul = is_q ? u : u - a.H;
        const float* src = is_q ? qr + u * a.dk : kr + ul * a.dk;
        float* dst = is_q ? qr + u * a.dk : a.kring + (row * a.G + ul) * a.dk;
        const float* wt = is_q ? a.qw : a.kw;
        if (wt && a.norm == CC_QK_NORM_ROW) wt += ul * a.dk;
        const float f = inv[u];
        const int rel = c - a.off;
        int pair = -1;                               // index of the pair this thread owns, -2: the pair's second column (its owner writes it)
        if (rel >= 0 && a.half > 0) {
            if (a.step == 1) pair = rel < a.half ? rel : rel < 2 * a.half ? -2 : -1;
            else if (rel < 2 * a.half) pair = (rel & 1) ? -2 : rel >> 1;
        }
        if (pair == -2) continue;
        const float x0 = wt ? src[c] * f * wt[c] : src[c] * f;
        if (pair >= 0) {
            const int c1 = c + a.gap;
            const float x1 = wt ? src[c1] * f * wt[c1] : src[c1] * f;
            float o0, o1;
            rotate_pair(x0, x1, pos, a.freq[pair], a.mag, o0, o1);
            dst[c] = o0; dst[c1] = o1;
        } else {
            dst[c] = x0;
        }
    }
    const float* vr = a.v + (int64_t)t * a.G * a.dv;
    float* vd = a.vring + row * a.G * a.dv;
    for (int c = threadIdx.x; c < a.G * a.dv; c += QKP_THREADS) vd[c] = vr[c];
}
extern "C" CC_API int cc_qk_prepare_append(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* kring, const cc_view* vring, int32_t qk_norm,
                                           const cc_view* q_w, const cc_view* k_w, float eps, const cc_view* freq, int32_t pairing, int32_t offset, float mag, int64_t pos0,
                                           int32_t H, int32_t G, int32_t dk, int32_t dv) {
    SEQ_ENTER(dev, "qk_prepare_append");
    SEQ_F32(dev, q, "qk_prepare_append q"); SEQ_F32(dev, k, "qk_prepare_append k"); SEQ_F32(dev, v, "qk_prepare_append v");
    SEQ_F32(dev, kring, "qk_prepare_append kring"); SEQ_F32(dev, vring, "qk_prepare_append vring");
    CC_REQUIRE(dev, H > 0 && G > 0 && dk > 0 && dv > 0 && q->ndim == 2 && kring->ndim == 2 && pos0 >= 0 && qk_norm >= CC_QK_NORM_NONE && qk_norm <= CC_QK_NORM_ROW,
               "qk_prepare_append: bad arguments");
    const int64_t T = q->shape[0], ring = kring->shape[0];
    CC_REQUIRE(dev, view_len(q) == T * H * dk && view_len(k) == T * G * dk && view_len(v) == T * G * dv && view_len(kring) == ring * G * dk && view_len(vring) == ring * G * dv,
               "qk_prepare_append: operand sizes do not fit heads=%d kv=%d dk=%d dv=%d", H, G, dk, dv);
    CC_REQUIRE(dev, T <= ring, "qk_prepare_append: %lld tokens do not fit a ring of %lld", (long long)T, (long long)ring);
    const int64_t wq = qk_norm == CC_QK_NORM_ROW ? (int64_t)H * dk : dk, wk = qk_norm == CC_QK_NORM_ROW ? (int64_t)G * dk : dk;
    if (q_w) { SEQ_F32(dev, q_w, "qk_prepare_append q_w"); CC_REQUIRE(dev, qk_norm != CC_QK_NORM_NONE && view_len(q_w) == wq, "qk_prepare_append: q_w must have %lld elements", (long long)wq); }
    if (k_w) { SEQ_F32(dev, k_w, "qk_prepare_append k_w"); CC_REQUIRE(dev, qk_norm != CC_QK_NORM_NONE && view_len(k_w) == wk, "qk_prepare_append: k_w must have %lld elements", (long long)wk); }
    int64_t half = 0;
    if (freq) {
        SEQ_F32(dev, freq, "qk_prepare_append freq");
        half = view_len(freq);
        CC_REQUIRE(dev, offset >= 0 && offset + 2 * half <= dk && (pairing == CC_ROPE_NEIGHBOURS || pairing == CC_ROPE_HALVES), "qk_prepare_append: %lld pairs at column %d do not fit heads of %d",
                   (long long)half, offset, dk);
    }
    if (T == 0) return CC_OK;
    QkPrepArgs a{};
    a.q = fptr(q); a.k = fptr(k); a.v = fptr(v); a.kring = fptr(kring); a.vring = fptr(vring); a.qw = q_w ? fptr(q_w) : nullptr; a.kw = k_w ? fptr(k_w) : nullptr;
    a.freq = freq ? fptr(freq) : nullptr; a.H = H; a.G = G; a.dk = dk; a.dv = dv; a.ring = (int)ring; a.norm = qk_norm; a.half = (int)half; a.off = offset;
    a.step = pairing == CC_ROPE_HALVES ? 1 : 2; a.gap = pairing == CC_ROPE_HALVES ? (int)half : 1; a.eps = eps; a.mag = mag; a.pos0 = pos0;
    const size_t smem = (size_t)(H + G + QKP_THREADS / 32) * 4;
    CC_REQUIRE(dev, smem <= 48 * 1024, "qk_prepare_append: too many heads");
    qk_prepare_kernel<<<(unsigned)T, QKP_THREADS, smem, dev->stream>>>(a);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- latent key/value cache ------------------------------------------------------------------------------------------------------------------
// one warp per token: the first `rank` columns are RMS-normalised and weighted, the pairs of the next columns rotated, the rest copied
__global__ void latent_ring_append_kernel(float* __restrict__ ring, const float* __restrict__ ckv, const float* __restrict__ nw, const float* __restrict__ freq, float eps,
                                          float mag, int64_t pos0, int ring_rows, int T, int rank, int rest, int half) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const int cols = rank + rest;
    const float* src = ckv + (int64_t)t * cols;
    float* dst = ring + ((pos0 + t) % ring_rows) * cols;
    float ss = 0.0f;
    for (int c = lane; c < rank; c += 32) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int c = lane; c < rank; c += 32) dst[c] = src[c] * inv * (nw ? nw[c] : 1.0f);
    for (int i = lane; i < half; i += 32) {
        float ou, ov;
        rotate_pair(src[rank + 2 * i], src[rank + 2 * i + 1], (float)(pos0 + t), freq[i], mag, ou, ov);
        dst[rank + 2 * i] = ou; dst[rank + 2 * i + 1] = ov;
    }
    for (int c = rank + 2 * half + lane; c < cols; c += 32) dst[c] = src[c];
}
extern "C" CC_API int cc_latent_ring_append(cc_device* dev, const cc_view* ring, const cc_view* ckv, const cc_view* norm_w, float eps, int32_t rank, const cc_view* freq,
                                            float mag, int64_t pos0) {
    SEQ_ENTER(dev, "latent_ring_append");
    SEQ_F32(dev, ring, "latent_ring_append ring"); SEQ_F32(dev, ckv, "latent_ring_append ckv");
    if (norm_w) SEQ_F32(dev, norm_w, "latent_ring_append norm_w");
    if (freq) SEQ_F32(dev, freq, "latent_ring_append freq");
    CC_REQUIRE(dev, ring->ndim == 2 && ckv->ndim == 2 && ring->shape[1] == ckv->shape[1] && pos0 >= 0, "latent_ring_append: ring and rows must be 2-D with equal columns");
    const int64_t cols = ckv->shape[1], T = ckv->shape[0], half = freq ? view_len(freq) : 0;
    CC_REQUIRE(dev, rank >= 1 && rank + 2 * half <= cols && (!norm_w || view_len(norm_w) == rank), "latent_ring_append: rank %d + %lld rotated pairs do not fit %lld columns", rank,
               (long long)half, (long long)cols);
    CC_REQUIRE(dev, T <= ring->shape[0], "latent_ring_append: %lld tokens do not fit a ring of %lld", (long long)T, (long long)ring->shape[0]);
    if (T == 0) return CC_OK;
    latent_ring_append_kernel<<<(unsigned)((T + 7) / 8), 256, 0, dev->stream>>>(fptr(ring), fptr(ckv), norm_w ? fptr(norm_w) : nullptr, freq ? fptr(freq) : nullptr, eps, mag, pos0,
                                                                                  (int)ring->shape[0], (int)T, rank, (int)(cols - rank), (int)half);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- per-head products: the up-projections of a latent cache, folded into the query and applied to the attention result ---------------------
#define HP_TOK 8
// grid (ceil(T / 8), H, ceil(n_out / 4)): the CTA stages 8 tokens' x[t, h, :n_in]; a warp owns one output coordinate for those tokens:
// lane-strided partial sums over n_in, then the butterfly -- one order per output, whatever T is.  W: [H * n_out, n_in], rows read
// contiguously.  The `rest` columns behind a head's n_in inputs are copied behind its n_out outputs.
__global__ void __launch_bounds__(128) head_project_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ out, int T, int H, int n_in, int rest,
                                                           int n_out, const float* __restrict__ freq, int half, float mag, int64_t pos0) {
    extern __shared__ float hp_sm[];
    const int t0 = blockIdx.x * HP_TOK, h = blockIdx.y;
    const int xs = n_in + rest, os = n_out + rest;
    for (int i = threadIdx.x; i < HP_TOK * n_in; i += 128) {
        const int tt = i / n_in, d = i - tt * n_in;
        hp_sm[i] = t0 + tt < T ? x[((int64_t)(t0 + tt) * H + h) * xs + d] : 0.0f;
    }
    if (blockIdx.z == 0) {
        // the carried columns: the first 2 * half of them are rotated on the way when a frequency table is given
        for (int i = threadIdx.x; i < HP_TOK * half; i += 128) {
            const int tt = i / half, p = i - tt * half;
            if (t0 + tt >= T) continue;
            const float* src = x + ((int64_t)(t0 + tt) * H + h) * xs + n_in + 2 * p;
            float* dst = out + ((int64_t)(t0 + tt) * H + h) * os + n_out + 2 * p;
            rotate_pair(src[0], src[1], (float)(pos0 + t0 + tt), freq[p], mag, dst[0], dst[1]);
        }
        const int plain = rest - 2 * half;
        for (int i = threadIdx.x; i < HP_TOK * plain; i += 128) {
            const int tt = i / plain, j = 2 * half + (i - tt * plain);
            if (t0 + tt < T) out[((int64_t)(t0 + tt) * H + h) * os + n_out + j] = x[((int64_t)(t0 + tt) * H + h) * xs + n_in + j];
        }
    }
    __syncthreads();
    const int v = blockIdx.z * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (v >= n_out) return;
    const float* wp = W + ((int64_t)h * n_out + v) * n_in;
    float acc[HP_TOK];
#pragma unroll
    for (int tt = 0; tt < HP_TOK; tt++) acc[tt] = 0.0f;
    for (int d = lane; d < n_in; d += 32) {
        const float wv = wp[d];
#pragma unroll
        for (int tt = 0; tt < HP_TOK; tt++) acc[tt] = fmaf(hp_sm[tt * n_in + d], wv, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < HP_TOK; tt++) {
        const float sum = warp_sum(acc[tt]);
        if (lane == 0 && t0 + tt < T) out[((int64_t)(t0 + tt) * H + h) * os + v] = sum;
    }
}
// many rows and nothing carried: a 64 x 64 output tile of one head per CTA, 16-deep slices of the inputs through shared memory, 4 x 4 outputs
// per thread, every sum over n_in in ascending order inside one thread.  grid (ceil(n_out / 64), ceil(T / 64), H)
#define HPT_TILE 64
#define HPT_K 16
__global__ void __launch_bounds__(256) head_project_tile_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ out, int T, int H, int n_in, int n_out) {
    __shared__ float sw[HPT_K][HPT_TILE + 4];
    __shared__ float sx[HPT_K][HPT_TILE + 4];
    const int o0 = blockIdx.x * HPT_TILE, t0 = blockIdx.y * HPT_TILE, h = blockIdx.z;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const float* Wh = W + (int64_t)h * n_out * n_in;
    const int64_t xrs = (int64_t)H * n_in, ors = (int64_t)H * n_out;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < n_in; k0 += HPT_K) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = threadIdx.x + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const bool kin = k0 + kk < n_in;
            sw[kk][r] = (kin && o0 + r < n_out) ? Wh[(int64_t)(o0 + r) * n_in + k0 + kk] : 0.0f;
            sx[kk][r] = (kin && t0 + r < T) ? x[(int64_t)(t0 + r) * xrs + h * n_in + k0 + kk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HPT_K; kk++) {
            const float4 wv = *(const float4*)&sw[kk][tx * 4];
            const float4 xv = *(const float4*)&sx[kk][ty * 4];
            const float wr[4] = {wv.x, wv.y, wv.z, wv.w}, xr[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xr[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int o = o0 + tx * 4 + j;
            if (o < n_out) out[(int64_t)t * ors + h * n_out + o] = acc[i][j];
        }
    }
}
extern "C" CC_API int cc_head_project(cc_device* dev, const cc_view* x, const cc_view* w, int32_t n_heads, int32_t rest, const cc_view* freq, float mag, int64_t pos0,
                                      cc_buf** out) {
    SEQ_ENTER(dev, "head_project");
    if (freq) { SEQ_F32(dev, freq, "head_project freq"); CC_REQUIRE(dev, 2 * view_len(freq) <= rest && pos0 >= 0, "head_project: more rotated pairs than carried columns"); }
    if (!out) return cc_fail(dev, CC_ERR_ARG, "head_project: out is NULL");
    SEQ_F32(dev, x, "head_project x"); SEQ_F32(dev, w, "head_project w");
    CC_REQUIRE(dev, x->ndim == 2 && w->ndim == 2 && n_heads > 0 && rest >= 0 && w->shape[0] % n_heads == 0 && x->shape[1] == (int64_t)n_heads * (w->shape[1] + rest),
               "head_project: x must be [T, heads * (n_in + rest)] and w [heads * n_out, n_in]");
    const int64_t T = x->shape[0], n_in = w->shape[1], n_out = w->shape[0] / n_heads;
    const size_t smem = (size_t)HP_TOK * n_in * 4;
    CC_REQUIRE(dev, smem <= 160 * 1024, "head_project: %lld inputs per head do not fit shared memory", (long long)n_in);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * n_heads * (n_out + rest), CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    if (rest == 0 && T >= 64) {          // a pass of many rows (a prompt): tiles; the sums differ from the few-row kernel's by their order only
        head_project_tile_kernel<<<dim3((unsigned)((n_out + HPT_TILE - 1) / HPT_TILE), (unsigned)((T + HPT_TILE - 1) / HPT_TILE), (unsigned)n_heads), 256, 0, dev->stream>>>(
            fptr(x), fptr(w), (float*)o->base, (int)T, n_heads, (int)n_in, (int)n_out);
        CC_LAUNCH_CHECK(dev);
        return CC_OK;
    }
    if (smem > 48 * 1024) CC_CUDA(dev, cudaFuncSetAttribute(head_project_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    head_project_kernel<<<dim3((unsigned)((T + HP_TOK - 1) / HP_TOK), (unsigned)n_heads, (unsigned)((n_out + 3) / 4)), 128, smem, dev->stream>>>(
        fptr(x), fptr(w), (float*)o->base, (int)T, n_heads, (int)n_in, rest, (int)n_out, freq ? fptr(freq) : nullptr, freq ? (int)view_len(freq) : 0, mag, pos0);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// out[j, h] = [ a[j, h, :dim] | shared[j, col0 : col0 + rest] ]: every head's part followed by the columns all heads share.  One thread per element.
__global__ void head_concat_shared_kernel(const float* __restrict__ a, const float* __restrict__ shared, float* __restrict__ out, int64_t n, int H, int dim, int rest, int scols,
                                          int col0) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int hs = dim + rest;
    const int c = (int)(idx % hs);
    const int64_t jh = idx / hs, j = jh / H;
    out[idx] = c < dim ? a[jh * dim + c] : shared[j * scols + col0 + (c - dim)];
}
extern "C" CC_API int cc_head_concat_shared(cc_device* dev, const cc_view* a, const cc_view* shared, int32_t n_heads, int32_t col0, int32_t rest, cc_buf** out) {
    SEQ_ENTER(dev, "head_concat_shared");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "head_concat_shared: out is NULL");
    SEQ_F32(dev, a, "head_concat_shared a"); SEQ_F32(dev, shared, "head_concat_shared shared");
    CC_REQUIRE(dev, a->ndim == 2 && shared->ndim == 2 && n_heads > 0 && a->shape[1] % n_heads == 0 && shared->shape[0] >= a->shape[0] && col0 >= 0 && rest >= 0 &&
                        col0 + rest <= shared->shape[1],
               "head_concat_shared: a must be [rows, heads * dim], shared [>= rows, cols] with cols >= col0 + rest");
    const int64_t rows = a->shape[0], dim = a->shape[1] / n_heads;
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, rows * n_heads * (dim + rest), CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    const int64_t n = rows * n_heads * (dim + rest);
    if (n == 0) return CC_OK;
    head_concat_shared_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(a), fptr(shared), (float*)o->base, n, n_heads, (int)dim, rest, (int)shared->shape[1], col0);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- column blocks of one product's result as separate tensors ------------------------------------------------------------------------------
#define SPLIT_MAX 16
struct SplitArgs {
    float* dst[SPLIT_MAX];
    int end[SPLIT_MAX];          // first column behind part p
    int n;
};
// grid (ceil(cols / 256), about rows / 8): a thread owns one column (its part is found once) and walks the rows of its grid line
__global__ void split_cols_kernel(const float* __restrict__ src, SplitArgs a, int64_t rows, int cols) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= cols) return;
    int p = 0;
    while (p + 1 < a.n && c >= a.end[p]) p++;
    const int begin = p ? a.end[p - 1] : 0, w = a.end[p] - begin;
    float* dst = a.dst[p] + (c - begin);
    for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) dst[r * w] = src[r * cols + c];
}
extern "C" CC_API int cc_split_cols(cc_device* dev, const cc_view* src, int32_t n_parts, const int32_t* widths, cc_buf** outs) {
    SEQ_ENTER(dev, "split_cols");
    if (!widths || !outs) return cc_fail(dev, CC_ERR_ARG, "split_cols: widths / outs is NULL");
    SEQ_F32(dev, src, "split_cols src");
    CC_REQUIRE(dev, src->ndim == 2 && n_parts >= 1 && n_parts <= SPLIT_MAX, "split_cols: src must be [rows, cols], 1..%d parts", SPLIT_MAX);
    const int64_t rows = src->shape[0], cols = src->shape[1];
    int64_t sum = 0;
    for (int p = 0; p < n_parts; p++) { CC_REQUIRE(dev, widths[p] >= 1, "split_cols: empty part %d", p); sum += widths[p]; }
    CC_REQUIRE(dev, sum == cols, "split_cols: the parts have %lld columns, src %lld", (long long)sum, (long long)cols);
    SplitArgs a;
    a.n = n_parts;
    int end = 0;
    for (int p = 0; p < n_parts; p++) {
        cc_buf* o = nullptr;
        int rc = cc_new_activation(dev, rows * widths[p], CC_F32, false, &o);
        if (rc) { for (int q = 0; q < p; q++) { cc_tensor_release(outs[q]); outs[q] = nullptr; } return rc; }
        outs[p] = o;
        a.dst[p] = (float*)o->base;
        a.end[p] = (end += widths[p]);
    }
    const int64_t total = rows * cols;
    if (total == 0) return CC_OK;
    const int64_t lines = (rows + 7) / 8;             // a thread copies about 8 rows of its column
    split_cols_kernel<<<dim3((unsigned)((cols + 255) / 256), (unsigned)(lines < 65535 ? lines : 65535)), 256, 0, dev->stream>>>(fptr(src), a, rows, (int)cols);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- PolyNorm ------------------------------------------------------------------------------------------------------------------------------
// one CTA per row: thread-strided sums of z^2, z^4, z^6, a fixed tree over the 256 partial sums, then the weighted sum of the three unit powers
__global__ void __launch_bounds__(256) poly_norm_kernel(float* __restrict__ z, const float* __restrict__ coef, int cols, float eps) {
    __shared__ float red[3][8];
    float* zr = z + (int64_t)blockIdx.x * cols;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int c = threadIdx.x; c < cols; c += 256) {
        const float v = zr[c], v2 = v * v, v3 = v2 * v;
        s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6);
    }
    s2 = warp_sum(s2); s4 = warp_sum(s4); s6 = warp_sum(s6);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][warp] = s2; red[1][warp] = s4; red[2][warp] = s6; }
    __syncthreads();
    float t2 = 0.0f, t4 = 0.0f, t6 = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) { t2 += red[0][w]; t4 += red[1][w]; t6 += red[2][w]; }
    const float i1 = 1.0f / sqrtf(t2 / (float)cols + eps), i2 = 1.0f / sqrtf(t4 / (float)cols + eps), i3 = 1.0f / sqrtf(t6 / (float)cols + eps);
    const float a = coef[0], b = coef[1], c3 = coef[2], e = coef[3];
    for (int c = threadIdx.x; c < cols; c += 256) {
        const float v = zr[c], v2 = v * v, v3 = v2 * v;
        zr[c] = a * (v * i1) + b * (v2 * i2) + c3 * (v3 * i3) + e;
    }
}
extern "C" CC_API int cc_poly_norm(cc_device* dev, const cc_view* z, const cc_view* coef, float eps) {
    SEQ_ENTER(dev, "poly_norm");
    SEQ_F32(dev, z, "poly_norm z"); SEQ_F32(dev, coef, "poly_norm coef");
    CC_REQUIRE(dev, z->ndim == 2 && view_len(coef) == 4, "poly_norm: z must be [rows, cols] and coef hold 4 numbers");
    if (z->shape[0] == 0) return CC_OK;
    poly_norm_kernel<<<(unsigned)z->shape[0], 256, 0, dev->stream>>>(fptr(z), fptr(coef), (int)z->shape[1], eps);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- gated sum of sublayer results into the residual stream -----------------------------------------------------------------------------------
__global__ void gated_sum_kernel(float* __restrict__ dst, const float* __restrict__ y1, const float* __restrict__ g1, const float* __restrict__ b1, const float* __restrict__ y2,
                                 const float* __restrict__ g2, const float* __restrict__ b2, int64_t n, int cols, int accumulate) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int c = (int)(i % cols);
    float v = y1[i];
    if (g1) v *= seq_sigmoid(g1[i] + (b1 ? b1[c] : 0.0f));
    if (y2) {
        float u = y2[i];
        if (g2) u *= seq_sigmoid(g2[i] + (b2 ? b2[c] : 0.0f));
        v += u;
    }
    dst[i] = accumulate ? dst[i] + v : v;
}
extern "C" CC_API int cc_gated_sum(cc_device* dev, const cc_view* dst, int32_t accumulate, const cc_view* y1, const cc_view* g1, const cc_view* b1, const cc_view* y2,
                                   const cc_view* g2, const cc_view* b2) {
    SEQ_ENTER(dev, "gated_sum");
    SEQ_F32(dev, dst, "gated_sum dst"); SEQ_F32(dev, y1, "gated_sum y1");
    CC_REQUIRE(dev, dst->ndim == 2, "gated_sum: dst must be [rows, cols]");
    const int64_t n = view_len(dst), cols = dst->shape[1];
    const cc_view* same[] = {y1, g1, y2, g2};
    for (const cc_view* v : same)
        if (v) { SEQ_F32(dev, v, "gated_sum operand"); CC_REQUIRE(dev, view_len(v) == n, "gated_sum: an operand has %lld elements, dst %lld", (long long)view_len(v), (long long)n); }
    const cc_view* bias[] = {b1, b2};
    for (const cc_view* v : bias)
        if (v) { SEQ_F32(dev, v, "gated_sum bias"); CC_REQUIRE(dev, view_len(v) == cols, "gated_sum: a bias needs one number per column"); }
    CC_REQUIRE(dev, (!b1 || g1) && (!b2 || g2) && (!g2 || y2), "gated_sum: a bias needs its gate, a gate its operand");
    if (n == 0) return CC_OK;
    gated_sum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(fptr(dst), fptr(y1), g1 ? fptr(g1) : nullptr, b1 ? fptr(b1) : nullptr, y2 ? fptr(y2) : nullptr,
                                                                           g2 ? fptr(g2) : nullptr, b2 ? fptr(b2) : nullptr, n, (int)cols, accumulate);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
