// seqops_diag.cu -- the gated diagonal recurrence of include/crabml_seqops.h (the real-gated linear recurrent unit): a state of one number per
// channel that every token first shrinks by a gate-dependent decay and then adds a gated, rescaled input to,
//     r = sigmoid(g_r + b_r) ; i = sigmoid(g_i + b_i) ; log a = -c r softplus(lam)
//     S <- a S + sqrt(1 - a^2) (i u) ; out = S * act(y + y_b)
// Everything is 32-bit (expf / log1pf / expm1f / tanhf of the CUDA math library).  1 - a^2 is taken as -expm1(2 log a): for a decay close to
// one the difference 1 - a * a would lose most of its digits.
//
// Only S ties a token to the one before it, and the tie is one fused multiply-add.  So the work is split: the threads of a CTA turn a block of
// tokens into the pairs (a, sqrt(1 - a^2) i u) side by side, a few threads then walk the block in order, and all threads write the gated
// read-outs.  A token's result depends on its inputs and the state alone; the order of the walk is the order of the tokens, whatever the
// call carries, so prompts, portions and decoding give the same bits.
#include "../../include/crabml_seqops.h"
#include "capi_checks.cuh"

#define DG_ENTER(dev, what)                                                                                           \
    if (!(dev)) return CC_ERR_ARG;                                                                                    \
    CC_ENTER(dev);                                                                                                    \
    if (LAZY(dev)) return cc_fail((dev), CC_ERR_UNSUPPORTED, "%s: not available on a lazy (graph / megakernel) device", what)
#define DG_F32(dev, v, what)                                                                                           \
    do {                                                                                                              \
        if (!view_ok(v)) return cc_fail((dev), CC_ERR_ARG, "%s: bad tensor view", what);                              \
        if (!view_in_bounds(v)) return cc_fail((dev), CC_ERR_TENSOR, "%s: view addresses element %lld of a buffer of %lld", what, \
                                               (long long)view_max_offset(v), (long long)(v)->buf->nelems);           \
        CC_REQUIRE(dev, view_contiguous(v), "%s: not contiguous", what);                                              \
        REQUIRE_F32(dev, v, what);                                                                                    \
    } while (0)
static inline float* dptr(const cc_view* v) { return (float*)v->buf->plane[0]; }

__device__ __forceinline__ float dg_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float dg_softplus(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float dg_act(float z, int act) {
    return act == CC_ACT_SILU        ? z / (1.0f + expf(-z))
           : act == CC_ACT_GELU_TANH ? 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)))
           : act == CC_ACT_SIGMOID   ? dg_sigmoid(z)
                                     : z;
}

#define DG_CH 4             // channels of a CTA
#define DG_ROWS 64          // token rows of the thread layout
#define DG_PER 2            // tokens per thread and block
#define DG_WALK 16          // tokens whose operands the walk keeps in registers at a time
#define DG_TB (DG_ROWS * DG_PER)
#define DG_THREADS (DG_CH * DG_ROWS)
struct DgArgs {
    const float *u, *gates, *gate_bias, *lam, *y, *y_bias;
    float *state, *out;
    int T, C, bs;           // bs: channels per gate block
    int y_act;
    float c;
};
// grid ceil(C / 4), 256 threads, blocks of 128 tokens.  Thread (row, l) = (threadIdx.x / 4, threadIdx.x % 4) is channel blockIdx.x * 4 + l
// for the block's tokens row and row + 64 -- independent chains of exponentials and roots; an SM holds two such CTAs, so that one computes
// gates while the other walks.  The walk over a block's tokens is done by the first 4 threads, one channel each: the operands of 16 tokens are
// read from shared memory into registers at once (they do not depend on S), then the chain is one fmaf per token.
__global__ void __launch_bounds__(DG_THREADS) gated_diag_kernel(DgArgs a) {
    __shared__ float s_a[DG_TB][DG_CH], s_b[DG_TB][DG_CH], s_s[DG_TB][DG_CH];
    const int l = threadIdx.x % DG_CH, row = threadIdx.x / DG_CH;
    const int ch = blockIdx.x * DG_CH + l;
    const bool live = ch < a.C;
    const int cc = live ? ch : a.C - 1;                       // idle threads shadow the last channel and never store
    const int blk = cc / a.bs, o = cc - blk * a.bs;
    const int col_r = blk * 2 * a.bs + o, col_i = col_r + a.bs;
    const float br = a.gate_bias[col_r], bi = a.gate_bias[col_i];
    const float rate = a.c * dg_softplus(a.lam[cc]);
    const float yb = a.y_bias ? a.y_bias[cc] : 0.0f;
    float S = row == 0 ? a.state[cc] : 0.0f;
    // a block's operands are fetched into registers one block ahead: the loads of block n + 1 are in flight while block n is walked and written
    float g_r[DG_PER], g_i[DG_PER], g_u[DG_PER], g_y[DG_PER];
    auto fetch = [&](int tb) {
#pragma unroll
        for (int e = 0; e < DG_PER; e++) {
            const int64_t t = tb + row + e * DG_ROWS;
            const bool in = t < a.T;
            const float* gr = a.gates + t * 2 * a.C;
            g_r[e] = in ? gr[col_r] : 0.0f;
            g_i[e] = in ? gr[col_i] : 0.0f;
            g_u[e] = in ? a.u[t * a.C + cc] : 0.0f;
            g_y[e] = (in && a.y) ? a.y[t * a.C + cc] : 0.0f;
        }
    };
    fetch(0);
    for (int tb = 0; tb < a.T; tb += DG_TB) {
        const int nt = min(DG_TB, a.T - tb);
        float yv[DG_PER];
#pragma unroll
        for (int e = 0; e < DG_PER; e++) {
            const int tt = row + e * DG_ROWS;
            const float r = dg_sigmoid(g_r[e] + br), i = dg_sigmoid(g_i[e] + bi);
            const float la = -(rate * r);
            s_a[tt][l] = expf(la);
            s_b[tt][l] = sqrtf(-expm1f(2.0f * la)) * (i * g_u[e]);
            yv[e] = a.y ? dg_act(g_y[e] + yb, a.y_act) : 1.0f;
        }
        if (tb + DG_TB < a.T) fetch(tb + DG_TB);
        __syncthreads();
        if (row == 0) {
            for (int k0 = 0; k0 < nt; k0 += DG_WALK) {
                float av[DG_WALK], bv[DG_WALK];
#pragma unroll
                for (int j = 0; j < DG_WALK; j++) { av[j] = s_a[k0 + j][l]; bv[j] = s_b[k0 + j][l]; }
#pragma unroll
                for (int j = 0; j < DG_WALK; j++) {
                    const float next = fmaf(av[j], S, bv[j]);
                    S = k0 + j < nt ? next : S;              // rows behind the last token hold values made from zeros: they are not applied
                    s_s[k0 + j][l] = S;
                }
            }
        }
        __syncthreads();
        if (live) {
#pragma unroll
            for (int e = 0; e < DG_PER; e++) {
                const int tt = row + e * DG_ROWS;
                if (tt < nt) a.out[(int64_t)(tb + tt) * a.C + ch] = s_s[tt][l] * yv[e];
            }
        }
    }
    if (row == 0 && live) a.state[ch] = S;
}

extern "C" CC_API int cc_gated_diagonal_recurrence(cc_device* dev, const cc_view* u, const cc_view* gates, const cc_view* gate_bias, const cc_view* lam, float c,
                                                   int32_t n_blocks, const cc_view* y, const cc_view* y_bias, int32_t y_act, const cc_view* state, cc_buf** out) {
    DG_ENTER(dev, "gated_diagonal_recurrence");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "gated_diagonal_recurrence: out is NULL");
    DG_F32(dev, u, "gated_diagonal_recurrence u"); DG_F32(dev, gates, "gated_diagonal_recurrence gates"); DG_F32(dev, gate_bias, "gated_diagonal_recurrence gate_bias");
    DG_F32(dev, lam, "gated_diagonal_recurrence lam"); DG_F32(dev, state, "gated_diagonal_recurrence state");
    if (y) DG_F32(dev, y, "gated_diagonal_recurrence y");
    if (y_bias) DG_F32(dev, y_bias, "gated_diagonal_recurrence y_bias");
    CC_REQUIRE(dev, u->ndim == 2 && u->shape[1] >= 1 && n_blocks >= 1 && u->shape[1] % n_blocks == 0, "gated_diagonal_recurrence: u must be [T, C] with C a multiple of the %d blocks",
               n_blocks);
    const int64_t T = u->shape[0], C = u->shape[1];
    CC_REQUIRE(dev, view_len(gates) == 2 * T * C && view_len(gate_bias) == 2 * C && view_len(lam) == C && view_len(state) == C && (!y || view_len(y) == T * C) &&
                        (!y_bias || (y && view_len(y_bias) == C)),
               "gated_diagonal_recurrence: operand sizes do not fit T=%lld channels=%lld", (long long)T, (long long)C);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * C, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    DgArgs a{};
    a.u = dptr(u); a.gates = dptr(gates); a.gate_bias = dptr(gate_bias); a.lam = dptr(lam); a.y = y ? dptr(y) : nullptr; a.y_bias = y_bias ? dptr(y_bias) : nullptr;
    a.state = dptr(state); a.out = (float*)o->base; a.T = (int)T; a.C = (int)C; a.bs = (int)(C / n_blocks); a.y_act = y_act; a.c = c;
    gated_diag_kernel<<<(unsigned)((C + DG_CH - 1) / DG_CH), DG_THREADS, 0, dev->stream>>>(a);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
