// seqops_linear.cu -- linear recurrences over a matrix state (include/crabml_seqops.h): the matrix memory with exponential gates, linear
// attention with a decay per key channel, and the selective state-space scan.  All three are
//     S <- D_t S + a_t k_t v_t^T ;  out_t = S^T q_t                 S: [dk, dv] per head, F32, carried between calls
// with D_t a number per (token, head), a fixed number per head or a vector over the key channels, and a_t a number per (token, head) or one
// constant.  One kernel runs that form
// (lr_kernel); a small kernel per mixer turns raw projections into D_t and a_t first, in 32-bit floats (expf / log1pf / tanhf of the CUDA
// math library).  The matrix memory's normaliser n_t = D_t n + a_t k_t is one more column of the state whose value is 1 for every token.
//
// As everywhere in the sequence ops, a token's result depends on its inputs and the state alone: sums run in a fixed order per output, so a
// prompt fed at once, in portions or token by token gives the same bits.
#include "../../include/crabml_seqops.h"
#include "capi_checks.cuh"

#define LIN_ENTER(dev, what)                                                                                          \
    if (!(dev)) return CC_ERR_ARG;                                                                                    \
    CC_ENTER(dev);                                                                                                    \
    if (LAZY(dev)) return cc_fail((dev), CC_ERR_UNSUPPORTED, "%s: not available on a lazy (graph / megakernel) device", what)
#define LIN_F32(dev, v, what)                                                                                          \
    do {                                                                                                              \
        if (!view_ok(v)) return cc_fail((dev), CC_ERR_ARG, "%s: bad tensor view", what);                              \
        if (!view_in_bounds(v)) return cc_fail((dev), CC_ERR_TENSOR, "%s: view addresses element %lld of a buffer of %lld", what, \
                                               (long long)view_max_offset(v), (long long)(v)->buf->nelems);           \
        CC_REQUIRE(dev, view_contiguous(v), "%s: not contiguous", what);                                              \
        REQUIRE_F32(dev, v, what);                                                                                    \
    } while (0)
static inline float* lptr(const cc_view* v) { return (float*)v->buf->plane[0]; }

__device__ __forceinline__ float lin_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float lin_softplus(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// ---- the recurrence ------------------------------------------------------------------------------------------------------------------------
struct LrArgs {
    const float *q, *k, *v;       // q, k: row t at + t * rs, the head group's dk numbers at + g * dk; v: row t at + t * v_rs, head h's at + h * v_hs
    const float* adec;            // [T, H * dk] decay per key channel, or NULL
    const float* sc;              // [T, H, 2] = {decay, weight of the outer product} per (token, head), or NULL (1, 1)
    const float* hdec;            // [H] one decay per head for every token, or NULL (1); read only when sc is NULL
    float wgt;                    // weight of the outer product when sc is NULL
    const float* skip;            // [H] or NULL: out += skip[h] * v
    float *state, *out;           // state [H, dk, dv]; out [T, H, dv]
    int T, H, G, dk, dv;          // dv: columns of the state
    int q_rs, k_rs, v_rs, v_hs;   // v_hs: value columns a head has in the input; column v_hs of the state (if dv > v_hs) takes the value 1
    int vec;                      // rows of q / k / adec may be copied 16 bytes at a time
    float q_scale;
};
// grid (H, ceil(dv / columns per CTA)).  A column j of the head's state is owned for the whole call by SPLIT adjacent threads.  DK > 0
// (dk = 32, 64, 128): a CTA is 32 columns x SPLIT threads, each thread keeps dk / SPLIT = 16 entries in registers -- the 4-float pieces
// part, part + SPLIT, ... of the column, so that the SPLIT threads of a column read neighbouring pieces of k and q (no bank conflicts) -- and
// the lanes' partial read-outs of a block of tokens go to shared memory and are added after the block, parts in ascending order: a short
// dependent chain per token with no shuffle in it, many warps per CTA.  DK == 0 (any
// dk): 64 columns, one thread each, the column in shared memory [dk][64].  k, q (and the channel decays) of LR_TB tokens at a time are staged
// in shared memory by asynchronous copies issued one block ahead; per token a thread runs once over its share:
//   S[i] = k[i] * (a v_j) + D[i] * S[i] ; out += S[i] * q[i]      as four interleaved partial sums added (p0 + p1) + (p2 + p3).
#define LR_COLS 32
#define LR_GENERIC_THREADS 64
#define LR_TB 16
__device__ __forceinline__ void lr_cp16(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void lr_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
// one staging buffer: k[TB][dk4], q[TB][dk4], (adec[TB][dk4]), sc[TB][2], v[TB][cols]
static __host__ __device__ __forceinline__ int lr_stage_floats(int dk4, bool adec, int cols) { return (adec ? 3 : 2) * LR_TB * dk4 + 2 * LR_TB + LR_TB * cols; }

template <int DK, int SPLIT, bool ADEC>
__global__ void __launch_bounds__(DK > 0 ? LR_COLS * SPLIT : LR_GENERIC_THREADS) lr_kernel(LrArgs a) {
    extern __shared__ __align__(16) float lr_sm[];           // two staging buffers, then (DK == 0) the state columns
    constexpr int THREADS = DK > 0 ? LR_COLS * SPLIT : LR_GENERIC_THREADS;
    constexpr int COLS = THREADS / SPLIT;
    constexpr int DKP = DK > 0 ? DK / SPLIT : 4;             // entries per thread (register path)
    const int dk = a.dk, dv = a.dv, T = a.T;
    const int dk4 = DK > 0 ? DK : (dk + 3) & ~3;
    const int stage_floats = lr_stage_floats(dk4, ADEC, COLS);
    const int h = blockIdx.x, g = h / (a.H / a.G);
    const int part = threadIdx.x % SPLIT, col = threadIdx.x / SPLIT;
    const int j = blockIdx.y * COLS + col;
    const bool live = j < dv;
    const int jj = live ? j : dv - 1;                      // idle threads shadow the last column and never store
    const bool ones = jj >= a.v_hs;
    float S[DKP];                                           // S[4 m + e] is row 4 (part + SPLIT m) + e of the column
    float* Ss = lr_sm + 2 * stage_floats + threadIdx.x;     // generic: row i at Ss[i * THREADS]
    float* pbuf = lr_sm + 2 * stage_floats;                 // SPLIT > 1: the lanes' partial read-outs of a block of tokens, [token][column][part]
    float* sp = a.state + (int64_t)h * dk * dv + jj;
    if (DK > 0) {
#pragma unroll
        for (int i = 0; i < DKP; i++) S[i] = sp[(int64_t)(4 * (part + SPLIT * (i >> 2)) + (i & 3)) * dv];
    } else {
        for (int i = 0; i < dk4; i++) Ss[i * THREADS] = i < dk ? sp[(int64_t)i * dv] : 0.0f;
    }
    const int n_rows = (ADEC ? 3 : 2) * LR_TB;
    // the pad lanes dk .. dk4 of both buffers are zero for the whole call (the copies below never touch them)
    if (dk4 != dk)
        for (int idx = threadIdx.x; idx < 2 * n_rows; idx += THREADS)
            for (int i = dk; i < dk4; i++) lr_sm[(idx / n_rows) * stage_floats + (idx % n_rows) * dk4 + i] = 0.0f;
    const float skip = a.skip ? a.skip[h] : 0.0f;
    const float head_dec = a.hdec ? a.hdec[h] : 1.0f;
    // a thread's first piece of a block of tokens, and how far the next one is: item idx = threadIdx.x + n THREADS is token idx / per,
    // piece idx % per of the block; walked without divisions
    const int per = a.vec ? dk >> 2 : dk, width = a.vec ? 4 : 1;
    const int tt0 = threadIdx.x / per, c0 = threadIdx.x % per, dtt = THREADS / per, dc = THREADS % per;
    auto stage = [&](int buf, int tb) {
        float* base = lr_sm + buf * stage_floats;
        const int nt = min(LR_TB, T - tb);
        for (int tt = tt0, c = c0; tt < nt;) {
            const int e = c * width;
            const float* ks = a.k + (int64_t)(tb + tt) * a.k_rs + g * dk + e;
            const float* qs = a.q + (int64_t)(tb + tt) * a.q_rs + g * dk + e;
            if (a.vec) {
                lr_cp16(base + tt * dk4 + e, ks);
                lr_cp16(base + (LR_TB + tt) * dk4 + e, qs);
                if (ADEC) lr_cp16(base + (2 * LR_TB + tt) * dk4 + e, a.adec + ((int64_t)(tb + tt) * a.H + h) * dk + e);
            } else {
                lr_cp4(base + tt * dk4 + e, ks);
                lr_cp4(base + (LR_TB + tt) * dk4 + e, qs);
                if (ADEC) lr_cp4(base + (2 * LR_TB + tt) * dk4 + e, a.adec + ((int64_t)(tb + tt) * a.H + h) * dk + e);
            }
            tt += dtt; c += dc;
            if (c >= per) { c -= per; tt++; }
        }
        float* ssc = base + n_rows * dk4;
        if (a.sc)
            for (int idx = threadIdx.x; idx < nt * 2; idx += THREADS) lr_cp4(ssc + idx, a.sc + ((int64_t)(tb + (idx >> 1)) * a.H + h) * 2 + (idx & 1));
        // the block's values of the CTA's columns: [token][column]
        float* sv = ssc + 2 * LR_TB;
        for (int idx = threadIdx.x; idx < nt * COLS; idx += THREADS) {
            const int tt = idx / COLS, cc = idx % COLS, jc = blockIdx.y * COLS + cc;
            if (jc < a.v_hs) lr_cp4(sv + idx, a.v + (int64_t)(tb + tt) * a.v_rs + h * a.v_hs + jc);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (T > 0) stage(0, 0);
    int buf = 0;
    for (int tb = 0; tb < T; tb += LR_TB, buf ^= 1) {
        const int nt = min(LR_TB, T - tb);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                      // this block has landed for everyone, and everyone is done with the other buffer
        if (tb + LR_TB < T) stage(buf ^ 1, tb + LR_TB);
        const float* base = lr_sm + buf * stage_floats;
        const float* ssc = base + n_rows * dk4;
        const float* sv = ssc + 2 * LR_TB + col;
        float* op = a.out + ((int64_t)tb * a.H + h) * dv + j;
        const int64_t o_rs = (int64_t)a.H * dv;
        // one token.  Only S ties a token to the one before it: in the unrolled loop of a full block the loads and the read-out's butterfly of
        // neighbouring tokens overlap
        auto token = [&](int tt) {
            const float* kt = base + tt * dk4 + 4 * part;
            const float* qt = base + (LR_TB + tt) * dk4 + 4 * part;
            const float* dt = base + (2 * LR_TB + tt) * dk4 + 4 * part;
            const float dec = a.sc ? ssc[tt * 2] : head_dec, wgt = a.sc ? ssc[tt * 2 + 1] : a.wgt;
            const float vj = ones ? 1.0f : sv[tt * COLS];
            const float u = wgt * vj;
            float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
            if (DK > 0) {
#pragma unroll
                for (int i = 0; i < DKP; i += 4) {
                    const float4 kv = *(const float4*)(kt + SPLIT * i);
                    const float4 qv = *(const float4*)(qt + SPLIT * i);
                    float4 dd = make_float4(dec, dec, dec, dec);
                    if (ADEC) dd = *(const float4*)(dt + SPLIT * i);
                    S[i] = fmaf(kv.x, u, dd.x * S[i]); S[i + 1] = fmaf(kv.y, u, dd.y * S[i + 1]); S[i + 2] = fmaf(kv.z, u, dd.z * S[i + 2]); S[i + 3] = fmaf(kv.w, u, dd.w * S[i + 3]);
                    o0 = fmaf(S[i], qv.x, o0); o1 = fmaf(S[i + 1], qv.y, o1); o2 = fmaf(S[i + 2], qv.z, o2); o3 = fmaf(S[i + 3], qv.w, o3);
                }
            } else {
                for (int i = 0; i < dk4; i += 4) {
                    const float4 kv = *(const float4*)(kt + i);
                    const float4 qv = *(const float4*)(qt + i);
                    float4 dd = make_float4(dec, dec, dec, dec);
                    if (ADEC) dd = *(const float4*)(dt + i);
                    const float s0 = fmaf(kv.x, u, dd.x * Ss[i * THREADS]), s1 = fmaf(kv.y, u, dd.y * Ss[(i + 1) * THREADS]);
                    const float s2 = fmaf(kv.z, u, dd.z * Ss[(i + 2) * THREADS]), s3 = fmaf(kv.w, u, dd.w * Ss[(i + 3) * THREADS]);
                    Ss[i * THREADS] = s0; Ss[(i + 1) * THREADS] = s1; Ss[(i + 2) * THREADS] = s2; Ss[(i + 3) * THREADS] = s3;
                    o0 = fmaf(s0, qv.x, o0); o1 = fmaf(s1, qv.y, o1); o2 = fmaf(s2, qv.z, o2); o3 = fmaf(s3, qv.w, o3);
                }
            }
            float outv = (o0 + o1) + (o2 + o3);
            if (SPLIT > 1) {
                pbuf[tt * THREADS + threadIdx.x] = outv;           // added up after the block: no shuffle waits between tokens
            } else {
                outv = fmaf(skip, vj, outv * a.q_scale);
                if (live) op[tt * o_rs] = outv;
            }
        };
        if (nt == LR_TB) {
#pragma unroll 4
            for (int tt = 0; tt < LR_TB; tt++) token(tt);
        } else {
#pragma unroll 1
            for (int tt = 0; tt < nt; tt++) token(tt);
        }
        if (SPLIT > 1) {
            // the block's read-outs: a column's SPLIT parts added in ascending order, one order whatever T is
            __syncthreads();
            for (int idx = threadIdx.x; idx < nt * COLS; idx += THREADS) {
                const int tt = idx / COLS, cc = idx % COLS, jc = blockIdx.y * COLS + cc;
                if (jc >= dv) continue;
                const float* pp = pbuf + idx * SPLIT;
                float sum = pp[0];
#pragma unroll
                for (int e = 1; e < SPLIT; e++) sum += pp[e];
                const float vj = jc >= a.v_hs ? 1.0f : ssc[2 * LR_TB + tt * COLS + cc];
                a.out[((int64_t)(tb + tt) * a.H + h) * dv + jc] = fmaf(skip, vj, sum * a.q_scale);
            }
        }
    }
    if (live) {
        if (DK > 0) {
#pragma unroll
            for (int i = 0; i < DKP; i++) sp[(int64_t)(4 * (part + SPLIT * (i >> 2)) + (i & 3)) * dv] = S[i];
        } else {
            for (int i = 0; i < dk; i++) sp[(int64_t)i * dv] = Ss[i * THREADS];
        }
    }
}

template <int DK, int SPLIT, bool ADEC>
static cudaError_t lr_launch_one(cc_device* dev, const LrArgs& a, size_t smem) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(lr_kernel<DK, SPLIT, ADEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int threads = DK > 0 ? LR_COLS * SPLIT : LR_GENERIC_THREADS, cols = threads / SPLIT;
    lr_kernel<DK, SPLIT, ADEC><<<dim3((unsigned)a.H, (unsigned)((a.dv + cols - 1) / cols)), threads, smem, dev->stream>>>(a);
    return cudaGetLastError();
}
template <bool ADEC>
static int lr_launch_sized(cc_device* dev, const LrArgs& a, const char* what) {
    const int dk4 = (a.dk + 3) & ~3;
    cudaError_t e;
    if (a.dk == 32 || a.dk == 64 || a.dk == 128) {
        const int split = a.dk / 16;
        const size_t stage = (size_t)2 * lr_stage_floats(dk4, ADEC, LR_COLS) * 4 + (size_t)LR_TB * LR_COLS * split * 4;
        e = a.dk == 32 ? lr_launch_one<32, 2, ADEC>(dev, a, stage) : a.dk == 64 ? lr_launch_one<64, 4, ADEC>(dev, a, stage) : lr_launch_one<128, 8, ADEC>(dev, a, stage);
    } else {
        const size_t smem = (size_t)2 * lr_stage_floats(dk4, ADEC, LR_GENERIC_THREADS) * 4 + (size_t)dk4 * LR_GENERIC_THREADS * 4;
        if (smem > 200 * 1024) return cc_fail(dev, CC_ERR_UNSUPPORTED, "%s: a state of %d rows per head is too large", what, a.dk);
        e = lr_launch_one<0, 1, ADEC>(dev, a, smem);
    }
    if (e != cudaSuccess) return cc_fail(dev, CC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    dev->launches++;
    return CC_OK;
}
static int lr_launch(cc_device* dev, LrArgs a, const char* what) {
    auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    a.vec = (a.dk % 4 == 0 && a.q_rs % 4 == 0 && a.k_rs % 4 == 0 && al(a.q) && al(a.k) && (!a.adec || al(a.adec))) ? 1 : 0;
    return a.adec ? lr_launch_sized<true>(dev, a, what) : lr_launch_sized<false>(dev, a, what);
}

// ---- matrix memory with exponential gates ----------------------------------------------------------------------------------------------------
// grid H, one warp: the running maximum is a scan over the tokens.  32 tokens at a time: lane l computes the two log gates of token
// t0 + l, the maximum walks through the 32 tokens by shuffles (every lane follows it, lane l keeps what its token saw), then lane l writes
// its token's {exp(f + m - m'), exp(i - m')} and exp(-m').
__global__ void __launch_bounds__(32) mm_gates_kernel(const float* __restrict__ gi, const float* __restrict__ gf, const float* __restrict__ bi, const float* __restrict__ bf,
                                                      float cap, float* __restrict__ mstate, float* __restrict__ sc, float* __restrict__ floor_out, int T, int H) {
    const int h = blockIdx.x, lane = threadIdx.x;
    float m = mstate[h];
    for (int t0 = 0; t0 < T; t0 += 32) {
        const int t = t0 + lane;
        float li = 0.0f, lf = 0.0f;
        if (t < T) {
            li = cap * tanhf((gi[(int64_t)t * H + h] + bi[h]) / cap);
            const float z = cap * tanhf((gf[(int64_t)t * H + h] + bf[h]) / cap);
            lf = -lin_softplus(-z);
        }
        float m_before = 0.0f, m_after = 0.0f;
        const int nt = min(32, T - t0);
        for (int l = 0; l < nt; l++) {
            const float fl = __shfl_sync(0xffffffffu, lf, l), il = __shfl_sync(0xffffffffu, li, l);
            const float mn = fmaxf(fl + m, il);
            if (l == lane) { m_before = m; m_after = mn; }
            m = mn;
        }
        if (t < T) {
            sc[((int64_t)t * H + h) * 2] = expf(lf + m_before - m_after);
            sc[((int64_t)t * H + h) * 2 + 1] = expf(li - m_after);
            floor_out[(int64_t)t * H + h] = expf(-m_after);
        }
    }
    if (lane == 0) mstate[h] = m;
}
// raw: [T, H, dv + 1], the read-out of the state and, in the last column, of the normaliser; out = raw / (max(|n . q|, floor) + 1e-6)
__global__ void mm_divide_kernel(const float* __restrict__ raw, const float* __restrict__ floor_in, float* __restrict__ out, int64_t n, int dv) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t th = i / dv;
    const int c = (int)(i - th * dv);
    const float* r = raw + th * (dv + 1);
    out[i] = r[c] / (fmaxf(fabsf(r[dv]), floor_in[th]) + 1e-6f);
}
extern "C" CC_API int cc_matrix_memory(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* gi, const cc_view* gf, const cc_view* bi,
                                       const cc_view* bf, float cap, float q_scale, const cc_view* state, const cc_view* mstate, int32_t H, int32_t dk, int32_t dv,
                                       cc_buf** out) {
    LIN_ENTER(dev, "matrix_memory");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "matrix_memory: out is NULL");
    LIN_F32(dev, q, "matrix_memory q"); LIN_F32(dev, k, "matrix_memory k"); LIN_F32(dev, v, "matrix_memory v"); LIN_F32(dev, gi, "matrix_memory gi");
    LIN_F32(dev, gf, "matrix_memory gf"); LIN_F32(dev, bi, "matrix_memory bi"); LIN_F32(dev, bf, "matrix_memory bf"); LIN_F32(dev, state, "matrix_memory state");
    LIN_F32(dev, mstate, "matrix_memory mstate");
    CC_REQUIRE(dev, H > 0 && dk > 0 && dv > 0 && q->ndim == 2 && cap > 0.0f, "matrix_memory: bad head counts / sizes");
    const int64_t T = q->shape[0];
    CC_REQUIRE(dev, view_len(q) == T * H * dk && view_len(k) == T * H * dk && view_len(v) == T * H * dv && view_len(gi) == T * H && view_len(gf) == T * H && view_len(bi) == H &&
                        view_len(bf) == H && view_len(state) == (int64_t)H * dk * (dv + 1) && view_len(mstate) == H,
               "matrix_memory: operand sizes do not fit T=%lld heads=%d dk=%d dv=%d (state [heads, dk, dv + 1])", (long long)T, H, dk, dv);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * H * dv, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    void* tmp = nullptr; size_t cls = 0;
    const size_t n_sc = (size_t)T * H * 2, n_floor = (size_t)T * H, n_raw = (size_t)T * H * (dv + 1);
    rc = cc_pool_alloc(dev, (n_sc + n_floor + n_raw) * 4, &tmp, &cls);
    if (rc) return rc;
    float* sc = (float*)tmp;
    float* fl = sc + n_sc;
    float* raw = fl + n_floor;
    mm_gates_kernel<<<(unsigned)H, 32, 0, dev->stream>>>(lptr(gi), lptr(gf), lptr(bi), lptr(bf), cap, lptr(mstate), sc, fl, (int)T, H);
    dev->launches++;
    LrArgs a{};
    a.q = lptr(q); a.k = lptr(k); a.v = lptr(v); a.adec = nullptr; a.sc = sc; a.skip = nullptr; a.state = lptr(state); a.out = raw;
    a.T = (int)T; a.H = H; a.G = H; a.dk = dk; a.dv = dv + 1; a.q_rs = a.k_rs = H * dk; a.v_rs = H * dv; a.v_hs = dv; a.q_scale = q_scale; a.wgt = 1.0f;
    rc = lr_launch(dev, a, "matrix_memory");
    if (rc == CC_OK) {
        const int64_t n = T * H * dv;
        mm_divide_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(raw, fl, (float*)o->base, n, dv);
    }
    cc_pool_free(dev, tmp, cls);
    if (rc) return rc;
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- linear attention with a decay per key channel ---------------------------------------------------------------------------------------------
// alpha = sigmoid(z + b)^(1 / tau) = exp(-softplus(-(z + b)) / tau)
__global__ void dla_decay_kernel(const float* __restrict__ z, const float* __restrict__ zb, float* __restrict__ adec, int64_t n, int cols, float inv_tau) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) adec[i] = expf(-lin_softplus(-(z[i] + zb[i % cols])) * inv_tau);
}
extern "C" CC_API int cc_decayed_linear_attention(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* z, const cc_view* zb, float tau,
                                                  float q_scale, const cc_view* state, int32_t H, int32_t dk, int32_t dv, cc_buf** out) {
    LIN_ENTER(dev, "decayed_linear_attention");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "decayed_linear_attention: out is NULL");
    LIN_F32(dev, q, "decayed_linear_attention q"); LIN_F32(dev, k, "decayed_linear_attention k"); LIN_F32(dev, v, "decayed_linear_attention v");
    LIN_F32(dev, z, "decayed_linear_attention z"); LIN_F32(dev, zb, "decayed_linear_attention zb"); LIN_F32(dev, state, "decayed_linear_attention state");
    CC_REQUIRE(dev, H > 0 && dk > 0 && dv > 0 && q->ndim == 2 && tau > 0.0f, "decayed_linear_attention: bad head counts / sizes");
    const int64_t T = q->shape[0];
    CC_REQUIRE(dev, view_len(q) == T * H * dk && view_len(k) == T * H * dk && view_len(z) == T * H * dk && view_len(v) == T * H * dv && view_len(zb) == (int64_t)H * dk &&
                        view_len(state) == (int64_t)H * dk * dv,
               "decayed_linear_attention: operand sizes do not fit T=%lld heads=%d dk=%d dv=%d", (long long)T, H, dk, dv);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * H * dv, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    void* tmp = nullptr; size_t cls = 0;
    rc = cc_pool_alloc(dev, (size_t)T * H * dk * 4, &tmp, &cls);
    if (rc) return rc;
    const int64_t n = T * H * dk;
    dla_decay_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(lptr(z), lptr(zb), (float*)tmp, n, H * dk, 1.0f / tau);
    dev->launches++;
    LrArgs a{};
    a.q = lptr(q); a.k = lptr(k); a.v = lptr(v); a.adec = (const float*)tmp; a.sc = nullptr; a.skip = nullptr; a.state = lptr(state); a.out = (float*)o->base;
    a.T = (int)T; a.H = H; a.G = H; a.dk = dk; a.dv = dv; a.q_rs = a.k_rs = H * dk; a.v_rs = H * dv; a.v_hs = dv; a.q_scale = q_scale; a.wgt = 1.0f;
    rc = lr_launch(dev, a, "decayed_linear_attention");
    cc_pool_free(dev, tmp, cls);
    if (rc) return rc;
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- retention: a fixed decay per head -------------------------------------------------------------------------------------------------------
extern "C" CC_API int cc_retention(cc_device* dev, const cc_view* q, const cc_view* k, const cc_view* v, const cc_view* decay, float k_scale, const cc_view* state, int32_t H,
                                   int32_t dk, int32_t dv, cc_buf** out) {
    LIN_ENTER(dev, "retention");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "retention: out is NULL");
    LIN_F32(dev, q, "retention q"); LIN_F32(dev, k, "retention k"); LIN_F32(dev, v, "retention v"); LIN_F32(dev, decay, "retention decay"); LIN_F32(dev, state, "retention state");
    CC_REQUIRE(dev, H > 0 && dk > 0 && dv > 0 && q->ndim == 2, "retention: bad head counts / sizes");
    const int64_t T = q->shape[0];
    CC_REQUIRE(dev, view_len(q) == T * H * dk && view_len(k) == T * H * dk && view_len(v) == T * H * dv && view_len(decay) == H && view_len(state) == (int64_t)H * dk * dv,
               "retention: operand sizes do not fit T=%lld heads=%d dk=%d dv=%d", (long long)T, H, dk, dv);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * H * dv, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    LrArgs a{};
    a.q = lptr(q); a.k = lptr(k); a.v = lptr(v); a.adec = nullptr; a.sc = nullptr; a.hdec = lptr(decay); a.wgt = k_scale; a.skip = nullptr; a.state = lptr(state);
    a.out = (float*)o->base;
    a.T = (int)T; a.H = H; a.G = H; a.dk = dk; a.dv = dv; a.q_rs = a.k_rs = H * dk; a.v_rs = H * dv; a.v_hs = dv; a.q_scale = 1.0f;
    rc = lr_launch(dev, a, "retention");
    if (rc) return rc;
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- selective state-space scan ------------------------------------------------------------------------------------------------------------------
// sc[(t * H + h) * 2] = {exp(-exp(a_log) d), d}, d = softplus(dt + dt_bias)
__global__ void ss_steps_kernel(const float* __restrict__ dt, const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ sc, int64_t n, int H) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int h = (int)(i % H);
    const float d = lin_softplus(dt[i] + dt_bias[h]);
    sc[i * 2] = expf(-expf(a_log[h]) * d);
    sc[i * 2 + 1] = d;
}
extern "C" CC_API int cc_state_space_scan(cc_device* dev, const cc_view* xbc, const cc_view* dt, const cc_view* dt_bias, const cc_view* a_log, const cc_view* d_skip,
                                          const cc_view* state, int32_t H, int32_t G, int32_t N, int32_t P, cc_buf** out) {
    LIN_ENTER(dev, "state_space_scan");
    if (!out) return cc_fail(dev, CC_ERR_ARG, "state_space_scan: out is NULL");
    LIN_F32(dev, xbc, "state_space_scan xbc"); LIN_F32(dev, dt, "state_space_scan dt"); LIN_F32(dev, dt_bias, "state_space_scan dt_bias");
    LIN_F32(dev, a_log, "state_space_scan a_log"); LIN_F32(dev, state, "state_space_scan state");
    if (d_skip) LIN_F32(dev, d_skip, "state_space_scan d_skip");
    CC_REQUIRE(dev, H > 0 && G > 0 && H % G == 0 && N > 0 && P > 0 && xbc->ndim == 2, "state_space_scan: bad head counts / sizes");
    const int64_t T = xbc->shape[0], row = (int64_t)H * P + 2 * (int64_t)G * N;
    CC_REQUIRE(dev, xbc->shape[1] == row && view_len(dt) == T * H && view_len(dt_bias) == H && view_len(a_log) == H && (!d_skip || view_len(d_skip) == H) &&
                        view_len(state) == (int64_t)H * N * P,
               "state_space_scan: operand sizes do not fit T=%lld heads=%d groups=%d state=%d head_dim=%d", (long long)T, H, G, N, P);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * H * P, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    void* tmp = nullptr; size_t cls = 0;
    rc = cc_pool_alloc(dev, (size_t)T * H * 2 * 4, &tmp, &cls);
    if (rc) return rc;
    ss_steps_kernel<<<(unsigned)((T * H + 255) / 256), 256, 0, dev->stream>>>(lptr(dt), lptr(dt_bias), lptr(a_log), (float*)tmp, T * H, H);
    dev->launches++;
    LrArgs a{};
    const float* base = lptr(xbc);
    a.v = base; a.k = base + (int64_t)H * P; a.q = base + (int64_t)H * P + (int64_t)G * N; a.adec = nullptr; a.sc = (const float*)tmp;
    a.skip = d_skip ? lptr(d_skip) : nullptr; a.state = lptr(state); a.out = (float*)o->base;
    a.T = (int)T; a.H = H; a.G = G; a.dk = N; a.dv = P; a.q_rs = a.k_rs = a.v_rs = (int)row; a.v_hs = P; a.q_scale = 1.0f; a.wgt = 1.0f;
    rc = lr_launch(dev, a, "state_space_scan");
    cc_pool_free(dev, tmp, cls);
    if (rc) return rc;
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
