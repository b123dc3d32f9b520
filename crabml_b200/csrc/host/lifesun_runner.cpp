// lifesun_runner.cpp -- host driver of the Lifesun decoder family over the C ABI (crabml_cuda.h + crabml_seqops.h).  Like the other runners it
// contains no arithmetic: it owns the weights' handles, says what a sequence holds (per layer RUN: key / value rings and either a diagonal
// state with a convolution tail or a retention matrix) and in which order the tensor ops run.  Slots, step and greedy generation are the
// shared ones of seq_runner.hpp.
//
//   pass:   before the first layer of every repetition of the loop: x = W_in [x | x0]
//   run:    h = LN(x) ; ONE product of everything that multiplies h, cut into its parts ; x += ls * left + rs * right + ff
//   left:   (q, k norms), (rotation) and keys and values into the run's rings, one kernel ; masked, capped softmax (+ sink) ; (gate per head) ; W_o
//   right:  diagonal: convolution of the x branch ; gates, one product per block ; the recurrence on the run's state, times act(y + b) ; W_o
//           retention: rotation ; the recurrence on the run's state ; unit RMS per head and silu gate ; W_o
//   ff:     gelu_tanh(gate) * up ; W_down
#include <cmath>
#include <string>
#include <vector>

#include "../../../include/crabml_lifesun.h"
#include "seq_runner.hpp"

using crabml::CudaTensor;
using crabml::TensorError;

namespace {

struct Layer {
    clr_layer_config c{};
    CudaTensor norm_w, norm_b, h_stack, x_bias, q_norm, k_norm, sink, rot_freq, left_o, right_o, conv, conv_bias, y_bias, gate_w, gate_b, lam, r_rot_freq, decay, down;
    std::vector<int32_t> widths;         // column blocks of the stacked product, in order
    int i_gate = -1, i_right = 0, i_ff = -1;     // block of the left gate (-1: none); first block of the right mixer; block of gate | up (-1: none)
    int64_t ring = 0;                    // rows of the key / value rings of one run
};
struct Run {
    int layer;
    bool re_enter;                       // the loop's product comes right before this run
};
struct RunState {
    CudaTensor kring, vring, S, tail;
};
struct State : crabml::SeqState {
    std::vector<RunState> runs;
};
const cc_view* opt(const CudaTensor& t, cc_view& store) {
    if (!t.valid()) return nullptr;
    store = t.view();
    return &store;
}

struct Runner : csr_runner {
    clr_config conf{};
    std::vector<Layer> layers;
    std::vector<Run> runs;
    CudaTensor embed, loop_in, final_w, final_b, head;

    std::unique_ptr<crabml::SeqState> make_state() override {
        auto s = std::make_unique<State>();
        for (const Run& run : runs) {
            const Layer& L = layers[run.layer];
            const auto& c = L.c;
            RunState r;
            r.kring = CudaTensor::alloc({L.ring, (int64_t)c.kv_heads * c.dim}, CC_F32, dev);
            r.vring = CudaTensor::alloc({L.ring, (int64_t)c.kv_heads * c.vdim}, CC_F32, dev);
            if (c.right == CLR_RIGHT_DIAGONAL) {
                r.S = CudaTensor::alloc({c.r_width}, CC_F32, dev);
                if (c.r_conv > 1) r.tail = CudaTensor::alloc({c.r_conv - 1, c.r_width}, CC_F32, dev);
            } else {
                r.S = CudaTensor::alloc({c.r_heads, c.r_dim, c.r_vdim}, CC_F32, dev);
            }
            s->runs.push_back(std::move(r));
        }
        return s;
    }
    // a reused slot starts like a new one: the recurrences and the convolutions see nothing before position 0.  The rings need no reset: a
    // query at position i only reads rows of positions <= i of ITS sequence, all written since the slot was opened.
    void reset_state(crabml::SeqState& base) override {
        State& s = static_cast<State&>(base);
        for (auto& r : s.runs)
            for (CudaTensor* t : {&r.S, &r.tail})
                if (t->valid()) { cc_view v = t->view(); check(cc_tensor_zero(dev, &v)); }
    }

    CudaTensor layer_norm(const CudaTensor& x, const CudaTensor& w, const CudaTensor& b) {
        CudaTensor h = CudaTensor::alloc(x.shape(), CC_F32, dev);
        cc_view hv = h.view(), xv = x.view(), wv = w.view(), bv{};
        check(cc_layer_norm(dev, &hv, &xv, &wv, opt(b, bv), conf.norm_eps));
        return h;
    }
    std::vector<CudaTensor> split(const CudaTensor& all, const std::vector<int32_t>& widths) {
        cc_view av = all.view();
        std::vector<cc_buf*> outs(widths.size(), nullptr);
        check(cc_split_cols(dev, &av, (int32_t)widths.size(), widths.data(), outs.data()));
        std::vector<CudaTensor> part;
        for (size_t p = 0; p < outs.size(); p++) part.push_back(adopt(outs[p], {all.shape()[0], widths[p]}));
        return part;
    }

    CudaTensor left_mixer(const Layer& L, RunState& st, std::vector<CudaTensor>& part, int64_t pos0) {
        const auto& c = L.c;
        CudaTensor &q = part[0], &k = part[1], &v = part[2];
        const int64_t n = q.shape()[0];
        if (c.window <= 0 && c.block <= 0 && pos0 + n > L.ring)
            throw TensorError("a sequence of " + std::to_string(pos0 + n) + " tokens does not fit the cache of " + std::to_string(L.ring));
        cc_view qv = q.view(), kv = k.view(), vv = v.view(), krv = st.kring.view(), vrv = st.vring.view(), tmp{}, qw{}, kw{}, fr{};
        // norms, rotation and the cache write in one pass
        const int norm = c.qk_norm == CLR_QK_UNIT_PER_HEAD ? CC_QK_NORM_HEAD : c.qk_norm == CLR_QK_WHOLE_WEIGHTED ? CC_QK_NORM_ROW : CC_QK_NORM_NONE;
        check(cc_qk_prepare_append(dev, &qv, &kv, &vv, &krv, &vrv, norm, opt(L.q_norm, qw), opt(L.k_norm, kw), conf.norm_eps, opt(L.rot_freq, fr), CC_ROPE_HALVES, 0, 1.0f, pos0,
                                   c.heads, c.kv_heads, c.dim, c.vdim));
        cc_buf* b = nullptr;
        check(cc_masked_attention_capped(dev, &qv, &krv, &vrv, pos0, c.heads, c.kv_heads, c.dim, c.vdim, c.window, c.block, c.scale, c.softcap, opt(L.sink, tmp), &b));
        CudaTensor o = adopt(b, {n, (int64_t)c.heads * c.vdim});
        if (L.i_gate >= 0) {
            cc_view ov = o.view(), gv = part[L.i_gate].view();
            check(cc_head_gate(dev, &ov, &gv, c.heads, CC_ACT_SIGMOID));
        }
        return L.left_o.matmul_vec(o);
    }

    CudaTensor diagonal_mixer(const Layer& L, RunState& st, std::vector<CudaTensor>& part) {
        const auto& c = L.c;
        const int64_t n = part[0].shape()[0];
        CudaTensor &y = part[L.i_right], &xb = part[L.i_right + 1];
        cc_view xv = xb.view(), cw = L.conv.view(), cb{}, tl{}, ib{};
        cc_buf* b = nullptr;
        // the projection's bias comes before the convolution: the kernel adds it to the inputs it reads
        check(cc_short_conv_biases(dev, &xv, &cw, opt(L.x_bias, ib), opt(L.conv_bias, cb), opt(st.tail, tl), CC_ACT_NONE, &b));
        CudaTensor u = adopt(b, {n, c.r_width});
        b = nullptr;
        cc_view uv = u.view(), gw = L.gate_w.view();
        check(cc_head_project(dev, &uv, &gw, c.r_blocks, 0, nullptr, 1.0f, 0, &b));
        CudaTensor gates = adopt(b, {n, 2 * (int64_t)c.r_width});
        b = nullptr;
        cc_view gv = gates.view(), gb = L.gate_b.view(), lv = L.lam.view(), yv = y.view(), yb{}, sv = st.S.view();
        check(cc_gated_diagonal_recurrence(dev, &uv, &gv, &gb, &lv, c.r_rate, c.r_blocks, &yv, opt(L.y_bias, yb), CC_ACT_GELU_TANH, &sv, &b));
        return L.right_o.matmul_vec(adopt(b, {n, c.r_width}));
    }

    CudaTensor retention_mixer(const Layer& L, RunState& st, std::vector<CudaTensor>& part, int64_t pos0) {
        const auto& c = L.c;
        const int64_t n = part[0].shape()[0];
        const int r0 = L.i_right;
        cc_view rq = part[r0].view(), rk = part[r0 + 1].view(), rv = part[r0 + 2].view(), rg = part[r0 + 3].view(), sv = st.S.view(), dv = L.decay.view();
        if (L.r_rot_freq.valid()) {
            cc_view f = L.r_rot_freq.view();
            check(cc_rope_halves_two(dev, &rq, &rk, c.r_heads, c.r_dim, 0, &f, 1.0f, pos0));
        }
        cc_buf* b = nullptr;
        check(cc_retention(dev, &rq, &rk, &rv, &dv, 1.0f / std::sqrt((float)c.r_dim), &sv, c.r_heads, c.r_dim, c.r_vdim, &b));
        CudaTensor o = adopt(b, {n, (int64_t)c.r_heads * c.r_vdim});
        cc_view ov = o.view();
        check(cc_gated_head_rms_norm(dev, &ov, &rg, nullptr, c.r_vdim, conf.norm_eps, CC_ACT_SILU));
        return L.right_o.matmul_vec(o);
    }

    CudaTensor forward_chunk(crabml::SeqState& base, int64_t pos0, const int64_t* tokens, int64_t n, int device_slot) override {
        State& s = static_cast<State&>(base);
        CudaTensor x = CudaTensor::alloc({n, conf.width}, CC_F32, dev);
        if (device_slot >= 0) x.copy_rows_from_slot(embed, device_slot);
        else x.copy_rows_from(embed, std::vector<int64_t>(tokens, tokens + n));
        CudaTensor x0;
        if (loop_in.valid()) x0 = x.dup();
        for (size_t ri = 0; ri < runs.size(); ri++) {
            const Layer& L = layers[runs[ri].layer];
            if (runs[ri].re_enter) {
                cc_view xv = x.view(), x0v = x0.view();
                cc_buf* b = nullptr;
                check(cc_concat_cols(dev, &xv, &x0v, &b));
                x = loop_in.matmul_vec(adopt(b, {n, 2 * (int64_t)conf.width}));
            }
            std::vector<CudaTensor> part;
            {
                part = split(L.h_stack.matmul_vec(layer_norm(x, L.norm_w, L.norm_b)), L.widths);
            }
            CudaTensor yl = left_mixer(L, s.runs[ri], part, pos0);
            CudaTensor yr = L.c.right == CLR_RIGHT_DIAGONAL ? diagonal_mixer(L, s.runs[ri], part) : retention_mixer(L, s.runs[ri], part, pos0);
            cc_view ylv = yl.view(), yrv = yr.view(), xv = x.view();
            if (L.i_ff >= 0) {
                cc_view gv = part[L.i_ff].view();
                cc_buf* b = nullptr;
                check(cc_glu_halves(dev, &gv, nullptr, CC_ACT_GELU_TANH, &b));
                CudaTensor yd = L.down.matmul_vec(adopt(b, {n, L.c.ff}));
                cc_view ydv = yd.view();
                check(cc_scaled_sum_accumulate(dev, &xv, &ylv, L.c.left_scale, &yrv, L.c.right_scale, &ydv));
            } else {
                check(cc_scaled_sum_accumulate(dev, &xv, &ylv, L.c.left_scale, &yrv, L.c.right_scale, nullptr));
            }
            x = std::move(x).with_name("run:" + std::to_string(ri) + ":" + std::to_string(pos0));
        }
        return x;
    }

    CudaTensor logits_of(const CudaTensor& x, const std::vector<int64_t>& rows) override {
        bool all = (int64_t)rows.size() == x.shape()[0];
        for (size_t i = 0; all && i < rows.size(); i++) all = rows[i] == (int64_t)i;
        CudaTensor lg;
        if (all) lg = head.matmul_vec(layer_norm(x, final_w, final_b));          // every row in order (a decoded token): no copy
        else {
            CudaTensor xs = CudaTensor::alloc({(int64_t)rows.size(), conf.width}, CC_F32, dev);
            xs.copy_rows_from(x, rows);
            lg = head.matmul_vec(layer_norm(xs, final_w, final_b));
        }
        if (conf.logit_scale != 1.0f) lg = std::move(lg).scale_inplace(conf.logit_scale);
        return lg;
    }
};

}  // namespace

extern "C" CC_API int clr_runner_create(cc_device* dev, const clr_config* conf, const clr_layer_config* lc, const clr_layer_weights* lw, cc_buf* embed, cc_buf* loop_in,
                                        cc_buf* final_norm_w, cc_buf* final_norm_b, cc_buf* head, csr_runner** out) {
    if (!dev || !conf || !lc || !lw || !embed || !final_norm_w || !head || !out) return CC_ERR_ARG;
    Runner* r = new Runner();
    r->dev = dev;
    r->conf = *conf;
    if (r->conf.chunk <= 0) r->conf.chunk = 256;
    if (r->conf.max_seq <= 0) r->conf.max_seq = 4096;
    r->width = conf->width; r->vocab = conf->vocab; r->chunk = r->conf.chunk;
    std::string err;
    int rc = crabml::seq_guarded(r, &err, [&] {
        const int64_t D = conf->width;
        if (conf->n_layers < 1 || D < 1 || conf->vocab < 1) throw TensorError("bad model sizes");
        r->embed = CudaTensor::wrap(dev, embed, {conf->vocab, D});
        r->final_w = CudaTensor::wrap(dev, final_norm_w, {D});
        if (final_norm_b) r->final_b = CudaTensor::wrap(dev, final_norm_b, {D});
        r->head = CudaTensor::wrap(dev, head, {conf->vocab, D});
        r->layers.resize(conf->n_layers);
        for (int i = 0; i < conf->n_layers; i++) {
            Layer& L = r->layers[i];
            const clr_layer_config& c = L.c = lc[i];
            const clr_layer_weights& w = lw[i];
            const std::string at = "layer " + std::to_string(i) + ": ";
            auto need = [&](cc_buf* b, const char* name, std::vector<int64_t> shape) {
                if (!b) throw TensorError(at + "tensor '" + name + "' is missing");
                return CudaTensor::wrap(dev, b, shape);
            };
            auto maybe = [&](cc_buf* b, std::vector<int64_t> shape) { return b ? CudaTensor::wrap(dev, b, shape) : CudaTensor(); };
            L.norm_w = need(w.norm_w, "norm1", {D}); L.norm_b = maybe(w.norm_b, {D});
            if (c.heads < 1 || c.kv_heads < 1 || c.heads % c.kv_heads || c.dim < 1 || c.vdim < 1) throw TensorError(at + "bad head counts / sizes of the left mixer");
            const int64_t hq = (int64_t)c.heads * c.dim, hk = (int64_t)c.kv_heads * c.dim, hv = (int64_t)c.kv_heads * c.vdim, ho = (int64_t)c.heads * c.vdim;
            L.widths = {(int32_t)hq, (int32_t)hk, (int32_t)hv};
            if (c.left_gate) { L.i_gate = (int)L.widths.size(); L.widths.push_back(c.heads); }
            L.i_right = (int)L.widths.size();
            int64_t right_out = 0;
            if (c.right == CLR_RIGHT_DIAGONAL) {
                if (c.r_width < 1 || c.r_blocks < 1 || c.r_width % c.r_blocks || c.r_conv < 1 || !(c.r_rate > 0.0f)) throw TensorError(at + "bad sizes / constants of the diagonal recurrence");
                const int64_t C = c.r_width, bs = C / c.r_blocks;
                L.widths.push_back((int32_t)C); L.widths.push_back((int32_t)C);
                L.conv = need(w.conv, "mix.right.conv", {C, c.r_conv}); L.conv_bias = maybe(w.conv_bias, {C}); L.x_bias = maybe(w.x_bias, {C}); L.y_bias = maybe(w.y_bias, {C});
                L.gate_w = need(w.gate_w, "the stack of mix.right.ra and mix.right.ri", {2 * C, bs}); L.gate_b = need(w.gate_b, "the stack of mix.right.ra.b and mix.right.ri.b", {2 * C});
                L.lam = need(w.lam, "mix.right.lam", {C});
                right_out = C;
            } else if (c.right == CLR_RIGHT_RETENTION) {
                if (c.r_heads < 1 || c.r_dim < 1 || c.r_vdim < 1) throw TensorError(at + "bad head counts / sizes of the right mixer");
                const int64_t rqk = (int64_t)c.r_heads * c.r_dim, rv = (int64_t)c.r_heads * c.r_vdim;
                for (int64_t v : {rqk, rqk, rv, rv}) L.widths.push_back((int32_t)v);
                L.decay = need(w.decay, "the decays of the right mixer", {c.r_heads});
                if (w.r_rot_freq) {
                    const int64_t pairs = cc_tensor_capacity(w.r_rot_freq);
                    if (2 * pairs > c.r_dim) throw TensorError(at + "more rotated pairs than a head of the right mixer holds");
                    L.r_rot_freq = CudaTensor::wrap(dev, w.r_rot_freq, {pairs});
                }
                right_out = rv;
            } else throw TensorError(at + "unknown right mixer");
            if (c.ff > 0) {
                L.i_ff = (int)L.widths.size();
                L.widths.push_back(2 * c.ff);
                L.down = need(w.down, "mlp.down", {D, c.ff});
            } else if (c.ff < 0) throw TensorError(at + "bad feed-forward width");
            int64_t on_h = 0;
            for (int32_t v : L.widths) on_h += v;
            L.h_stack = need(w.h_stack, "the stack of the layer's projections", {on_h, D});
            if (c.qk_norm == CLR_QK_WHOLE_WEIGHTED) { L.q_norm = need(w.q_norm, "mix.left.q.norm", {hq}); L.k_norm = need(w.k_norm, "mix.left.k.norm", {hk}); }
            else if (c.qk_norm != CLR_QK_NONE && c.qk_norm != CLR_QK_UNIT_PER_HEAD) throw TensorError(at + "unknown query / key norm");
            L.sink = maybe(w.sink, {c.heads});
            if (w.rot_freq) {
                const int64_t pairs = cc_tensor_capacity(w.rot_freq);
                if (2 * pairs > c.dim) throw TensorError(at + "more rotated pairs than a head holds");
                L.rot_freq = CudaTensor::wrap(dev, w.rot_freq, {pairs});
            }
            L.left_o = need(w.left_o, "mix.left.o", {D, ho}); L.right_o = need(w.right_o, "mix.right.o", {D, right_out});
            // a ring holds what the mask lets the first token of a pass see, plus the pass
            int64_t reach = 0;
            if (c.window > 0) reach = c.window;
            if (c.block > 0 && (reach == 0 || c.block < reach)) reach = c.block;
            L.ring = reach > 0 ? reach - 1 + r->conf.chunk : std::max<int64_t>(r->conf.max_seq, r->conf.chunk);
        }
        // the order of the runs
        const int n = conf->n_layers;
        if (conf->loop_times >= 1) {
            const int a = conf->loop_start, b = conf->loop_stop;
            if (a < 0 || b < a || b > n) throw TensorError("the loop does not lie inside the layers");
            if (b > a) {
                if (!loop_in) throw TensorError("tensor 'loop.in' is missing");
                r->loop_in = CudaTensor::wrap(dev, loop_in, {D, 2 * D});
            }
            for (int i = 0; i < a; i++) r->runs.push_back({i, false});
            for (int t = 0; t < conf->loop_times; t++)
                for (int i = a; i < b; i++) r->runs.push_back({i, i == a});
            for (int i = b; i < n; i++) r->runs.push_back({i, false});
        } else {
            for (int i = 0; i < n; i++) r->runs.push_back({i, false});
        }
        // a looped layer holds its state once per run
        for (const Run& run : r->runs) {
            const Layer& L = r->layers[run.layer];
            const auto& c = L.c;
            int64_t floats = L.ring * (int64_t)c.kv_heads * (c.dim + c.vdim);
            floats += c.right == CLR_RIGHT_DIAGONAL ? (int64_t)c.r_width * c.r_conv : (int64_t)c.r_heads * c.r_dim * c.r_vdim;
            r->state_bytes_per_slot += floats * 4;
        }
    });
    if (rc != CC_OK) {
        crabml::seq_set_create_error(err);
        delete r;
        return rc;
    }
    *out = r;
    return CC_OK;
}
