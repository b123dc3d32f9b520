// vuzinex_runner.cpp -- host driver of the Vuzinex decoder family over the C ABI (crabml_cuda.h + crabml_seqops.h).  Like the other
// runners it contains no arithmetic: it owns the weights' handles, says what a sequence holds (per layer RUN: key / value rings and a
// recurrent matrix, or a state-space matrix and a convolution tail; per sequence: its last token) and in which order the tensor ops run.
// Slots, step and greedy generation are the shared ones of seq_runner.hpp.
//
//   run:    x += mult * norm_b(mixer(norm_a(x))) ; x += mult * norm_d(ff(norm_c(x)))
//   pair:   ONE product of the stacked projections (+ biases), cut into its parts ; left: (q, k norms) ; rotation ; keys and values into the
//           run's rings ; masked softmax (+ sink) ; (sigmoid gate) ; W_o.  right: the recurrence on the run's state ; per-head norm and gate
//           ; W_o.  Then left_scale * left + right_scale * right.
//   state space: in-projection cut into z | x B C | dt ; convolution + silu ; scan ; gate, then group norm ; W_o
//   ff:     one product [gate ; up] ; silu(gate + b) * (up + b) ; W_down + b
#include <cmath>
#include <string>
#include <vector>

#include "../../../include/crabml_vuzinex.h"
#include "seq_runner.hpp"

using crabml::CudaTensor;
using crabml::TensorError;

namespace {

struct Layer {
    cvr_layer_config c{};
    CudaTensor norm_a, norm_b, norm_c, norm_d, h_stack, h_bias, q_norm, k_norm, sink, rot_freq, left_o, right_norm, right_o, gate_bias_i, gate_bias_f, decay_up, decay_bias, in,
        conv, conv_bias, dt_bias, a_log, d_skip, s_norm, s_o, gate_up, gate_up_bias, down, down_bias;
    std::vector<int32_t> widths;         // column blocks of the stacked product, in order
    int i_gate = -1, i_right = 0;        // block of the left gate (-1: none); first block of the right mixer
    int64_t ring = 0;                    // pair: rows of the key / value rings of one run
};
struct RunState {
    CudaTensor kring, vring, S, m, tail;
};
struct State : crabml::SeqState {
    std::vector<RunState> runs;
    CudaTensor last;                     // I32 [1]: 1 + the sequence's last token, 0 before the first
};
const cc_view* opt(const CudaTensor& t, cc_view& store) {
    if (!t.valid()) return nullptr;
    store = t.view();
    return &store;
}

struct Runner : csr_runner {
    cvr_config conf{};
    std::vector<Layer> layers;
    std::vector<int> runs;               // the layer of every run, in order
    CudaTensor embed, pair_table, final_norm, head;

    std::unique_ptr<crabml::SeqState> make_state() override {
        auto s = std::make_unique<State>();
        for (int li : runs) {
            const Layer& L = layers[li];
            const auto& c = L.c;
            RunState r;
            if (c.mixer == CVR_MIXER_PAIR) {
                r.kring = CudaTensor::alloc({L.ring, (int64_t)c.kv_heads * c.dim}, CC_F32, dev);
                r.vring = CudaTensor::alloc({L.ring, (int64_t)c.kv_heads * c.vdim}, CC_F32, dev);
                if (c.right == CVR_RIGHT_MATRIX_MEMORY) {
                    r.S = CudaTensor::alloc({c.r_heads, c.r_dim, (int64_t)c.r_vdim + 1}, CC_F32, dev);
                    r.m = CudaTensor::alloc({c.r_heads}, CC_F32, dev);
                } else {
                    r.S = CudaTensor::alloc({c.r_heads, c.r_dim, c.r_vdim}, CC_F32, dev);
                }
            } else {
                r.S = CudaTensor::alloc({c.s_heads, c.s_state, c.s_vdim}, CC_F32, dev);
                if (c.s_conv > 1) r.tail = CudaTensor::alloc({c.s_conv - 1, (int64_t)c.s_heads * c.s_vdim + 2 * (int64_t)c.s_groups * c.s_state}, CC_F32, dev);
            }
            s->runs.push_back(std::move(r));
        }
        if (pair_table.valid()) s->last = CudaTensor::alloc({1}, CC_I32, dev);
        return s;
    }
    // a reused slot starts like a new one: the recurrences, the convolutions and the token pair see nothing before position 0.  The rings
    // need no reset: a query at position i only reads rows of positions <= i of ITS sequence, all written since the slot was opened.
    void reset_state(crabml::SeqState& base) override {
        State& s = static_cast<State&>(base);
        for (auto& r : s.runs)
            for (CudaTensor* t : {&r.S, &r.m, &r.tail})
                if (t->valid()) { cc_view v = t->view(); check(cc_tensor_zero(dev, &v)); }
        if (s.last.valid()) { cc_view v = s.last.view(); check(cc_tensor_zero(dev, &v)); }
    }

    CudaTensor norm(const CudaTensor& x, const CudaTensor& w) {
        CudaTensor h = CudaTensor::alloc(x.shape(), CC_F32, dev);
        cc_view hv = h.view(), xv = x.view(), wv = w.view();
        check(cc_group_rms_norm(dev, &hv, &xv, &wv, 1, conf.norm_eps));
        return h;
    }
    // x += mult * norm(y) * w
    void add_normed(CudaTensor& x, const CudaTensor& y, const CudaTensor& w) {
        cc_view xv = x.view(), yv = y.view(), wv = w.view();
        check(cc_rms_norm_gain_mult(dev, &xv, &yv, &wv, conf.norm_eps, conf.residual_mult));
    }
    std::vector<CudaTensor> split(const CudaTensor& all, const std::vector<int32_t>& widths) {
        cc_view av = all.view();
        std::vector<cc_buf*> outs(widths.size(), nullptr);
        check(cc_split_cols(dev, &av, (int32_t)widths.size(), widths.data(), outs.data()));
        std::vector<CudaTensor> part;
        for (size_t p = 0; p < outs.size(); p++) part.push_back(adopt(outs[p], {all.shape()[0], widths[p]}));
        return part;
    }

    CudaTensor pair_mixer(const Layer& L, RunState& st, const CudaTensor& h, int64_t pos0) {
        const auto& c = L.c;
        const int64_t n = h.shape()[0];
        if (c.window <= 0 && c.block <= 0 && pos0 + n > L.ring)
            throw TensorError("a sequence of " + std::to_string(pos0 + n) + " tokens does not fit the cache of " + std::to_string(L.ring));
        std::vector<CudaTensor> part;
        {
            CudaTensor all = L.h_stack.matmul_vec(h);
            if (L.h_bias.valid()) { cc_view av = all.view(), bv = L.h_bias.view(); check(cc_add_row_bias(dev, &av, &bv)); }
            part = split(all, L.widths);
        }
        cc_buf* b = nullptr;
        // ---- left: softmax attention over the run's rings
        CudaTensor &q = part[0], &k = part[1], &v = part[2];
        cc_view qv = q.view(), kv = k.view(), vv = v.view(), tmp{};
        if (L.q_norm.valid()) {
            cc_view w = L.q_norm.view();
            check(cc_gated_head_rms_norm(dev, &qv, nullptr, &w, c.dim, conf.norm_eps, CC_ACT_NONE));
            w = L.k_norm.view();
            check(cc_gated_head_rms_norm(dev, &kv, nullptr, &w, c.dim, conf.norm_eps, CC_ACT_NONE));
        }
        if (L.rot_freq.valid()) {
            cc_view f = L.rot_freq.view();
            check(cc_rope_pairs(dev, &qv, c.heads, c.dim, 0, &f, c.rot_mag, pos0));
            check(cc_rope_pairs(dev, &kv, c.kv_heads, c.dim, 0, &f, c.rot_mag, pos0));
        }
        cc_view krv = st.kring.view(), vrv = st.vring.view();
        check(cc_kv_ring_append(dev, &krv, &vrv, &kv, &vv, nullptr, 0.0f, pos0, c.kv_heads, c.dim, c.vdim));
        check(cc_masked_attention(dev, &qv, &krv, &vrv, pos0, c.heads, c.kv_heads, c.dim, c.vdim, c.window, c.block, c.scale, opt(L.sink, tmp), &b));
        CudaTensor ol = adopt(b, {n, (int64_t)c.heads * c.vdim});
        b = nullptr;
        if (L.i_gate >= 0) {
            cc_view ov = ol.view(), gv = part[L.i_gate].view();
            check(cc_gated_sum(dev, &ov, 0, &ov, &gv, nullptr, nullptr, nullptr, nullptr));
        }
        CudaTensor yl = L.left_o.matmul_vec(ol);
        // ---- right: the recurrence on the run's state
        const int r0 = L.i_right;
        cc_view rq = part[r0].view(), rk = part[r0 + 1].view(), rv = part[r0 + 2].view(), rg = part[r0 + 3].view(), sv = st.S.view(), nw = L.right_norm.view();
        CudaTensor orr;
        if (c.right == CVR_RIGHT_MATRIX_MEMORY) {
            cc_view gi = part[r0 + 4].view(), gf = part[r0 + 5].view(), bi = L.gate_bias_i.view(), bf = L.gate_bias_f.view(), mv = st.m.view();
            check(cc_matrix_memory(dev, &rq, &rk, &rv, &gi, &gf, &bi, &bf, c.gate_cap, c.r_q_scale, &sv, &mv, c.r_heads, c.r_dim, c.r_vdim, &b));
            orr = adopt(b, {n, (int64_t)c.r_heads * c.r_vdim});
            cc_view ov = orr.view();
            check(cc_gated_head_rms_norm(dev, &ov, &rg, &nw, c.r_vdim, conf.norm_eps, CC_ACT_SIGMOID));
        } else {
            CudaTensor z = L.decay_up.matmul_vec(part[r0 + 4]);
            cc_view zv = z.view(), zb = L.decay_bias.view();
            check(cc_decayed_linear_attention(dev, &rq, &rk, &rv, &zv, &zb, c.tau, c.r_q_scale, &sv, c.r_heads, c.r_dim, c.r_vdim, &b));
            orr = adopt(b, {n, (int64_t)c.r_heads * c.r_vdim});
            cc_view ov = orr.view();
            check(cc_gated_head_rms_norm(dev, &ov, &rg, &nw, c.r_vdim, conf.norm_eps, CC_ACT_SILU));
        }
        CudaTensor yr = L.right_o.matmul_vec(orr);
        cc_view ylv = yl.view(), yrv = yr.view();
        check(cc_scaled_sum(dev, &ylv, &ylv, c.left_scale, &yrv, c.right_scale));
        return yl;
    }

    CudaTensor state_space_mixer(const Layer& L, RunState& st, const CudaTensor& h) {
        const auto& c = L.c;
        const int64_t n = h.shape()[0], inner = (int64_t)c.s_heads * c.s_vdim;
        std::vector<CudaTensor> part = split(L.in.matmul_vec(h), L.widths);          // z | x B C | dt
        cc_view xv = part[1].view(), cw = L.conv.view(), cb{}, tl{};
        cc_buf* b = nullptr;
        check(cc_short_conv_bias(dev, &xv, &cw, opt(L.conv_bias, cb), opt(st.tail, tl), CC_ACT_SILU, &b));
        CudaTensor xc = adopt(b, {n, part[1].shape()[1]});
        b = nullptr;
        cc_view xcv = xc.view(), dtv = part[2].view(), db = L.dt_bias.view(), al = L.a_log.view(), ds{}, sv = st.S.view();
        check(cc_state_space_scan(dev, &xcv, &dtv, &db, &al, opt(L.d_skip, ds), &sv, c.s_heads, c.s_groups, c.s_state, c.s_vdim, &b));
        CudaTensor y = adopt(b, {n, inner});
        cc_view yv = y.view(), zv = part[0].view(), nw = L.s_norm.view();
        check(cc_gated_group_rms_norm(dev, &yv, &yv, &zv, &nw, c.s_norm_groups, conf.norm_eps, CC_ACT_SILU));
        return L.s_o.matmul_vec(y);
    }

    CudaTensor feed_forward(const Layer& L, const CudaTensor& h) {
        CudaTensor gu = L.gate_up.matmul_vec(h);
        cc_view gv = gu.view(), bv{};
        cc_buf* b = nullptr;
        check(cc_glu_halves(dev, &gv, opt(L.gate_up_bias, bv), CC_ACT_SILU, &b));
        CudaTensor z = adopt(b, {h.shape()[0], L.c.ff});
        CudaTensor y = L.down.matmul_vec(z);
        if (L.down_bias.valid()) { cc_view yv = y.view(), dv = L.down_bias.view(); check(cc_add_row_bias(dev, &yv, &dv)); }
        return y;
    }

    CudaTensor forward_chunk(crabml::SeqState& base, int64_t pos0, const int64_t* tokens, int64_t n, int device_slot) override {
        State& s = static_cast<State&>(base);
        CudaTensor x = CudaTensor::alloc({n, conf.width}, CC_F32, dev);
        if (device_slot >= 0) x.copy_rows_from_slot(embed, device_slot);
        else x.copy_rows_from(embed, std::vector<int64_t>(tokens, tokens + n));
        if (pair_table.valid()) {
            cc_view xv = x.view(), tv = pair_table.view(), lv = s.last.view();
            check(cc_pair_hash_rows_add(dev, &xv, &tv, device_slot >= 0 ? nullptr : tokens, (int32_t)n, device_slot, &lv, conf.hash_mul_prev, conf.hash_mul_cur, conf.hash_buckets));
        }
        for (size_t ri = 0; ri < runs.size(); ri++) {
            const Layer& L = layers[runs[ri]];
            {
                CudaTensor h = norm(x, L.norm_a);
                CudaTensor y = L.c.mixer == CVR_MIXER_PAIR ? pair_mixer(L, s.runs[ri], h, pos0) : state_space_mixer(L, s.runs[ri], h);
                add_normed(x, y, L.norm_b);
            }
            if (L.c.ff > 0) {
                CudaTensor y = feed_forward(L, norm(x, L.norm_c));
                add_normed(x, y, L.norm_d);
            }
            x = std::move(x).with_name("run:" + std::to_string(ri) + ":" + std::to_string(pos0));
        }
        return x;
    }

    CudaTensor logits_of(const CudaTensor& x, const std::vector<int64_t>& rows) override {
        bool all = (int64_t)rows.size() == x.shape()[0];
        for (size_t i = 0; all && i < rows.size(); i++) all = rows[i] == (int64_t)i;
        CudaTensor lg;
        if (all) lg = head.matmul_vec(norm(x, final_norm));                   // every row in order (a decoded token): no copy
        else {
            CudaTensor xs = CudaTensor::alloc({(int64_t)rows.size(), conf.width}, CC_F32, dev);
            xs.copy_rows_from(x, rows);
            lg = head.matmul_vec(norm(xs, final_norm));
        }
        if (conf.logit_scale != 1.0f) lg = std::move(lg).scale_inplace(conf.logit_scale);
        return lg;
    }
};

}  // namespace

extern "C" CC_API int cvr_runner_create(cc_device* dev, const cvr_config* conf, const cvr_layer_config* lc, const cvr_layer_weights* lw, cc_buf* embed, cc_buf* pair_table,
                                        cc_buf* final_norm, cc_buf* head, csr_runner** out) {
    if (!dev || !conf || !lc || !lw || !embed || !final_norm || !head || !out) return CC_ERR_ARG;
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
        r->final_norm = CudaTensor::wrap(dev, final_norm, {D});
        r->head = CudaTensor::wrap(dev, head, {conf->vocab, D});
        if (conf->hash_buckets > 0) {
            if (!pair_table) throw TensorError("the table of the token-pair rows is missing");
            if (conf->hash_mul_prev < 0 || conf->hash_mul_cur < 0) throw TensorError("the multipliers of the token-pair hash must not be negative");
            // the hash is taken in 64-bit integers: token ids are below vocab
            if ((double)conf->vocab * ((double)conf->hash_mul_prev + (double)conf->hash_mul_cur) > 9.0e18) throw TensorError("the token-pair hash would overflow 64 bits");
            r->pair_table = CudaTensor::wrap(dev, pair_table, {conf->hash_buckets + 1, D});
        }
        r->layers.resize(conf->n_layers);
        for (int i = 0; i < conf->n_layers; i++) {
            Layer& L = r->layers[i];
            const cvr_layer_config& c = L.c = lc[i];
            const cvr_layer_weights& w = lw[i];
            const std::string at = "layer " + std::to_string(i) + ": ";
            auto need = [&](cc_buf* b, const char* name, std::vector<int64_t> shape) {
                if (!b) throw TensorError(at + "tensor '" + name + "' is missing");
                return CudaTensor::wrap(dev, b, shape);
            };
            auto maybe = [&](cc_buf* b, std::vector<int64_t> shape) { return b ? CudaTensor::wrap(dev, b, shape) : CudaTensor(); };
            L.norm_a = need(w.norm_a, "norm1", {D}); L.norm_b = need(w.norm_b, "norm1b", {D});
            if (c.mixer == CVR_MIXER_PAIR) {
                if (c.heads < 1 || c.kv_heads < 1 || c.heads % c.kv_heads || c.dim < 1 || c.vdim < 1) throw TensorError(at + "bad head counts / sizes of the left mixer");
                if (c.r_heads < 1 || c.r_dim < 1 || c.r_vdim < 1) throw TensorError(at + "bad head counts / sizes of the right mixer");
                const int64_t hq = (int64_t)c.heads * c.dim, hk = (int64_t)c.kv_heads * c.dim, hv = (int64_t)c.kv_heads * c.vdim, ho = (int64_t)c.heads * c.vdim;
                const int64_t rqk = (int64_t)c.r_heads * c.r_dim, rv = (int64_t)c.r_heads * c.r_vdim;
                L.widths = {(int32_t)hq, (int32_t)hk, (int32_t)hv};
                if (c.left_gate) { L.i_gate = (int)L.widths.size(); L.widths.push_back((int32_t)ho); }
                L.i_right = (int)L.widths.size();
                for (int64_t v : {rqk, rqk, rv, rv}) L.widths.push_back((int32_t)v);
                if (c.right == CVR_RIGHT_MATRIX_MEMORY) {
                    if (!(c.gate_cap > 0.0f)) throw TensorError(at + "the cap of the gates must be positive");
                    L.widths.push_back(c.r_heads); L.widths.push_back(c.r_heads);
                    L.gate_bias_i = need(w.gate_bias_i, "mix.right.i.b", {c.r_heads}); L.gate_bias_f = need(w.gate_bias_f, "mix.right.f.b", {c.r_heads});
                    L.right_norm = need(w.right_norm, "mix.right.norm", {rv});
                } else if (c.right == CVR_RIGHT_DECAYED) {
                    if (c.r_rank < 1 || !(c.tau > 0.0f)) throw TensorError(at + "bad sizes / constants of the decay");
                    L.widths.push_back(c.r_rank);
                    L.decay_up = need(w.decay_up, "mix.right.a2", {rqk, c.r_rank}); L.decay_bias = need(w.decay_bias, "mix.right.a2.b", {rqk});
                    L.right_norm = need(w.right_norm, "mix.right.norm", {c.r_vdim});
                } else throw TensorError(at + "unknown right mixer");
                int64_t on_h = 0;
                for (int32_t v : L.widths) on_h += v;
                L.h_stack = need(w.h_stack, "the stack of the mixer's projections", {on_h, D});
                L.h_bias = maybe(w.h_bias, {on_h});
                if ((w.q_norm == nullptr) != (w.k_norm == nullptr)) throw TensorError(at + "query and key norms come together");
                L.q_norm = maybe(w.q_norm, {c.dim}); L.k_norm = maybe(w.k_norm, {c.dim});
                L.sink = maybe(w.sink, {c.heads});
                if (w.rot_freq) {
                    const int64_t pairs = cc_tensor_capacity(w.rot_freq);
                    if (2 * pairs > c.dim) throw TensorError(at + "more rotated pairs than a head holds");
                    L.rot_freq = CudaTensor::wrap(dev, w.rot_freq, {pairs});
                }
                L.left_o = need(w.left_o, "mix.left.o", {D, ho}); L.right_o = need(w.right_o, "mix.right.o", {D, rv});
                // a ring holds what the mask lets the first token of a pass see, plus the pass
                int64_t reach = 0;
                if (c.window > 0) reach = c.window;
                if (c.block > 0 && (reach == 0 || c.block < reach)) reach = c.block;
                L.ring = reach > 0 ? reach - 1 + r->conf.chunk : std::max<int64_t>(r->conf.max_seq, r->conf.chunk);
            } else if (c.mixer == CVR_MIXER_STATE_SPACE) {
                if (c.s_heads < 1 || c.s_vdim < 1 || c.s_state < 1 || c.s_groups < 1 || c.s_heads % c.s_groups || c.s_conv < 1) throw TensorError(at + "bad sizes of the state-space mixer");
                const int64_t inner = (int64_t)c.s_heads * c.s_vdim, bc = 2 * (int64_t)c.s_groups * c.s_state;
                if (c.s_norm_groups < 1 || inner % c.s_norm_groups) throw TensorError(at + "the norm's groups do not divide the inner width");
                L.widths = {(int32_t)inner, (int32_t)(inner + bc), c.s_heads};
                L.in = need(w.in, "mix.in", {2 * inner + bc + c.s_heads, D});
                L.conv = need(w.conv, "mix.conv", {inner + bc, c.s_conv}); L.conv_bias = maybe(w.conv_bias, {inner + bc});
                L.dt_bias = need(w.dt_bias, "mix.dt_bias", {c.s_heads}); L.a_log = need(w.a_log, "mix.A_log", {c.s_heads}); L.d_skip = maybe(w.d_skip, {c.s_heads});
                L.s_norm = need(w.s_norm, "mix.norm", {inner}); L.s_o = need(w.s_o, "mix.o", {D, inner});
            } else throw TensorError(at + "unknown mixer");
            if (c.ff > 0) {
                L.norm_c = need(w.norm_c, "norm2", {D}); L.norm_d = need(w.norm_d, "norm2b", {D});
                L.gate_up = need(w.gate_up, "the stack of mlp.gate and mlp.up", {2 * (int64_t)c.ff, D}); L.gate_up_bias = maybe(w.gate_up_bias, {2 * (int64_t)c.ff});
                L.down = need(w.down, "mlp.down", {D, c.ff}); L.down_bias = maybe(w.down_bias, {D});
            } else if (c.ff < 0) throw TensorError(at + "bad feed-forward width");
        }
        // the order of the runs
        const int n = conf->n_layers;
        int a = conf->loop_start, b = conf->loop_stop, times = conf->loop_times;
        if (times <= 1 || b <= a) { a = b = 0; times = 1; }
        if (a < 0 || b > n) throw TensorError("the loop does not lie inside the layers");
        for (int i = 0; i < a; i++) r->runs.push_back(i);
        for (int t = 0; t < times; t++)
            for (int i = a; i < b; i++) r->runs.push_back(i);
        for (int i = b; i < n; i++) r->runs.push_back(i);
        // a looped layer holds its state once per run
        for (int li : r->runs) {
            const Layer& L = r->layers[li];
            const auto& c = L.c;
            if (c.mixer == CVR_MIXER_PAIR)
                r->state_bytes_per_slot += (L.ring * (int64_t)c.kv_heads * (c.dim + c.vdim) + (int64_t)c.r_heads * c.r_dim * (c.r_vdim + (c.right == CVR_RIGHT_MATRIX_MEMORY ? 1 : 0)) +
                                            (c.right == CVR_RIGHT_MATRIX_MEMORY ? c.r_heads : 0)) * 4;
            else
                r->state_bytes_per_slot += ((int64_t)c.s_heads * c.s_state * c.s_vdim + (int64_t)(c.s_conv - 1) * ((int64_t)c.s_heads * c.s_vdim + 2 * (int64_t)c.s_groups * c.s_state)) * 4;
        }
        if (conf->hash_buckets > 0) r->state_bytes_per_slot += 4;
    });
    if (rc != CC_OK) {
        crabml::seq_set_create_error(err);
        delete r;
        return rc;
    }
    *out = r;
    return CC_OK;
}
