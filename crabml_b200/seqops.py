"""Python handles on the sequence-mixing / routing ops of include/crabml_seqops.h (ctypes over the C ABI; used by the tests and
by anyone who builds a model out of these mechanisms in Python).  Arguments are CudaTensors; outputs are new CudaTensors."""
from __future__ import annotations

import ctypes as C

from . import capi
from .tensor import CudaTensor, TensorStrider, _Buf


def _v(t):
    return C.byref(t._view()) if t is not None else None


def _new(dev, handle, shape):
    return CudaTensor(_Buf(dev, handle), TensorStrider(shape), dev)


def tensor_zero(x):
    x.device.check(x.device.lib.cc_tensor_zero(x.device.handle, _v(x)))


def rms_norm_gain(dst, y, gain, eps, accumulate=False):
    dst.device.check(dst.device.lib.cc_rms_norm_gain(dst.device.handle, _v(dst), _v(y), _v(gain), float(eps), int(accumulate)))
    return dst


def gated_head_rms_norm(x, gate, w, head_size, eps, gate_act=capi.ACT_SILU):
    x.device.check(x.device.lib.cc_gated_head_rms_norm(x.device.handle, _v(x), _v(gate), _v(w), int(head_size), float(eps), int(gate_act)))
    return x


def glu_inplace(gate, up, act=capi.ACT_SILU):
    gate.device.check(gate.device.lib.cc_glu_inplace(gate.device.handle, _v(gate), _v(up), int(act)))
    return gate


def short_conv(x, w, tail, act=capi.ACT_SILU, head_size=0, unit_norm=False, unit_eps=1e-6, unit_scale=1.0):
    h = C.c_void_p()
    x.device.check(x.device.lib.cc_short_conv(x.device.handle, _v(x), _v(w), _v(tail), int(act), int(head_size), int(unit_norm), float(unit_eps),
                                              float(unit_scale), C.byref(h)))
    return _new(x.device, h, x.shape())


def gated_delta_rule(q, k, v, a, b, a_log, dt_bias, state, n_heads, n_kv, dk, dv):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_gated_delta_rule(q.device.handle, _v(q), _v(k), _v(v), _v(a), _v(b), _v(a_log), _v(dt_bias), _v(state), n_heads, n_kv, dk, dv,
                                                    C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def kv_ring_append(kring, vring, k, v, k_norm_w, eps, pos0, n_kv, dk, dv):
    kring.device.check(kring.device.lib.cc_kv_ring_append(kring.device.handle, _v(kring), _v(vring), _v(k), _v(v), _v(k_norm_w), float(eps), int(pos0), n_kv, dk, dv))


def window_attention(q, q_norm_w, eps, kring, vring, pos0, n_heads, n_kv, dk, dv, window, scale, r1=None, r2=None):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_window_attention(q.device.handle, _v(q), _v(q_norm_w), float(eps), _v(kring), _v(vring), int(pos0), n_heads, n_kv, dk, dv,
                                                    int(window), float(scale), _v(r1), _v(r2), C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def moe_route(x, router_w, correction, top, n_groups=1, keep_groups=1, renormalise=False):
    """-> (ids I32 [T, top] as a CudaTensor, weights F32 [T, top])"""
    hi, hw = C.c_void_p(), C.c_void_p()
    x.device.check(x.device.lib.cc_moe_route(x.device.handle, _v(x), _v(router_w), _v(correction), int(top), int(n_groups), int(keep_groups), int(renormalise),
                                             C.byref(hi), C.byref(hw)))
    T = x.shape()[0]
    return _new(x.device, hi, [T, top]), _new(x.device, hw, [T, top])


def moe_experts(x, ids, weights, w_gate, w_up, w_down, n_experts, ff, act=capi.ACT_SILU):
    h = C.c_void_p()
    x.device.check(x.device.lib.cc_moe_experts(x.device.handle, _v(x), _v(ids), _v(weights), _v(w_gate), _v(w_up), _v(w_down), int(n_experts), int(ff), int(act),
                                               C.byref(h)))
    return _new(x.device, h, list(x.shape()))


def split_cols(src, widths):
    n = len(widths)
    w = (C.c_int32 * n)(*[int(v) for v in widths])
    outs = (C.c_void_p * n)()
    src.device.check(src.device.lib.cc_split_cols(src.device.handle, _v(src), n, w, outs))
    return [_new(src.device, C.c_void_p(outs[i]), [src.shape()[0], int(widths[i])]) for i in range(n)]


def group_rms_norm(x, w, groups, eps, dst=None):
    dst = dst if dst is not None else type(x).alloc(x.shape(), capi.F32, x.device)
    x.device.check(x.device.lib.cc_group_rms_norm(x.device.handle, _v(dst), _v(x), _v(w), int(groups), float(eps)))
    return dst


def poly_norm(z, coef, eps):
    z.device.check(z.device.lib.cc_poly_norm(z.device.handle, _v(z), _v(coef), float(eps)))
    return z


def gated_sum(dst, y1, g1=None, b1=None, y2=None, g2=None, b2=None, accumulate=True):
    dst.device.check(dst.device.lib.cc_gated_sum(dst.device.handle, _v(dst), int(accumulate), _v(y1), _v(g1), _v(b1), _v(y2), _v(g2), _v(b2)))
    return dst


def rope_pairs(x, n_heads, head_size, offset, freq, mag, pos0):
    x.device.check(x.device.lib.cc_rope_pairs(x.device.handle, _v(x), int(n_heads), int(head_size), int(offset), _v(freq), float(mag), int(pos0)))
    return x


def latent_ring_append(ring, ckv, norm_w, eps, rank, freq, mag, pos0):
    ring.device.check(ring.device.lib.cc_latent_ring_append(ring.device.handle, _v(ring), _v(ckv), _v(norm_w), float(eps), int(rank), _v(freq), float(mag), int(pos0)))


def head_project(x, w, n_heads, rest=0, freq=None, mag=1.0, pos0=0):
    """freq: the first 2 * len(freq) carried columns are rotated on the way (rows are positions pos0 ..)"""
    h = C.c_void_p()
    x.device.check(x.device.lib.cc_head_project(x.device.handle, _v(x), _v(w), int(n_heads), int(rest), _v(freq), float(mag), int(pos0), C.byref(h)))
    return _new(x.device, h, [x.shape()[0], n_heads * (w.shape()[0] // n_heads + rest)])


def head_concat_shared(a, shared, n_heads, col0, rest):
    h = C.c_void_p()
    a.device.check(a.device.lib.cc_head_concat_shared(a.device.handle, _v(a), _v(shared), int(n_heads), int(col0), int(rest), C.byref(h)))
    return _new(a.device, h, [a.shape()[0], a.shape()[1] + n_heads * rest])


def window_attention_sink(q, kring, vring, pos0, n_heads, n_kv, dk, dv, window, scale, sink=None, q_norm_w=None, eps=0.0, r1=None, r2=None):
    """vring None: a key row's first dv columns are its value"""
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_window_attention_sink(q.device.handle, _v(q), _v(q_norm_w), float(eps), _v(kring), _v(vring), int(pos0), n_heads, n_kv, dk, dv,
                                                         int(window), float(scale), _v(r1), _v(r2), _v(sink), C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def moe_route_ex(x, router_w, correction, top, n_groups=1, keep_groups=1, score=capi.ROUTE_SOFTMAX, group_top=1, renormalise=False, renorm_eps=0.0):
    hi, hw = C.c_void_p(), C.c_void_p()
    rp = capi.cc_route_params(int(score), int(top), int(n_groups), int(keep_groups), int(group_top), int(renormalise), float(renorm_eps))
    x.device.check(x.device.lib.cc_moe_route_ex(x.device.handle, _v(x), _v(router_w), _v(correction), C.byref(rp), C.byref(hi), C.byref(hw)))
    T = x.shape()[0]
    return _new(x.device, hi, [T, top]), _new(x.device, hw, [T, top])


def moe_experts_glu(x, ids, weights, w_gate, w_up, w_down, n_experts, ff, act=capi.ACT_SILU, alpha=1.0, limit=0.0, up_shift=0.0):
    h = C.c_void_p()
    gp = capi.cc_glu_params(int(act), float(alpha), float(limit), float(up_shift))
    x.device.check(x.device.lib.cc_moe_experts_glu(x.device.handle, _v(x), _v(ids), _v(weights), _v(w_gate), _v(w_up), _v(w_down), int(n_experts), int(ff), C.byref(gp),
                                                   C.byref(h)))
    return _new(x.device, h, list(x.shape()))


def rms_norm_gain_mult(dst, y, gain, eps, mult):
    dst.device.check(dst.device.lib.cc_rms_norm_gain_mult(dst.device.handle, _v(dst), _v(y), _v(gain), float(eps), float(mult)))
    return dst


def head_rms_norm(x, w, head_size, eps, gate=None, gate_act=capi.ACT_NONE):
    """cc_gated_head_rms_norm with its optional operands: w None (no weight), [head_size] or one per column; gate None (no gate)"""
    x.device.check(x.device.lib.cc_gated_head_rms_norm(x.device.handle, _v(x), _v(gate), _v(w), int(head_size), float(eps), int(gate_act)))
    return x


def gated_group_rms_norm(x, gate, w, groups, eps, gate_act=capi.ACT_SILU, dst=None):
    dst = dst if dst is not None else type(x).alloc(x.shape(), capi.F32, x.device)
    x.device.check(x.device.lib.cc_gated_group_rms_norm(x.device.handle, _v(dst), _v(x), _v(gate), _v(w), int(groups), float(eps), int(gate_act)))
    return dst


def glu_halves(src, bias=None, act=capi.ACT_SILU):
    h = C.c_void_p()
    src.device.check(src.device.lib.cc_glu_halves(src.device.handle, _v(src), _v(bias), int(act), C.byref(h)))
    return _new(src.device, h, [src.shape()[0], src.shape()[1] // 2])


def add_row_bias(x, bias):
    x.device.check(x.device.lib.cc_add_row_bias(x.device.handle, _v(x), _v(bias)))
    return x


def scaled_sum(dst, a, sa, b, sb):
    dst.device.check(dst.device.lib.cc_scaled_sum(dst.device.handle, _v(dst), _v(a), float(sa), _v(b), float(sb)))
    return dst


def pair_hash_rows_add(dst, table, tokens, last, mul_prev, mul_cur, buckets, slot=-1):
    """tokens: a list of ids, or None to take ONE id from device slot `slot`; last: I32 [1] state"""
    n = len(tokens) if tokens is not None else 1
    arr = (C.c_int64 * n)(*[int(t) for t in tokens]) if tokens is not None else None
    dst.device.check(dst.device.lib.cc_pair_hash_rows_add(dst.device.handle, _v(dst), _v(table), arr, n, int(slot), _v(last), int(mul_prev), int(mul_cur), int(buckets)))
    return dst


def short_conv_bias(x, w, bias, tail, act=capi.ACT_SILU):
    h = C.c_void_p()
    x.device.check(x.device.lib.cc_short_conv_bias(x.device.handle, _v(x), _v(w), _v(bias), _v(tail), int(act), C.byref(h)))
    return _new(x.device, h, x.shape())


def masked_attention(q, kring, vring, pos0, n_heads, n_kv, dk, dv, scale, window=0, block=0, sink=None):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_masked_attention(q.device.handle, _v(q), _v(kring), _v(vring), int(pos0), n_heads, n_kv, dk, dv, int(window), int(block), float(scale),
                                                    _v(sink), C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def matrix_memory(q, k, v, gi, gf, bi, bf, cap, q_scale, state, mstate, n_heads, dk, dv):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_matrix_memory(q.device.handle, _v(q), _v(k), _v(v), _v(gi), _v(gf), _v(bi), _v(bf), float(cap), float(q_scale), _v(state), _v(mstate),
                                                 n_heads, dk, dv, C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def decayed_linear_attention(q, k, v, z, zb, tau, q_scale, state, n_heads, dk, dv):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_decayed_linear_attention(q.device.handle, _v(q), _v(k), _v(v), _v(z), _v(zb), float(tau), float(q_scale), _v(state), n_heads, dk, dv,
                                                            C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def state_space_scan(xbc, dt, dt_bias, a_log, d_skip, state, n_heads, n_groups, n_state, head_dim):
    h = C.c_void_p()
    xbc.device.check(xbc.device.lib.cc_state_space_scan(xbc.device.handle, _v(xbc), _v(dt), _v(dt_bias), _v(a_log), _v(d_skip), _v(state), n_heads, n_groups, n_state,
                                                        head_dim, C.byref(h)))
    return _new(xbc.device, h, [xbc.shape()[0], n_heads * head_dim])


def layer_norm(x, w, b, eps, dst=None):
    dst = dst if dst is not None else type(x).alloc(x.shape(), capi.F32, x.device)
    x.device.check(x.device.lib.cc_layer_norm(x.device.handle, _v(dst), _v(x), _v(w), _v(b), float(eps)))
    return dst


def head_gate(x, g, n_heads, act=capi.ACT_SIGMOID):
    x.device.check(x.device.lib.cc_head_gate(x.device.handle, _v(x), _v(g), int(n_heads), int(act)))
    return x


def concat_cols(a, b):
    h = C.c_void_p()
    a.device.check(a.device.lib.cc_concat_cols(a.device.handle, _v(a), _v(b), C.byref(h)))
    return _new(a.device, h, [a.shape()[0], a.shape()[1] + b.shape()[1]])


def rope_halves(x, n_heads, head_size, offset, freq, mag, pos0):
    x.device.check(x.device.lib.cc_rope_halves(x.device.handle, _v(x), int(n_heads), int(head_size), int(offset), _v(freq), float(mag), int(pos0)))
    return x


def masked_attention_capped(q, kring, vring, pos0, n_heads, n_kv, dk, dv, scale, window=0, block=0, softcap=0.0, sink=None):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_masked_attention_capped(q.device.handle, _v(q), _v(kring), _v(vring), int(pos0), n_heads, n_kv, dk, dv, int(window), int(block),
                                                           float(scale), float(softcap), _v(sink), C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def retention(q, k, v, decay, k_scale, state, n_heads, dk, dv):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_retention(q.device.handle, _v(q), _v(k), _v(v), _v(decay), float(k_scale), _v(state), n_heads, dk, dv, C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def gated_diagonal_recurrence(u, gates, gate_bias, lam, c, n_blocks, state, y=None, y_bias=None, y_act=capi.ACT_NONE):
    """gates / gate_bias: per block of channels the recurrence gate followed by the input gate, [n_blocks][2][C / n_blocks]"""
    h = C.c_void_p()
    u.device.check(u.device.lib.cc_gated_diagonal_recurrence(u.device.handle, _v(u), _v(gates), _v(gate_bias), _v(lam), float(c), int(n_blocks), _v(y), _v(y_bias),
                                                             int(y_act), _v(state), C.byref(h)))
    return _new(u.device, h, list(u.shape()))


def scaled_sum_accumulate(dst, a, sa, b, sb, c=None):
    dst.device.check(dst.device.lib.cc_scaled_sum_accumulate(dst.device.handle, _v(dst), _v(a), float(sa), _v(b), float(sb), _v(c)))
    return dst


def qk_prepare_append(q, k, v, kring, vring, pos0, n_heads, n_kv, dk, dv, qk_norm=capi.QK_NORM_NONE, q_w=None, k_w=None, eps=0.0, freq=None, pairing=capi.ROPE_HALVES, offset=0,
                      mag=1.0):
    """norms, rotation and the cache write between the projections and the attention, one kernel; q is overwritten"""
    q.device.check(q.device.lib.cc_qk_prepare_append(q.device.handle, _v(q), _v(k), _v(v), _v(kring), _v(vring), int(qk_norm), _v(q_w), _v(k_w), float(eps), _v(freq), int(pairing),
                                                     int(offset), float(mag), int(pos0), n_heads, n_kv, dk, dv))
    return q


def rope_halves_two(x1, x2, n_heads, head_size, offset, freq, mag, pos0):
    x1.device.check(x1.device.lib.cc_rope_halves_two(x1.device.handle, _v(x1), _v(x2), int(n_heads), int(head_size), int(offset), _v(freq), float(mag), int(pos0)))
    return x1, x2


def short_conv_biases(x, w, in_bias, bias, tail, act=capi.ACT_NONE):
    """the convolution over x + in_bias (zeros before the sequence), plus bias, then the activation"""
    h = C.c_void_p()
    x.device.check(x.device.lib.cc_short_conv_biases(x.device.handle, _v(x), _v(w), _v(in_bias), _v(bias), _v(tail), int(act), C.byref(h)))
    return _new(x.device, h, x.shape())
