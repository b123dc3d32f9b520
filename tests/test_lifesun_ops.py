"""The mechanisms the Lifesun family added to include/crabml_seqops.h, each alone, against its function in the plain reference
(tests/lifesun_ref.py).  Where random inputs would hide a fault (a block's or a window's edge, a far key, the extra 1 in the denominator,
a decay close to one) the inputs are made so that it shows."""
import numpy as np
import pytest

from crabml_b200 import capi, seqops
from crabml_b200.capi import TensorError
from tests import lifesun_ref as R
from tests.gpu_common import make_device

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = make_device()
    yield d
    d.close()


def T32(dev, a, shape=None):
    from crabml_b200 import CudaTensor
    a = np.asarray(a, np.float32)
    return CudaTensor.new(a, list(shape if shape is not None else a.shape), dev)


def zeros(dev, shape):
    from crabml_b200 import CudaTensor
    t = CudaTensor.alloc(list(shape), capi.F32, dev)
    seqops.tensor_zero(t)
    return t


def f32(a):
    return np.asarray(a, np.float32).astype(np.float64)


def cuts(T, sizes):
    """portions of the given sizes, repeated until T tokens are covered"""
    out, at, i = [], 0, 0
    while at < T:
        n = min(sizes[i % len(sizes)], T - at)
        out.append((at, at + n))
        at += n
        i += 1
    return out


# ---- small ops ----------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cols", [1, 5, 32, 33, 200, 1500])
def test_layer_norm(dev, cols):
    rng = np.random.default_rng(cols)
    x = f32(rng.standard_normal((7, cols)) * 3 + 5.0)            # a mean far from zero: E[x^2] - mean^2 would lose digits
    w, b = f32(1 + 0.3 * rng.standard_normal(cols)), f32(rng.standard_normal(cols))
    got = seqops.layer_norm(T32(dev, x), T32(dev, w), T32(dev, b), 1e-5).export().reshape(7, cols)
    assert np.abs(got - R.layer_norm(x, w, b, 1e-5)).max() < 2e-5
    got = seqops.layer_norm(T32(dev, x), T32(dev, w), None, 1e-2).export().reshape(7, cols)
    assert np.abs(got - R.layer_norm(x, w, 0.0, 1e-2)).max() < 2e-5
    t = T32(dev, x)
    seqops.layer_norm(t, T32(dev, w), T32(dev, b), 1e-5, dst=t)       # in place
    assert np.abs(t.export().reshape(7, cols) - R.layer_norm(x, w, b, 1e-5)).max() < 2e-5
    with pytest.raises(TensorError):
        seqops.layer_norm(T32(dev, x), T32(dev, np.ones(cols + 1)), None, 1e-5)


def test_head_gate_and_concat(dev):
    rng = np.random.default_rng(2)
    x, g = f32(rng.standard_normal((9, 5 * 7))), f32(rng.standard_normal((9, 5)) * 3)
    got = seqops.head_gate(T32(dev, x), T32(dev, g), 5).export().reshape(9, 5, 7)
    assert np.abs(got - x.reshape(9, 5, 7) * R.sigmoid(g)[:, :, None]).max() < 1e-6
    a, b = f32(rng.standard_normal((6, 11))), f32(rng.standard_normal((6, 3)))
    assert np.array_equal(seqops.concat_cols(T32(dev, a), T32(dev, b)).export().reshape(6, 14), np.concatenate([a, b], 1).astype(np.float32))
    d, e, c = f32(rng.standard_normal((6, 11))), f32(rng.standard_normal((6, 11))), f32(rng.standard_normal((6, 11)))
    assert np.abs(seqops.scaled_sum_accumulate(T32(dev, a), T32(dev, d), 0.8, T32(dev, e), 1.3, T32(dev, c)).export().reshape(6, 11) - (a + 0.8 * d + 1.3 * e + c)).max() < 1e-6
    assert np.abs(seqops.scaled_sum_accumulate(T32(dev, a), T32(dev, d), 0.8, T32(dev, e), 1.3).export().reshape(6, 11) - (a + 0.8 * d + 1.3 * e)).max() < 1e-6
    with pytest.raises(TensorError):
        seqops.concat_cols(T32(dev, a), T32(dev, b[:5]))
    with pytest.raises(TensorError):
        seqops.head_gate(T32(dev, x), T32(dev, g[:, :4]), 5)


@pytest.mark.parametrize("heads,hs,dims,base", [(3, 10, 6, 100.0), (1, 8, 8, 1e4), (4, 7, 2, 50.0), (2, 64, 32, 2e5)])
def test_rotation_of_half_pairs(dev, heads, hs, dims, base):
    rng = np.random.default_rng(dims)
    x = f32(rng.standard_normal((12, heads * hs)))
    f = T32(dev, (float(base) ** (-2.0 * np.arange(dims // 2) / dims)).astype(np.float32))
    want = R.rotate_half(x.reshape(12, heads, hs), np.arange(12), dims, base).reshape(12, -1)
    got = seqops.rope_halves(T32(dev, x), heads, hs, 0, f, 1.0, 0).export().reshape(12, -1)
    assert np.abs(got - want).max() < 2e-5
    # rows 5 .. as positions 5 ..: a portion of a prompt
    got = seqops.rope_halves(T32(dev, x[5:]), heads, hs, 0, f, 1.0, 5).export().reshape(7, -1)
    assert np.abs(got - want[5:]).max() < 2e-5
    # two tensors in one pass
    x2 = f32(rng.standard_normal((12, heads * hs)))
    a, b = seqops.rope_halves_two(T32(dev, x), T32(dev, x2), heads, hs, 0, f, 1.0, 0)
    assert np.abs(a.export().reshape(12, -1) - want).max() < 2e-5
    assert np.abs(b.export().reshape(12, -1) - R.rotate_half(x2.reshape(12, heads, hs), np.arange(12), dims, base).reshape(12, -1)).max() < 2e-5
    # far positions: the angle is a 32-bit product, so compare against the reference fed that product
    far = np.array([100000 + i for i in range(12)])
    ang = (far[:, None].astype(np.float32) * f.export()[None, :].astype(np.float32)).astype(np.float64)
    xr = x.reshape(12, heads, hs)
    u, v = xr[..., :dims // 2], xr[..., dims // 2:dims]
    wf = xr.copy()
    wf[..., :dims // 2] = u * np.cos(ang)[:, None] - v * np.sin(ang)[:, None]
    wf[..., dims // 2:dims] = v * np.cos(ang)[:, None] + u * np.sin(ang)[:, None]
    got = seqops.rope_halves(T32(dev, x), heads, hs, 0, f, 1.0, 100000).export().reshape(12, heads, hs)
    assert np.abs(got - wf).max() < 2e-5


# ---- attention: cap, blocks, window, the extra 1 ----------------------------------------------------------------------------------------------
def run_attention(dev, q, k, v, scale, window, block, softcap, sink, portions, ring):
    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    kr, vr = zeros(dev, [ring, G * dk]), zeros(dev, [ring, G * dv])
    out = []
    for a, b in portions:
        seqops.kv_ring_append(kr, vr, T32(dev, k[a:b].reshape(b - a, -1)), T32(dev, v[a:b].reshape(b - a, -1)), None, 0.0, a, G, dk, dv)
        o = seqops.masked_attention_capped(T32(dev, q[a:b].reshape(b - a, -1)), kr, vr, a, H, G, dk, dv, scale, window=window, block=block, softcap=softcap,
                                           sink=T32(dev, np.zeros(H)) if sink else None)
        out.append(o.export().reshape(b - a, H, dv))
    return np.concatenate(out)


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 12, 8), (6, 2, 10, 6), (3, 3, 7, 5), (5, 1, 16, 20)])
@pytest.mark.parametrize("kind", ["blocks", "window"])
def test_attention_in_portions_against_the_reference(dev, H, G, dk, dv, kind):
    rng = np.random.default_rng(H * 10 + dk)
    T, size = 90, 13
    q, k, v = f32(rng.standard_normal((T, H, dk))), f32(rng.standard_normal((T, G, dk))), f32(rng.standard_normal((T, G, dv)))
    if kind == "blocks":
        want = R.attention(q, k, v, 0.5, R.block_mask(T, size), one_in_denominator=True)
        args = dict(window=0, block=size, softcap=0.0, sink=True)
    else:
        want = R.attention(q, k, v, 0.5, R.window_mask(T, size), softcap=1.7)
        args = dict(window=size, block=0, softcap=1.7, sink=False)
    for sizes in ([90], [1], [2], [40, 1, 1, 7], [5, 2, 31]):
        ring = size - 1 + max(sizes)
        got = run_attention(dev, q, k, v, 0.5, portions=cuts(T, sizes), ring=ring, **args)
        assert np.abs(got - want).max() < 3e-5, sizes


def test_keys_just_inside_and_just_outside_an_edge_tower(dev):
    """One key gets a score far above the rest.  Seen, it takes all the weight; one position further it must be invisible."""
    rng = np.random.default_rng(5)
    T, H, G, dk, dv, size = 64, 2, 1, 8, 4, 9
    q, k, v = f32(rng.standard_normal((T, H, dk)) * 0.1), f32(rng.standard_normal((T, G, dk)) * 0.1), f32(rng.standard_normal((T, G, dv)))
    tower = 20
    k[tower, 0] = 0.0
    k[tower, 0, 3] = 30.0
    q[:, :, 3] = 2.0
    for kind in ("blocks", "window"):
        if kind == "blocks":
            want = R.attention(q, k, v, 1.0, R.block_mask(T, size), one_in_denominator=True)
            args = dict(window=0, block=size, softcap=0.0, sink=True)
            last_seeing = (tower // size + 1) * size - 1
        else:
            want = R.attention(q, k, v, 1.0, R.window_mask(T, size))
            args = dict(window=size, block=0, softcap=0.0, sink=False)
            last_seeing = tower + size - 1
        assert np.abs(want[last_seeing, 0] - v[tower, 0]).max() < 1e-6 and np.abs(want[last_seeing + 1, 0] - v[tower, 0]).max() > 1e-2
        for sizes in ([64], [1], [2], [last_seeing, 1, 1, 40], [tower + 1, 3, 64]):
            got = run_attention(dev, q, k, v, 1.0, portions=cuts(T, sizes), ring=size - 1 + max(sizes), **args)
            assert np.abs(got - want).max() < 3e-5, (kind, sizes)


def test_far_key_without_a_mask_and_the_cap_keeps_a_huge_score_finite(dev):
    rng = np.random.default_rng(6)
    T, H, G, dk, dv = 700, 2, 2, 6, 3
    q, k, v = f32(rng.standard_normal((T, H, dk)) * 0.2), f32(rng.standard_normal((T, G, dk)) * 0.2), f32(rng.standard_normal((T, G, dv)))
    k[3, :, 0] = 50.0
    q[:, :, 0] = 40.0                                           # raw score 2000: without the cap the far key would take everything
    want = R.attention(q, k, v, 1.0, R.window_mask(T, 10000), softcap=2.5)
    assert np.abs(want[-1] - v[3]).max() > 0.05
    got = run_attention(dev, q, k, v, 1.0, 0, 0, 2.5, False, cuts(T, [600, 1]), ring=700)
    assert np.abs(got - want).max() < 3e-5
    want = R.attention(q, k, v, 1.0, R.window_mask(T, 10000))
    got = run_attention(dev, q, k, v, 1.0, 0, 0, 0.0, False, cuts(T, [256, 3, 1]), ring=700)
    assert np.abs(got[-1] - v[3]).max() < 1e-5 and np.abs(got - want).max() < 3e-5


def test_the_extra_one_weighs_in_when_scores_are_small(dev):
    T, H, dk, dv = 5, 1, 4, 2
    q, k, v = np.zeros((T, H, dk)), np.zeros((T, H, dk)), np.ones((T, H, dv))
    got = run_attention(dev, q, k, v, 1.0, 0, 3, 0.0, True, [(0, 5)], ring=8)
    assert np.allclose(got[:, 0, 0], [1 / 2, 2 / 3, 3 / 4, 1 / 2, 2 / 3], atol=1e-6)         # n keys of score 0 beside the 1: n / (n + 1)
    k[:] = 1.0
    q[:] = -20.0                                                  # all scores -80: the 1 holds almost all the weight
    got = run_attention(dev, q, k, v, 1.0, 0, 3, 0.0, True, [(0, 2), (2, 5)], ring=8)
    assert np.abs(got).max() < 1e-30 and np.isfinite(got).all()


# ---- retention ------------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,dk,dv", [(2, 32, 16), (3, 64, 40), (1, 128, 33), (2, 8, 10), (3, 5, 1), (1, 1, 7)])
def test_retention_in_portions_against_the_reference(dev, H, dk, dv):
    rng = np.random.default_rng(dk + dv)
    T = 70
    q, k, v = f32(rng.standard_normal((T, H, dk))), f32(rng.standard_normal((T, H, dk))), f32(rng.standard_normal((T, H, dv)))
    decay = f32([0.5, 0.9375, 0.998046875][:H])
    scale = dk ** -0.5
    want = R.retention(q, k * np.float32(scale), v, decay)
    tol = 2e-5 * max(1.0, np.abs(want).max())
    for sizes in ([70], [1], [2], [16, 17, 1, 3], [33, 37]):
        S = zeros(dev, [H, dk, dv])
        got = []
        for a, b in cuts(T, sizes):
            got.append(seqops.retention(T32(dev, q[a:b].reshape(b - a, -1)), T32(dev, k[a:b].reshape(b - a, -1)), T32(dev, v[a:b].reshape(b - a, -1)), T32(dev, decay), scale, S,
                                        H, dk, dv).export().reshape(b - a, H, dv))
        assert np.abs(np.concatenate(got) - want).max() < tol, sizes


def test_retention_remembers_a_key_from_far_back_by_its_decay(dev):
    T, H, dk, dv = 600, 2, 4, 2
    q, k, v = np.zeros((T, H, dk)), np.zeros((T, H, dk)), np.zeros((T, H, dv))
    k[2, :, 1] = 1.0
    v[2, :, 0] = 1.0
    q[:, :, 1] = 1.0
    decay = f32([0.998046875, 0.9375])
    S = zeros(dev, [H, dk, dv])
    got = np.concatenate([seqops.retention(T32(dev, q[a:b].reshape(b - a, -1)), T32(dev, k[a:b].reshape(b - a, -1)), T32(dev, v[a:b].reshape(b - a, -1)), T32(dev, decay), 1.0, S, H, dk,
                                           dv).export().reshape(b - a, H, dv) for a, b in cuts(T, [100, 1])])
    for h in range(H):
        want = np.where(np.arange(T) >= 2, decay[h] ** np.maximum(np.arange(T) - 2, 0), 0.0)
        assert np.allclose(got[:, h, 0], want, rtol=2e-4, atol=1e-30), h
    assert got[2, 0, 0] == 1.0 and got[1, 0, 0] == 0.0
    with pytest.raises(TensorError):
        seqops.retention(T32(dev, q.reshape(T, -1)), T32(dev, k.reshape(T, -1)), T32(dev, v.reshape(T, -1)), T32(dev, decay[:1]), 1.0, S, H, dk, dv)


# ---- the gated diagonal recurrence ----------------------------------------------------------------------------------------------------------------
def interleave(r, i, blocks):
    """[T, C] gate inputs -> the op's layout: per block of channels the recurrence gate, then the input gate"""
    T, C = r.shape
    bs = C // blocks
    return np.concatenate([r.reshape(T, blocks, 1, bs), i.reshape(T, blocks, 1, bs)], 2).reshape(T, 2 * C)


@pytest.mark.parametrize("C,blocks", [(24, 3), (32, 1), (33, 33), (100, 4), (7, 1)])
def test_diagonal_recurrence_in_portions_against_the_reference(dev, C, blocks):
    rng = np.random.default_rng(C)
    T = 75
    u, gr, gi, y = (f32(rng.standard_normal((T, C)) * s) for s in (1.0, 2.0, 2.0, 1.5))
    br, bi, yb, lam = f32(rng.standard_normal(C)), f32(rng.standard_normal(C)), f32(rng.standard_normal(C)), f32(rng.uniform(-6, 2, C))
    S = R.gated_diagonal_recurrence(u, R.sigmoid(gr + br), R.sigmoid(gi + bi), lam)
    want, want_plain = S * R.gelu_tanh(y + yb), S
    gates, gb = interleave(gr, gi, blocks), interleave(br[None], bi[None], blocks).reshape(-1)
    for sizes in ([75], [1], [2], [32, 33, 1, 9], [40, 35]):
        st, st2 = zeros(dev, [C]), zeros(dev, [C])
        got, plain = [], []
        for a, b in cuts(T, sizes):
            got.append(seqops.gated_diagonal_recurrence(T32(dev, u[a:b]), T32(dev, gates[a:b]), T32(dev, gb), T32(dev, lam), 8.0, blocks, st, y=T32(dev, y[a:b]), y_bias=T32(dev, yb),
                                                        y_act=capi.ACT_GELU_TANH).export().reshape(b - a, C))
            plain.append(seqops.gated_diagonal_recurrence(T32(dev, u[a:b]), T32(dev, gates[a:b]), T32(dev, gb), T32(dev, lam), 8.0, blocks, st2).export().reshape(b - a, C))
        assert np.abs(np.concatenate(got) - want).max() < 2e-5, sizes
        assert np.abs(np.concatenate(plain) - want_plain).max() < 2e-5, sizes


def test_diagonal_recurrence_with_decays_close_to_one_and_a_long_decode(dev):
    """softplus(lam) tiny: a = 1 - 1e-5 or so, and sqrt(1 - a^2) must keep its digits; 600 tokens one by one after a prompt"""
    rng = np.random.default_rng(9)
    T, C = 640, 6
    lam = f32([-13.0, -11.0, -9.0, -7.0, -3.0, 1.0])
    u, gr, gi = f32(np.ones((T, C))), f32(rng.standard_normal((T, C))), f32(rng.standard_normal((T, C)) + 2.0)
    want = R.gated_diagonal_recurrence(u, R.sigmoid(gr), R.sigmoid(gi), lam)
    st = zeros(dev, [C])
    got = np.concatenate([seqops.gated_diagonal_recurrence(T32(dev, u[a:b]), T32(dev, interleave(gr[a:b], gi[a:b], 2)), T32(dev, np.zeros(2 * C)), T32(dev, lam), 8.0, 2,
                                                           st).export().reshape(b - a, C) for a, b in cuts(T, [40] + [1] * 600)])
    assert np.abs(got / want - 1.0).max() < 2e-4 and want[-1, 0] > 1.5 * want[300, 0]          # the slowest channel is still far from saturated
    assert np.abs(st.export() - want[-1]).max() < 1e-4 * np.abs(want[-1]).max()
    with pytest.raises(TensorError):
        seqops.gated_diagonal_recurrence(T32(dev, u), T32(dev, interleave(gr, gi, 2)), T32(dev, np.zeros(2 * C)), T32(dev, lam), 8.0, 4, st)      # 4 blocks do not divide 6 channels


def test_convolution_with_bias_without_activation_carries_its_tail(dev):
    rng = np.random.default_rng(10)
    for C, K in ((24, 4), (5, 1), (40, 3), (33, 2)):
        T = 50
        x, w, b = f32(rng.standard_normal((T, C))), f32(rng.standard_normal((C, K))), f32(rng.standard_normal(C))
        want = R.causal_conv(x, w, b)
        for sizes in ([50], [1], [2], [7, 1, 30]):
            tail = zeros(dev, [K - 1, C]) if K > 1 else None
            got = np.concatenate([seqops.short_conv_bias(T32(dev, x[a:b_]), T32(dev, w), T32(dev, b), tail, act=capi.ACT_NONE).export().reshape(b_ - a, C) for a, b_ in cuts(T, sizes)])
            assert np.abs(got - want).max() < 1e-5, (C, K, sizes)
            # the bias of the projection that made x, added inside: zeros before the sequence stay zeros
            xb = f32(rng.standard_normal(C))
            tail = zeros(dev, [K - 1, C]) if K > 1 else None
            got = np.concatenate([seqops.short_conv_biases(T32(dev, x[a:b_]), T32(dev, w), T32(dev, xb), T32(dev, b), tail).export().reshape(b_ - a, C) for a, b_ in cuts(T, sizes)])
            assert np.abs(got - R.causal_conv(x + xb, w, b)).max() < 1e-5, (C, K, sizes)


@pytest.mark.parametrize("T,H,n_in,n_out", [(64, 3, 8, 16), (200, 2, 70, 33), (130, 1, 128, 256), (7, 2, 20, 9)])
def test_products_per_block_many_rows_and_few(dev, T, H, n_in, n_out):
    rng = np.random.default_rng(T)
    x, w = f32(rng.standard_normal((T, H, n_in))), f32(rng.standard_normal((H, n_out, n_in)))
    want = np.einsum("thi,hoi->tho", x, w).reshape(T, -1)
    got = seqops.head_project(T32(dev, x.reshape(T, -1)), T32(dev, w.reshape(H * n_out, n_in)), H).export().reshape(T, -1)
    assert np.abs(got - want).max() < 1e-4
    one = seqops.head_project(T32(dev, x[:3].reshape(3, -1)), T32(dev, w.reshape(H * n_out, n_in)), H).export().reshape(3, -1)      # the few-row kernel
    assert np.abs(one - want[:3]).max() < 1e-4


@pytest.mark.parametrize("norm", ["none", "head", "row"])
@pytest.mark.parametrize("pairing,dims,offset", [("halves", 6, 0), ("halves", 10, 0), ("neighbours", 4, 2), (None, 0, 0)])
def test_norms_rotation_and_cache_write_in_one_pass(dev, norm, pairing, dims, offset):
    """against the reference's steps one after the other; the ring wraps, and rows of other positions stay as they were"""
    rng = np.random.default_rng(dims + len(norm))
    T, H, G, dk, dv, ring, pos0, eps = 9, 3, 2, 10, 7, 12, 20, 1e-3
    q, k, v = f32(rng.standard_normal((T, H, dk)) * 2), f32(rng.standard_normal((T, G, dk)) * 2), f32(rng.standard_normal((T, G, dv)))
    qw = f32(1 + 0.3 * rng.standard_normal(H * dk if norm == "row" else dk))
    kw = f32(1 + 0.3 * rng.standard_normal(G * dk if norm == "row" else dk))
    if norm == "head":
        wq, wk = R.unit_rms(q, eps) * qw, R.unit_rms(k, eps) * kw
    elif norm == "row":
        wq, wk = (R.unit_rms(q.reshape(T, -1), eps) * qw).reshape(T, H, dk), (R.unit_rms(k.reshape(T, -1), eps) * kw).reshape(T, G, dk)
    else:
        wq, wk = q.copy(), k.copy()
    f = None
    if pairing:
        base, pos = 50.0, np.arange(pos0, pos0 + T)
        f = T32(dev, (base ** (-2.0 * np.arange(dims // 2) / dims)).astype(np.float32))
        if pairing == "halves":
            wq, wk = R.rotate_half(wq, pos, dims, base), R.rotate_half(wk, pos, dims, base)
        else:                                                   # neighbouring columns from `offset` on: the half layout of the reordered columns
            order = [offset + 2 * i for i in range(dims // 2)] + [offset + 2 * i + 1 for i in range(dims // 2)]
            for w_ in (wq, wk):
                w_[..., order] = R.rotate_half(w_[..., order], pos, dims, base)
    kr, vr = T32(dev, np.full((ring, G * dk), 7.0)), T32(dev, np.full((ring, G * dv), 7.0))
    tq = T32(dev, q.reshape(T, -1))
    seqops.qk_prepare_append(tq, T32(dev, k.reshape(T, -1)), T32(dev, v.reshape(T, -1)), kr, vr, pos0, H, G, dk, dv,
                             qk_norm={"none": capi.QK_NORM_NONE, "head": capi.QK_NORM_HEAD, "row": capi.QK_NORM_ROW}[norm], q_w=None if norm == "none" else T32(dev, qw),
                             k_w=None if norm == "none" else T32(dev, kw), eps=eps, freq=f, pairing=capi.ROPE_NEIGHBOURS if pairing == "neighbours" else capi.ROPE_HALVES, offset=offset)
    assert np.abs(tq.export().reshape(T, H, dk) - wq).max() < 2e-5
    gk, gv = kr.export().reshape(ring, G, dk), vr.export().reshape(ring, G, dv)
    rows = [(pos0 + t) % ring for t in range(T)]
    assert np.abs(gk[rows] - wk).max() < 2e-5 and np.array_equal(gv[rows], v.astype(np.float32))
    others = [r for r in range(ring) if r not in rows]
    assert np.all(gk[others] == 7.0) and np.all(gv[others] == 7.0)
