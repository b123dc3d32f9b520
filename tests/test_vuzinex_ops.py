"""The mechanisms the Vuzinex family added to include/crabml_seqops.h, each alone, against its function in the plain reference
(tests/vuzinex_ref.py).  The reference's mixers start from projections; here the projections are selection matrices, so that the columns
of a random input ARE the queries, keys, values and gates the op gets.  Where random inputs would hide a fault (a block's edge, a far
key, a sink) the inputs are made so that it shows."""
import numpy as np
import pytest

from crabml_b200 import capi, seqops
from tests import vuzinex_ref as R
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


def zeros(dev, shape, dtype=capi.F32):
    from crabml_b200 import CudaTensor
    return CudaTensor.alloc(list(shape), dtype, dev)


def sel(total, start, n):
    m = np.zeros((n, total))
    m[np.arange(n), start + np.arange(n)] = 1.0
    return m


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
def test_pair_hash_rows_follow_the_sequence_across_calls(dev):
    rng = np.random.default_rng(0)
    conf = {"embedding": {"scale": 1.0, "bigram": {"buckets": 11, "mul_prev": 13, "mul_cur": 5}}}
    w = {"embed": np.zeros((40, 6)), "bigram": f32(rng.standard_normal((12, 6)))}
    toks = rng.integers(0, 40, 23).tolist()
    want = R.embed(conf, w, toks)
    table, last = T32(dev, w["bigram"]), zeros(dev, [1], capi.I32)
    got = []
    for a, b in cuts(23, [1, 4, 2, 9]):
        x = zeros(dev, [b - a, 6])
        seqops.pair_hash_rows_add(x, table, toks[a:b], last, 13, 5, 11)
        got.append(x.export().reshape(b - a, 6))
    assert np.array_equal(np.concatenate(got), want.astype(np.float32))
    # a state that is zeroed starts a new sequence: the first token takes the last row again
    seqops.tensor_zero(last)
    x = zeros(dev, [1, 6])
    seqops.pair_hash_rows_add(x, table, [toks[5]], last, 13, 5, 11)
    assert np.array_equal(x.export().reshape(6), w["bigram"][11].astype(np.float32))


def test_norm_with_residual_multiplier_and_bias_ops(dev):
    rng = np.random.default_rng(1)
    x, y, g = f32(rng.standard_normal((5, 20))), f32(rng.standard_normal((5, 20)) * 4), f32(rng.standard_normal(20) * 0.2)
    got = seqops.rms_norm_gain_mult(T32(dev, x), T32(dev, y), T32(dev, 1.0 + g), 1e-5, 0.37).export().reshape(5, 20)
    assert np.abs(got - (x + np.float32(0.37) * R.norm_around_zero(y, g, 1e-5))).max() < 1e-5
    b = f32(rng.standard_normal(20))
    assert np.abs(seqops.add_row_bias(T32(dev, x), T32(dev, b)).export().reshape(5, 20) - (x + b)).max() < 1e-6
    got = seqops.scaled_sum(T32(dev, x), T32(dev, x), 1.2, T32(dev, y), -0.7).export().reshape(5, 20)
    assert np.abs(got - (np.float32(1.2) * x + np.float32(-0.7) * y)).max() < 1e-5
    ff = 7
    src, bias = f32(rng.standard_normal((5, 2 * ff)) * 2), f32(rng.standard_normal(2 * ff))
    got = seqops.glu_halves(T32(dev, src), T32(dev, bias)).export().reshape(5, ff)
    assert np.abs(got - R.silu(src[:, :ff] + bias[:ff]) * (src[:, ff:] + bias[ff:])).max() < 1e-5
    got = seqops.glu_halves(T32(dev, src)).export().reshape(5, ff)
    assert np.abs(got - R.silu(src[:, :ff]) * src[:, ff:]).max() < 1e-5


@pytest.mark.parametrize("heads,hs", [(1, 5), (3, 8), (2, 48), (4, 70)])
def test_head_norm_forms(dev, heads, hs):
    rng = np.random.default_rng(hs)
    x, g = f32(rng.standard_normal((6, heads * hs)) * 3), f32(rng.standard_normal((6, heads * hs)))
    w1, wc = f32(rng.standard_normal(hs)), f32(rng.standard_normal(heads * hs))
    unit = R.unit_rms(x.reshape(6, heads, hs), 1e-5)
    got = seqops.head_rms_norm(T32(dev, x), T32(dev, w1), hs, 1e-5).export().reshape(6, heads, hs)
    assert np.abs(got - unit * w1).max() < 1e-5
    got = seqops.head_rms_norm(T32(dev, x), T32(dev, wc), hs, 1e-5, gate=T32(dev, g), gate_act=capi.ACT_SIGMOID).export().reshape(6, heads * hs)
    assert np.abs(got - unit.reshape(6, -1) * wc * R.sigmoid(g)).max() < 1e-5
    got = seqops.head_rms_norm(T32(dev, x), None, hs, 1e-5).export().reshape(6, heads, hs)
    assert np.abs(got - unit).max() < 1e-5


@pytest.mark.parametrize("cols,groups", [(12, 1), (36, 3), (384, 2), (10, 10)])
def test_gate_before_group_norm(dev, cols, groups):
    rng = np.random.default_rng(cols)
    x, z, w = f32(rng.standard_normal((7, cols)) * 2), f32(rng.standard_normal((7, cols))), f32(rng.standard_normal(cols))
    got = seqops.gated_group_rms_norm(T32(dev, x), T32(dev, z), T32(dev, w), groups, 1e-5).export().reshape(7, cols)
    want = R.unit_rms((x * R.silu(z)).reshape(7, groups, cols // groups), 1e-5).reshape(7, cols) * w
    assert np.abs(got - want).max() < 2e-5


# ---- attention masks ------------------------------------------------------------------------------------------------------------------------
def attention_case(dev, T, H, G, dk, dv, block, window, sink, portions, ring, seed, spikes=()):
    """runs queries / keys / values of T positions through ring caches in `portions` and compares with the reference's softmax mixer.
    spikes: (query position, key position) pairs whose score is made to tower over all others IF the key is visible."""
    rng = np.random.default_rng(seed)
    D = H * dk + G * dk + G * dv
    h = f32(rng.standard_normal((T, D)))
    e = np.zeros(dk); e[0] = 1.0
    for qi, kj in spikes:
        h[qi, :H * dk] = np.tile(6.0 * e, H)
        h[kj, H * dk:H * dk + G * dk] = np.tile(6.0 * e, G)
        h[kj, H * dk + G * dk:] = 50.0 + kj                  # a value that shows when it leaks into a result
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": 0.7}
    if block:
        m["mask"] = {"size": block}
    w = {"a.q": sel(D, 0, H * dk), "a.k": sel(D, H * dk, G * dk), "a.v": sel(D, H * dk + G * dk, G * dv), "a.o": np.eye(H * dv)}
    sk = None
    if sink:
        w["a.sink"] = f32(rng.standard_normal(H) + 1.0)
        sk = T32(dev, w["a.sink"])
    want = R.attention(h, m, w, "a.", 0.0) if not window else None
    kring, vring = zeros(dev, [ring, G * dk]), zeros(dev, [ring, G * dv])
    got = []
    for a, b in portions:
        q, k, v = T32(dev, h[a:b, :H * dk]), T32(dev, h[a:b, H * dk:H * dk + G * dk]), T32(dev, h[a:b, H * dk + G * dk:])
        seqops.kv_ring_append(kring, vring, k, v, None, 0.0, a, G, dk, dv)
        got.append(seqops.masked_attention(q, kring, vring, a, H, G, dk, dv, 0.7, window=window, block=block, sink=sk).export().reshape(b - a, H * dv))
    return np.concatenate(got), want


@pytest.mark.parametrize("sizes", [[300], [1], [2], [64, 1, 1, 3, 17], [5, 90, 2, 2, 31]])
def test_blocks_of_positions_edges_in_prompts_and_decoding(dev, sizes):
    T, block = 300, 32
    # for queries at the start, the middle and the end of a block: the key just inside (the block's first position) and the key just
    # outside (the position before it) tower over everything -- the first must count, the second must not
    spikes = [(64, 64), (65, 64), (95, 64), (96, 95), (127, 96), (128, 127), (131, 127), (200, 191), (200, 192), (31, 0), (32, 31), (299, 288), (299, 287)]
    got, want = attention_case(dev, T, 4, 2, 16, 12, block, 0, True, cuts(T, sizes), block - 1 + max(sizes), 3, spikes)
    assert np.abs(got - want).max() < 2e-4 * np.abs(want).max()


@pytest.mark.parametrize("H,G,dk,dv", [(1, 1, 8, 8), (6, 2, 20, 7), (8, 1, 64, 64), (5, 5, 33, 9), (3, 3, 128, 40)])
def test_causal_far_keys_among_hundreds(dev, H, G, dk, dv):
    T = 700
    spikes = [(699, 3), (698, 0), (650, 255), (651, 256), (400, 17)]
    for sizes in ([700], [667] + [1] * 33, [256, 256, 100, 2, 2]):
        got, want = attention_case(dev, T, H, G, dk, dv, 0, 0, False, cuts(T, sizes), T, 5, spikes)
        assert np.abs(got - want).max() < 2e-4 * np.abs(want).max(), sizes


def test_block_of_one_and_block_larger_than_the_sequence(dev):
    for block in (1, 1000):
        got, want = attention_case(dev, 40, 2, 1, 8, 8, block, 0, True, cuts(40, [7, 1, 2]), (block if block < 40 else 40) - 1 + 7, 9)
        assert np.abs(got - want).max() < 1e-4


def test_window_and_block_together(dev):
    # both limits hold: with window 5 inside blocks of 8, position 14 sees 10..14 and position 17 sees 16..17
    rng = np.random.default_rng(2)
    T, H, dk = 24, 1, 4
    q, k, v = f32(rng.standard_normal((T, dk))), f32(rng.standard_normal((T, dk))), f32(rng.standard_normal((T, dk)))
    kring, vring = zeros(dev, [T, dk]), zeros(dev, [T, dk])
    seqops.kv_ring_append(kring, vring, T32(dev, k), T32(dev, v), None, 0.0, 0, 1, dk, dk)
    got = seqops.masked_attention(T32(dev, q), kring, vring, 0, 1, 1, dk, dk, 1.0, window=5, block=8).export().reshape(T, dk)
    for i in range(T):
        lo = max(i - 4, (i // 8) * 8)
        s = (k[lo:i + 1] @ q[i])
        p = np.exp(s - s.max()); p /= p.sum()
        assert np.abs(got[i] - p @ v[lo:i + 1]).max() < 1e-5, i


# ---- recurrences ----------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,dk,dv,T,sizes", [(2, 40, 56, 90, [90]), (2, 40, 56, 90, [1]), (3, 32, 20, 70, [2, 33, 1]), (1, 64, 64, 50, [17, 2]), (2, 128, 96, 40, [16, 5]),
                                              (4, 10, 7, 45, [3, 40]), (1, 5, 70, 33, [33])])
def test_matrix_memory(dev, H, dk, dv, T, sizes):
    rng = np.random.default_rng(dk + dv)
    cap = 6.0
    D = 2 * H * dk + 2 * H * dv + 2 * H
    h = f32(rng.standard_normal((T, D)))
    at = np.cumsum([0, H * dk, H * dk, H * dv, H * dv, H, H])
    h[:, at[4]:] *= 8.0                                       # gate inputs far beyond the cap on both sides
    m = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    names = ["q", "k", "v", "g", "i", "f"]
    w = {"r." + n: sel(D, at[j], at[j + 1] - at[j]) for j, n in enumerate(names)}
    w.update({"r.i.b": f32(rng.standard_normal(H)), "r.f.b": f32(rng.standard_normal(H) + 2), "r.norm": f32(rng.standard_normal(H * dv)), "r.o": np.eye(H * dv)})
    want = R.matrix_memory(h, m, w, "r.", 1e-5)
    S, ms = zeros(dev, [H, dk, dv + 1]), zeros(dev, [H])
    bi, bf, nw = T32(dev, w["r.i.b"]), T32(dev, w["r.f.b"]), T32(dev, w["r.norm"])
    got = []
    for a, b in cuts(T, sizes):
        p = [T32(dev, h[a:b, at[j]:at[j + 1]]) for j in range(6)]
        o = seqops.matrix_memory(p[0], p[1], p[2], p[4], p[5], bi, bf, cap, dk ** -0.5, S, ms, H, dk, dv)
        got.append(seqops.head_rms_norm(o, nw, dv, 1e-5, gate=p[3], gate_act=capi.ACT_SIGMOID).export().reshape(b - a, H * dv))
    assert np.abs(np.concatenate(got) - want).max() < 3e-4 * max(1.0, np.abs(want).max())


def test_matrix_memory_long_decoding_keeps_its_maximum(dev):
    # 600 single-token calls with input gates that keep growing: without the running maximum the state would overflow
    rng = np.random.default_rng(8)
    H, dk, dv, T, cap = 1, 8, 8, 600, 40.0
    D = 2 * dk + 2 * dv + 2
    h = f32(rng.standard_normal((T, D)))
    h[:, -2] = np.linspace(-30, 39, T)
    at = np.cumsum([0, dk, dk, dv, dv, 1, 1])
    w = {"r." + n: sel(D, at[j], at[j + 1] - at[j]) for j, n in enumerate(["q", "k", "v", "g", "i", "f"])}
    w.update({"r.i.b": np.zeros(1), "r.f.b": np.zeros(1), "r.norm": np.ones(dv), "r.o": np.eye(dv)})
    want = R.matrix_memory(h, {"heads": 1, "dim": dk, "vdim": dv, "gate_cap": cap}, w, "r.", 1e-5)
    S, ms, z1, ones = zeros(dev, [1, dk, dv + 1]), zeros(dev, [1]), T32(dev, [0.0]), T32(dev, np.ones(dv))
    got = []
    for t in range(T):
        p = [T32(dev, h[t:t + 1, at[j]:at[j + 1]]) for j in range(6)]
        o = seqops.matrix_memory(p[0], p[1], p[2], p[4], p[5], z1, z1, cap, dk ** -0.5, S, ms, 1, dk, dv)
        got.append(seqops.head_rms_norm(o, ones, dv, 1e-5, gate=p[3], gate_act=capi.ACT_SIGMOID).export().reshape(1, dv))
    got = np.concatenate(got)
    assert np.isfinite(got).all() and np.abs(got - want).max() < 3e-4


@pytest.mark.parametrize("H,dk,dv,tau,T,sizes", [(2, 32, 48, 8.0, 80, [80]), (2, 32, 48, 8.0, 80, [1]), (3, 12, 9, 2.0, 60, [2, 5, 40]), (1, 64, 32, 1.0, 40, [40]),
                                                  (2, 128, 128, 8.0, 36, [16, 1]), (1, 7, 130, 4.0, 30, [30])])
def test_decayed_linear_attention(dev, H, dk, dv, tau, T, sizes):
    rng = np.random.default_rng(dk * 3 + dv)
    rank = 5
    D = 2 * H * dk + 2 * H * dv + rank
    h = f32(rng.standard_normal((T, D)))
    at = np.cumsum([0, H * dk, H * dk, H * dv, H * dv, rank])
    m = {"heads": H, "dim": dk, "vdim": dv, "tau": tau}
    w = {"r." + n: sel(D, at[j], at[j + 1] - at[j]) for j, n in enumerate(["q", "k", "v", "g", "a1"])}
    w.update({"r.a2": f32(rng.standard_normal((H * dk, rank))), "r.a2.b": f32(rng.standard_normal(H * dk) + 2), "r.norm": f32(rng.standard_normal(dv)), "r.o": np.eye(H * dv)})
    want = R.decayed_linear_attention(h, m, w, "r.", 1e-5)
    z = (h[:, at[4]:at[5]] @ w["r.a2"].T).astype(np.float32)
    S, zb, nw = zeros(dev, [H, dk, dv]), T32(dev, w["r.a2.b"]), T32(dev, w["r.norm"])
    got = []
    for a, b in cuts(T, sizes):
        p = [T32(dev, h[a:b, at[j]:at[j + 1]]) for j in range(4)]
        o = seqops.decayed_linear_attention(p[0], p[1], p[2], T32(dev, z[a:b]), zb, tau, dk ** -0.5, S, H, dk, dv)
        got.append(seqops.head_rms_norm(o, nw, dv, 1e-5, gate=p[3], gate_act=capi.ACT_SILU).export().reshape(b - a, H * dv))
    assert np.abs(np.concatenate(got) - want).max() < 3e-4 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("H,P,N,G,K,ng,T,sizes", [(6, 40, 32, 1, 4, 1, 70, [70]), (6, 40, 32, 1, 4, 1, 70, [1]), (4, 6, 8, 2, 4, 2, 50, [2, 3, 30]), (6, 10, 64, 3, 2, 3, 40, [17, 1]),
                                                   (2, 64, 128, 1, 4, 4, 36, [20, 2]), (3, 5, 7, 3, 1, 1, 30, [4]), (2, 70, 16, 2, 5, 1, 40, [40])])
def test_state_space_mixer(dev, H, P, N, G, K, ng, T, sizes):
    rng = np.random.default_rng(P * 7 + N)
    inner, bc = H * P, 2 * G * N
    D = 2 * inner + bc + H
    h = f32(rng.standard_normal((T, D)))
    m = {"heads": H, "vdim": P, "state": N, "groups": G, "conv": K, "norm_groups": ng}
    w = {"s.in": np.eye(D), "s.conv": f32(rng.standard_normal((inner + bc, K)) * 0.6), "s.conv.b": f32(rng.standard_normal(inner + bc) * 0.3),
         "s.dt_bias": f32(rng.uniform(-3, 1, H)), "s.A_log": f32(rng.uniform(-1, 1.5, H)), "s.D": f32(rng.standard_normal(H)), "s.norm": f32(rng.standard_normal(inner)),
         "s.o": np.eye(inner)}
    want = R.state_space(h, m, w, "s.", 1e-5)
    S = zeros(dev, [H, N, P])
    tail = zeros(dev, [K - 1, inner + bc]) if K > 1 else None
    cw, cb, dtb, al, dsk, nw = (T32(dev, w["s." + n]) for n in ("conv", "conv.b", "dt_bias", "A_log", "D", "norm"))
    got = []
    for a, b in cuts(T, sizes):
        z, xbc, dt = T32(dev, h[a:b, :inner]), T32(dev, h[a:b, inner:2 * inner + bc]), T32(dev, h[a:b, 2 * inner + bc:])
        xc = seqops.short_conv_bias(xbc, cw, cb, tail)
        y = seqops.state_space_scan(xc, dt, dtb, al, dsk, S, H, G, N, P)
        got.append(seqops.gated_group_rms_norm(y, z, nw, ng, 1e-5, dst=y).export().reshape(b - a, inner))
    assert np.abs(np.concatenate(got) - want).max() < 3e-4 * max(1.0, np.abs(want).max())


def test_recurrences_refuse_misshaped_operands(dev):
    q = zeros(dev, [3, 8])
    with pytest.raises(capi.TensorError):
        seqops.decayed_linear_attention(q, q, q, q, zeros(dev, [8]), 2.0, 1.0, zeros(dev, [2, 4, 5]), 2, 4, 4)
    with pytest.raises(capi.TensorError):
        seqops.state_space_scan(zeros(dev, [3, 10]), zeros(dev, [3, 2]), zeros(dev, [2]), zeros(dev, [2]), None, zeros(dev, [2, 2, 3]), 2, 1, 2, 2)
    with pytest.raises(capi.TensorError):
        seqops.masked_attention(zeros(dev, [40, 4]), zeros(dev, [16, 4]), zeros(dev, [16, 4]), 0, 1, 1, 4, 4, 1.0)      # 40 positions, a ring of 16
