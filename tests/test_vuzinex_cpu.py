"""CPU tests of the Vuzinex family: the plain reference (tests/vuzinex_ref.py) pinned on cases worked out by hand, and the package's
host-side parts (configuration, tensor lists, frequency tables) against it."""
import math

import numpy as np
import pytest

from crabml_b200 import rotary, vuzinex
from crabml_b200.capi import TensorError
from tests import vuzinex_ref as R
from tests.vuzinex_common import bands, config, decayed_layer, memory_layer, mixed_config, space_layer, yarn


def test_ref_pair_hash_rows_and_the_first_token():
    conf = config([space_layer()], bigram=(7, 5, 3), embed_scale=2.0)
    w = {"embed": np.arange(53 * 36, dtype=np.float64).reshape(53, 36), "bigram": 1000.0 * np.arange(8)[:, None] + np.zeros((8, 36))}
    x = R.embed(conf, w, [4, 9, 9])
    # first token: the last row (7); then (4 * 5 + 9 * 3) % 7 = 5 and (9 * 5 + 9 * 3) % 7 = 2
    assert np.allclose(x[:, 0], [2 * 4 * 36 + 7000, 2 * 9 * 36 + 5000, 2 * 9 * 36 + 2000])


def test_ref_norm_weight_is_an_offset_from_one():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(R.norm_around_zero(x, np.array([0.0, 1.0]), 0.0), [[3 / math.sqrt(12.5), 2 * 4 / math.sqrt(12.5)]])


def test_ref_rotation_pairs_neighbours_and_leaves_the_rest():
    x = np.array([[[1.0, 0.0, 0.0, 1.0, 5.0, 6.0]], [[1.0, 0.0, 0.0, 1.0, 5.0, 6.0]]])
    out = R.rotate(x, {"dims": 4, "base": 100.0})
    assert np.allclose(out[0], x[0])
    f = [1.0, 100.0 ** -0.5]
    assert np.allclose(out[1, 0], [math.cos(f[0]), math.sin(f[0]), -math.sin(f[1]), math.cos(f[1]), 5.0, 6.0])


def test_frequency_tables_of_the_package_agree_with_the_reference():
    for rot in (bands(8), bands(16, base=1e6, factor=8.0, original=64, low=1.0, high=4.0), bands(64, base=5e5, factor=32.0, original=8192), yarn(6), yarn(32, original=16),
                {"dims": 10, "base": 77.0}):
        f, mag = rotary.table_of(rot)
        rf, rmag = R.rot_frequencies(rot)
        assert np.allclose(f, rf, rtol=1e-6, atol=0) and abs(mag - rmag) < 1e-12
    # the three bands all occur: an untouched pair, a slowed-down pair, a blended pair
    f, _ = R.rot_frequencies(bands(16, base=1e4, factor=8.0, original=64))
    plain = 1e4 ** (-np.arange(8) / 8.0)
    ratio = f / plain
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8.0) < 1e-12 and ((ratio > 1 / 8.0 + 1e-9) & (ratio < 1.0 - 1e-9)).any()


def _sel(total, start, n):
    m = np.zeros((n, total))
    m[np.arange(n), start + np.arange(n)] = 1.0
    return m


def test_ref_blocks_count_from_position_zero_and_the_sink_counts_once_unscaled():
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 123.0, "mask": {"size": 2}}
    w = {"a.q": np.zeros((2, 4)), "a.k": _sel(4, 0, 2), "a.v": _sel(4, 2, 2), "a.o": np.eye(2)}
    h = np.array([[0, 0, 1.0, 0], [0, 0, 0, 1.0], [0, 0, 2.0, 2.0], [0, 0, 4.0, 0]])
    # queries are zero: every visible key scores 0, so a result is the mean of the visible values.  Blocks: {0, 1}, {2, 3}
    out = R.attention(h, m, w, "a.", 0.0)
    assert np.allclose(out, [[1, 0], [0.5, 0.5], [2, 2], [3, 1]])
    w["a.sink"] = np.array([0.0])                         # exp(0) = 1 joins the denominator whatever the scale is
    out = R.attention(h, m, w, "a.", 0.0)
    assert np.allclose(out, [[0.5, 0], [1 / 3, 1 / 3], [1, 1], [2, 2 / 3]])


def test_ref_matrix_memory_first_steps_by_hand():
    # one head, dk = dv = 1, cap large enough not to matter: i = gi, f = logsigmoid(gf)
    m = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 1e6}
    D = 6
    w = {"r.q": _sel(D, 0, 1), "r.k": _sel(D, 1, 1), "r.v": _sel(D, 2, 1), "r.i": _sel(D, 3, 1), "r.f": _sel(D, 4, 1), "r.g": _sel(D, 5, 1), "r.i.b": np.zeros(1), "r.f.b": np.zeros(1),
         "r.norm": np.ones(1), "r.o": np.eye(1)}
    # token 0: i = -3, f = logsigmoid(0) = -ln 2: the maximum starts at 0, so m = max(-ln 2 + 0, -3) = -ln 2 (not -3)
    h = np.array([[2.0, 1.0, 5.0, -3.0, 0.0, 50.0]])
    top = -math.log(2.0)
    S = math.exp(-3.0 - top) * 1.0 * 5.0
    n = math.exp(-3.0 - top) * 1.0
    want = (S * 2.0) / (max(abs(n * 2.0), math.exp(-top)) + 1e-6)
    got_raw = want / math.sqrt(want * want + 1e-5)          # the per-head unit RMS of a single number
    out = R.matrix_memory(h, m, w, "r.", 1e-5)
    assert np.allclose(out, [[got_raw]])


def test_ref_decay_acts_on_key_channels_and_state_space_by_hand():
    m = {"heads": 1, "dim": 2, "vdim": 1, "tau": 2.0}
    D = 8
    w = {"r.q": _sel(D, 0, 2), "r.k": _sel(D, 2, 2), "r.v": _sel(D, 4, 1), "r.g": _sel(D, 5, 1), "r.a1": _sel(D, 6, 2), "r.a2": np.eye(2), "r.a2.b": np.array([0.0, math.log(3.0)]),
         "r.norm": np.ones(1), "r.o": np.eye(1)}
    # decays: sigmoid(0)^(1/2) = sqrt(1/2) on key channel 0, sigmoid(ln 3)^(1/2) = sqrt(3/4) on channel 1
    h = np.array([[0, 0, 1.0, 1.0, 2.0, 50.0, 0, 0], [1.0, 1.0, 0, 0, 0, 50.0, 0, 0]])
    S1 = np.array([2.0, 2.0]) * np.array([math.sqrt(0.5), math.sqrt(0.75)])
    o = (S1 @ np.array([1.0, 1.0])) * 2 ** -0.5
    out = R.decayed_linear_attention(h, m, w, "r.", 1e-30)
    assert np.allclose(out[1], o / abs(o) * R.silu(50.0))
    # state space: one head, N = 1, P = 1, one tap: y_0 = dt B x C + D x with dt = softplus(dt_raw + bias)
    ms = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    ws = {"s.in": np.eye(5), "s.conv": np.ones((3, 1)), "s.conv.b": np.zeros(3), "s.dt_bias": np.array([0.5]), "s.A_log": np.array([0.0]), "s.D": np.array([2.0]),
          "s.norm": np.ones(1), "s.o": np.eye(1)}
    hs = np.array([[50.0, 1.0, 2.0, 3.0, 0.25]])
    x, B, Cc = R.silu(1.0), R.silu(2.0), R.silu(3.0)
    y = R.softplus(0.75) * B * x * Cc + 2.0 * x
    y = y * R.silu(50.0)
    assert np.allclose(R.state_space(hs, ms, ws, "s.", 0.0), [[y / abs(y)]])


def test_ref_layer_runs_follow_the_loop():
    assert R.layer_runs(config([space_layer()] * 5, loop=(2, 4, 3))) == [0, 1, 2, 3, 2, 3, 2, 3, 4]
    assert R.layer_runs(config([space_layer()] * 2)) == [0, 1]
    assert R.layer_runs(config([space_layer()] * 2, loop=(0, 2, 2))) == [0, 1, 0, 1]


def test_config_is_validated_and_the_tensor_list_fits_the_reference():
    c = vuzinex.parse_config(mixed_config())
    assert [L["type"] for L in c["layers"]] == ["parallel", "parallel_2", "mamba2", "mamba2"]
    assert c["layers"][0]["mixer"]["right"]["kind"] == "matrix_memory" and c["layers"][1]["mixer"]["right"]["kind"] == "decayed"
    assert c["layers"][0]["mixer"]["left"]["mask"] == {"size": 7, "window": 0} and c["layers"][1]["mixer"]["left"]["mask"] == {"size": 0, "window": 0}
    w = vuzinex.random_weights(c, 1)
    # every tensor the reference touches exists, with the shape it needs: a forward pass runs
    lg = R.forward(mixed_config(), w, [1, 2, 3, 4, 5, 6, 7, 8, 9])
    assert lg.shape == (9, 53) and np.isfinite(lg).all()
    for bad in (dict(mixed_config(), architecture="Other"), config([dict(space_layer(), type="conv")]), config([space_layer()], loop=(0, 3, 2)),
                config([memory_layer(left_kw=dict(heads=3, kv_heads=2))]), config([space_layer(heads=3, groups=2)])):
        with pytest.raises(TensorError):
            vuzinex.parse_config(bad)
    broken = mixed_config()
    del broken["layers"][0]["mixer"]["right"]["gate_cap"]
    with pytest.raises(TensorError):
        vuzinex.parse_config(broken)


def test_reference_does_not_depend_on_later_tokens():
    conf = mixed_config()
    w = vuzinex.random_weights(vuzinex.parse_config(conf), 5)
    toks = list(np.random.default_rng(0).integers(0, 53, 30))
    a, b = R.forward(conf, w, toks), R.forward(conf, w, toks[:17])
    assert np.abs(a[:17] - b).max() < 1e-9
