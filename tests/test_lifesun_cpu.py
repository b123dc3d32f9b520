"""Pins the plain Lifesun reference (tests/lifesun_ref.py) with cases small enough to do by hand, and checks the package's host-side parts
(configuration, tensor inventory, frequency table, run order) against it.  No GPU."""
import numpy as np
import pytest

from crabml_b200 import lifesun, rotary
from crabml_b200.capi import TensorError
from tests import lifesun_ref as R
from tests.lifesun_common import config, dense, lru_layer, mixed_config, retention_layer


def test_layer_norm_takes_the_mean_off_and_uses_the_biased_variance():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    w, b = np.array([1.0, 2.0, 1.0, 0.5]), np.array([0.0, 1.0, 0.0, -1.0])
    var = (4.0 + 1.0 + 0.0 + 9.0) / 4.0
    want = (x - 3.0) / np.sqrt(var + 0.5) * w + b
    assert np.allclose(R.layer_norm(x, w, b, 0.5), want)


def test_unit_rms_has_eps_inside_the_root():
    x = np.array([3.0, 4.0])
    assert np.allclose(R.unit_rms(x, 2.5), x / np.sqrt(12.5 + 2.5))


def test_masks_blocks_count_from_position_zero_and_the_window_holds_itself():
    m = R.block_mask(7, 3)
    assert m[2].tolist() == [True, True, True, False, False, False, False]
    assert m[3].tolist() == [False, False, False, True, False, False, False]          # the first position of a block sees itself only
    assert m[5].tolist() == [False, False, False, True, True, True, False]
    w = R.window_mask(6, 3)
    assert w[5].tolist() == [False, False, False, True, True, True]                    # itself and the two before it
    assert w[1].tolist() == [True, True, False, False, False, False]


def test_one_in_the_denominator_counts_once_and_has_no_value():
    q, k, v = np.zeros((1, 1, 2)), np.zeros((1, 1, 2)), np.array([[[6.0, -2.0]]])
    # one key with score 0 beside the extra 1: weight 1/2
    assert np.allclose(R.attention(q, k, v, 1.0, R.block_mask(1, 4), one_in_denominator=True)[0, 0], [3.0, -1.0])
    assert np.allclose(R.attention(q, k, v, 1.0, R.block_mask(1, 4))[0, 0], [6.0, -2.0])
    # a large score drowns it, a very negative one leaves almost nothing
    q2, k2 = np.array([[[10.0, 0.0]]]), np.array([[[3.0, 0.0]]])
    assert np.allclose(R.attention(q2, k2, v, 1.0, R.block_mask(1, 4), one_in_denominator=True)[0, 0], np.array([6.0, -2.0]) / (1 + np.exp(-30.0)))
    assert np.abs(R.attention(q2, -k2, v, 1.0, R.block_mask(1, 4), one_in_denominator=True)[0, 0]).max() < 1e-11


def test_score_cap_comes_after_the_scale():
    q, k = np.array([[[4.0]], [[4.0]]]), np.array([[[1.0]], [[5.0]]])
    v = np.array([[[1.0]], [[0.0]]])
    s = 2.0 * np.tanh(np.array([4.0 * 1.0 * 0.5, 4.0 * 5.0 * 0.5]) / 2.0)
    p = np.exp(s) / np.exp(s).sum()
    assert np.allclose(R.attention(q, k, v, 0.5, R.window_mask(2, 8), softcap=2.0)[1, 0, 0], p[0])


def test_rotation_pairs_column_i_with_i_plus_half_and_leaves_the_rest():
    x = np.arange(1.0, 7.0).reshape(1, 1, 6)           # dims 4 of 6: pairs (0, 2) and (1, 3)
    out = R.rotate_half(x, [3], 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(out[0, 0], [1 * np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1), 3 * np.cos(a0) + 1 * np.sin(a0), 4 * np.cos(a1) + 2 * np.sin(a1), 5.0, 6.0])
    assert np.allclose(R.rotate_half(x, [0], 4, 100.0), x)


def test_frequency_table_of_the_package_is_the_reference_rule():
    for dims, base in ((2, 10.0), (6, 100.0), (64, 3e6), (40, 2e5)):
        f, mag = rotary.table_of({"dims": dims, "base": base})
        assert mag == 1.0 and f.dtype == np.float32 and len(f) == dims // 2
        assert np.allclose(f, float(base) ** (-2.0 * np.arange(dims // 2) / dims), rtol=1e-7)


def test_convolution_sees_zeros_before_the_start_and_its_last_tap_is_the_current_token():
    x = np.array([[1.0], [10.0], [100.0]])
    y = R.causal_conv(x, np.array([[3.0, 2.0, 1.0]]), np.array([0.5]))
    assert np.allclose(y[:, 0], [1.0 + 0.5, 10.0 + 2.0 + 0.5, 100.0 + 20.0 + 3.0 + 0.5])


def test_diagonal_recurrence_by_hand():
    lam = np.array([0.0])
    sp = np.log(2.0)
    u, r, i = np.array([[2.0], [1.0]]), np.array([[0.5], [0.25]]), np.array([[0.5], [1.0]])
    a0, a1 = np.exp(-8 * 0.5 * sp), np.exp(-8 * 0.25 * sp)
    s0 = np.sqrt(1 - a0 ** 2) * 0.5 * 2.0               # the first token is no special case: S = 0 before it
    s1 = a1 * s0 + np.sqrt(1 - a1 ** 2) * 1.0
    assert np.allclose(R.gated_diagonal_recurrence(u, r, i, lam)[:, 0], [s0, s1])


def test_diagonal_gates_are_block_diagonal():
    rng = np.random.default_rng(0)
    conf = config([lru_layer(width=6, blocks=2, conv=1, mlp=None)], width=5)
    W = {k: np.asarray(v, np.float64) for k, v in lifesun.random_weights(conf, 1).items()}
    h = rng.standard_normal((3, 5))
    base = R.right_rglru(h, W, "l0.mix.right.", conf["layers"][0]["mixer"]["right"])
    # the gates of block 1 must not see block 0's inputs: make the off-diagonal blocks explicit and compare
    u = h @ W["l0.mix.right.x"].T + W["l0.mix.right.x.b"]
    u = u * W["l0.mix.right.conv"][:, 0] + W["l0.mix.right.conv.b"]
    full_r, full_i = np.zeros((6, 6)), np.zeros((6, 6))
    for b in range(2):
        full_r[3 * b:3 * b + 3, 3 * b:3 * b + 3] = W["l0.mix.right.ra"][b]
        full_i[3 * b:3 * b + 3, 3 * b:3 * b + 3] = W["l0.mix.right.ri"][b]
    r = R.sigmoid(u @ full_r.T + W["l0.mix.right.ra.b"].reshape(-1))
    i = R.sigmoid(u @ full_i.T + W["l0.mix.right.ri.b"].reshape(-1))
    y = R.gelu_tanh(h @ W["l0.mix.right.y"].T + W["l0.mix.right.y.b"])
    assert np.allclose(base, (R.gated_diagonal_recurrence(u, r, i, W["l0.mix.right.lam"]) * y) @ W["l0.mix.right.o"].T)


def test_retention_by_hand():
    q = np.array([[[1.0, 0.0]], [[1.0, 1.0]]])
    k = np.array([[[2.0, 1.0]], [[0.0, 3.0]]])
    v = np.array([[[5.0]], [[7.0]]])
    out = R.retention(q, k, v, [0.5])
    s0 = np.array([[10.0], [5.0]])
    s1 = 0.5 * s0 + np.array([[0.0], [21.0]])
    assert np.allclose(out[0, 0], [10.0]) and np.allclose(out[1, 0], [s1[0, 0] + s1[1, 0]])


def test_run_order_and_where_the_streams_are_joined():
    conf = config([lru_layer()] * 5, loop=(1, 3, 3))
    assert R.run_order(conf) == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]
    assert R.run_order(config([lru_layer()] * 2)) == [(0, False), (1, False)]
    assert R.run_order(config([lru_layer()] * 2, loop=(0, 2, 1))) == [(0, True), (1, False)]          # a single repetition still joins the streams once


def test_forward_is_causal_and_the_loop_matters():
    conf = mixed_config()
    w = lifesun.random_weights(conf, 3)
    a = [5, 9, 2, 44, 1, 0, 17, 30, 30, 8, 3, 21, 40]
    b = a[:7] + [31] + a[8:]
    la, lb = R.forward(conf, w, a), R.forward(conf, w, b)
    assert np.allclose(la[:7], lb[:7]) and np.abs(la[7:] - lb[7:]).max() > 1e-3
    once = dict(conf, loop={"start": 1, "stop": 3, "times": 1})
    assert np.abs(R.forward(once, w, a) - la).max() > 1e-3
    taps = []
    R.forward(conf, w, a, taps)
    assert len(taps) == 1 + 2 * 2 + 1 and taps[0].shape == (len(a), conf["width"])


def test_config_defaults_and_refusals():
    c = lifesun.parse_config(mixed_config())
    assert c["layers"][0]["mixer"]["left"]["rot"] == {"dims": 6, "base": 100.0} and c["layers"][1]["mlp"] is None and c["loop"]["times"] == 2
    assert lifesun.parse_config(c) == c                  # parsing what was parsed changes nothing
    bare = config([retention_layer(rot=None, softcap=0, r_rot=None)])
    del bare["logit_scale"]
    p = lifesun.parse_config(bare)
    assert p["logit_scale"] == 1.0 and p["loop"] is None and p["layers"][0]["mixer"]["left"]["rot"] is None and p["layers"][0]["mixer"]["left"]["softcap"] == 0.0
    for bad in (config([lru_layer(heads=5, kv_heads=2)]), config([lru_layer(width=10, blocks=3)]), config([retention_layer(decay=(0.5,), r_heads=2)]),
                config([retention_layer(rot=(5, 10.0))]), config([retention_layer(rot=(14, 10.0))]), config([lru_layer()], loop=(0, 2, 1)),
                config([dict(lru_layer(), type="mamba2")]), config([dict(lru_layer(), mlp={"kind": "moe"})]), dict(mixed_config(), architecture="Other")):
        with pytest.raises(TensorError):
            lifesun.parse_config(bad)


def test_tensor_inventory():
    c = lifesun.parse_config(mixed_config())
    t = lifesun.expected_tensors(c)
    assert t["loop.in"] == [36, 72] and t["l1.mix.left.g"] == [6, 36] and t["l1.mix.right.ra"] == [3, 8, 8] and t["l1.mix.right.ri.b"] == [3, 8]
    assert t["l0.mix.left.q.norm"] == [48] and t["l0.mix.left.k.norm"] == [24] and t["l0.mix.right.g"] == [30, 36] and t["l3.mix.right.conv"] == [20, 2]
    assert "l1.mlp.gate" not in t and t["l0.mlp.down"] == [36, 24] and t["final.norm.b"] == [36] and t["head"] == [53, 36]
    assert "loop.in" not in lifesun.expected_tensors(lifesun.parse_config(config([lru_layer()])))
    w = lifesun.random_weights(mixed_config(), 0)
    assert sorted(w) == sorted(t) and all(list(w[n].shape) == t[n] for n in t)
