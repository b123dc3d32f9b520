"""The Lifesun runner (config -> weights -> slots -> steps) against the plain reference on small random models: whole prompts,
token-by-token decoding, portions of several sizes, interleaved requests, reused slots, ring wrap-around, other sizes, greedy
generation and the trace replay tool."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from crabml_b200 import lifesun, models
from crabml_b200.safetensors import write_safetensors
from tests import lifesun_ref as R
from tests.gpu_common import make_device
from tests.lifesun_common import config, dense, lru_layer, mixed_config, rel_err, retention_layer, run_portions

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


@pytest.fixture(scope="module")
def dev():
    d = make_device()
    yield d
    d.close()


def build(dev, conf, seed, dtype="float32", chunk=0, max_seq=0):
    c = lifesun.parse_config(conf)
    w = lifesun.random_weights(c, seed)
    return c, w, lifesun.LifesunModel(dev, conf, w, dtype, chunk, max_seq)


def check(err, dtype, what):
    if dtype == "float32":
        assert err.max() < TOL[dtype], (what, err.max())
    else:
        assert np.median(err) < TOL[dtype] / 4 and err.max() < 3 * TOL[dtype], (what, err.max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_decode_and_portions_agree_with_the_reference(dev, dtype):
    c, w, m = build(dev, mixed_config(), 11, dtype, chunk=16)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, c["vocab"], 70).tolist()
    want = R.forward(mixed_config(), w, toks)
    for portions in ([70], [1] * 70, [38] + [1] * 32, [2, 3, 35, 2, 17, 1, 1, 9], [2] * 35):
        check(rel_err(run_portions(m, toks, portions), want), dtype, portions)
    assert m.stats()["live"] == 0 and m.stats()["slots"] == 1
    m.close()


def test_residual_stream_after_every_run(dev):
    from crabml_b200 import CudaTensorDevice
    d = CudaTensorDevice(debug_named_tensors=True)
    c, w, m = build(d, mixed_config(), 21)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    res = []
    R.forward(mixed_config(), w, toks, res)
    assert len(res) == 1 + 2 * 2 + 1
    s = m.open(); m.step(s, toks, []); m.close_seq(s)
    for i, want in enumerate(res):
        got = d.dump_debug_tensor(f"run:{i}:0").reshape(len(toks), -1)
        assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max()), i
    m.close(); d.close()


def test_first_tokens_and_single_token_sequence(dev):
    c, w, m = build(dev, mixed_config(), 12)
    for toks in ([5], [5, 9], [0, 0, 0, 0], [52, 0]):
        assert rel_err(run_portions(m, toks, [len(toks)]), R.forward(mixed_config(), w, toks)).max() < TOL["float32"]
        assert rel_err(run_portions(m, toks, [1] * len(toks)), R.forward(mixed_config(), w, toks)).max() < TOL["float32"]
    m.close()


def test_interleaved_requests_equal_each_alone_and_slots_are_reused(dev):
    c, w, m = build(dev, mixed_config(), 13, chunk=8)
    rng = np.random.default_rng(1)
    A, B, Cq = (rng.integers(0, c["vocab"], n).tolist() for n in (41, 17, 29))
    alone = {k: run_portions(m, t, [len(t)]) for k, t in (("A", A), ("B", B), ("C", Cq))}
    sa, sb = m.open(), m.open()
    assert (sa, sb) == (0, 1)
    got = {"A": [], "B": [], "C": []}
    got["A"].append(m.step(sa, A[:20], range(20))); got["B"].append(m.step(sb, B[:3], range(3)))
    got["A"].append(m.step(sa, A[20:21], [0])); got["B"].append(m.step(sb, B[3:], range(14)))
    m.close_seq(sb)
    sc = m.open()                                             # takes B's slot: its rings, states and tails hold B's leftovers
    assert sc == 1
    got["C"].append(m.step(sc, Cq[:2], range(2))); got["A"].append(m.step(sa, A[21:], range(20))); got["C"].append(m.step(sc, Cq[2:], range(27)))
    for k in got:
        assert rel_err(np.concatenate(got[k]), alone[k]).max() < 1e-5, k
    for k, t in (("A", A), ("B", B), ("C", Cq)):
        assert rel_err(np.concatenate(got[k]), R.forward(mixed_config(), w, t)).max() < TOL["float32"]
    m.close_seq(sa); m.close_seq(sc)
    assert m.stats() == {"slots": 2, "live": 0, "state_bytes_per_slot": m.stats()["state_bytes_per_slot"]}
    m.close()


def test_long_decoding_past_every_block_window_and_ring_lap(dev):
    conf = config([lru_layer(block=6), retention_layer(window=11, mlp=None), lru_layer(block=4, heads=2, kv_heads=2, dim=6, vdim=4, conv=2)], loop=(0, 2, 2))
    c, w, m = build(dev, conf, 14, chunk=4)                   # rings of 9, 14 and 7 rows: many laps
    rng = np.random.default_rng(2)
    toks = rng.integers(0, c["vocab"], 150).tolist()
    want = R.forward(conf, w, toks)
    assert rel_err(run_portions(m, toks, [30] + [1] * 120), want).max() < TOL["float32"]
    assert rel_err(run_portions(m, toks, [3, 4, 1, 2] * 15), want).max() < TOL["float32"]
    m.close()


def test_a_layer_without_a_mask_is_causal_and_sized_by_the_token_budget(dev):
    layer = retention_layer()
    del layer["mixer"]["left"]["mask"]
    conf = config([layer])
    c, w, m = build(dev, conf, 18, chunk=8, max_seq=40)
    toks = list(np.random.default_rng(5).integers(0, c["vocab"], 41))
    full = lifesun.parse_config(conf)
    full["layers"][0]["mixer"]["left"]["mask"]["size"] = 1000          # the reference's window, wider than the prompt: every earlier key
    assert rel_err(run_portions(m, toks[:40], [33, 7]), R.forward(full, w, toks[:40])).max() < TOL["float32"]
    s = m.open()
    m.step(s, toks[:40], [])
    with pytest.raises(lifesun.TensorError):
        m.step(s, toks[40:], [0])                             # the 41st token does not fit
    m.close_seq(s)
    m.close()


CONFIGS = {
    "one_of_everything": config([lru_layer(block=3, heads=1, kv_heads=1, dim=5, vdim=3, width=4, blocks=1, conv=1, ls=1.0, rs=1.0, mlp=dense(9)),
                                 retention_layer(window=1, heads=1, kv_heads=1, dim=4, vdim=2, rot=(2, 10.0), r_heads=1, r_dim=2, r_vdim=1, decay=(1.0,), r_rot=(2, 7.0), ls=1.0, rs=1.0)],
                                width=24, vocab=19, logit_scale=1.0),
    "no_loop_no_rotation_no_cap": config([retention_layer(rot=None, softcap=0, r_rot=None), lru_layer(block=20, heads=6, kv_heads=1)], width=40, vocab=33),
    "loop_is_the_whole_stack": config([lru_layer(block=64, width=32, blocks=2), retention_layer(window=16, r_heads=1, r_dim=32, r_vdim=16, decay=(0.75,), r_rot=(32, 1e4))],
                                      width=48, vocab=128, loop=(0, 2, 3)),
    "loop_of_one_layer_at_the_end_run_once_and_four_times": config([retention_layer(mlp=dense(7)), lru_layer(mlp=None)], loop=(1, 2, 4)),
    "single_repetition_still_joins_the_streams": config([lru_layer(), retention_layer()], loop=(0, 1, 1)),
    "block_and_window_longer_than_the_prompt": config([lru_layer(block=500), retention_layer(window=300)]),
    "rotation_of_the_whole_head_and_of_two_columns": config([retention_layer(dim=12, rot=(12, 3e6), r_dim=8, r_rot=(2, 2.0)), retention_layer(dim=10, rot=(2, 30.0), r_rot=(8, 2e5))]),
    "aligned_for_tensor_cores": config([retention_layer(window=20, heads=4, kv_heads=2, dim=32, vdim=32, rot=(16, 1e4), r_heads=2, r_dim=64, r_vdim=64, decay=(0.9, 0.99), r_rot=(64, 1e4),
                                                        mlp=dense(256)),
                                        lru_layer(block=24, heads=8, kv_heads=4, dim=32, vdim=32, width=128, blocks=4, conv=4, mlp=dense(128)),
                                        retention_layer(window=70, heads=2, kv_heads=1, dim=64, vdim=64, rot=(64, 2e5), r_heads=1, r_dim=128, r_vdim=32, decay=(0.97,), r_rot=(32, 1e3)),
                                        lru_layer(block=33, heads=3, kv_heads=1, dim=64, vdim=32, width=64, blocks=1, conv=3)], width=128, vocab=256, loop=(1, 3, 2)),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes_and_layer_orders(dev, name, dtype):
    c, w, m = build(dev, CONFIGS[name], 20, dtype, chunk=64)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, c["vocab"], 90).tolist()
    want = R.forward(CONFIGS[name], w, toks)
    for portions in ([90], [40, 7, 2, 1, 40], [64, 26]):
        check(rel_err(run_portions(m, toks, portions), want), dtype, (name, portions))
    m.close()


def random_config(seed):
    """sizes drawn so that odd widths and head sizes, both layer types in every place, every loop shape and masks on both sides of the
    prompt length all come up over the seeds"""
    rng = np.random.default_rng(3000 + seed)
    width = int(rng.integers(5, 70))
    n_layers = int(rng.integers(1, 5))
    layers = []
    for _ in range(n_layers):
        mlp = dense(int(rng.integers(1, 120))) if rng.random() < 0.6 else None
        g = int(rng.integers(1, 4)); heads = g * int(rng.integers(1, 5)); dim = int(rng.integers(2, 40)); vdim = int(rng.integers(1, 40))
        size = int(rng.choice([1, 2, 7, 33, 64, 65, 300]))
        ls, rs = float(rng.uniform(0.3, 1.5)), float(rng.uniform(0.3, 1.5))
        if rng.random() < 0.5:
            blocks = int(rng.integers(1, 6))
            layers.append(lru_layer(block=size, mlp=mlp, heads=heads, kv_heads=g, dim=dim, vdim=vdim, scale=float(rng.uniform(0.2, 1.5)), width=blocks * int(rng.integers(1, 20)),
                                    blocks=blocks, conv=int(rng.integers(1, 6)), ls=ls, rs=rs))
        else:
            rd = 2 * int(rng.integers(1, dim // 2 + 1))
            rh, rdim = int(rng.integers(1, 4)), int(rng.integers(2, 50))
            layers.append(retention_layer(window=size, mlp=mlp, heads=heads, kv_heads=g, dim=dim, vdim=vdim, scale=float(rng.uniform(0.05, 0.5)),
                                          rot=None if rng.random() < 0.15 else (rd, float(rng.choice([50.0, 1e4, 3e6]))), softcap=float(rng.choice([0.0, 1.0, 15.0])), r_heads=rh,
                                          r_dim=rdim, r_vdim=int(rng.integers(1, 50)), decay=tuple(float(x) for x in rng.choice([0.5, 0.9, 0.9375, 0.998046875, 1.0], rh)),
                                          r_rot=None if rng.random() < 0.15 else (2 * int(rng.integers(1, rdim // 2 + 1)), float(rng.choice([10.0, 1e4, 3e6]))), ls=ls, rs=rs))
    a = int(rng.integers(0, n_layers + 1)); b = int(rng.integers(a, n_layers + 1))
    return config(layers, width=width, vocab=int(rng.integers(2, 200)), eps=float(rng.choice([1e-6, 1e-5, 1e-3])),
                  loop=(a, b, int(rng.integers(1, 4))) if rng.random() < 0.7 else None, logit_scale=float(rng.choice([1.0, 0.5, 0.07])))


@pytest.mark.parametrize("seed", range(30))
def test_random_configurations(dev, seed):
    conf = random_config(seed)
    c, w, m = build(dev, conf, seed, "float32", chunk=int(np.random.default_rng(seed).choice([8, 32, 70])))
    rng = np.random.default_rng(seed)
    toks = rng.integers(0, c["vocab"], 75).tolist()
    want = R.forward(conf, w, toks)
    for portions in ([75], [40] + [1] * 35, [2, 33, 3, 30, 7]):
        err = rel_err(run_portions(m, toks, portions), want)
        assert err.max() < TOL["float32"], (seed, portions, err.max())
    m.close()
    c, w, m = build(dev, conf, seed, "bfloat16", chunk=32)
    err = rel_err(run_portions(m, toks, [37, 1, 37]), want)
    assert np.median(err) < TOL["bfloat16"] / 2 and err.max() < 5 * TOL["bfloat16"], (seed, err.max())
    m.close()


def test_greedy_generation_through_the_runner(dev):
    c, w, m = build(dev, mixed_config(), 15)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    s = m.open()
    ids = m.generate_greedy(s, prompt, 24)
    m.close_seq(s)
    assert len(ids) == 24
    # the same chain through the step interface (what a host-side sampler would do): the LAST maximum, as the device sampler takes
    s = m.open()
    lg = m.step(s, prompt, [len(prompt) - 1])[0]
    chain = []
    for _ in range(24):
        t = int(len(lg) - 1 - np.argmax(lg[::-1]))
        chain.append(t)
        lg = m.step(s, [t], [0])[0]
    m.close_seq(s)
    assert ids == chain
    # and against the reference wherever its own choice is not a close call
    seq = list(prompt)
    for t in ids:
        ref = R.forward(mixed_config(), w, seq)[-1]
        top2 = np.sort(ref)[-2:]
        if top2[1] - top2[0] > 1e-3:
            assert t == int(np.argmax(ref))
        seq.append(t)
    with pytest.raises(lifesun.TensorError):
        m.step(s, [1], [0])                                   # a closed slot is refused
    m.close()


def test_trace_replay_tool(dev, tmp_path):
    c = lifesun.parse_config(mixed_config())
    w = lifesun.random_weights(c, 16)
    mdir = os.path.join(tmp_path, "model"); out = os.path.join(tmp_path, "out")
    os.makedirs(mdir)
    with open(os.path.join(mdir, "config.json"), "w") as f:
        json.dump(mixed_config(), f)
    write_safetensors(os.path.join(mdir, "model.safetensors"), w)
    assert models.architecture_of(mdir) == "Lifesun"
    rng = np.random.default_rng(4)
    a, b = rng.integers(0, c["vocab"], 25).tolist(), rng.integers(0, c["vocab"], 6).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[20:22], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[22:], "want": [2]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [1, 5]}], "end": ["b"]}]
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", mdir, "--dtype", dtype, "--out", out, "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        assert not os.path.exists(os.path.join(out, "1.f32"))
        ra, rb = R.forward(mixed_config(), w, a), R.forward(mixed_config(), w, b)
        for step, want in ((0, ra[[0, 19]]), (2, ra[[24]]), (3, rb[[1, 5]])):
            got = np.fromfile(os.path.join(out, f"{step}.f32"), "<f4").reshape(-1, c["vocab"])
            assert rel_err(got, want).max() < TOL[dtype] * (1 if dtype == "float32" else 3)


def test_loader_refuses_a_model_that_does_not_fit_its_config(dev):
    c = lifesun.parse_config(mixed_config())
    w = lifesun.random_weights(c, 17)
    for name, change in (("l1.mix.right.conv.b", None), ("loop.in", None), ("l0.mix.right.q", lambda a: a[:-1]), ("l1.mix.right.ra", lambda a: a[:, :-1]), ("final.norm.b", lambda a: a[:-1])):
        bad = dict(w)
        if change is None:
            del bad[name]
        else:
            bad[name] = change(bad[name])
        with pytest.raises(lifesun.TensorError):
            lifesun.LifesunModel(dev, c, bad, "float32")
