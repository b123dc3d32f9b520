"""The Vuzinex runner (config -> weights -> slots -> steps) against the plain reference on small random models: whole prompts,
token-by-token decoding, portions of several sizes, interleaved requests, reused slots, ring wrap-around, other sizes, greedy
generation and the trace replay tool."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from crabml_b200 import models, vuzinex
from crabml_b200.safetensors import write_safetensors
from tests import vuzinex_ref as R
from tests.gpu_common import make_device
from tests.vuzinex_common import bands, config, decayed_layer, dense, memory_layer, mixed_config, rel_err, run_portions, space_layer, yarn

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


@pytest.fixture(scope="module")
def dev():
    d = make_device()
    yield d
    d.close()


def build(dev, conf, seed, dtype="float32", chunk=0, extras=None, max_seq=0):
    c = vuzinex.parse_config(conf)
    w = vuzinex.random_weights(c, seed, extras=extras)
    return c, w, vuzinex.VuzinexModel(dev, conf, w, dtype, chunk, max_seq)


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
    sc = m.open()                                             # takes B's slot: its rings, states, tails and last token hold B's leftovers
    assert sc == 1
    got["C"].append(m.step(sc, Cq[:2], range(2))); got["A"].append(m.step(sa, A[21:], range(20))); got["C"].append(m.step(sc, Cq[2:], range(27)))
    for k in got:
        assert rel_err(np.concatenate(got[k]), alone[k]).max() < 1e-5, k
    for k, t in (("A", A), ("B", B), ("C", Cq)):
        assert rel_err(np.concatenate(got[k]), R.forward(mixed_config(), w, t)).max() < TOL["float32"]
    m.close_seq(sa); m.close_seq(sc)
    assert m.stats() == {"slots": 2, "live": 0, "state_bytes_per_slot": m.stats()["state_bytes_per_slot"]}
    m.close()


def test_long_decoding_past_every_block_and_ring_lap(dev):
    conf = config([memory_layer(block=6), memory_layer(block=11, mlp=None, left_kw=dict(heads=2, kv_heads=2, dim=6, vdim=4)), space_layer()], loop=(0, 2, 2))
    c, w, m = build(dev, conf, 14, chunk=4)                   # rings of 9 and 14 rows: many laps
    rng = np.random.default_rng(2)
    toks = rng.integers(0, c["vocab"], 150).tolist()
    want = R.forward(conf, w, toks)
    assert rel_err(run_portions(m, toks, [30] + [1] * 120), want).max() < TOL["float32"]
    assert rel_err(run_portions(m, toks, [3, 4, 1, 2] * 15), want).max() < TOL["float32"]
    m.close()


def test_causal_cache_is_sized_by_the_token_budget(dev):
    conf = config([decayed_layer()])
    c, w, m = build(dev, conf, 18, chunk=8, max_seq=40)
    toks = list(np.random.default_rng(5).integers(0, c["vocab"], 41))
    assert rel_err(run_portions(m, toks[:40], [33, 7]), R.forward(conf, w, toks[:40])).max() < TOL["float32"]
    s = m.open()
    m.step(s, toks[:40], [])
    with pytest.raises(vuzinex.TensorError):
        m.step(s, toks[40:], [0])                             # the 41st token does not fit
    m.close_seq(s)
    m.close()


CONFIGS = {
    "state_space_first_one_group_of_everything": config([space_layer(heads=1, vdim=16, state=4, groups=1, conv=2, norm_groups=1, mlp=dense(9)), memory_layer(block=3)],
                                                        width=24, vocab=19, bigram=(2, 1, 1), mult=1.0, logit_scale=1.0),
    "no_pair_table_plain_rotation_no_loop": config([decayed_layer(left_kw=dict(rot={"dims": 4, "base": 50.0})), memory_layer(left_kw=dict(rot=None, heads=6, kv_heads=1), block=20)],
                                                   width=40, vocab=33, bigram=None),
    "loop_is_the_whole_stack": config([memory_layer(block=64, heads=1, dim=32, vdim=16), space_layer(state=16, conv=5)], width=48, vocab=128, loop=(0, 2, 3)),
    "loop_of_one_layer_at_the_end": config([space_layer(mlp=dense(7)), decayed_layer(mlp=None, tau=1.0)], loop=(1, 2, 4), embed_scale=1.0),
    "block_longer_than_the_prompt_and_a_window": config([memory_layer(block=500, cap=2.0), decayed_layer(left_kw=dict(window=9))], mult=0.25),
    "rotation_of_part_of_a_head_bands_on_the_causal_side": config([decayed_layer(left_kw=dict(dim=12, rot=bands(8, original=16))), memory_layer(left_kw=dict(dim=10, rot=yarn(4)))]),
    "aligned_for_tensor_cores": config([memory_layer(block=20, left_kw=dict(heads=4, kv_heads=2, dim=32, vdim=32), heads=2, dim=64, vdim=64, mlp=dense(256)),
                                        decayed_layer(left_kw=dict(heads=8, kv_heads=4, dim=32, vdim=32, rot=yarn(32)), heads=2, dim=32, vdim=64, mlp=dense(128)),
                                        space_layer(heads=8, vdim=32, state=64, groups=1, conv=4, norm_groups=1), space_layer(heads=4, vdim=64, state=128, groups=2, norm_groups=4)],
                                       width=128, vocab=256, loop=(1, 3, 2)),
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
    """sizes drawn so that odd widths and head sizes, every layer type in every place, every loop shape and blocks on both sides of the
    prompt length all come up over the seeds"""
    rng = np.random.default_rng(2000 + seed)
    width = int(rng.integers(5, 70))
    n_layers = int(rng.integers(1, 5))
    layers = []
    for _ in range(n_layers):
        kind = rng.choice(["memory", "decayed", "space"])
        mlp = dense(int(rng.integers(1, 120))) if rng.random() < 0.6 else None
        g = int(rng.integers(1, 4)); dim = int(rng.integers(2, 40))
        rd = 2 * int(rng.integers(1, dim // 2 + 1))
        rot = None if rng.random() < 0.15 else {"dims": rd, "base": float(rng.choice([50.0, 1e4, 1e6]))}
        if rot and rng.random() < 0.7:
            rot = bands(rd, base=rot["base"], original=int(rng.choice([8, 32, 256]))) if rng.random() < 0.5 else yarn(rd, base=rot["base"], original=int(rng.choice([8, 64])))
        lk = dict(heads=g * int(rng.integers(1, 5)), kv_heads=g, dim=dim, vdim=int(rng.integers(1, 40)), scale=float(rng.uniform(0.05, 0.5)), rot=rot)
        if kind == "memory":
            layers.append(memory_layer(block=int(rng.choice([1, 2, 7, 33, 64, 65, 300])), mlp=mlp, left_kw=lk, heads=int(rng.integers(1, 4)), dim=int(rng.integers(1, 50)),
                                       vdim=int(rng.integers(1, 50)), cap=float(rng.choice([1.0, 12.0, 30.0])), ls=float(rng.uniform(0.3, 1.5)), rs=float(rng.uniform(0.3, 1.5))))
        elif kind == "decayed":
            layers.append(decayed_layer(mlp=mlp, left_kw=lk, heads=int(rng.integers(1, 4)), dim=int(rng.integers(1, 50)), vdim=int(rng.integers(1, 50)),
                                        tau=float(rng.choice([1.0, 4.0, 32.0])), ls=float(rng.uniform(0.3, 1.5)), rs=float(rng.uniform(0.3, 1.5))))
        else:
            sg = int(rng.integers(1, 4)); heads = sg * int(rng.integers(1, 4)); vd = int(rng.integers(1, 30))
            ng = int(rng.choice([d for d in (1, 2, 3, 4) if (heads * vd) % d == 0]))
            layers.append(space_layer(heads=heads, vdim=vd, state=int(rng.integers(1, 40)), groups=sg, conv=int(rng.integers(1, 6)), norm_groups=ng, mlp=mlp))
    a = int(rng.integers(0, n_layers + 1)); b = int(rng.integers(a, n_layers + 1))
    return config(layers, width=width, vocab=int(rng.integers(2, 200)), eps=float(rng.choice([1e-6, 1e-5, 1e-3])),
                  loop=(a, b, int(rng.integers(1, 4))) if rng.random() < 0.7 else None, embed_scale=float(rng.choice([1.0, 0.5, 8.0])),
                  bigram=(int(rng.integers(1, 300)), int(rng.integers(0, 200)), int(rng.integers(0, 200))) if rng.random() < 0.85 else None,
                  mult=float(rng.choice([1.0, 0.5, 0.3])), logit_scale=float(rng.choice([1.0, 0.5, 0.07])))


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


def test_optional_parts_of_the_left_mixer_follow_the_tensors(dev):
    # a block-masked layer WITH biases, norms and a gate but no sink; a causal one with a sink only
    conf = config([memory_layer(), decayed_layer()])
    extras = {0: ("bias", "qk_norm", "gate"), 1: ("sink",)}
    c, w, m = build(dev, conf, 22, extras=extras)
    assert "l0.mix.left.g" in w and "l0.mix.left.sink" not in w and "l1.mix.left.sink" in w and "l1.mix.left.q.b" not in w
    toks = list(range(30))
    assert rel_err(run_portions(m, toks, [13, 17]), R.forward(conf, w, toks)).max() < TOL["float32"]
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
    with pytest.raises(vuzinex.TensorError):
        m.step(s, [1], [0])                                   # a closed slot is refused
    m.close()


def test_trace_replay_tool(dev, tmp_path):
    c = vuzinex.parse_config(mixed_config())
    w = vuzinex.random_weights(c, 16)
    mdir = os.path.join(tmp_path, "model"); out = os.path.join(tmp_path, "out")
    os.makedirs(mdir)
    with open(os.path.join(mdir, "config.json"), "w") as f:
        json.dump(mixed_config(), f)
    write_safetensors(os.path.join(mdir, "model.safetensors"), w)
    assert models.architecture_of(mdir) == "Vuzinex"
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
    c = vuzinex.parse_config(mixed_config())
    w = vuzinex.random_weights(c, 17)
    bad = dict(w); del bad["l2.mix.conv.b"]
    with pytest.raises(vuzinex.TensorError):
        vuzinex.VuzinexModel(dev, c, bad, "float32")
    bad = dict(w); bad["l0.mix.right.q"] = bad["l0.mix.right.q"][:-1]
    with pytest.raises(vuzinex.TensorError):
        vuzinex.VuzinexModel(dev, c, bad, "float32")
    bad = dict(w); bad["bigram"] = bad["bigram"][:-1]
    with pytest.raises(vuzinex.TensorError):
        vuzinex.VuzinexModel(dev, c, bad, "float32")
    bad = dict(w); del bad["l1.mix.right.a1"]
    with pytest.raises(vuzinex.TensorError):
        vuzinex.VuzinexModel(dev, c, bad, "float32")
