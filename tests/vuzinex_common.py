"""Small Vuzinex configurations for the tests.  Sizes differ from layer to layer and avoid values that would make two of them equal by
accident (head counts, head sizes, value sizes, taps, groups)."""
from tests.meresun_common import rel_err, run_portions  # noqa: F401  (helpers that only drive the runner)


def bands(dims, base=10000.0, factor=4.0, original=32, low=1.0, high=4.0):
    return {"dims": dims, "base": base, "scaling": {"factor": factor, "original": original, "low": low, "high": high}}


def yarn(dims, base=10000.0, factor=8.0, original=64, fast=16.0, slow=2.0):
    return {"dims": dims, "base": base, "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def left(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.3, rot="default", block=0, window=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": bands(dim) if rot == "default" else rot}
    if block or window:
        m["mask"] = {k: v for k, v in (("size", block), ("window", window)) if v}
    return m


def memory_layer(block=7, mlp="default", left_kw=None, heads=2, dim=12, vdim=10, cap=12.0, ls=1.2, rs=0.8):
    """softmax attention in blocks of positions with a sink, beside the matrix memory"""
    return {"type": "parallel", "mlp": dense() if mlp == "default" else mlp,
            "mixer": {"left": left(block=block, **(left_kw or {})), "right": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "left_scale": ls, "right_scale": rs}}


def decayed_layer(mlp="default", left_kw=None, heads=3, dim=8, vdim=12, tau=8.0, ls=0.9, rs=1.3):
    """causal attention with biases, query / key norms and an output gate, beside the decayed linear attention"""
    kw = dict(heads=6, kv_heads=3, dim=10, vdim=8, rot=yarn(6))
    kw.update(left_kw or {})
    return {"type": "parallel_2", "mlp": dense(24) if mlp == "default" else mlp,
            "mixer": {"left": left(**kw), "right": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "left_scale": ls, "right_scale": rs}}


def space_layer(heads=4, vdim=6, state=8, groups=2, conv=3, norm_groups=2, mlp=None):
    return {"type": "mamba2", "mlp": mlp, "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def config(layers, width=36, vocab=53, eps=1e-5, loop=None, embed_scale=3.0, bigram=(31, 5, 3), mult=0.7, logit_scale=0.4):
    c = {"architecture": "Vuzinex", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps}, "residual_mult": mult,
         "logit_scale": logit_scale, "layers": layers}
    if bigram:
        c["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def mixed_config():
    """a matrix-memory layer, then a looped block (decayed, state space with a feed-forward) that runs twice, then a state-space layer"""
    return config([memory_layer(), decayed_layer(), space_layer(mlp=dense(20)), space_layer(heads=3, vdim=10, state=5, groups=1, conv=4, norm_groups=1)], loop=(1, 3, 2))
