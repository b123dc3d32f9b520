"""Small Lifesun configurations for the tests.  Sizes differ from layer to layer and avoid values that would make two of them equal by
accident (head counts, head sizes, value sizes, taps, blocks, decays)."""
from tests.meresun_common import rel_err, run_portions  # noqa: F401  (helpers that only drive the runner)


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def lru_layer(block=7, mlp="default", heads=6, kv_heads=2, dim=10, vdim=6, scale=0.6, width=24, blocks=3, conv=4, ls=1.25, rs=0.75):
    """attention without positions in blocks of positions, unit-RMS queries and keys, one more 1 in the denominator, a gate per head; beside
    the gated diagonal recurrence"""
    return {"type": "parallel", "mlp": dense() if mlp == "default" else mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": block}},
                      "right": {"width": width, "blocks": blocks, "conv": conv}, "left_scale": ls, "right_scale": rs}}


def retention_layer(window=5, mlp="default", heads=4, kv_heads=2, dim=12, vdim=8, scale=0.4, rot=(6, 100.0), softcap=3.0, r_heads=3, r_dim=8, r_vdim=10,
                    decay=(0.9, 0.97, 0.6), r_rot=(8, 1000.0), ls=0.85, rs=1.3):
    """windowed attention with whole-projection norms, half-paired rotation and capped scores; beside retention"""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}
    if rot:
        left["rot"] = {"dims": rot[0], "base": rot[1]}
    if softcap:
        left["softcap"] = softcap
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay)[:r_heads]}
    if r_rot:
        right["rot"] = {"dims": r_rot[0], "base": r_rot[1]}
    return {"type": "parallel_2", "mlp": dense(24) if mlp == "default" else mlp, "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}}


def config(layers, width=36, vocab=53, eps=1e-5, loop=None, logit_scale=0.4):
    c = {"architecture": "Lifesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def mixed_config():
    """a retention layer, then a looped pair (diagonal without a feed-forward, retention) that runs twice, then a diagonal layer"""
    return config([retention_layer(), lru_layer(mlp=None), retention_layer(window=9, heads=3, kv_heads=3, dim=8, vdim=12, rot=(8, 50.0), softcap=1.5, r_heads=2, r_dim=6, r_vdim=4,
                                                                           decay=(0.99, 0.8), r_rot=(4, 10.0)),
                   lru_layer(block=11, heads=2, kv_heads=1, dim=14, vdim=10, width=20, blocks=5, conv=2)], loop=(1, 3, 2))
