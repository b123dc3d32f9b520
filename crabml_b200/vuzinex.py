"""The Vuzinex decoder family: configuration, weight loading and the Python handle on its C++ runner
(crabml_b200/csrc/host/vuzinex_runner.cpp; the stack is described in include/crabml_vuzinex.h).

A model folder holds config.json and model.safetensors.  config.json gives every size and every constant that can differ between
models of the family: `vocab`, `width`, `embedding` (`scale`, `bigram`: `buckets`, `mul_prev`, `mul_cur`), `norm.eps`, `residual_mult`,
`logit_scale`, `loop` (`start`, `stop`, `times`) and `layers`, a list whose entries name the layer's mixer (`type`: "parallel",
"parallel_2" or "mamba2"), the mixer's sizes (`mixer`) and its feed-forward (`mlp`: kind "dense", or null).  A parallel mixer has a
`left` (softmax attention: `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `rot`, `mask`) and a `right` (`heads`, `dim`, `vdim` and
`gate_cap` for the matrix memory or `tau` for the decayed linear attention) with `left_scale` / `right_scale`.  Tensor names: `embed`,
`bigram`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`.

What a left mixer has beyond its projections is read from the tensors the file holds: biases (`.q.b`, `.k.b`, `.v.b`), query / key norms
(`.q.norm`, `.k.norm`), a sink (`.sink`), an output gate (`.g`).  The mask is `mask.size` (blocks of positions) or `mask.window` (a
sliding window) or none (causal).

Precision: `dtype="bfloat16"` keeps the matrices of the dense products in bfloat16 (activations are rounded to bfloat16 at the input
of a product, sums are 32-bit); `dtype="float32"` widens them and every product is a true 32-bit one.  In both modes the residual
stream, norms, rotations, attention scores and sums, gates, decays, step sizes and all recurrent state are 32-bit.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np

from . import capi, rotary
from .capi import CudaError, TensorError
from .safetensors import bf16_to_f32, f32_to_bf16, read_safetensors
from .seqmodel import SeqModel, Uploader, handle_of
from .tensor import CudaTensorDevice

ARCHITECTURE = "Vuzinex"
PAIR_TYPES = ("parallel", "parallel_2")


# ---- configuration ----------------------------------------------------------------------------------------------------------------
def _rot(r, dim, at):
    if not r or int(r.get("dims", 0)) <= 0:
        return None
    sc = r.get("scaling")
    out = {"dims": int(r["dims"]), "base": float(r["base"]), "scaling": {k: float(v) for k, v in sc.items()} if sc else None}
    if out["dims"] > dim or out["dims"] % 2:
        raise TensorError(f"{at}: rot.dims must be even and at most the head size")
    return out


def parse_config(conf: dict) -> dict:
    """Validates a config.json dict and fills the optional keys, so that the rest of the code reads one shape of dict."""
    if conf.get("architecture", ARCHITECTURE) != ARCHITECTURE:
        raise TensorError(f"not a {ARCHITECTURE} config: architecture = {conf.get('architecture')!r}")
    emb = conf.get("embedding") or {}
    big = emb.get("bigram")
    out = {"architecture": ARCHITECTURE, "vocab": int(conf["vocab"]), "width": int(conf["width"]),
           "embedding": {"scale": float(emb.get("scale", 1.0)),
                         "bigram": {k: int(big[k]) for k in ("buckets", "mul_prev", "mul_cur")} if big else None},
           "norm": {"eps": float(conf["norm"]["eps"])}, "residual_mult": float(conf.get("residual_mult", 1.0)),
           "logit_scale": float(conf.get("logit_scale", 1.0)), "layers": []}
    n = len(conf["layers"])
    lp = conf.get("loop")
    out["loop"] = {"start": int(lp["start"]), "stop": int(lp["stop"]), "times": int(lp["times"])} if lp else {"start": 0, "stop": 0, "times": 1}
    if not (0 <= out["loop"]["start"] <= out["loop"]["stop"] <= n) or out["loop"]["times"] < 1:
        raise TensorError(f"loop {out['loop']} does not fit {n} layers")
    for i, L in enumerate(conf["layers"]):
        at, m = f"layer {i}", L["mixer"]
        if L["type"] in PAIR_TYPES:
            a, b = m["left"], m["right"]
            left = {k: int(a[k]) for k in ("heads", "kv_heads", "dim", "vdim")}
            left["scale"] = float(a["scale"])
            left["rot"] = _rot(a.get("rot"), left["dim"], at)
            mask = a.get("mask") or {}
            left["mask"] = {"size": int(mask.get("size", 0)), "window": int(mask.get("window", 0))}
            if left["heads"] % left["kv_heads"]:
                raise TensorError(f"{at}: kv_heads does not divide heads")
            right = {k: int(b[k]) for k in ("heads", "dim", "vdim")}
            if "gate_cap" in b:
                right["kind"], right["gate_cap"] = "matrix_memory", float(b["gate_cap"])
            elif "tau" in b:
                right["kind"], right["tau"] = "decayed", float(b["tau"])
            else:
                raise TensorError(f"{at}: the right mixer has neither gate_cap nor tau")
            mixer = {"left": left, "right": right, "left_scale": float(m.get("left_scale", 1.0)), "right_scale": float(m.get("right_scale", 1.0))}
        elif L["type"] == "mamba2":
            mixer = {k: int(m[k]) for k in ("heads", "vdim", "state", "conv")}
            mixer["groups"], mixer["norm_groups"] = int(m.get("groups", 1)), int(m.get("norm_groups", 1))
            if mixer["heads"] % mixer["groups"] or (mixer["heads"] * mixer["vdim"]) % mixer["norm_groups"]:
                raise TensorError(f"{at}: groups / norm_groups do not divide the heads / the inner width")
        else:
            raise TensorError(f"{at}: unknown mixer type {L['type']!r}")
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise TensorError(f"{at}: unknown feed-forward kind {mlp.get('kind')!r}")
            mlp = {"kind": "dense", "ff": int(mlp["ff"])}
        out["layers"].append({"type": L["type"], "mixer": mixer, "mlp": mlp})
    return out


# what a layer type's left mixer has when nothing else is said (random_weights, tests); a file's own tensors decide for a loaded model
LEFT_EXTRAS = {"parallel": ("sink",), "parallel_2": ("bias", "qk_norm", "gate")}


def expected_tensors(conf: dict, extras=None) -> dict:
    """name -> shape of every tensor a model of this config has.  extras: per layer index the left mixer's optional parts (a subset of
    "bias", "qk_norm", "sink", "gate"); default by layer type."""
    D, V = conf["width"], conf["vocab"]
    t = {"embed": [V, D], "final.norm": [D]}
    if conf["embedding"]["bigram"]:
        t["bigram"] = [conf["embedding"]["bigram"]["buckets"] + 1, D]
    for i, L in enumerate(conf["layers"]):
        m, p = L["mixer"], f"l{i}."
        t.update({p + "norm1": [D], p + "norm1b": [D]})
        if L["type"] in PAIR_TYPES:
            a, b = m["left"], m["right"]
            ex = (extras or {}).get(i, LEFT_EXTRAS[L["type"]])
            q = p + "mix.left."
            t.update({q + "q": [a["heads"] * a["dim"], D], q + "k": [a["kv_heads"] * a["dim"], D], q + "v": [a["kv_heads"] * a["vdim"], D],
                      q + "o": [D, a["heads"] * a["vdim"]]})
            if "bias" in ex:
                t.update({q + "q.b": [a["heads"] * a["dim"]], q + "k.b": [a["kv_heads"] * a["dim"]], q + "v.b": [a["kv_heads"] * a["vdim"]]})
            if "qk_norm" in ex:
                t.update({q + "q.norm": [a["dim"]], q + "k.norm": [a["dim"]]})
            if "sink" in ex:
                t[q + "sink"] = [a["heads"]]
            if "gate" in ex:
                t[q + "g"] = [a["heads"] * a["vdim"], D]
            r = p + "mix.right."
            qk, hv = b["heads"] * b["dim"], b["heads"] * b["vdim"]
            t.update({r + "q": [qk, D], r + "k": [qk, D], r + "v": [hv, D], r + "g": [hv, D], r + "o": [D, hv]})
            if b["kind"] == "matrix_memory":
                t.update({r + "norm": [hv], r + "i": [b["heads"], D], r + "i.b": [b["heads"]], r + "f": [b["heads"], D], r + "f.b": [b["heads"]]})
            else:
                t[r + "norm"] = [b["vdim"]]
        else:
            inner, bc = m["heads"] * m["vdim"], 2 * m["groups"] * m["state"]
            q = p + "mix."
            t.update({q + "in": [2 * inner + bc + m["heads"], D], q + "conv": [inner + bc, m["conv"]], q + "conv.b": [inner + bc], q + "dt_bias": [m["heads"]],
                      q + "A_log": [m["heads"]], q + "D": [m["heads"]], q + "norm": [inner], q + "o": [D, inner]})
        if L["mlp"]:
            ff = L["mlp"]["ff"]
            t.update({p + "norm2": [D], p + "norm2b": [D], p + "mlp.gate": [ff, D], p + "mlp.gate.b": [ff], p + "mlp.up": [ff, D], p + "mlp.up.b": [ff],
                      p + "mlp.down": [D, ff], p + "mlp.down.b": [D]})
    return t


def _decay_rank(conf, weights, i):
    """the inner width of the decay's two projections is a tensor's shape, not a config key"""
    return int(np.shape(weights[f"l{i}.mix.right.a1"])[0])


def random_weights(conf: dict, seed: int = 0, scale: float = 1.0, extras=None, decay_rank: int = 6) -> dict:
    """Random weights of a config (float32 arrays whose values are exact in bfloat16), sized so that activations stay O(1)."""
    rng = np.random.default_rng(seed)
    shapes = expected_tensors(conf, extras)
    for i, L in enumerate(conf["layers"]):
        if L["type"] in PAIR_TYPES and L["mixer"]["right"]["kind"] == "decayed":
            b, r = L["mixer"]["right"], f"l{i}.mix.right."
            shapes.update({r + "a1": [decay_rank, conf["width"]], r + "a2": [b["heads"] * b["dim"], decay_rank], r + "a2.b": [b["heads"] * b["dim"]]})
    out = {}
    for name, shape in shapes.items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            a = 0.1 * rng.standard_normal(shape)                       # stored around zero
        elif leaf == "norm":
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf in ("sink", "D"):
            a = rng.standard_normal(shape)
        elif leaf == "A_log":
            a = rng.uniform(-1.0, 1.0, shape)
        elif leaf == "dt_bias":
            a = rng.uniform(-3.0, 0.0, shape)
        elif name.endswith("a2.b"):
            a = 2.0 + rng.standard_normal(shape)
        elif name.endswith("f.b"):
            a = 2.0 + rng.standard_normal(shape)
        elif leaf == "b":
            a = rng.standard_normal(shape) * 0.5
        elif leaf == "conv":
            a = rng.standard_normal(shape) * 0.5
        elif name in ("embed", "bigram"):
            a = rng.standard_normal(shape) * (1.0 if name == "embed" else 0.5)
        else:
            a = rng.standard_normal(shape) * (scale / np.sqrt(shape[-1]))
        out[name] = bf16_to_f32(f32_to_bf16(np.asarray(a, np.float32))).reshape(shape)
    return out


# ---- the model on a device ------------------------------------------------------------------------------------------------------------
class VuzinexModel(SeqModel):
    """Weights of one model on one device + its runner (sequences, steps and generation: seqmodel.SeqModel).  `weights`: {name: float32
    ndarray} or the pair read_safetensors returns."""

    def __init__(self, device: CudaTensorDevice, conf: dict, weights, dtype: str = "bfloat16", chunk: int = 0, max_seq: int = 0):
        self.device, self.conf, self.dtype = device, parse_config(conf), dtype
        up = Uploader(device, weights, dtype)
        c, names = self.conf, up.weights
        extras = {}
        for i, L in enumerate(c["layers"]):
            if L["type"] in PAIR_TYPES:
                q = f"l{i}.mix.left."
                extras[i] = tuple(e for e, n in (("bias", "q.b"), ("qk_norm", "q.norm"), ("sink", "sink"), ("gate", "g")) if q + n in names)
        want = expected_tensors(c, extras)
        for i, L in enumerate(c["layers"]):
            if L["type"] in PAIR_TYPES and L["mixer"]["right"]["kind"] == "decayed":
                b, r = L["mixer"]["right"], f"l{i}.mix.right."
                if r + "a1" not in names:
                    raise TensorError(f"model is missing tensor {r}a1")
                rank = _decay_rank(c, names, i)
                want.update({r + "a1": [rank, c["width"]], r + "a2": [b["heads"] * b["dim"], rank], r + "a2.b": [b["heads"] * b["dim"]]})
        up.check(want)
        nl, D = len(c["layers"]), c["width"]

        def one_plus(name):                          # the layer norms store their weight as an offset from one
            return up.table(np.float32(1.0) + up.f32(name).reshape(-1))
        # the embedding scale is folded into the (32-bit) table: one rounding, as when it is applied to the looked-up row
        self.tensors = {"embed": up.table(up.f32("embed") * np.float32(c["embedding"]["scale"])), "final.norm": one_plus("final.norm"), "head": up.mat("embed")}
        big = c["embedding"]["bigram"]
        if big:
            self.tensors["bigram"] = up.mat32("bigram")
        lcs = (capi.cvr_layer_config * nl)()
        lws = (capi.cvr_layer_weights * nl)()
        for i, L in enumerate(c["layers"]):
            m, mlp, p = L["mixer"], L["mlp"], f"l{i}."
            lc = lcs[i]
            t = {"norm_a": one_plus(p + "norm1"), "norm_b": one_plus(p + "norm1b")}
            if L["type"] in PAIR_TYPES:
                a, b, q, r = m["left"], m["right"], p + "mix.left.", p + "mix.right."
                ex = extras[i]
                lc.mixer = 0
                lc.heads, lc.kv_heads, lc.dim, lc.vdim = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
                lc.window, lc.block, lc.left_gate, lc.scale, lc.rot_mag = a["mask"]["window"], a["mask"]["size"], int("gate" in ex), a["scale"], 1.0
                lc.r_heads, lc.r_dim, lc.r_vdim = b["heads"], b["dim"], b["vdim"]
                lc.r_q_scale = float(b["dim"]) ** -0.5
                lc.left_scale, lc.right_scale = m["left_scale"], m["right_scale"]
                # one product for everything that multiplies the mixer's input (the order include/crabml_vuzinex.h gives)
                stack = [q + "q", q + "k", q + "v"] + ([q + "g"] if "gate" in ex else []) + [r + "q", r + "k", r + "v", r + "g"]
                if b["kind"] == "matrix_memory":
                    lc.right, lc.gate_cap = 0, b["gate_cap"]
                    stack += [r + "i", r + "f"]
                    t["gate_bias_i"], t["gate_bias_f"] = up.vec(r + "i.b"), up.vec(r + "f.b")
                else:
                    lc.right, lc.tau, lc.r_rank = 1, b["tau"], _decay_rank(c, names, i)
                    stack += [r + "a1"]
                    t["decay_up"], t["decay_bias"] = up.mat(r + "a2"), up.vec(r + "a2.b")
                t["h_stack"] = up.stack(stack)
                if "bias" in ex:
                    t["h_bias"] = up.table(np.concatenate([up.f32(n + ".b").reshape(-1) if n in (q + "q", q + "k", q + "v") else np.zeros(np.shape(names[n])[0], np.float32)
                                                           for n in stack]))
                if "qk_norm" in ex:
                    t["q_norm"], t["k_norm"] = up.vec(q + "q.norm"), up.vec(q + "k.norm")
                if "sink" in ex:
                    t["sink"] = up.vec(q + "sink")
                if a["rot"]:
                    freq, mag = rotary.table_of(a["rot"])
                    t["rot_freq"], lc.rot_mag = up.table(freq), mag
                t["left_o"], t["right_o"], t["right_norm"] = up.mat(q + "o"), up.mat(r + "o"), up.vec(r + "norm")
            else:
                q = p + "mix."
                lc.mixer = 1
                lc.s_heads, lc.s_vdim, lc.s_state, lc.s_groups, lc.s_conv, lc.s_norm_groups = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
                t.update({"in": up.mat(q + "in"), "conv": up.mat32(q + "conv"), "conv_bias": up.vec(q + "conv.b"), "dt_bias": up.vec(q + "dt_bias"),
                          "a_log": up.vec(q + "A_log"), "d_skip": up.vec(q + "D"), "s_norm": up.vec(q + "norm"), "s_o": up.mat(q + "o")})
            if mlp:
                lc.ff = mlp["ff"]
                t.update({"norm_c": one_plus(p + "norm2"), "norm_d": one_plus(p + "norm2b"), "gate_up": up.stack([p + "mlp.gate", p + "mlp.up"]),
                          "gate_up_bias": up.table(np.concatenate([up.f32(p + "mlp.gate.b").reshape(-1), up.f32(p + "mlp.up.b").reshape(-1)])),
                          "down": up.mat(p + "mlp.down"), "down_bias": up.vec(p + "mlp.down.b")})
            for k, v in t.items():
                setattr(lws[i], k, handle_of(v))
                self.tensors[f"{p}{k}"] = v                                  # keep alive
        lp = c["loop"]
        cc = capi.cvr_config(nl, D, c["vocab"], c["norm"]["eps"], c["residual_mult"], c["logit_scale"], lp["start"], lp["stop"], lp["times"],
                             big["buckets"] if big else 0, big["mul_prev"] if big else 0, big["mul_cur"] if big else 0, int(chunk), int(max_seq))
        h = C.c_void_p()
        rc = device.lib.cvr_runner_create(device.handle, C.byref(cc), lcs, lws, self.tensors["embed"].buf.handle, self.tensors["bigram"].buf.handle if big else None,
                                          self.tensors["final.norm"].buf.handle, self.tensors["head"].buf.handle, C.byref(h))
        if rc != capi.CC_OK:
            raise (TensorError if rc == capi.CC_ERR_TENSOR else CudaError)(f"cvr_runner_create failed [{rc}]: {device.lib.csr_last_create_error().decode()}")
        self.handle = h
        self.vocab = c["vocab"]
        self._keep = (lcs, lws)


def load(path: str, device: CudaTensorDevice, dtype: str = "bfloat16", chunk: int = 0, max_seq: int = 0) -> VuzinexModel:
    """path: a folder with config.json and model.safetensors"""
    with open(os.path.join(path, "config.json")) as f:
        conf = json.load(f)
    return VuzinexModel(device, conf, read_safetensors(os.path.join(path, "model.safetensors")), dtype, chunk, max_seq)
