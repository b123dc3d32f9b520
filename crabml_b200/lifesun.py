"""The Lifesun decoder family: configuration, weight loading and the Python handle on its C++ runner
(crabml_b200/csrc/host/lifesun_runner.cpp; the stack is described in include/crabml_lifesun.h).

A model folder holds config.json and model.safetensors.  config.json gives every size and every constant that can differ between
models of the family: `vocab`, `width`, `norm.eps`, `logit_scale`, `loop` (`start`, `stop`, `times`) and `layers`, a list whose entries
name the layer's mixer (`type`: "parallel" or "parallel_2"), the mixer's sizes (`mixer`: `left`, `right`, `left_scale`, `right_scale`)
and its feed-forward (`mlp`: kind "dense" with `ff`, or null).
  parallel    left: `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `mask.size` (blocks of positions); right: `width`, `blocks`, `conv`
  parallel_2  left: the same sizes, `rot` (`dims`, `base`), `softcap`, `mask.size` (a sliding window); right: `heads`, `dim`, `vdim`, `decay`
              (one number per head), `rot`
Tensor names: `embed`, `loop.in`, `final.norm`, `final.norm.b`, `head`, and per layer i `l<i>.norm1`, `l<i>.norm1.b`, `l<i>.mix.left.*`,
`l<i>.mix.right.*`, `l<i>.mlp.*`.

Precision: `dtype="bfloat16"` keeps the matrices of the dense products in bfloat16 (activations are rounded to bfloat16 at the input
of a product, sums are 32-bit); `dtype="float32"` widens them and every product is a true 32-bit one.  In both modes the residual
stream, norms, rotations, attention scores and sums, gates, decays, the gate products of the diagonal recurrence and all recurrent state
are 32-bit.
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

ARCHITECTURE = "Lifesun"
LRU_RATE = 8.0          # the constant c of the diagonal recurrence, log a = -c r softplus(lam)
QK_UNIT_PER_HEAD, QK_WHOLE_WEIGHTED = 1, 2
RIGHT_DIAGONAL, RIGHT_RETENTION = 0, 1


# ---- configuration ----------------------------------------------------------------------------------------------------------------
def _rot(r, dim, at):
    if not r or int(r.get("dims", 0)) <= 0:
        return None
    out = {"dims": int(r["dims"]), "base": float(r["base"])}
    if out["dims"] > dim or out["dims"] % 2:
        raise TensorError(f"{at}: rot.dims must be even and at most the head size")
    return out


def parse_config(conf: dict) -> dict:
    """Validates a config.json dict and fills the optional keys, so that the rest of the code reads one shape of dict."""
    if conf.get("architecture", ARCHITECTURE) != ARCHITECTURE:
        raise TensorError(f"not a {ARCHITECTURE} config: architecture = {conf.get('architecture')!r}")
    out = {"architecture": ARCHITECTURE, "vocab": int(conf["vocab"]), "width": int(conf["width"]), "norm": {"eps": float(conf["norm"]["eps"])},
           "logit_scale": float(conf.get("logit_scale", 1.0)), "layers": []}
    n = len(conf["layers"])
    lp = conf.get("loop")
    out["loop"] = {"start": int(lp["start"]), "stop": int(lp["stop"]), "times": int(lp["times"])} if lp else None
    if lp and (not (0 <= out["loop"]["start"] <= out["loop"]["stop"] <= n) or out["loop"]["times"] < 1):
        raise TensorError(f"loop {out['loop']} does not fit {n} layers")
    for i, L in enumerate(conf["layers"]):
        at, m = f"layer {i}", L["mixer"]
        if L["type"] not in ("parallel", "parallel_2"):
            raise TensorError(f"{at}: unknown mixer type {L['type']!r}")
        a, b = m["left"], m["right"]
        left = {k: int(a[k]) for k in ("heads", "kv_heads", "dim", "vdim")}
        left["scale"] = float(a["scale"])
        left["mask"] = {"size": int((a.get("mask") or {}).get("size", 0))}
        if left["heads"] % left["kv_heads"]:
            raise TensorError(f"{at}: kv_heads does not divide heads")
        if L["type"] == "parallel":
            right = {k: int(b[k]) for k in ("width", "blocks", "conv")}
            if right["width"] % right["blocks"] or right["conv"] < 1:
                raise TensorError(f"{at}: blocks must divide the recurrence's width, and the convolution needs a tap")
        else:
            left["rot"] = _rot(a.get("rot"), left["dim"], at)
            left["softcap"] = float(a.get("softcap") or 0.0)
            right = {k: int(b[k]) for k in ("heads", "dim", "vdim")}
            right["decay"] = [float(d) for d in b["decay"]]
            right["rot"] = _rot(b.get("rot"), right["dim"], at)
            if len(right["decay"]) != right["heads"]:
                raise TensorError(f"{at}: the right mixer needs one decay per head")
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise TensorError(f"{at}: unknown feed-forward kind {mlp.get('kind')!r}")
            mlp = {"kind": "dense", "ff": int(mlp["ff"])}
        out["layers"].append({"type": L["type"], "mlp": mlp,
                              "mixer": {"left": left, "right": right, "left_scale": float(m.get("left_scale", 1.0)), "right_scale": float(m.get("right_scale", 1.0))}})
    return out


def expected_tensors(conf: dict) -> dict:
    """name -> shape of every tensor a model of this (parsed) config has"""
    D, V = conf["width"], conf["vocab"]
    t = {"embed": [V, D], "final.norm": [D], "final.norm.b": [D], "head": [V, D]}
    if conf.get("loop") and conf["loop"]["stop"] > conf["loop"]["start"]:
        t["loop.in"] = [D, 2 * D]
    for i, L in enumerate(conf["layers"]):
        m, p = L["mixer"], f"l{i}."
        a, b, q, r = m["left"], m["right"], p + "mix.left.", p + "mix.right."
        hq, hk, hv, ho = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"], a["heads"] * a["vdim"]
        t.update({p + "norm1": [D], p + "norm1.b": [D], q + "q": [hq, D], q + "k": [hk, D], q + "v": [hv, D], q + "o": [D, ho]})
        if L["type"] == "parallel":
            Cw, B = b["width"], b["blocks"]
            bs = Cw // B
            t.update({q + "g": [a["heads"], D], r + "y": [Cw, D], r + "y.b": [Cw], r + "x": [Cw, D], r + "x.b": [Cw], r + "conv": [Cw, b["conv"]], r + "conv.b": [Cw],
                      r + "ra": [B, bs, bs], r + "ra.b": [B, bs], r + "ri": [B, bs, bs], r + "ri.b": [B, bs], r + "lam": [Cw], r + "o": [D, Cw]})
        else:
            qk, rv = b["heads"] * b["dim"], b["heads"] * b["vdim"]
            t.update({q + "q.norm": [hq], q + "k.norm": [hk], r + "q": [qk, D], r + "k": [qk, D], r + "v": [rv, D], r + "g": [rv, D], r + "o": [D, rv]})
        if L["mlp"]:
            ff = L["mlp"]["ff"]
            t.update({p + "mlp.gate": [ff, D], p + "mlp.up": [ff, D], p + "mlp.down": [D, ff]})
    return t


def random_weights(conf: dict, seed: int = 0, scale: float = 1.0) -> dict:
    """Random weights of a (parsed) config (float32 arrays whose values are exact in bfloat16), sized so that activations stay O(1)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in expected_tensors(parse_config(conf)).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm") and not name.endswith(("q.norm", "k.norm")):
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif name.endswith(("q.norm", "k.norm")):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "lam":
            a = rng.uniform(-5.0, -1.0, shape)
        elif leaf == "b":
            a = rng.standard_normal(shape) * (0.1 if name.endswith(("norm1.b", "norm.b")) else 0.5)
        elif leaf == "conv":
            a = rng.standard_normal(shape) * 0.5
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif name == "loop.in":
            a = rng.standard_normal(shape) * (scale / np.sqrt(shape[-1] / 2))
        else:
            a = rng.standard_normal(shape) * (scale / np.sqrt(shape[-1]))
        out[name] = bf16_to_f32(f32_to_bf16(np.asarray(a, np.float32))).reshape(shape)
    return out


# ---- the model on a device ------------------------------------------------------------------------------------------------------------
class LifesunModel(SeqModel):
    """Weights of one model on one device + its runner (sequences, steps and generation: seqmodel.SeqModel).  `weights`: {name: float32
    ndarray} or the pair read_safetensors returns."""

    def __init__(self, device: CudaTensorDevice, conf: dict, weights, dtype: str = "bfloat16", chunk: int = 0, max_seq: int = 0):
        self.device, self.conf, self.dtype = device, parse_config(conf), dtype
        up = Uploader(device, weights, dtype)
        c = self.conf
        up.check(expected_tensors(c))
        nl, D = len(c["layers"]), c["width"]
        self.tensors = {"embed": up.table(up.f32("embed")), "final.norm": up.vec("final.norm"), "final.norm.b": up.vec("final.norm.b"), "head": up.mat("head")}
        if "loop.in" in expected_tensors(c):
            self.tensors["loop.in"] = up.mat("loop.in")
        lcs = (capi.clr_layer_config * nl)()
        lws = (capi.clr_layer_weights * nl)()
        for i, L in enumerate(c["layers"]):
            m, mlp, p = L["mixer"], L["mlp"], f"l{i}."
            a, b, q, r = m["left"], m["right"], p + "mix.left.", p + "mix.right."
            lc = lcs[i]
            lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.scale = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"]
            lc.left_scale, lc.right_scale = m["left_scale"], m["right_scale"]
            t = {"norm_w": up.vec(p + "norm1"), "norm_b": up.vec(p + "norm1.b"), "left_o": up.mat(q + "o"), "right_o": up.mat(r + "o")}
            # one product for everything that multiplies the layer's normed input (the order include/crabml_lifesun.h gives)
            stack = [q + "q", q + "k", q + "v"]
            if L["type"] == "parallel":
                lc.block, lc.window, lc.qk_norm, lc.left_gate, lc.softcap = a["mask"]["size"], 0, QK_UNIT_PER_HEAD, 1, 0.0
                lc.right, lc.r_width, lc.r_blocks, lc.r_conv, lc.r_rate = RIGHT_DIAGONAL, b["width"], b["blocks"], b["conv"], LRU_RATE
                stack += [q + "g", r + "y", r + "x"]
                bs = b["width"] // b["blocks"]
                # per block of channels the recurrence gate's matrix over the input gate's: one product per block gives both gates
                t.update({"sink": up.table(np.zeros(a["heads"], np.float32)),          # a key whose score is 0 and which has no value: 1 in the denominator
                          "x_bias": up.vec(r + "x.b"), "y_bias": up.vec(r + "y.b"), "conv": up.mat32(r + "conv"), "conv_bias": up.vec(r + "conv.b"), "lam": up.vec(r + "lam"),
                          "gate_w": up.table(np.concatenate([up.f32(r + "ra"), up.f32(r + "ri")], 1).reshape(2 * b["width"], bs)),
                          "gate_b": up.table(np.concatenate([up.f32(r + "ra.b"), up.f32(r + "ri.b")], 1).reshape(-1))})
            else:
                lc.window, lc.block, lc.qk_norm, lc.left_gate, lc.softcap = a["mask"]["size"], 0, QK_WHOLE_WEIGHTED, 0, a["softcap"]
                lc.right, lc.r_heads, lc.r_dim, lc.r_vdim = RIGHT_RETENTION, b["heads"], b["dim"], b["vdim"]
                stack += [r + "q", r + "k", r + "v", r + "g"]
                t.update({"q_norm": up.vec(q + "q.norm"), "k_norm": up.vec(q + "k.norm"), "decay": up.table(np.asarray(b["decay"], np.float32))})
                if a["rot"]:
                    t["rot_freq"] = up.table(rotary.table_of(a["rot"])[0])
                if b["rot"]:
                    t["r_rot_freq"] = up.table(rotary.table_of(b["rot"])[0])
            if mlp:
                lc.ff = mlp["ff"]
                stack += [p + "mlp.gate", p + "mlp.up"]
                t["down"] = up.mat(p + "mlp.down")
            t["h_stack"] = up.stack(stack)
            for k, v in t.items():
                setattr(lws[i], k, handle_of(v))
                self.tensors[f"{p}{k}"] = v                                  # keep alive
        lp = c["loop"]
        cc = capi.clr_config(nl, D, c["vocab"], c["norm"]["eps"], c["logit_scale"], lp["start"] if lp else 0, lp["stop"] if lp else 0, lp["times"] if lp else 0,
                             int(chunk), int(max_seq))
        h = C.c_void_p()
        rc = device.lib.clr_runner_create(device.handle, C.byref(cc), lcs, lws, self.tensors["embed"].buf.handle,
                                          self.tensors["loop.in"].buf.handle if "loop.in" in self.tensors else None, self.tensors["final.norm"].buf.handle,
                                          self.tensors["final.norm.b"].buf.handle, self.tensors["head"].buf.handle, C.byref(h))
        if rc != capi.CC_OK:
            raise (TensorError if rc == capi.CC_ERR_TENSOR else CudaError)(f"clr_runner_create failed [{rc}]: {device.lib.csr_last_create_error().decode()}")
        self.handle = h
        self.vocab = c["vocab"]
        self._keep = (lcs, lws)


def load(path: str, device: CudaTensorDevice, dtype: str = "bfloat16", chunk: int = 0, max_seq: int = 0) -> LifesunModel:
    """path: a folder with config.json and model.safetensors"""
    with open(os.path.join(path, "config.json")) as f:
        conf = json.load(f)
    return LifesunModel(device, conf, read_safetensors(os.path.join(path, "model.safetensors")), dtype, chunk, max_seq)
