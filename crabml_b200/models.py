"""Model registry: which loader serves which architecture.

A model is either a GGUF file (the llama family of the reference: llama / qwen2 / gemma, crabml-llama2/src/model.rs:21-27) or a folder
with config.json + model.safetensors whose "architecture" key names a registered family.  `load_model` returns an object with the
family's serving interface; `architecture_of` only reads the metadata."""
from __future__ import annotations

import json
import os

from .capi import TensorError

_FOLDER_LOADERS = {}


def register(architecture: str, loader):
    """loader(path, device, **options) -> model"""
    _FOLDER_LOADERS[architecture] = loader


def architectures():
    return sorted(_FOLDER_LOADERS) + ["llama (GGUF)"]


def architecture_of(path: str) -> str:
    if os.path.isdir(path):
        with open(os.path.join(path, "config.json")) as f:
            return str(json.load(f).get("architecture"))
    return "gguf"


def load_model(path: str, device, **options):
    arch = architecture_of(path)
    if arch == "gguf":
        from . import runner
        conf, weights, tok = runner.load_gguf(path, device)
        return runner.LlamaRunner(device, conf, weights, options.get("kv_seq_len", conf.seq_len), options.get("f16_kv", False))
    if arch not in _FOLDER_LOADERS:
        raise TensorError(f"no loader for architecture {arch!r}; known: {architectures()}")
    return _FOLDER_LOADERS[arch](path, device, **options)


def _load_zatorax(path, device, dtype="bfloat16", chunk=0, **_):
    from . import zatorax
    return zatorax.load(path, device, dtype, chunk)


register("Zatorax", _load_zatorax)


def _load_meresun(path, device, dtype="bfloat16", chunk=0, max_tokens=0, **_):
    from . import meresun
    return meresun.load(path, device, dtype, chunk, max_tokens)


register("Meresun", _load_meresun)


def _load_vuzinex(path, device, dtype="bfloat16", chunk=0, max_tokens=0, **_):
    from . import vuzinex
    return vuzinex.load(path, device, dtype, chunk, max_tokens)


register("Vuzinex", _load_vuzinex)


def _load_lifesun(path, device, dtype="bfloat16", chunk=0, max_tokens=0, **_):
    from . import lifesun
    return lifesun.load(path, device, dtype, chunk, max_tokens)


register("Lifesun", _load_lifesun)
