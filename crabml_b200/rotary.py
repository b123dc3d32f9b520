"""Frequency tables for cc_rope_pairs / cc_latent_ring_append (include/crabml_seqops.h): one frequency per rotated pair and one factor
on cos and sin.  The kernels multiply position and frequency in 32-bit; whatever a model does to its frequencies lives in the table."""
from __future__ import annotations

import math

import numpy as np


def plain_table(dims: int, base: float):
    """pair i turns by position * base^(-2 i / dims)"""
    i = np.arange(dims // 2, dtype=np.float64)
    return np.power(float(base), -2.0 * i / dims), 1.0


def yarn_table(dims: int, base: float, factor: float, original: float, fast: float, slow: float):
    """YaRN: pairs that turn more than `fast` times over the original context keep their frequency, pairs that turn less than `slow`
    times have it divided by `factor`, a linear ramp over the pair index joins the two; cos and sin grow by 0.1 ln(factor) + 1."""
    f, _ = plain_table(dims, base)

    def pair_of(turns):                       # the (fractional) pair index that makes `turns` full turns over the original context
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    i = np.arange(dims // 2, dtype=np.float64)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def wavelength_band_table(dims: int, base: float, factor: float, original: float, low: float, high: float):
    """Scaling by wavelength bands (the Llama 3.1 rule): a pair whose wavelength is shorter than original / high keeps its frequency, one
    whose wavelength is longer than original / low has it divided by `factor`, and between the two the frequency is the blend
    (1 - s) f / factor + s f with s = (original / wavelength - low) / (high - low)."""
    f, _ = plain_table(dims, base)
    wave = 2.0 * math.pi / f
    s = (original / wave - low) / (high - low)
    blend = (1.0 - s) * f / factor + s * f
    return np.where(wave < original / high, f, np.where(wave > original / low, f / factor, blend)), 1.0


def table_of(rot: dict):
    """rot: {"dims", "base", optional "scaling"} -> (float32 frequencies [dims / 2], factor on cos and sin).  The scaling's keys say which
    rule it is: {"factor", "original", "fast", "slow"} is YaRN, {"factor", "original", "low", "high"} the wavelength bands."""
    dims, base = int(rot["dims"]), float(rot["base"])
    sc = rot.get("scaling")
    if not sc:
        f, mag = plain_table(dims, base)
    elif "low" in sc or "high" in sc:
        f, mag = wavelength_band_table(dims, base, float(sc["factor"]), float(sc["original"]), float(sc["low"]), float(sc["high"]))
    else:
        f, mag = yarn_table(dims, base, float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
    return f.astype(np.float32), float(mag)
