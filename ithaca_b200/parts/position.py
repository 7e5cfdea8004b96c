"""Rotary position encoding: the table of inverse frequencies and how pairs are formed.

inv_freq[i] = theta^(-2i/rot) / rscale / factor_i  (src/model.cpp:229-237).  ``rscale`` is
the ``linear`` scaling factor.  The reference reads the per-frequency divisors
``factor_i`` from a tensor (``rope_freqs.weight``, src/model.cpp:230, 235); a model
folder gives the ``llama3`` rule instead, from which they are computed here: a
frequency whose wavelength is shorter than original_max/high_freq_factor is kept,
one longer than original_max/low_freq_factor is divided by ``factor``, and between
the two the divisor is interpolated so that the frequency moves linearly from one
regime to the other.  The table is computed once in float64 and rounded to
float32; the angle pos * inv_freq[i] is formed in float32 by the kernel, as the
reference forms it on the host (src/model.cpp:698-713).

Pairing: ``half`` rotates (i, i + rot/2), ``interleaved`` rotates (2i, 2i+1); the
reference has both behind its ``neox`` flag (src/model.cpp:643).
"""
from __future__ import annotations

import json
import math
from typing import Dict, Mapping

import numpy as np
import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorReq
from .base import Runtime, register_position

_PAIRINGS = {"half": 0, "interleaved": 1}


def inverse_frequencies(rotary_dim: int, theta: float, scaling) -> np.ndarray:
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ValueError(f"rotary: the rotated width must be a positive even number, found {rotary_dim}")
    exponent = np.arange(0, rotary_dim, 2, dtype=np.float64) / rotary_dim
    freq = 1.0 / np.power(float(theta), exponent)
    kind = None if not scaling else scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        pass
    elif kind == "linear":
        freq = freq / float(scaling["factor"])
    elif kind == "llama3":
        factor = float(scaling["factor"])
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        original = float(scaling["original_max_position_embeddings"])
        turns = original * freq / (2.0 * math.pi)          # rotations over the original context
        out = np.empty_like(freq)
        for n, (f, r) in enumerate(zip(freq, turns)):
            if r > high:            # short wavelength: keep
                out[n] = f
            elif r < low:           # long wavelength: slow down by the factor
                out[n] = f / factor
            else:
                mix = (r - low) / (high - low)
                out[n] = (1.0 - mix) * f / factor + mix * f
        freq = out
    else:
        raise ValueError(f"rotary: scaling type {kind!r} is not supported (llama3, linear, default)")
    return freq.astype(np.float32)


_TABLES: Dict[tuple, torch.Tensor] = {}      # one device copy per distinct table: layers with equal settings share it


class RotaryPosition:
    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        return {}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.rotary_dim = int(spec["rotary_dim"])
        pairing = spec.get("pairing", "half")
        if pairing not in _PAIRINGS:
            raise ValueError(f"rotary: pairing {pairing!r} is not known (half, interleaved)")
        self.pairing = _PAIRINGS[pairing]
        scaling = spec.get("scaling")
        self.key = ("rotary", self.rotary_dim, float(spec["theta"]), json.dumps(scaling, sort_keys=True), str(runtime.device))
        if self.key not in _TABLES:
            table = inverse_frequencies(self.rotary_dim, float(spec["theta"]), scaling)
            _TABLES[self.key] = torch.from_numpy(table).to(runtime.device)
        self.inv_freq = _TABLES[self.key]


register_position("rotary", RotaryPosition)
