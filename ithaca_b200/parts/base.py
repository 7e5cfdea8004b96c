"""What every part shares: the runtime it is built for, and the registries by kind.

A part is built from a ``PartSpec`` (its sizes and constants), the tensors its
spec names, and a ``Runtime``.  It never learns which architecture it is in.
Adding a part means: write a class with the interface of its family (below),
and call the family's ``register_*`` with a new kind; a configuration then names
that kind in its layer records.

Interfaces
----------
Every part class has ``manifest(spec) -> {tensor name: TensorReq}``, a class
method that states the tensors it needs with their shapes, and a constructor
``(spec, tensors, runtime)``.

* norm:          ``forward(x[T, d] float32, rows=None) -> [rows, d]`` in the activation dtype.
* position:      exposes what its mixer needs (for rotary: ``inv_freq``, ``rotary_dim``, ``pairing``).
* mixer:         ``cache_requests() -> [KVRequest | StateRequest, ...]`` and
                 ``forward(x, ctx, cache, residual, writes_cache)``: reads the normed
                 activations ``x[T, d]``, updates its cache entry for the step's tokens,
                 and adds its output into ``residual[T, d]`` (float32).
* feed-forward:  ``forward(x, ctx, residual)``: adds its output into ``residual``.
* block:         ``forward(residual, ctx, cache, writes_cache)``: arranges norms, mixer and
                 feed-forward around the residual stream.
* embedding:     ``forward(ids[T] int32, ctx) -> [T, d]`` float32 (the residual stream's start); it has
                 ``table``, the matrix a tied head shares.
* head:          ``forward(xn[rows, d]) -> [rows, vocab]`` float32 logits; ``weight_names()`` lists the
                 tensors it reads in full at every step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorReq

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass
class Runtime:
    """``dtype`` is the compute path: ``bfloat16`` (the serving kernels: 16-bit operands,
    float accumulation, float residual stream) or ``float32`` (everything in true
    32-bit arithmetic on the CUDA cores, 32-bit cache)."""
    dtype: str = "bfloat16"
    device: str = "cuda"
    status: Optional[torch.Tensor] = None      # int32[1]: set by a kernel that met an index out of range

    def __post_init__(self):
        if self.dtype not in _DTYPES:
            raise ValueError(f"dtype {self.dtype!r} is not supported (bfloat16, float32)")
        if self.status is None and self.device != "cpu" and torch.cuda.is_available():
            from ..csrc.ops import device_status
            self.status = device_status(self.device)

    @property
    def act_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype]

    @property
    def kv_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype]


class Registry:
    def __init__(self, family: str):
        self.family = family
        self._kinds: Dict[str, type] = {}

    def register(self, kind: str, cls: type, replace: bool = False) -> None:
        if kind in self._kinds and not replace:
            raise ValueError(f"{self.family} kind '{kind}' is already registered")
        self._kinds[kind] = cls

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> type:
        try:
            return self._kinds[kind]
        except KeyError:
            raise ValueError(f"unknown {self.family} kind '{kind}' (registered: {', '.join(sorted(self._kinds))})") from None

    def kinds(self):
        return sorted(self._kinds)


NORMS = Registry("norm")
POSITIONS = Registry("position")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")

register_norm = NORMS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register


def to_device(t: torch.Tensor, runtime: Runtime) -> torch.Tensor:
    return t.to(runtime.device, non_blocking=True) if str(t.device) != str(runtime.device) else t


def as_float32(t: torch.Tensor, runtime: Runtime) -> torch.Tensor:
    """Small vectors (norm weights) are used in float32 by the kernels; widening is exact."""
    return to_device(t, runtime).to(torch.float32).contiguous()
