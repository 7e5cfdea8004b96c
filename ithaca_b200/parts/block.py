"""The arrangement of a layer's parts around the residual stream.

``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x)) -- the order of the
reference's layer loop (src/model.cpp:1460-1565).  The residual stream is float32
and the parts add into it, so the sum never passes through 16 bits.
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Mapping

import torch

from ..cache.cache import LayerCache
from ..config.spec import BlockSpec
from ..weights.loader import TensorReq
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Runtime, register_block


def _merge(into: Dict[str, TensorReq], more: Mapping[str, TensorReq]) -> None:
    for name, req in more.items():
        if name in into and tuple(into[name].shape) != tuple(req.shape):
            raise ValueError(f"tensor '{name}' is asked for with shapes {into[name].shape} and {req.shape}")
        into[name] = req


class PreNormBlock:
    @classmethod
    def manifest(cls, spec: BlockSpec) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        _merge(out, MIXERS.get(spec.mixer.kind).manifest(spec.mixer))
        _merge(out, FEED_FORWARDS.get(spec.feed_forward.kind).manifest(spec.feed_forward))
        for n in spec.norms.values():
            _merge(out, NORMS.get(n.kind).manifest(n))
        if spec.position is not None:
            _merge(out, POSITIONS.get(spec.position.kind).manifest(spec.position))
        return out

    def __init__(self, spec: BlockSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        for need in ("mixer", "feed_forward"):
            if need not in spec.norms:
                raise ValueError(f"prenorm block: the spec has no '{need}' norm")
        position = None
        if spec.position is not None:
            position = POSITIONS.get(spec.position.kind)(spec.position, tensors, runtime)
        mixer_cls = MIXERS.get(spec.mixer.kind)
        if "position" in inspect.signature(mixer_cls.__init__).parameters:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime, position=position)
        else:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, tensors, runtime)
        self.mixer_norm = NORMS.get(spec.norms["mixer"].kind)(spec.norms["mixer"], tensors, runtime)
        self.ff_norm = NORMS.get(spec.norms["feed_forward"].kind)(spec.norms["feed_forward"], tensors, runtime)

    def cache_requests(self) -> List[object]:
        return list(self.mixer.cache_requests())

    def forward(self, residual: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True) -> None:
        self.mixer.forward(self.mixer_norm.forward(residual), ctx, cache, residual, writes_cache)
        self.feed_forward.forward(self.ff_norm.forward(residual), ctx, residual)


register_block("prenorm", PreNormBlock)
