"""The generic decoder: embedding, the scheduled runs of the layers, final norm, head.

It is built from a ``ModelSpec`` alone.  The schedule is data: a list of runs,
each naming a layer and the cache entry its mixer works on (the reference's layer
loop is ``for L in layers`` with per-layer flags, src/model.cpp:1130-1259, 1457-1566).
Final norm and head run only on the rows whose logits are wanted, as the reference
does for the last row (src/model.cpp:1588-1594).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..cache.cache import SequenceCache
from ..config import ConfigError, config_from_model_dir
from ..config.spec import ModelSpec, validate_schedule
from ..parts import BLOCKS, NORMS, Runtime
from ..parts.block import _merge
from ..parts.embedding import Embedding, OutputHead
from ..weights.loader import TensorReq, WeightError, check_tensors, load_checkpoint, read_model_tensors, _storage_form


def weight_manifest(spec: ModelSpec) -> Dict[str, TensorReq]:
    """Every tensor the model needs, with its shape."""
    out: Dict[str, TensorReq] = {}
    _merge(out, Embedding.manifest(spec.embedding))
    for b in spec.layers:
        _merge(out, BLOCKS.get(b.kind).manifest(b))
    _merge(out, NORMS.get(spec.final_norm.kind).manifest(spec.final_norm))
    _merge(out, OutputHead.manifest(spec.head))
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        validate_schedule(spec)
        self.spec = spec
        self.runtime = runtime
        self.embedding = Embedding(spec.embedding, tensors, runtime)
        self.layers = [BLOCKS.get(b.kind)(b, tensors, runtime) for b in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, tensors, runtime)
        if spec.head.weights["weight"] == spec.embedding.weights["weight"]:
            tensors = dict(tensors)
            tensors[spec.head.weights["weight"]] = self.embedding.table      # one copy on the device for both
        self.head = OutputHead(spec.head, tensors, runtime)

    @property
    def graph_safe(self) -> bool:
        """True when every mixer and feed-forward says that a captured step may be replayed for
        other slots and positions (they read those from the step's device arrays, never from
        host values).  A part that does not say so is stepped eagerly."""
        return all(getattr(l.mixer, "graph_safe", False) and getattr(l.feed_forward, "graph_safe", False)
                   for l in self.layers)

    def cache_requests(self) -> Dict[int, List[object]]:
        out: Dict[int, List[object]] = {}
        for e in self.spec.schedule:
            if e.writes_cache:
                out[e.cache] = self.layers[e.layer].cache_requests()
        return out

    def forward(self, ctx, cache: SequenceCache) -> Optional[torch.Tensor]:
        """Runs the step's tokens through every scheduled run; returns float32 logits
        [wanted rows, vocab], or None when no row is wanted."""
        h = self.embedding.forward(ctx.token_ids)
        for e in self.spec.schedule:
            self.layers[e.layer].forward(h, ctx, cache.layer(e.cache), e.writes_cache)
        if ctx.n_logit_rows == 0:
            return None
        xn = self.final_norm.forward(h, rows=ctx.logit_rows)
        return self.head.forward(xn)

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads once (matrices and the head; for roofline figures)."""
        seen, total = set(), 0

        def add(t: torch.Tensor):
            nonlocal total
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        for layer in self.layers:
            for part in (layer.mixer, layer.feed_forward):
                for v in vars(part).values():
                    if hasattr(v, "weight") and isinstance(v.weight, torch.Tensor):
                        add(v.weight)
        add(self.head.linear.weight)
        return total


def build_model(arch, config, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
    spec = config.model_spec()
    if arch.build_model is not None:
        return arch.build_model(spec, tensors, runtime)
    return DecoderModel(spec, tensors, runtime)


def load_model(model_dir: str, runtime: Runtime):
    """Reads ``config.json``, picks the architecture from the registry, checks the
    folder's tensors against what the architecture's parts ask for, and builds the
    model on the runtime's device.  Returns (model, config)."""
    arch, config = config_from_model_dir(model_dir)
    spec = config.model_spec()
    manifest = weight_manifest(spec)
    found = read_model_tensors(model_dir)
    ignore = []
    head_name, emb_name = spec.head.weights["weight"], spec.embedding.weights["weight"]
    if head_name == emb_name and "lm_head.weight" in found and "lm_head.weight" not in manifest:
        # a tied model may still store the head; it must then be the embedding matrix itself
        if emb_name in found and found["lm_head.weight"].shape == found[emb_name].shape and \
                torch.equal(found["lm_head.weight"], found[emb_name]):
            ignore.append("lm_head.weight")
        else:
            raise WeightError("the configuration ties the output head to the embedding, but the folder holds a "
                              "different 'lm_head.weight'")
    check_tensors(found, manifest, ignore)
    tensors = {n: _storage_form(n, found[n], manifest[n]) for n in manifest if n in found}
    return build_model(arch, config, tensors, runtime), config
