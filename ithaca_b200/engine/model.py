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
from ..parts import BLOCKS, EMBEDDINGS, HEADS, NORMS, Runtime
from ..parts.block import _merge
from ..weights.loader import TensorReq, WeightError, check_tensors, load_checkpoint, read_model_tensors, _storage_form


def weight_manifest(spec: ModelSpec) -> Dict[str, TensorReq]:
    """Every tensor the model needs, with its shape."""
    out: Dict[str, TensorReq] = {}
    _merge(out, EMBEDDINGS.get(spec.embedding.kind).manifest(spec.embedding))
    for b in spec.layers:
        _merge(out, BLOCKS.get(b.kind).manifest(b))
    _merge(out, NORMS.get(spec.final_norm.kind).manifest(spec.final_norm))
    _merge(out, HEADS.get(spec.head.kind).manifest(spec.head))
    return out


def streamed_tensor_names(spec: ModelSpec) -> List[str]:
    """The tensors a step reads in full whatever it brings: what the layers' mixers and feed-forwards and the
    head ask for (their manifests), each once.  Norm vectors are left out (a few KB), and so is the embedding
    matrix, of which a step reads one row per token, unless the head shares it."""
    names: List[str] = []
    for e in spec.schedule:
        b = spec.layers[e.layer]
        from ..parts import FEED_FORWARDS, MIXERS
        for part, reg in ((b.mixer, MIXERS), (b.feed_forward, FEED_FORWARDS)):
            names += list(reg.get(part.kind).manifest(part))
    names += list(HEADS.get(spec.head.kind).manifest(spec.head))
    return list(dict.fromkeys(names))


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        validate_schedule(spec)
        self.spec = spec
        self.runtime = runtime
        # bytes of the matrices a step streams, in the form the kernels read them: 16-bit on the bfloat16 path
        # (a matrix stored in 32-bit is rounded once when it is loaded), as stored on the float32 path
        self._streamed_bytes = sum(
            tensors[n].numel() * (2 if runtime.dtype == "bfloat16" and tensors[n].dtype.is_floating_point
                                  else tensors[n].element_size())
            for n in streamed_tensor_names(spec) if n in tensors)
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, tensors, runtime)
        self.layers = [BLOCKS.get(b.kind)(b, tensors, runtime) for b in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, tensors, runtime)
        shared = set(spec.head.weights.values()) & set(spec.embedding.weights.values())
        if shared and hasattr(self.embedding, "table"):
            tensors = dict(tensors)
            for name in shared:
                tensors[name] = self.embedding.table                        # one copy on the device for both
        self.head = HEADS.get(spec.head.kind)(spec.head, tensors, runtime)

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
        h = self.embedding.forward(ctx.token_ids, ctx)
        for e in self.spec.schedule:
            self.layers[e.layer].forward(h, ctx, cache.layer(e.cache), e.writes_cache)
        if ctx.n_logit_rows == 0:
            return None
        xn = self.final_norm.forward(h, rows=ctx.logit_rows)
        return self.head.forward(xn)

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads once (the matrices of the scheduled layers and the head, each
        counted once; for roofline figures)."""
        return self._streamed_bytes


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
    for name, same_as in spec.aliases.items():
        if name in found and name not in manifest:
            # a tensor that repeats another one may be stored; it must then hold the same values
            if same_as in found and found[name].shape == found[same_as].shape and torch.equal(found[name], found[same_as]):
                ignore.append(name)
            else:
                raise WeightError(f"the configuration says that '{name}' repeats '{same_as}', but the folder holds a "
                                  f"different '{name}'")
    check_tensors(found, manifest, ignore)
    tensors = {n: _storage_form(n, found[n], manifest[n]) for n in manifest if n in found}
    return build_model(arch, config, tensors, runtime), config
