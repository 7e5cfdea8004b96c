"""Architecture-neutral description of a decoder: what the engine builds from.

An architecture's typed configuration (for instance ``LlamaConfig``) turns
itself into a ``ModelSpec``.  Everything below the configuration works from the
spec only: no part, cache or kernel knows which architecture it serves.

The reference describes a layer with boolean flags on one ``Layer`` struct and
``if (L.x)`` chains in the layer loop (src/model.h:27-57, src/model.cpp:1153-1163).
Here each layer is a record that names its parts, and the order in which layers
run is a list of its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` selects the class in the part registry,
    ``params`` are that class's sizes and constants, ``weights`` maps the part's
    own tensor roles (``"q"``, ``"gate"``, ``"weight"`` ...) to tensor names in
    the checkpoint."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class BlockSpec:
    """A layer: the arrangement ``kind`` (for instance ``"prenorm"``) and the
    parts it arranges.  ``position`` is handed to the mixer (rotary angles are
    applied inside attention); ``None`` means the mixer sees no positions."""

    kind: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]
    position: Optional[PartSpec] = None
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` (a layer may
    be named more than once).  ``cache`` is the cache entry the mixer works on;
    ``writes_cache=False`` lets a run read a cache that an earlier run filled."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    stop_token_ids: Tuple[int, ...] = ()
    # tensors a folder may hold although the model does not ask for them, because they repeat another one:
    # name -> the tensor it must equal (a tied output matrix stored beside the embedding, for instance)
    aliases: Dict[str, str] = field(default_factory=dict)

    def n_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))


def validate_schedule(spec: ModelSpec) -> None:
    """A schedule is sound when every entry names an existing layer, every cache
    entry has exactly one writer, and no run reads a cache entry before its
    writer has run in the same pass."""
    written: Dict[int, int] = {}
    for n, e in enumerate(spec.schedule):
        if not 0 <= e.layer < len(spec.layers):
            raise ValueError(f"schedule[{n}] names layer {e.layer}, but the model has {len(spec.layers)} layers")
        if e.cache < 0:
            raise ValueError(f"schedule[{n}] has a negative cache entry {e.cache}")
        if e.writes_cache:
            if e.cache in written:
                raise ValueError(
                    f"schedule[{n}] writes cache entry {e.cache}, which schedule[{written[e.cache]}] already writes")
            written[e.cache] = n
        elif e.cache not in written:
            raise ValueError(f"schedule[{n}] reads cache entry {e.cache} before any run has written it")
    missing = sorted(set(range(spec.n_cache_entries())) - set(written))
    if missing:
        raise ValueError(f"cache entries {missing} are never written")


def describe(spec: ModelSpec) -> List[str]:
    """Human-readable lines, one per scheduled run (used by the command line)."""
    out = []
    for n, e in enumerate(spec.schedule):
        b = spec.layers[e.layer]
        out.append(f"run {n}: layer {e.layer} [{b.kind}: {b.mixer.kind} + {b.feed_forward.kind}] cache {e.cache}"
                   + ("" if e.writes_cache else " (read only)"))
    return out
