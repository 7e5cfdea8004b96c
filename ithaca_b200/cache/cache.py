"""The cache a model steps on: page pools and block tables plus the device storage.

Each mixer states what it keeps per sequence: keys and values that grow with the
sequence (``KVRequest``) and/or a state of fixed size (``StateRequest``).  Cache
entries with equal key/value needs share a group: one pool of pages, one block
table per slot, and one pair of tensors ``[entries, pages, kv_heads, page_size,
head_dim]``.  Fixed-size state lies beside it as ``[entries, max_slots, *shape]``
and is cleared when a slot is handed out (the reference zeroes recurrent state
when a sequence restarts, src/model.cpp:1047-1055).

The reference's layout is one buffer per layer ``[positions][kv_heads*head_dim]``
(src/model.cpp:440-448); pages keep each kv head's ``page_size`` positions
contiguous, which is what the attention kernels stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from .pages import CacheError, CacheFull, KVGroupLayout, SlotTable, StateGroupLayout

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVRequest:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    name: str
    shape: Tuple[int, ...]
    dtype: str = "float32"


_TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class LayerCache:
    """What one run of a mixer sees of the cache."""
    entry: int
    kv_group: Optional[int] = None          # index into StepContext.tables
    k_pages: Optional[torch.Tensor] = None  # [pages, kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor] = None
    window: Optional[int] = None
    states: Optional[Dict[str, torch.Tensor]] = None   # name -> [max_slots, *shape]

    def state(self, name: str) -> torch.Tensor:
        if not self.states or name not in self.states:
            raise CacheError(f"cache entry {self.entry} has no state '{name}'")
        return self.states[name]


def plan_groups(requests: Mapping[int, Sequence[object]]):
    """Groups cache entries by what they keep.  Returns (kv groups, state groups,
    entry -> kv group index, entry -> {state name: (state group index, row)})."""
    kv_keys: Dict[tuple, List[int]] = {}
    st_keys: Dict[tuple, List[int]] = {}
    for entry in sorted(requests):
        seen_kv = False
        for r in requests[entry]:
            if isinstance(r, KVRequest):
                if seen_kv:
                    raise CacheError(f"cache entry {entry} asks for keys and values twice")
                seen_kv = True
                kv_keys.setdefault((r.n_kv_heads, r.head_dim, r.window), []).append(entry)
            elif isinstance(r, StateRequest):
                if r.dtype not in _TORCH:
                    raise CacheError(f"state '{r.name}': dtype {r.dtype} is not supported")
                st_keys.setdefault((r.name, tuple(r.shape), r.dtype), []).append(entry)
            else:
                raise CacheError(f"cache entry {entry}: unknown request {r!r}")
    kv_groups = [KVGroupLayout(k[0], k[1], k[2], tuple(v)) for k, v in kv_keys.items()]
    st_groups = [StateGroupLayout(k[1], k[2], tuple(v), k[0]) for k, v in st_keys.items()]
    return kv_groups, st_groups


class SequenceCache:
    def __init__(self, requests: Mapping[int, Sequence[object]], max_tokens: int, max_slots: Optional[int] = None,
                 kv_dtype: torch.dtype = torch.bfloat16, device: Optional[str] = "cuda", page_size: int = PAGE_SIZE):
        """``max_tokens``: the most positions that live sequences hold at any time, each
        sequence's count rounded up to a multiple of ``page_size``.  Every key/value
        group gets that many positions' worth of pages."""
        if max_tokens < page_size:
            max_tokens = page_size
        n_pages = max_tokens // page_size
        self.page_size = page_size
        self.kv_groups, self.state_groups = plan_groups(requests)
        if max_slots is None:
            max_slots = max(1, n_pages)        # a live sequence holds at least one page
        self.max_slots = max_slots
        self.n_pages = n_pages
        self.table = SlotTable(self.kv_groups, [n_pages] * len(self.kv_groups), max_slots, page_size)
        self.device = device
        self.kv_dtype = kv_dtype
        self._views: Dict[int, LayerCache] = {}
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        self.state: List[torch.Tensor] = []
        if device is not None:
            for g in self.kv_groups:
                shape = (len(g.cache_entries), n_pages, g.n_kv_heads, page_size, g.head_dim)
                self.k.append(torch.zeros(shape, dtype=kv_dtype, device=device))
                self.v.append(torch.zeros(shape, dtype=kv_dtype, device=device))
            for s in self.state_groups:
                self.state.append(torch.zeros((len(s.cache_entries), max_slots) + tuple(s.shape),
                                              dtype=_TORCH[s.dtype], device=device))
        entries = set(requests)
        for e in entries:
            view = LayerCache(entry=e, states={})
            for gi, g in enumerate(self.kv_groups):
                if e in g.cache_entries:
                    row = g.cache_entries.index(e)
                    view.kv_group, view.window = gi, g.window
                    if device is not None:
                        view.k_pages, view.v_pages = self.k[gi][row], self.v[gi][row]
            for si, s in enumerate(self.state_groups):
                if e in s.cache_entries and device is not None:
                    view.states[s.name] = self.state[si][s.cache_entries.index(e)]
            self._views[e] = view

    # -- what a model run needs ----------------------------------------------------------------
    def layer(self, entry: int) -> LayerCache:
        v = self._views.get(entry)
        return v if v is not None else LayerCache(entry=entry, states={})

    def bytes_per_token(self) -> int:
        el = torch.empty((), dtype=self.kv_dtype).element_size()
        return sum(2 * len(g.cache_entries) * g.n_kv_heads * g.head_dim * el for g in self.kv_groups)

    # -- slots ---------------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        s = self.table.alloc_slot()
        for t in self.state:
            t[:, s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.table.free_slot(slot)

    def length(self, slot: int) -> int:
        self.table._check_slot(slot)
        return int(self.table.length[slot])

    def truncate(self, slot: int, n: int) -> None:
        """Keeps the first ``n`` positions of the slot.  Fixed-size state cannot be rolled back: a
        sequence that has some goes back to 0 only, and its state is cleared then (the reference
        restarts a recurrent model from zero when it is rewound, src/model.cpp:1047-1055)."""
        if self.state_groups and n not in (0, self.length(slot)):
            raise CacheError("a sequence with fixed-size state can only be truncated to 0")
        shorter = n < self.length(slot)
        self.table.truncate(slot, n)
        if n == 0 and shorter:
            for t in self.state:
                t[:, slot].zero_()

    def reserve(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """Pages for a whole step, or CacheFull with nothing changed for the step's later
        sequences (earlier ones keep pages they can use at the next try)."""
        need = [0] * len(self.kv_groups)
        for s, n in zip(slots, n_new):
            for g, c in enumerate(self.table.pages_needed(s, n)):
                need[g] += c
        for g, pool in enumerate(self.table.pools):
            if pool.n_free < need[g]:
                raise CacheFull(f"the cache is full: this step needs {need[g]} more pages of {self.page_size} positions "
                                f"in group {g}, {pool.n_free} of {pool.n_pages} are free")
        for s, n in zip(slots, n_new):
            self.table.reserve(s, n)

    def commit(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        for s, n in zip(slots, n_new):
            self.table.commit(s, n)
