"""Bookkeeping of the cache: slots, pages and block tables.  No device memory here.

The reference holds exactly one sequence: a scalar ``n_past`` and one key/value
buffer per layer that grows by doubling (src/model.h:93, src/model.cpp:1001-1035).
Here a *slot* stands for one sequence of a batch.  Keys and values live in pages
of ``page_size`` positions drawn from a pool; a slot's block table maps
position // page_size to a page.  Layers with different needs form groups with
pools of their own: a group that keeps every key never releases a page before
the slot is freed; a group with a window releases pages that no later query can
reach.  Slots and pages go back to their pools when a sequence ends and are
handed out again.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    pass


class PagePool:
    """A fixed set of page ids.  A page is either free or held by exactly one owner."""

    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise CacheError(f"a pool cannot have {n_pages} pages")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))   # pop() hands out low ids first
        self._held = np.zeros(n_pages, dtype=bool)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"the cache is full: all {self.n_pages} pages are in use")
        p = self._free.pop()
        if self._held[p]:
            raise CacheError(f"page {p} was on the free list while held")
        self._held[p] = True
        return p

    def give_back(self, page: int) -> None:
        if not 0 <= page < self.n_pages:
            raise CacheError(f"page {page} does not belong to this pool of {self.n_pages}")
        if not self._held[page]:
            raise CacheError(f"page {page} is freed twice")
        self._held[page] = False
        self._free.append(page)

    def held(self) -> int:
        return int(self._held.sum())


@dataclass(frozen=True)
class KVGroupLayout:
    """Layers that keep keys and values with the same shape and reach."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int]            # None: every key is kept
    cache_entries: tuple             # cache entries (of the schedule) stored in this group, in order


@dataclass(frozen=True)
class StateGroupLayout:
    """Layers that keep a fixed-size state per sequence."""
    shape: tuple
    dtype: str
    cache_entries: tuple
    name: str = "state"


class SlotTable:
    """Slots and, for every key/value group, each slot's block table."""

    def __init__(self, kv_groups: Sequence[KVGroupLayout], n_pages: Sequence[int], max_slots: int, page_size: int):
        if page_size <= 0 or max_slots <= 0:
            raise CacheError("page_size and max_slots must be positive")
        if len(n_pages) != len(kv_groups):
            raise CacheError("one page count per key/value group is needed")
        self.page_size = page_size
        self.max_slots = max_slots
        self.kv_groups = list(kv_groups)
        self.pools = [PagePool(n) for n in n_pages]
        self._free_slots: List[int] = list(range(max_slots - 1, -1, -1))
        self._in_use = np.zeros(max_slots, dtype=bool)
        self.length = np.zeros(max_slots, dtype=np.int64)             # positions each slot holds
        self._reserved = np.zeros(max_slots, dtype=np.int64)           # positions that have pages
        self.epoch = np.zeros(max_slots, dtype=np.int64)               # how often each slot has been handed out
        # tables[g][slot, i] = page of positions [i*page_size, (i+1)*page_size), -1 = none
        self._cols = 4
        self.tables = [np.full((max_slots, self._cols), -1, dtype=np.int32) for _ in kv_groups]
        self._first_live = [np.zeros(max_slots, dtype=np.int64) for _ in kv_groups]  # first table column not yet released

    # -- slots ---------------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.max_slots} slots are in use")
        s = self._free_slots.pop()
        if self._in_use[s]:
            raise CacheError(f"slot {s} was on the free list while in use")
        self._in_use[s] = True
        self.epoch[s] += 1
        self.length[s] = 0
        self._reserved[s] = 0
        for g in range(len(self.kv_groups)):
            self._first_live[g][s] = 0
        return s

    def free_slot(self, slot: int) -> None:
        self._check_slot(slot)
        for g, pool in enumerate(self.pools):
            row = self.tables[g][slot]
            for i in np.nonzero(row >= 0)[0]:
                pool.give_back(int(row[i]))
            row[:] = -1
        self._in_use[slot] = False
        self.length[slot] = 0
        self._reserved[slot] = 0
        self._free_slots.append(slot)

    def in_use(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and bool(self._in_use[slot])

    def n_slots_in_use(self) -> int:
        return int(self._in_use.sum())

    def _check_slot(self, slot: int) -> None:
        if not 0 <= slot < self.max_slots:
            raise CacheError(f"slot {slot} is out of range (0..{self.max_slots - 1})")
        if not self._in_use[slot]:
            raise CacheError(f"slot {slot} is not in use (freed twice, or never allocated)")

    # -- pages ---------------------------------------------------------------------------------
    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        """Pages each group would have to take so that ``slot`` can grow by ``n_new``."""
        self._check_slot(slot)
        end = int(self.length[slot]) + n_new
        have = -(-int(self._reserved[slot]) // self.page_size)
        need = -(-end // self.page_size)
        return [max(0, need - have) for _ in self.kv_groups]

    def reserve(self, slot: int, n_new: int) -> None:
        """Gives ``slot`` pages for positions [length, length + n_new) in every group.
        Either all groups get theirs or nothing changes."""
        self._check_slot(slot)
        if n_new < 0:
            raise CacheError("cannot grow by a negative number of positions")
        end = int(self.length[slot]) + n_new
        if end <= self._reserved[slot]:
            return
        first = -(-int(self._reserved[slot]) // self.page_size)
        last = -(-end // self.page_size)
        for g, pool in enumerate(self.pools):
            if pool.n_free < last - first:
                raise CacheFull(
                    f"the cache is full: slot {slot} needs {last - first} more pages of {self.page_size} positions, "
                    f"group {g} has {pool.n_free} free of {pool.n_pages}")
        if last > self._cols:
            cols = max(last, 2 * self._cols)
            for g in range(len(self.tables)):
                t = np.full((self.max_slots, cols), -1, dtype=np.int32)
                t[:, :self._cols] = self.tables[g]
                self.tables[g] = t
            self._cols = cols
        for g, pool in enumerate(self.pools):
            for i in range(first, last):
                self.tables[g][slot, i] = pool.take()
        self._reserved[slot] = last * self.page_size

    def commit(self, slot: int, n_new: int) -> None:
        """The positions have been written: the slot is that much longer.  Groups with a
        window give back the pages that no later query can reach."""
        self._check_slot(slot)
        new_len = int(self.length[slot]) + n_new
        if new_len > self._reserved[slot]:
            raise CacheError(f"slot {slot}: {new_len} positions committed but only {int(self._reserved[slot])} reserved")
        self.length[slot] = new_len
        for g, grp in enumerate(self.kv_groups):
            if grp.window is None:
                continue
            # the next query sits at position new_len and reaches back to new_len + 1 - window
            first_needed = max(0, new_len + 1 - grp.window)
            dead_cols = first_needed // self.page_size
            row = self.tables[g][slot]
            for i in range(int(self._first_live[g][slot]), dead_cols):
                if row[i] >= 0:
                    self.pools[g].give_back(int(row[i]))
                    row[i] = -1
            self._first_live[g][slot] = max(int(self._first_live[g][slot]), dead_cols)

    def truncate(self, slot: int, n: int) -> None:
        """Keeps the first ``n`` positions (the reference's ``rewind``, src/model.cpp:1047-1058).
        Pages past them are kept for reuse by the same slot.  A windowed group cannot go
        back behind pages it has already released, except to 0: then the slot gives all its
        pages back and starts again.  On refusal nothing has changed."""
        self._check_slot(slot)
        if not 0 <= n <= self.length[slot]:
            raise CacheError(f"slot {slot}: cannot truncate to {n}, it holds {int(self.length[slot])}")
        if n == 0 and any(self._first_live[g][slot] > 0 for g in range(len(self.kv_groups))):
            for g, pool in enumerate(self.pools):
                row = self.tables[g][slot]
                for i in np.nonzero(row >= 0)[0]:
                    pool.give_back(int(row[i]))
                row[:] = -1
                self._first_live[g][slot] = 0
            self.length[slot] = 0
            self._reserved[slot] = 0
            return
        for g, grp in enumerate(self.kv_groups):
            if grp.window is not None and n < self.length[slot]:
                first_needed = max(0, n + 1 - grp.window)
                if first_needed // self.page_size < self._first_live[g][slot]:
                    raise CacheError(f"slot {slot}: group {g} has released the pages a truncation to {n} would need")
        self.length[slot] = n

    def table_rows(self, group: int, slots: Sequence[int], n_cols: int) -> np.ndarray:
        """[len(slots), n_cols] block table of the given slots (padded with -1)."""
        t = self.tables[group]
        out = np.full((len(slots), n_cols), -1, dtype=np.int32)
        c = min(n_cols, t.shape[1])
        out[:, :c] = t[np.asarray(slots, dtype=np.int64), :c]
        return out

    def check_consistent(self) -> None:
        """Every page is free or held by exactly one table entry (used by the tests)."""
        for g, pool in enumerate(self.pools):
            t = self.tables[g]
            used = t[t >= 0]
            if len(np.unique(used)) != len(used):
                raise CacheError(f"group {g}: a page is held twice")
            if len(used) != pool.held():
                raise CacheError(f"group {g}: {pool.held()} pages are held but the tables name {len(used)}")
            if len(used) + pool.n_free != pool.n_pages:
                raise CacheError(f"group {g}: pages were lost ({len(used)} held + {pool.n_free} free != {pool.n_pages})")
            if np.any(t[~self._in_use] >= 0):
                raise CacheError(f"group {g}: a free slot still holds pages")
