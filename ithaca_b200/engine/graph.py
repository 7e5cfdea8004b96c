"""Decode steps replayed from CUDA graphs.

A decode step is some hundreds of small launches; issued one by one from Python
they cost more than the step itself.  The reference captures its whole
single-token forward into one graph and replays it, reading the position from
device memory (src/model.cpp:1341-1350, src/cuda_tier.cpp:630-651).  Here a graph
is captured per (number of sequences, block-table width): the step's description
(tokens, positions, lengths, block tables) lives in one device buffer that is
refilled before each replay, so the same graph serves every step of that shape.
The graph covers the forward pass, the greedy pick, and a copy of the kernels'
status word next to the picked ids, so that one read-back per step brings both.

In the greedy generation loop the next step is launched before the current one has been read
back: its token ids are fed on the device from the current step's picks, so the GPU does not
wait for the host between steps.  If the host then decides otherwise (a sequence ended, the
caller asks for something else), the step launched ahead is dropped and the lengths it advanced
are taken back; what it wrote lies beyond those lengths and is never read.

The host side of a replayed step is kept short: the description is written
straight into one of two pinned staging buffers (the other may still be in
flight), only the fields that change from step to step are rewritten, and the
cache's bookkeeping for "one more position per sequence" is done with array
operations.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.pages import CacheError
from ..csrc import ops
from .context import StepContext, field_offsets
from .step import StepError, Stepper


@dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    buffer: torch.Tensor                 # device int32: the step's description
    offsets: List[int]
    sizes: List[int]
    stages: List[torch.Tensor]           # two pinned copies of the description
    stage_events: List[Optional[torch.cuda.Event]]
    stage_slots: List[Optional[Tuple[int, ...]]]
    logits: torch.Tensor
    out: torch.Tensor                    # device int32 [B + 1]: greedy ids, then the status word
    launches: int
    pick_scratch: Optional[torch.Tensor] = None      # kept alive with the graph that writes it
    turn: int = 0


@dataclass
class _Launched:
    """A decode step that has been put on the stream and not yet read back."""
    cap: _Captured
    slots: Tuple[int, ...]
    epochs: np.ndarray
    new_lengths: np.ndarray
    host_out: torch.Tensor               # pinned [B + 1]: greedy ids, then the status word
    done: torch.cuda.Event
    input_tokens: Optional[List[int]]    # the tokens this step was given (None until known: fed on the device)


def _bucket(cols: int) -> int:
    """Block-table widths are rounded up so that a growing sequence re-captures rarely: to multiples of 4 up to 32,
    then in four steps per doubling (40, 48, 56, 64, 80, ...).  What a captured step derives from the length of its
    longest sequence (grid sizes, the chunk length of decode attention) it derives from the width's upper end, so
    beyond 1,024 positions no graph is replayed for a longest sequence shorter than four fifths of what it was shaped for."""
    p = 4
    while 2 * p < cols:
        p *= 2
    step = max(4, p // 4)                     # cols lies in (p, 2p] (or is at most 8)
    return -(-cols // step) * step


class GraphDecoder:
    def __init__(self, stepper: Stepper):
        self.stepper = stepper
        self.graphs: Dict[Tuple[int, int], _Captured] = {}
        self.launches_last_step = 0
        self.last_upload_bytes = 0
        self._ahead: Optional[_Launched] = None          # the step launched before its tokens reached the host
        self._host_bufs: Dict[int, List[torch.Tensor]] = {}
        self._host_turn = 0
        self.steps_dropped = 0

    # -- one decode step -------------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]]) -> Tuple[torch.Tensor, torch.Tensor]:
        """One token per slot.  Returns (logits [B, vocab], greedy ids [B]) on the device; both are
        the graph's own buffers and are overwritten by the next step of the same shape."""
        self.flush()
        cap = self._run(slots, [t[0] for t in self._check_tokens(tokens)], None, strict=True)
        return cap.logits, cap.out[:len(slots)]

    def flush(self) -> None:
        """Drops the step that was launched ahead, if any: the positions it added are taken back."""
        a, self._ahead = self._ahead, None
        if a is None:
            return
        table = self.stepper.cache.table
        for i, s in enumerate(a.slots):
            if table._in_use[s] and table.epoch[s] == a.epochs[i] and table.length[s] == a.new_lengths[i]:
                table.length[s] -= 1
        self.steps_dropped += 1

    def _check_tokens(self, tokens):
        if any(len(t) != 1 for t in tokens):
            raise StepError("a decode step brings exactly one token per slot")
        return tokens

    def _host_buffer(self, n: int) -> torch.Tensor:
        bufs = self._host_bufs.get(n)
        if bufs is None:
            bufs = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(3)]
            self._host_bufs[n] = bufs
        self._host_turn = (self._host_turn + 1) % 3
        return bufs[self._host_turn]

    def _launch(self, slots, tokens: Optional[List[int]], feed: Optional[_Captured], strict: bool) -> Optional[_Launched]:
        table = self.stepper.cache.table
        idx = np.asarray(slots, dtype=np.int64)
        cap = self._run(slots, tokens, feed, strict)
        if cap is None:
            return None
        host = self._host_buffer(len(slots) + 1)
        host.copy_(cap.out, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return _Launched(cap, tuple(slots), table.epoch[idx].copy(), table.length[idx].copy(), host, ev, tokens)

    def greedy_step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]]) -> List[int]:
        """One greedy decode step: returns the picked ids on the host.  The following step is put on
        the stream before this one is read back."""
        toks = [int(t[0]) for t in self._check_tokens(tokens)]
        key = tuple(slots)
        cur, self._ahead = self._ahead, None
        if cur is not None:
            table = self.stepper.cache.table
            idx = np.asarray(cur.slots, dtype=np.int64)
            same = (cur.slots == key and cur.input_tokens == toks and bool((table.epoch[idx] == cur.epochs).all())
                    and bool((table.length[idx] == cur.new_lengths).all()))
            if not same:
                self._ahead = cur
                self.flush()
                cur = None
        if cur is None:
            cur = self._launch(slots, toks, None, strict=True)
        nxt = None
        if not any(g.window is not None for g in self.stepper.cache.kv_groups):
            nxt = self._launch(slots, None, cur.cap, strict=False)      # tokens: this step's picks, on the device
        cur.done.synchronize()
        got = cur.host_out.tolist()
        if got[-1] != 0:
            self._ahead = nxt
            self.flush()
            self.stepper.check_status()
        if nxt is not None:
            nxt.input_tokens = got[:-1]
            self._ahead = nxt
        return got[:-1]

    def _run(self, slots, tokens: Optional[List[int]], feed: Optional[_Captured], strict: bool) -> Optional[_Captured]:
        """Puts one decode step on the stream.  ``tokens``: host token ids, or None to take the ids
        ``feed`` picked (on the device).  Not ``strict``: returns None instead of raising, with nothing
        changed, when the step cannot run (no page left, a sequence at its limit, no graph yet)."""
        st = self.stepper
        table = st.cache.table
        page = st.cache.page_size
        B = len(slots)
        try:
            if B == 0 or (tokens is not None and len(tokens) != B):
                raise StepError("one token per slot is needed")
            idx = np.asarray(slots, dtype=np.int64)
            if idx.min() < 0 or idx.max() >= table.max_slots or not table._in_use[idx].all():
                raise StepError("a slot of this step is not in use")
            if len(set(slots)) != B:
                raise StepError("a slot appears twice in one step")
            if tokens is not None:
                toks = np.asarray(tokens, dtype=np.int64)
                if toks.min() < 0 or toks.max() >= st.vocab_size:
                    raise StepError(f"a token id is outside the vocabulary [0, {st.vocab_size})")
            lens = table.length[idx].copy()
            if int(lens.max()) + 1 > st.max_position:
                raise StepError(f"a sequence would exceed the model's limit of {st.max_position} positions")
            cols = _bucket(int(-(-(int(lens.max()) + 1) // page)))
            cap = self.graphs.get((B, cols))
            if cap is None:
                if tokens is None:
                    return None                               # a new shape is captured with real tokens only
                cap = self._capture(slots, [[t] for t in tokens], cols)
                self.graphs[(B, cols)] = cap
                self.launches_last_step = cap.launches
                return cap
            # pages: a sequence needs a new one only when it stands at a page boundary
            for s in idx[table._reserved[idx] <= lens]:
                table.reserve(int(s), 1)
        except (StepError, CacheError):
            if strict:
                raise
            return None
        # the description, into the staging buffer that is not in flight
        cap.turn ^= 1
        k = cap.turn
        if cap.stage_events[k] is not None:
            cap.stage_events[k].synchronize()
        sn = cap.stages[k].numpy()
        o = cap.offsets
        if tokens is not None:
            sn[o[0]:o[0] + B] = toks
        sn[o[2]:o[2] + B] = lens
        sn[o[5]:o[5] + B] = lens + 1
        key = tuple(slots)
        if cap.stage_slots[k] != key:
            sn[o[1]:o[1] + B] = np.arange(B)
            sn[o[3]:o[3] + B + 1] = np.arange(B + 1)
            sn[o[4]:o[4] + B] = idx
            sn[o[6]:o[6] + B] = np.arange(B)
            cap.stage_slots[k] = key
        for g in range(len(st.cache.kv_groups)):
            t = table.tables[g]
            dst = sn[o[7 + g]:o[7 + g] + B * cols].reshape(B, cols)
            c = min(cols, t.shape[1])
            dst[:, :c] = t[idx, :c]
            if c < cols:
                dst[:, c:] = -1
        cap.buffer.copy_(cap.stages[k], non_blocking=True)
        if cap.stage_events[k] is None:
            cap.stage_events[k] = torch.cuda.Event()
        cap.stage_events[k].record()
        if tokens is None:
            cap.buffer[o[0]:o[0] + B].copy_(feed.out[:B])      # the previous step's picks, device to device
        self.last_upload_bytes = cap.buffer.numel() * 4
        cap.graph.replay()
        # the sequences are one position longer
        if any(g.window is not None for g in st.cache.kv_groups):
            for s in slots:
                table.commit(int(s), 1)
        else:
            table.length[idx] += 1
        self.launches_last_step = cap.launches
        return cap

    def _capture(self, slots, tokens, cols) -> _Captured:
        """The first step of a shape runs eagerly (it also compiles whatever the model still
        needs) and is then captured; capture does not execute, so the cache is written once more
        with the same values when the fresh graph is replayed."""
        st = self.stepper
        page = st.cache.page_size
        B = len(slots)
        n_groups = len(st.cache.kv_groups)
        offsets, sizes, total = field_offsets([B, B, B, B + 1, B, B, B] + [B * cols] * n_groups)
        buffer = torch.empty(total, dtype=torch.int32, device=st.runtime.device)
        ctx = st.prepare(slots, tokens, "last", into=buffer, table_cols=cols)
        ctx.kv_len_bound = cols * page
        torch.cuda.current_stream().synchronize()
        st.model.forward(ctx, st.cache)                      # eager warm-up: writes this step's keys and values
        torch.cuda.current_stream().synchronize()
        ctx.shared.clear()            # what the warm-up computed once per step has to be computed inside the graph too
        out = torch.empty(B + 1, dtype=torch.int32, device=st.runtime.device)
        pick_scratch = ops.argmax_scratch(st.runtime.device, fresh=True)      # this graph's own: its replays follow one another
        graph = torch.cuda.CUDAGraph()
        n0 = ops.launch_count()
        with torch.cuda.graph(graph):
            logits = st.model.forward(ctx, st.cache)
            ops.argmax(logits, out=out[:B], scratch=pick_scratch)
            out[B:].copy_(st.runtime.status)
        launches = ops.launch_count() - n0
        graph.replay()                                       # same tokens again: rewrites the same cache entries
        st.finish(ctx)
        stages = [torch.empty(total, dtype=torch.int32).pin_memory() for _ in range(2)]
        for s in stages:
            s.copy_(buffer)                                  # both start as the captured step's description
        torch.cuda.current_stream().synchronize()
        key = tuple(slots)
        return _Captured(graph, buffer, offsets, sizes, stages, [None, None], [key, key], logits, out, launches, pick_scratch)

    # -- used by the generation loop -------------------------------------------------------------
    def step_and_sample(self, slots, tokens, streams, counters, recent, sampler) -> List[int]:
        o = sampler.options
        if o.greedy and (o.rep_pen == 1.0 or not any(len(r) for r in recent)):
            return self.greedy_step(slots, tokens)
        logits, _ = self.step(slots, tokens)
        host = sampler.sample(logits, streams, counters, recent).cpu()
        self.stepper.check_status()
        return host.tolist()
