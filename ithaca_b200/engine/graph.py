"""Decode steps replayed from CUDA graphs.

A decode step is some hundreds of small launches; issued one by one from Python
they cost more than the step itself.  The reference captures its whole
single-token forward into one graph and replays it, reading the position from
device memory (src/model.cpp:1341-1350, src/cuda_tier.cpp:630-651).  Here a graph
is captured per (number of sequences, block-table width): the step's description
(tokens, positions, lengths, block tables) lives in one device buffer that is
refilled before each replay, so the same graph serves every step of that shape.
The graph covers the forward pass and, for greedy sampling, the argmax.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..csrc import ops
from .context import StepContext
from .step import Stepper


@dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    buffer: torch.Tensor
    logits: torch.Tensor
    ids: torch.Tensor
    launches: int


def _bucket(cols: int) -> int:
    """Block-table widths are rounded up so that a growing sequence re-captures rarely."""
    b = 4
    while b < cols:
        b *= 2
    return b


class GraphDecoder:
    def __init__(self, stepper: Stepper):
        self.stepper = stepper
        self.graphs: Dict[Tuple[int, int], _Captured] = {}
        self.launches_last_step = 0

    def _table_cols(self, slots: Sequence[int]) -> int:
        page = self.stepper.cache.page_size
        need = max(-(-(self.stepper.cache.length(s) + 1) // page) for s in slots)
        return _bucket(need)

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]]) -> Tuple[torch.Tensor, torch.Tensor]:
        """One token per slot.  Returns (logits [B, vocab], argmax ids [B]); both are the
        graph's own buffers and are overwritten by the next step of the same shape."""
        st = self.stepper
        B = len(slots)
        cols = self._table_cols(slots)
        key = (B, cols)
        cap = self.graphs.get(key)
        if cap is None:
            cap = self._capture(slots, tokens, cols)
            self.graphs[key] = cap
            self.launches_last_step = cap.launches
            return cap.logits, cap.ids
        ctx = st.prepare(slots, tokens, "last", into=cap.buffer, table_cols=cols)
        cap.graph.replay()
        st.finish(ctx)
        self.launches_last_step = cap.launches
        return cap.logits, cap.ids

    def _capture(self, slots, tokens, cols) -> _Captured:
        """The first step of a shape runs eagerly (it also compiles whatever the model still
        needs) and is then captured; capture does not execute, so the cache is written once."""
        st = self.stepper
        page = st.cache.page_size
        probe = st.prepare(slots, tokens, "last", table_cols=cols)
        buffer = torch.empty(max(self._buffer_size(probe), 4), dtype=torch.int32, device=st.runtime.device)
        ctx = st.prepare(slots, tokens, "last", into=buffer, table_cols=cols)
        ctx.kv_len_bound = cols * page
        torch.cuda.current_stream().synchronize()
        st.model.forward(ctx, st.cache)                      # eager warm-up: writes this step's keys and values
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = ops.launch_count()
        with torch.cuda.graph(graph):
            logits = st.model.forward(ctx, st.cache)
            ids = ops.argmax(logits)
        launches = ops.launch_count() - n0
        graph.replay()                                       # same tokens again: rewrites the same cache entries
        st.finish(ctx)
        return _Captured(graph, buffer, logits, ids, launches)

    @staticmethod
    def _buffer_size(ctx: StepContext) -> int:
        n = 0
        for t in [ctx.token_ids, ctx.token_seq, ctx.token_pos, ctx.cu_seqlens, ctx.slots, ctx.kv_lens, ctx.logit_rows,
                  *ctx.tables]:
            n += (t.numel() + 3) // 4 * 4
        return n

    def step_and_sample(self, slots, tokens, streams, counters, recent, sampler) -> torch.Tensor:
        logits, ids = self.step(slots, tokens)
        o = sampler.options
        if o.greedy and (o.rep_pen == 1.0 or not any(len(r) for r in recent)):
            return ids
        return sampler.sample(logits, streams, counters, recent)
