"""The step function: a batch of sequences, each bringing its next tokens.

The reference's ``Model::eval(toks, n)`` appends n tokens of its single sequence
and returns the last token's logits; ``eval_all`` returns all n rows
(src/model.h:85-90, src/model.cpp:1312).  Here one call serves a batch: every
sequence brings one or more tokens (all prompts in one step, then one token each;
mixtures are legal), the step runs exactly those tokens as one batch against the
cache that earlier steps left, and returns float32 logits at the wanted places.

Nothing is padded: activations are token-major [T, ...] with T the number of
tokens the step brings, so what else is in the batch cannot change a row.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.cache import SequenceCache
from ..cache.pages import CacheError
from .context import ContextBuilder, StepContext


class StepError(ValueError):
    pass


class Stepper:
    def __init__(self, model, cache: SequenceCache, max_position: Optional[int] = None,
                 max_step_tokens: Optional[int] = None):
        """``max_step_tokens``: the workspace limit.  A step that brings more tokens is run as
        several passes of at most that many, cut along the token-major order; the result is the
        same (bit for bit in float32, to rounding in bfloat16).  The reference cuts a prompt into
        pieces of at most 512 tokens (src/model.cpp:1364-1368)."""
        if max_step_tokens is not None and max_step_tokens < 1:
            raise ValueError("max_step_tokens must be positive")
        self.max_step_tokens = max_step_tokens
        self.passes_last_step = 0
        self.model = model
        self.cache = cache
        self.runtime = model.runtime
        self.vocab_size = model.spec.vocab_size
        self.max_position = max_position if max_position is not None else model.spec.max_position
        self.builder = ContextBuilder(self.runtime.device)

    # -- validation (host only; nothing has changed when it raises) ----------------------------
    def _validate(self, slots, tokens, want) -> List[List[int]]:
        if len(slots) != len(tokens):
            raise StepError("one token list per slot is needed")
        if len(set(slots)) != len(slots):
            raise StepError("a slot appears twice in one step")
        for s, t in zip(slots, tokens):
            if not self.cache.table.in_use(s):
                raise StepError(f"slot {s} is not in use")
            if len(t) < 1:
                raise StepError(f"slot {s} brings no token")
            lo, hi = min(t), max(t)
            if lo < 0 or hi >= self.vocab_size:
                raise StepError(f"slot {s}: token id {lo if lo < 0 else hi} is outside the vocabulary [0, {self.vocab_size})")
            end = self.cache.length(s) + len(t)
            if end > self.max_position:
                raise StepError(f"slot {s}: {end} positions exceed the model's limit of {self.max_position}")
        if want == "last":
            return [[len(t) - 1] for t in tokens]
        if want == "all":
            return [list(range(len(t))) for t in tokens]
        if want is None:
            return [[] for _ in tokens]
        if len(want) != len(tokens):
            raise StepError("one list of wanted places per slot is needed")
        out = []
        for s, t, w in zip(slots, tokens, want):
            w = [int(x) for x in w]
            if any(x < 0 or x >= len(t) for x in w):
                raise StepError(f"slot {s}: a wanted place lies outside its {len(t)} tokens")
            out.append(w)
        return out

    def prepare(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
                want: Union[str, None, Sequence[Sequence[int]]] = "last",
                into: Optional[torch.Tensor] = None, table_cols: Optional[int] = None) -> StepContext:
        """Validates, reserves pages and uploads the step's description."""
        want_lists = self._validate(slots, tokens, want)
        n_new = [len(t) for t in tokens]
        self.cache.reserve(slots, n_new)
        start = [self.cache.length(s) for s in slots]
        page = self.cache.page_size
        cols = max(1, max(-(-(st + n) // page) for st, n in zip(start, n_new)))
        if table_cols is not None:
            if table_cols < cols:
                raise StepError("the block table is narrower than the longest sequence")
            cols = table_cols
        tables = [self.cache.table.table_rows(g, slots, cols) for g in range(len(self.cache.kv_groups))]
        return self.builder.build(slots, tokens, start, want_lists, tables, into=into)

    def finish(self, ctx: StepContext) -> None:
        self.cache.commit(ctx.host_slots, ctx.host_n_new)

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Union[str, None, Sequence[Sequence[int]]] = "last") -> Optional[torch.Tensor]:
        """Runs the tokens and returns float32 logits [wanted, vocab] on the device (None if
        nothing is wanted), rows in the order of the slots and of each slot's wanted places."""
        if self.max_step_tokens is not None and sum(len(t) for t in tokens) > self.max_step_tokens:
            return self._step_in_passes(slots, tokens, want)
        ctx = self.prepare(slots, tokens, want)
        logits = self.model.forward(ctx, self.cache)
        self.finish(ctx)
        self.passes_last_step = 1
        return logits

    def _step_in_passes(self, slots, tokens, want) -> Optional[torch.Tensor]:
        """A step over the workspace limit: the flat token list is cut every ``max_step_tokens`` tokens;
        each pass runs its pieces of sequences as an ordinary step behind what the passes before left
        in the cache.  Everything is checked and every page taken before the first pass runs."""
        want_lists = self._validate(slots, tokens, want)
        self.cache.reserve(slots, [len(t) for t in tokens])
        limit = self.max_step_tokens
        passes: List[List[tuple]] = [[]]                    # per pass: (sequence index, first token, end)
        room = limit
        for b, t in enumerate(tokens):
            lo = 0
            while lo < len(t):
                if room == 0:
                    passes.append([])
                    room = limit
                hi = min(len(t), lo + room)
                passes[-1].append((b, lo, hi))
                room -= hi - lo
                lo = hi
        outs: List[torch.Tensor] = []
        where = {}                                          # (sequence, index in its want list) -> row of the passes' outputs
        row = 0
        for pieces in passes:
            piece_want = []
            for b, lo, hi in pieces:
                idx = [i for i, w in enumerate(want_lists[b]) if lo <= w < hi]
                piece_want.append([want_lists[b][i] - lo for i in idx])
                for i in idx:
                    where[(b, i)] = row
                    row += 1
            ctx = self.prepare([slots[b] for b, _, _ in pieces], [tokens[b][lo:hi] for b, lo, hi in pieces], piece_want)
            out = self.model.forward(ctx, self.cache)
            self.finish(ctx)
            if out is not None:
                outs.append(out)
        self.passes_last_step = len(passes)
        if not outs:
            return None
        logits = outs[0] if len(outs) == 1 else torch.cat(outs, 0)
        order = [where[(b, i)] for b in range(len(tokens)) for i in range(len(want_lists[b]))]
        if order != list(range(len(order))):
            logits = logits[torch.as_tensor(order, dtype=torch.long, device=logits.device)]
        return logits

    def check_status(self) -> None:
        """Reads the word in which kernels record what they refused to do (this waits for the
        device) and clears it.  The kernels skip such an access; the results of the steps since
        the last check are not to be used."""
        st = self.runtime.status
        if st is not None:
            v = int(st.item())
            if v != 0:
                st.zero_()
                raise CacheError("a kernel reported " + describe_status(v) + wait_detail(v))


STATUS_EVENTS = {1: "a token id outside the vocabulary", 2: "a cache write without a page",
                 3: "a cache read without a page", 4: "a matrix-product block that gave up waiting for its data",
                 5: "shared memory that is not aligned for the tensor-core tiles"}


def wait_detail(word: int) -> str:
    """For a wait that ran out: which wait of which kernel it was."""
    if not word & (1 << 3):
        return ""
    from ..csrc import ops
    where = ops.wait_records()
    return f" [{where}]" if where else ""


def describe_status(word: int) -> str:
    """The status word holds one bit per kind of event (bit code - 1)."""
    found = [what for code, what in STATUS_EVENTS.items() if word & (1 << (code - 1))]
    rest = word & ~sum(1 << (c - 1) for c in STATUS_EVENTS)
    if rest:
        found.append(f"unknown bits {rest:#x}")
    return "; ".join(found)
