"""The generation loop above the step function.

The reference's loop serves one sequence (src/chat.cpp:292-492): evaluate the
prompt, then sample, check for a stop token, evaluate the token, until the budget
is spent.  The stop token is neither emitted nor evaluated (:447), and the last
sampled token is not evaluated (:489).  Here the same loop serves batches: all
prompts of a batch in one step (unequal lengths), then one token for each
sequence that is still running; a sequence that ends leaves the batch at once and
its slot and pages go back to the cache; when a batch is empty the next requests
form the next batch, in slots that are used again.

The loop's decisions (who is in a batch, who has ended, what the budget is) use
only the small ``Backend`` interface, so they are testable without a device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Protocol, Sequence

from ..sampling.sampler import RECENT_WINDOW, SamplingOptions


@dataclass(frozen=True)
class GenerationOptions:
    """``max_tokens``, ``temp``, ``top_k``, ``top_p``, ``rep_pen`` are the reference's
    ``GenOpts`` (src/chat.h:10-16) with the command line's defaults ``-n 128`` and
    ``--temp 0`` (src/main.cpp:944).  The others are this library's."""
    max_tokens: int = 128
    temp: float = 0.0
    top_k: int = 40
    top_p: float = 0.9
    rep_pen: float = 1.1
    seed: int = 0
    stop_token_ids: Optional[Sequence[int]] = None     # None: the model's own (eos_token_id)
    include_stop: bool = False                         # the reference does not emit the stop token
    max_batch: Optional[int] = None                    # None: as many as the cache has slots and room for

    def sampling(self) -> SamplingOptions:
        return SamplingOptions(self.temp, self.top_k, self.top_p, self.rep_pen, self.seed)


@dataclass
class GenStats:
    """The reference's ``GenStats`` (src/chat.h:27) summed over the requests."""
    prompt_tokens: int = 0
    gen_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    batches: int = 0
    steps: int = 0
    reused_tokens: int = 0          # prompt positions found in the cache (src/chat.h:27 ``reused``)

    @property
    def prefill_tps(self) -> float:
        return self.prompt_tokens / max(1e-9, self.prefill_seconds)

    @property
    def gen_tps(self) -> float:
        return self.gen_tokens / max(1e-9, self.decode_seconds)


class Backend(Protocol):
    context_length: int          # the most positions one sequence may hold

    def room_for(self, lengths: Sequence[int], slots: Optional[Sequence[Optional[int]]] = None) -> bool:
        """Can sequences that will grow to these lengths live at the same time?  ``slots[i]`` names the slot
        sequence i already lives in (what that slot holds needs no new room), or None."""

    def free_slots(self) -> int: ...
    def alloc_slot(self) -> int: ...
    def free_slot(self, slot: int) -> None: ...

    def step_and_sample(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], streams: Sequence[int],
                        counters: Sequence[int], recent: Sequence[Sequence[int]]) -> List[int]:
        """Runs one step and returns one sampled id per slot."""


@dataclass
class _Running:
    request: int
    slot: int
    budget: int
    cached: int = 0            # positions of the prompt that the slot held already (a resumed request)
    owned: bool = True         # the loop took the slot and gives it back; a resumed request's slot is its caller's
    out: List[int] = field(default_factory=list)
    recent: List[int] = field(default_factory=list)
    next_token: int = -1


def budget_for(prompt_len: int, max_tokens: int, context_length: int) -> int:
    """New tokens a request may get: what it asks for, cut to what the context leaves
    (src/chat.cpp:308).  The reference also raises small requests to 64 and caps at
    half the context (:295); a library call gets what it asks for."""
    return max(0, min(max_tokens, context_length - prompt_len))


def next_batch(pending: Sequence[int], prompts: Sequence[Sequence[int]], budgets: Sequence[int], backend: Backend,
               max_batch: Optional[int], resume: Optional[Sequence[Optional[tuple]]] = None) -> List[int]:
    """The longest run of pending requests, in order, that fits the free slots and the
    cache when every one of them grows to its full budget.  A resumed request brings its slot."""
    chosen: List[int] = []
    fresh = 0
    for r in pending:
        held = resume[r][0] if resume is not None and resume[r] is not None else None
        if max_batch is not None and len(chosen) >= max_batch:
            break
        if held is None and fresh >= backend.free_slots():
            break
        grown = [len(prompts[c]) + budgets[c] for c in chosen + [r]]
        if resume is None:
            fits = backend.room_for(grown)
        else:
            fits = backend.room_for(grown, [resume[c][0] if resume[c] is not None else None for c in chosen + [r]])
        if not fits:
            break
        chosen.append(r)
        fresh += held is None
    return chosen


def generate_loop(prompts: Sequence[Sequence[int]], options: GenerationOptions, backend: Backend,
                  stop_token_ids: Sequence[int] = (), on_token: Optional[Callable[[int, int], bool]] = None,
                  clock: Callable[[], float] = time.perf_counter,
                  resume: Optional[Sequence[Optional[tuple]]] = None):
    """Returns (generated ids per request, GenStats).  ``on_token(request, id)`` may
    return False to end that request (the reference's ``on_text`` callback, src/chat.cpp:481).

    ``resume[r] = (slot, n)``: request r goes on in a slot its caller holds, whose first n positions
    are the first n tokens of its prompt already (the reference's reuse of the cache for a shared
    prefix, src/chat.cpp:311-318): only the rest of the prompt is evaluated, and the slot stays
    with the caller when the request ends.  n must be less than the prompt's length."""
    stops = set(options.stop_token_ids if options.stop_token_ids is not None else stop_token_ids)
    ctx = backend.context_length
    for n, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {n}: empty prompt")                    # src/chat.cpp:298
        if len(p) > ctx:
            raise ValueError(f"request {n}: the prompt of {len(p)} tokens is longer than the context of {ctx}")
        if resume is not None and resume[n] is not None and not 0 <= resume[n][1] < len(p):
            raise ValueError(f"request {n}: {resume[n][1]} cached positions do not leave a token of the prompt to evaluate")
    budgets = [budget_for(len(p), options.max_tokens, ctx) for p in prompts]
    results: List[List[int]] = [[] for _ in prompts]
    stats = GenStats()
    pending = list(range(len(prompts)))

    def settle(run: _Running, tok: int) -> bool:
        """Takes the sampled token; True if the sequence goes on."""
        if tok in stops:
            if options.include_stop:
                run.out.append(tok)
            return False
        run.out.append(tok)
        stats.gen_tokens += 1
        run.recent.append(tok)
        if len(run.recent) > RECENT_WINDOW:
            del run.recent[0]
        if on_token is not None and on_token(run.request, tok) is False:
            return False
        if len(run.out) >= run.budget:
            return False
        run.next_token = tok
        return True

    while pending:
        batch = next_batch(pending, prompts, budgets, backend, options.max_batch, resume)
        if not batch:
            raise RuntimeError(f"request {pending[0]} does not fit the cache even alone "
                               f"({len(prompts[pending[0]])} prompt tokens + {budgets[pending[0]]} new)")
        pending = pending[len(batch):]
        stats.batches += 1
        running = []
        for r in batch:
            if resume is not None and resume[r] is not None:
                running.append(_Running(r, resume[r][0], budgets[r], cached=resume[r][1], owned=False))
            else:
                running.append(_Running(r, backend.alloc_slot(), budgets[r]))
        try:
            # requests with no budget produce nothing and need no step
            for run in [x for x in running if x.budget == 0 and x.owned]:
                backend.free_slot(run.slot)
            running = [x for x in running if x.budget > 0]
            if running:
                t0 = clock()
                toks = backend.step_and_sample([x.slot for x in running],
                                               [list(prompts[x.request][x.cached:]) for x in running],
                                               [x.request for x in running], [0] * len(running),
                                               [x.recent for x in running])
                stats.prefill_seconds += clock() - t0
                stats.prompt_tokens += sum(len(prompts[x.request]) - x.cached for x in running)
                stats.reused_tokens += sum(x.cached for x in running)
                stats.steps += 1
                t1 = clock()
                while True:
                    still = []
                    for run, tok in zip(running, toks):
                        if settle(run, int(tok)):
                            still.append(run)
                        else:
                            results[run.request] = run.out
                            if run.owned:
                                backend.free_slot(run.slot)
                            run.slot = -1
                    running = still
                    if not running:
                        break
                    toks = backend.step_and_sample([x.slot for x in running], [[x.next_token] for x in running],
                                                   [x.request for x in running], [len(x.out) for x in running],
                                                   [x.recent for x in running])
                    stats.steps += 1
                stats.decode_seconds += clock() - t1
        finally:
            for run in running:
                if run.slot >= 0 and run.owned:
                    backend.free_slot(run.slot)
    return results, stats
