"""Sampling options and their device kernels.

Names, defaults and meanings follow the reference's ``GenOpts`` and
``Chat::sample`` (src/chat.h:10-16, src/chat.cpp:124-145): ``temp`` (<= 0 takes
the largest logit), ``top_k`` (clamped to [1, vocab]), ``top_p``, ``rep_pen``
(applied to each of the last 64 generated ids, once per occurrence, before
anything else -- also before the greedy pick).  The command line's default
temperature is 0, as the reference's (src/main.cpp:944).  The reference seeds its
generator from the system and offers no seed; here ``seed`` fixes the draws:
the uniform number of (sequence ``stream``, generated token ``counter``) is
Philox-4x32-10(seed; counter, stream), so a sequence's draws do not depend on
what else is in its batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..csrc import ops

RECENT_WINDOW = 64      # src/chat.cpp:479: the penalty covers the last 64 generated ids


@dataclass(frozen=True)
class SamplingOptions:
    temp: float = 0.0
    top_k: int = 40
    top_p: float = 0.9
    rep_pen: float = 1.1
    seed: int = 0

    def validate(self) -> None:
        if not self.rep_pen > 0:
            raise ValueError(f"rep_pen must be > 0, found {self.rep_pen}")
        if not self.top_p > 0:
            raise ValueError(f"top_p must be > 0, found {self.top_p}")

    @property
    def greedy(self) -> bool:
        return self.temp <= 0


class Sampler:
    def __init__(self, options: SamplingOptions, device: str):
        options.validate()
        self.options = options
        self.device = device

    def sample(self, logits: torch.Tensor, streams: Sequence[int], counters: Sequence[int],
               recent: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """One id per row of ``logits`` (device int32).  ``recent[r]``: the ids the penalty
        covers for row r, oldest first (at most the last 64 are used)."""
        o = self.options
        rows = logits.shape[0]
        if o.greedy and (o.rep_pen == 1.0 or recent is None or not any(len(r) for r in recent)):
            return ops.argmax(logits)
        rec = None
        if o.rep_pen != 1.0 and recent is not None and any(len(r) for r in recent):
            host = torch.full((rows, RECENT_WINDOW), -1, dtype=torch.int32)
            for r, ids in enumerate(recent):
                ids = list(ids)[-RECENT_WINDOW:]
                if ids:
                    host[r, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
            rec = host.to(self.device, non_blocking=True)
        st = torch.tensor(list(streams), dtype=torch.int32).to(self.device, non_blocking=True)
        ct = torch.tensor(list(counters), dtype=torch.int32).to(self.device, non_blocking=True)
        return ops.sample(logits, o.temp, o.top_k, o.top_p, o.rep_pen, rec, o.seed, st, ct)
