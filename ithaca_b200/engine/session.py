"""A sequence that outlives one call to generate: the next prompt reuses the cache of the prefix it shares.

The reference's ``Chat`` keeps the token ids its model's cache holds (``cache_``, src/chat.h:58).  Each turn it
counts how many leading tokens of the new prompt equal that record, rewinds the model to there and evaluates only
the rest (src/chat.cpp:311-318); a model with recurrent state starts over instead (src/model.cpp:1047-1055).  A
``Session`` is that for one slot of the engine's cache, beside whatever else the engine is serving.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

from ..cache.pages import CacheError
from .generate import GenerationOptions


class Session:
    def __init__(self, engine):
        self.engine = engine
        self.slot: Optional[int] = engine.alloc_slot()
        self.tokens: List[int] = []          # the token ids whose keys and values the slot holds, in order
        self.reused_last = 0

    def close(self) -> None:
        if self.slot is not None:
            self.engine.free_slot(self.slot)
            self.slot = None
            self.tokens = []

    def __enter__(self) -> "Session":
        return self

    def __exit__(self, *exc) -> bool:
        self.close()
        return False

    def shared_prefix(self, prompt: Sequence[int]) -> int:
        """Leading tokens of ``prompt`` that the slot holds; at most len(prompt) - 1, because the prompt's
        last token has to be evaluated to give the first logits (src/chat.cpp:313-314)."""
        n = 0
        limit = min(len(self.tokens), len(prompt))
        while n < limit and self.tokens[n] == prompt[n]:
            n += 1
        return min(n, len(prompt) - 1)

    def generate(self, prompt: Sequence[int], options: Optional[GenerationOptions] = None,
                 on_token: Optional[Callable[[int], bool]] = None, **kw) -> List[int]:
        """Generates behind ``prompt`` (the whole conversation so far, as token ids).  What the slot holds of
        it is kept; the rest is evaluated.  Returns the new ids; ``reused_last`` says how many positions
        were found in the cache."""
        if self.slot is None:
            raise CacheError("this session is closed")
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        eng = self.engine
        keep = self.shared_prefix(prompt)
        try:
            eng.truncate(self.slot, keep)
        except CacheError:
            # fixed-size state cannot be rolled back, and a window may have let go of what the cut needs:
            # start over, as the reference does for a recurrent model
            keep = 0
            eng.truncate(self.slot, 0)
        self.tokens = self.tokens[:keep]
        cb = None if on_token is None else (lambda request, tok: on_token(tok))
        try:
            out = eng.generate([list(prompt)], options, on_token=cb, resume=[(self.slot, keep)], **kw)[0]
        except BaseException:
            # the slot's contents are unknown now: forget them
            self.tokens = []
            eng.truncate(self.slot, 0)
            raise
        self.reused_last = keep
        self.tokens = (list(prompt) + out)[:eng.length(self.slot)]       # the last sampled token was not evaluated
        return out
