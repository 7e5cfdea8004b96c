"""What one step tells the kernels: which tokens, whose they are, where they sit.

All of it is small int32 data.  It is assembled on the host into one pinned
buffer and reaches the device in one copy; the fields below are views of that
device buffer.  Positions are implied by the cache: token k of a sequence sits at
the sequence's length before the step plus k.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    n_logit_rows: int
    token_ids: torch.Tensor            # [T]
    token_seq: torch.Tensor            # [T] index of the token's sequence in this step
    token_pos: torch.Tensor            # [T] absolute position
    cu_seqlens: torch.Tensor           # [B + 1] first token of each sequence
    slots: torch.Tensor                # [B]
    kv_lens: torch.Tensor              # [B] positions each sequence holds after this step
    logit_rows: torch.Tensor           # [R] token indices whose logits are wanted
    tables: List[torch.Tensor]         # per key/value group: [B, pages] block table
    is_decode: bool                    # every sequence brings exactly one token
    max_new: int
    max_kv_len: int
    kv_len_bound: int = 0              # no sequence is longer than this (sizes grids; >= max_kv_len)
    host_slots: List[int] = field(default_factory=list)
    host_n_new: List[int] = field(default_factory=list)
    host_kv_lens: List[int] = field(default_factory=list)
    shared: dict = field(default_factory=dict)     # what the layers of one step compute once and share (rotary tables)


def field_offsets(sizes):
    """Where each field of a step's description starts in the packed int32 buffer: every field on a
    16-byte boundary.  Returns (offsets, sizes, total length)."""
    offs, total = [], 0
    for n in sizes:
        offs.append(total)
        total += (n + 3) // 4 * 4
    return offs, list(sizes), max(total, 4)


class ContextBuilder:
    """Reusable pinned staging so that a step costs one host-to-device copy."""

    def __init__(self, device: str):
        self.device = device
        self.last_upload_bytes = 0
        self._pinned: Optional[torch.Tensor] = None
        self._copied: Optional[torch.cuda.Event] = None      # the last upload from the staging buffer

    def _staging(self, n: int) -> torch.Tensor:
        if self._pinned is None or self._pinned.numel() < n:
            cap = max(4096, 1 << (n - 1).bit_length())
            self._pinned = torch.empty(cap, dtype=torch.int32).pin_memory()
        return self._pinned

    def build(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], start: Sequence[int],
              want: Sequence[Sequence[int]], tables: Sequence[np.ndarray],
              into: Optional[torch.Tensor] = None) -> StepContext:
        """``start[b]``: positions sequence b holds before the step.  ``tables[g]``: the
        [B, pages] block table of group g (pages already reserved for the new tokens).
        ``into``: a device buffer to fill instead of a fresh one (its layout must be the
        same as at its first use; CUDA graphs replay on it)."""
        B = len(slots)
        n_new = [len(t) for t in tokens]
        T = int(sum(n_new))
        cu = np.zeros(B + 1, dtype=np.int32)
        cu[1:] = np.cumsum(n_new)
        token_ids = np.fromiter((x for t in tokens for x in t), dtype=np.int32, count=T)
        token_seq = np.repeat(np.arange(B, dtype=np.int32), n_new)
        token_pos = (np.arange(T, dtype=np.int32) - cu[token_seq] + np.asarray(start, dtype=np.int32)[token_seq])
        rows = np.fromiter((cu[b] + w for b in range(B) for w in want[b]), dtype=np.int32)
        kv_lens = np.asarray(start, dtype=np.int32) + np.asarray(n_new, dtype=np.int32)
        parts = [token_ids, token_seq, token_pos, cu, np.asarray(slots, dtype=np.int32), kv_lens, rows]
        parts += [np.ascontiguousarray(t, dtype=np.int32).reshape(-1) for t in tables]
        offs, sizes, total = field_offsets([p.size for p in parts])
        if self._copied is not None:
            self._copied.synchronize()                        # the staging buffer is free again
        stage = self._staging(total)
        sn = stage.numpy()
        for p, o in zip(parts, offs):
            sn[o:o + p.size] = p
        if into is None:
            dev = torch.empty(total, dtype=torch.int32, device=self.device)
        else:
            if into.numel() < total:
                raise ValueError("the context buffer is too small for this step")
            dev = into
        dev[:total].copy_(stage[:total], non_blocking=True)
        if self._copied is None:
            self._copied = torch.cuda.Event()
        self._copied.record()
        self.last_upload_bytes = total * 4

        def view(i):
            return dev[offs[i]:offs[i] + sizes[i]]

        tabs = [view(7 + g).view(B, tables[g].shape[1]) for g in range(len(tables))]
        return StepContext(
            n_tokens=T, n_seqs=B, n_logit_rows=int(rows.size), token_ids=view(0), token_seq=view(1),
            token_pos=view(2), cu_seqlens=view(3), slots=view(4), kv_lens=view(5), logit_rows=view(6), tables=tabs,
            is_decode=all(n == 1 for n in n_new), max_new=max(n_new) if n_new else 0,
            max_kv_len=int(kv_lens.max()) if B else 0, kv_len_bound=int(kv_lens.max()) if B else 0, host_slots=list(slots), host_n_new=n_new,
            host_kv_lens=[int(x) for x in kv_lens])
