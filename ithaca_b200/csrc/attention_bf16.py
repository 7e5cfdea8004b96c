"""Attention kernels for the bfloat16 path: which kernel takes which shape."""
from __future__ import annotations

from typing import Optional

import torch


def attend(q, k_pages, v_pages, ctx, table, n_heads: int, scale: float, window: int,
           status) -> Optional[torch.Tensor]:
    """Returns None when no specialised kernel takes these sizes (the caller then uses the
    CUDA-core kernel)."""
    return None
