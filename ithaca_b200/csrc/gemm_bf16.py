"""Products with bfloat16 operands and float accumulation: which kernel takes which shape."""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
         out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return ops.gemm_simt(x, w, out=out, accumulate=accumulate, out_dtype=out_dtype)
