"""Products with bfloat16 operands and float accumulation: which kernel takes which shape."""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
         out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    done = ops.gemm_bf16_mma(x, w, out=out, accumulate=accumulate)
    if done is None:        # K not a multiple of 8 or unaligned rows: the CUDA-core product takes anything
        ops.gemm_simt(x, w, out=out, accumulate=accumulate)
    return out
