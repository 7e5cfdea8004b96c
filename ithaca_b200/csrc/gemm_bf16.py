"""Products with bfloat16 operands and float accumulation: which kernel takes which shape.

* up to 16 tokens: the skinny warp-level kernel (weights streamed once, no wasted tensor work);
* more tokens: the tcgen05 kernel (TMA-fed, accumulators in TMEM), for decode batches and prefill;
* K not a multiple of 8 or unaligned rows: the CUDA-core product, which takes anything.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

SKINNY_MAX_TOKENS = 16


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
         out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    if x.shape[0] <= SKINNY_MAX_TOKENS:
        done = ops.gemm_bf16_mma(x, w, out=out, accumulate=accumulate, kind=1)
    else:
        done = ops.gemm_tcgen05(x, w, out=out, accumulate=accumulate, status=ops.device_status(x.device))
    if done is None:
        ops.gemm_simt(x, w, out=out, accumulate=accumulate)
    return out
