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


def gemm_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """h = silu(x Wg^T) * (x Wu^T) in one kernel.  ``w_interleaved``: [2 ff, d] with gate j in row 2j and
    up j in row 2j + 1, so that a product tile holds both halves of every pair it covers and the
    [tokens, 2 ff] intermediate is never written."""
    M, ff = x.shape[0], w_interleaved.shape[0] // 2
    out = torch.empty((M, ff), dtype=out_dtype, device=x.device)
    if M <= SKINNY_MAX_TOKENS:
        done = ops.gemm_bf16_mma(x, w_interleaved, out=out, kind=1, swiglu=True)
    else:
        done = ops.gemm_tcgen05(x, w_interleaved, out=out, status=ops.device_status(x.device), swiglu=True)
    if done is None:
        gu = ops.gemm_simt(x, w_interleaved, out_dtype=torch.float32)
        ops.swiglu(gu, out_dtype, out=out, interleaved=True)
    return out
