"""Products with bfloat16 operands and float accumulation: which kernel takes which shape.

* up to 8 tokens, and up to 16 for matrices under 96 MB: the skinny warp-level kernel (weights streamed once, no
  wasted tensor work);
* otherwise: the tcgen05 kernel (TMA-fed, accumulators in TMEM), for decode batches and prefill;
* K not a multiple of 8 or unaligned rows: the CUDA-core product, which takes anything.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

SKINNY_MAX_TOKENS = 16
SKINNY_FULL_TOKENS = 8            # one 8-token column tile: the skinny kernel at its best
BIG_WEIGHT_BYTES = 96e6


def takes_skinny(n_tokens: int, n_out: int, n_in: int) -> bool:
    """Up to 8 tokens the skinny kernel streams every weight at the copy rate.  With 9-16 tokens (two column tiles,
    half the loads in flight per thread) it falls behind the tcgen05 kernel on the large matrices (measured on B200,
    12 tokens: gate/up 28672 x 4096 61 against 39 us, down 4096 x 14336 30 against 25 us) and stays ahead on the
    small ones (q/k/v 13 against 14 us, output 11 against 12 us), whose time is start-up and tail."""
    if n_tokens <= SKINNY_FULL_TOKENS:
        return True
    return n_tokens <= SKINNY_MAX_TOKENS and 2.0 * n_out * n_in < BIG_WEIGHT_BYTES


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
         out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    if takes_skinny(x.shape[0], w.shape[0], w.shape[1]):
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
    if takes_skinny(M, w_interleaved.shape[0], w_interleaved.shape[1]):
        done = ops.gemm_bf16_mma(x, w_interleaved, out=out, kind=1, swiglu=True)
    else:
        done = ops.gemm_tcgen05(x, w_interleaved, out=out, status=ops.device_status(x.device), swiglu=True)
    if done is None:
        gu = ops.gemm_simt(x, w_interleaved, out_dtype=torch.float32)
        ops.swiglu(gu, out_dtype, out=out, interleaved=True)
    return out
