"""A weight matrix and the product with it: y = x W^T, W stored [out, in] as the
reference binds it (rows = out features, cols = in features, src/model.cpp:33).

Which kernel runs depends on the runtime's dtype and the shape:

* float32 path: the CUDA-core product (true 32-bit arithmetic, ascending-k sums);
  the weight stays as stored (bfloat16 is widened exactly when it is loaded).
* bfloat16 path: 16-bit operands with float accumulation.  A weight stored in
  32-bit is rounded to bfloat16 once, here, because this path's products are 16-bit.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..csrc import ops
from .base import Runtime, to_device


class Linear:
    def __init__(self, weights: Sequence[torch.Tensor], runtime: Runtime):
        """``weights``: one matrix, or several with equal ``in`` that are stacked along
        ``out`` so that one product serves them all (q/k/v; gate/up)."""
        ws = [to_device(w, runtime) for w in weights]
        if runtime.dtype == "bfloat16":
            ws = [w.to(torch.bfloat16) for w in ws]
        elif len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.weight = ws[0].contiguous() if len(ws) == 1 else torch.cat(ws, dim=0).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.runtime = runtime

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                 out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise ValueError(f"linear: input has {x.shape[-1]} features, the weight takes {self.in_features}")
        return gemm(x, self.weight, out=out, accumulate=accumulate, out_dtype=out_dtype)


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
         out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Dispatch by operand type and shape.  Every branch is this library's own kernel."""
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from ..csrc import gemm_bf16
        return gemm_bf16.gemm(x, w, out=out, accumulate=accumulate, out_dtype=out_dtype)
    return ops.gemm_simt(x, w, out=out, accumulate=accumulate, out_dtype=out_dtype)
