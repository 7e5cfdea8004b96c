"""RMS norm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, in float32
(src/model.cpp:626-633; GPU kernel src/gpu_kernels.cpp:1177-1195)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, as_float32, register_norm


class RMSNorm:
    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        return {spec.weights["weight"]: TensorReq((spec["size"],), init="ones")}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = as_float32(tensors[spec.weights["weight"]], runtime)
        self.runtime = runtime

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype or self.runtime.act_dtype, rows_in=rows)


register_norm("rmsnorm", RMSNorm)
