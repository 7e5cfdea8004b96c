"""Token embedding and the output head.

x[t, :] = E[id_t, :] * scale (src/model.cpp:1381-1383).  The reference clamps an id
outside the vocabulary; here the step function rejects it before anything runs.
logits = W_out xn, where W_out is the embedding matrix when the model has no
output matrix of its own (src/model.cpp:132, 1590-1592).
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, register_embedding, register_head, to_device
from .linear import Linear


class Embedding:
    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        return {spec.weights["weight"]: TensorReq((spec["vocab_size"], spec["hidden_size"]))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.vocab_size = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.scale = float(spec.get("scale", 1.0))
        self.table = to_device(tensors[spec.weights["weight"]], runtime).contiguous()
        self.runtime = runtime

    def forward(self, ids: torch.Tensor, ctx=None) -> torch.Tensor:
        return ops.embed(ids, self.table, self.scale, self.runtime.status)


class OutputHead:
    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        return {spec.weights["weight"]: TensorReq((spec["vocab_size"], spec["hidden_size"]))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.vocab_size = int(spec["vocab_size"])
        self.linear = Linear([tensors[spec.weights["weight"]]], runtime)

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        return self.linear(xn, out_dtype=torch.float32)


register_embedding("embedding", Embedding)
register_head("lm_head", OutputHead)
