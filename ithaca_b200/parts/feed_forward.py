"""Gated feed-forward: g = Wg x, u = Wu x, h = act(g) * u, y = Wd h, added to the
residual stream (src/model.cpp:1559-1565; silu(x) = x / (1 + exp(-x)), :1309).
Gate and up are stacked into one product ([gate; up], the split the reference
applies to a fused ``ffn_up``, src/model.cpp:1553-1557)."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, register_feed_forward
from .linear import Linear


class GatedMLP:
    graph_safe = True

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, ff = spec["hidden_size"], spec["intermediate_size"]
        w = spec.weights
        return {w["gate"]: TensorReq((ff, d)), w["up"]: TensorReq((ff, d)), w["down"]: TensorReq((d, ff))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        act = spec.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp: activation {act!r} is not supported (silu)")
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        w = spec.weights
        self.gate_up = Linear([tensors[w["gate"]], tensors[w["up"]]], runtime)
        self.down = Linear([tensors[w["down"]]], runtime)
        self.runtime = runtime
        # bfloat16 path: rows interleaved (gate 0, up 0, gate 1, up 1, ...) so that the product's epilogue
        # can apply silu(gate) * up itself and the [tokens, 2 ff] intermediate never exists
        self.fused = runtime.dtype == "bfloat16"
        if self.fused:
            ff, d = self.intermediate, self.hidden
            wgu = self.gate_up.weight
            self.gate_up.weight = torch.stack((wgu[:ff], wgu[ff:]), dim=1).reshape(2 * ff, d).contiguous()

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        if self.fused:
            from ..csrc import gemm_bf16
            h = gemm_bf16.gemm_swiglu(x, self.gate_up.weight, self.runtime.act_dtype)
        else:
            gu = self.gate_up(x, out_dtype=torch.float32)
            h = ops.swiglu(gu, self.runtime.act_dtype)
        self.down(h, out=residual, accumulate=True)


register_feed_forward("gated_mlp", GatedMLP)
