"""Grouped-query attention over the paged cache.

Per token: q, k, v projections; rotary encoding of q and k; k and v appended to the
sequence's pages; attention of each query head over the keys of its kv head
(head h uses kv head h / (n_heads / n_kv_heads)) from position j0 to its own, where
j0 = pos + 1 - window under a window and 0 otherwise; output projection added to
the residual stream.  Scores are (q . k) * scale with scale = 1/sqrt(head_dim)
unless the spec gives one; softmax and the weighted sum are float32
(src/model.cpp:1479-1535; GPU path src/model.cpp:1164-1216).

The three projections are stacked into one product, as the reference does for a
fused ``attn_qkv`` tensor (src/model.cpp:1164-1170).
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

from ..cache.cache import KVRequest, LayerCache
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, register_mixer
from .linear import Linear


class Attention:
    graph_safe = True       # reads slots, positions and lengths from device arrays only

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, nh, nkv, hd = spec["hidden_size"], spec["n_heads"], spec["n_kv_heads"], spec["head_dim"]
        w = spec.weights
        return {w["q"]: TensorReq((nh * hd, d)), w["k"]: TensorReq((nkv * hd, d)),
                w["v"]: TensorReq((nkv * hd, d)), w["o"]: TensorReq((d, nh * hd))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime, position=None):
        self.hidden = int(spec["hidden_size"])
        self.n_heads = int(spec["n_heads"])
        self.n_kv_heads = int(spec["n_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"attention: {self.n_heads} heads cannot share {self.n_kv_heads} kv heads evenly")
        self.window = spec.get("window")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"attention: window must be positive, found {self.window}")
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = position
        if position is not None and position.rotary_dim > self.head_dim:
            raise ValueError("attention: the rotated width exceeds the head size")
        w = spec.weights
        wq, wk = tensors[w["q"]], tensors[w["k"]]
        # bfloat16 path with the whole head rotated: the rows of the q and k weights are reordered so that the
        # two members of a rotary pair are neighbours, (i, i + hd/2) -> (2i, 2i + 1).  Scores do not change (q and k
        # are reordered alike, and the cache holds k in that order); the product's epilogue can then rotate a pair
        # and write q and the cache entries itself, without the [tokens, q+k+v] intermediate.
        self.pairing = position.pairing if position is not None else 0
        self.fused_rope = (runtime.dtype == "bfloat16" and position is not None and position.rotary_dim == self.head_dim
                           and self.head_dim % 2 == 0)
        if self.fused_rope and self.pairing == 0:
            half = self.head_dim // 2
            order = torch.stack((torch.arange(half), torch.arange(half) + half), dim=1).reshape(-1)
            wq = wq.view(self.n_heads, self.head_dim, -1)[:, order].reshape(wq.shape)
            wk = wk.view(self.n_kv_heads, self.head_dim, -1)[:, order].reshape(wk.shape)
            self.pairing = 1                                       # pairs are (2i, 2i + 1) from here on
        self.qkv = Linear([wq, wk, tensors[w["v"]]], runtime)
        self.o = Linear([tensors[w["o"]]], runtime)
        self.runtime = runtime

    def cache_requests(self) -> List[object]:
        return [KVRequest(self.n_kv_heads, self.head_dim, self.window)]

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor,
                writes_cache: bool = True) -> None:
        rt = self.runtime
        T = x.shape[0]
        q = torch.empty((T, self.n_heads * self.head_dim), dtype=rt.act_dtype, device=x.device)
        table = ctx.tables[cache.kv_group]
        pos = self.position
        done = False
        if self.fused_rope:
            key = pos.key
            cos_sin = ctx.shared.get(key)
            if cos_sin is None:                                   # once per step, shared by the layers
                cos_sin = ctx.shared[key] = ops.rope_table(ctx.token_pos, pos.inv_freq)
            done = ops.gemm_qkv_rope(x, self.qkv.weight, q, cache.k_pages, cache.v_pages, cos_sin, ctx.token_seq,
                                     ctx.token_pos, table, self.n_heads, self.n_kv_heads, self.head_dim, writes_cache,
                                     rt.status)
        if not done:
            qkv = self.qkv(x, out_dtype=torch.float32)
            ops.rope_append(qkv, q, cache.k_pages, cache.v_pages, ctx.token_seq, ctx.token_pos, table,
                            pos.inv_freq if pos is not None else None, self.n_heads, self.n_kv_heads, self.head_dim,
                            pos.rotary_dim if pos is not None else 0, self.pairing, writes_cache, rt.status)
        att = attend(q, cache, ctx, table, self.n_heads, self.scale, self.window or 0, rt)
        self.o(att, out=residual, accumulate=True)


def attend(q: torch.Tensor, cache: LayerCache, ctx, table: torch.Tensor, n_heads: int, scale: float, window: int,
           rt: Runtime) -> torch.Tensor:
    """Chooses the attention kernel: tensor-core kernels for bfloat16 when they take the
    head size, else the CUDA-core kernel (always for float32)."""
    if q.dtype == torch.bfloat16:
        from ..csrc import attention_bf16
        out = attention_bf16.attend(q, cache.k_pages, cache.v_pages, ctx, table, n_heads, scale, window, rt.status)
        if out is not None:
            return out
    return ops.attention_simt(q, cache.k_pages, cache.v_pages, ctx.token_seq, ctx.token_pos, table, n_heads, scale,
                              window, rt.status)


register_mixer("attention", Attention)
