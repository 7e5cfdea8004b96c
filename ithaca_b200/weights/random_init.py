"""Random weights from a configuration and a seed.

The reference has no random-weights mode (its self-tests draw *inputs* from a
linear congruential generator, src/model.cpp:1646).  Each tensor is drawn from a
generator seeded by the seed and the tensor's own name, so a tensor's values do
not depend on which other tensors exist or in which order they are made.
Linear and embedding matrices are N(0, 0.02); norm weights are 1 + N(0, 0.01).
Values are drawn in float32 and rounded to the storage type.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping

import torch

from .loader import TensorReq
from .safetensors_io import write_file

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _name_seed(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return (h ^ (seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF


def random_tensors(manifest: Mapping[str, TensorReq], seed: int, dtype: str = "bfloat16",
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Tensors for every entry of the manifest.  On ``cpu`` the values are the
    ones a model folder written by ``write_random_model`` holds; on a CUDA
    device they come from that device's generator (same law, other values), for
    models too large to be worth writing to disk."""
    if dtype not in _STORAGE:
        raise ValueError(f"random weights: dtype {dtype!r} is not supported (bfloat16, float32)")
    out: Dict[str, torch.Tensor] = {}
    for name, req in manifest.items():
        gen = torch.Generator(device=device)
        gen.manual_seed(_name_seed(seed, name))
        if req.integer:
            out[name] = torch.zeros(req.shape, dtype=torch.int32, device=device)
            continue
        std = 0.01 if req.init == "ones" else req.std
        t = torch.empty(req.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=gen)
        if req.init == "ones":
            t += 1.0
        out[name] = t.to(_STORAGE[dtype])
    return out


def write_random_model(model_dir: str, config_dict: Dict[str, Any], seed: int, dtype: str | None = None) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for the architecture the
    dictionary names.  Returns the folder."""
    from ..config import config_from_dict
    from ..engine.model import weight_manifest

    _, cfg = config_from_dict(config_dict)
    dtype = dtype or config_dict.get("torch_dtype", "bfloat16")
    manifest = weight_manifest(cfg.model_spec())
    tensors = random_tensors(manifest, seed, dtype)
    os.makedirs(model_dir, exist_ok=True)
    full = dict(cfg.to_dict()) if hasattr(cfg, "to_dict") else dict(config_dict)
    full["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(full, f, indent=1)
    write_file(os.path.join(model_dir, "model.safetensors"), tensors, {"format": "pt", "seed": str(seed)})
    return model_dir
