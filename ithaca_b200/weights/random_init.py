"""Random weights from a configuration and a seed.

The reference has no random-weights mode (its self-tests draw *inputs* from a
linear congruential generator, src/model.cpp:1646).  Here every element of every
tensor is a function of (seed, tensor name, flat index) alone: a counter-based
generator, so a tensor's values do not depend on which other tensors exist, in
which order they are made, or where.  The same function exists twice, in numpy
(``hashed_normal``) and as a CUDA kernel (``csrc/elementwise.cu``); both use
integer arithmetic and one float multiply and add, and give the same bits.  A
model made on the device therefore has exactly the weights that the folder
``write_random_model`` writes for the same configuration and seed, and whoever
wants to check the device's results can make those weights on the host.

Element i of a tensor: the splitmix64 outputs 2i+1 and 2i+2 of the sequence that
starts at the tensor's key are cut into eight 16-bit fields; their sum minus its
mean, times std / 53510.85 (the standard deviation of such a sum), is close to
N(0, std).  Linear and embedding matrices have std 0.02; norm weights are
1 + N(0, 0.01).  Values are formed in float32 and rounded to the storage type.
"""
from __future__ import annotations

import json
import math
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, Mapping

import numpy as np
import torch

from .loader import TensorReq
from .safetensors_io import write_file

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32}
_MASK = 0xFFFFFFFFFFFFFFFF
_GOLDEN = 0x9E3779B97F4A7C15
_FIELD_SUM_MEAN = 4 * 65535                                   # eight fields, each 0..65535
_FIELD_SUM_STD = math.sqrt(8 * (65536.0 ** 2 - 1.0) / 12.0)


def _mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's sequence: FNV-1a of the name, mixed with the seed."""
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return _mix64(h ^ ((seed * _GOLDEN) & _MASK))


def _scale(std: float) -> np.float32:
    return np.float32(std / _FIELD_SUM_STD)


_CHUNK = 1 << 18          # elements per piece: its temporaries stay in the cache


def hashed_normal(key: int, n: int, std: float, offset: float = 0.0, first: int = 0) -> np.ndarray:
    """float32 values of elements [first, first + n) of the sequence with this key."""
    out = np.empty(n, dtype=np.float32)
    scale, off = _scale(std), np.float32(offset)
    m1, m2 = np.uint64(0xBF58476D1CE4E5B9), np.uint64(0x94D049BB133111EB)
    f = np.uint64(0xFFFF)

    def piece(lo: int) -> None:
        hi = min(n, lo + _CHUNK)
        idx = np.arange(first + lo, first + hi, dtype=np.uint64)
        total = np.zeros(hi - lo, dtype=np.int64)
        with np.errstate(over="ignore"):
            for j in (1, 2):
                z = np.uint64(key) + (idx * np.uint64(2) + np.uint64(j)) * np.uint64(_GOLDEN)
                z = (z ^ (z >> np.uint64(30))) * m1
                z = (z ^ (z >> np.uint64(27))) * m2
                z = z ^ (z >> np.uint64(31))
                total += ((z & f) + ((z >> np.uint64(16)) & f) + ((z >> np.uint64(32)) & f) + (z >> np.uint64(48))).astype(np.int64)
        out[lo:hi] = off + scale * (total - _FIELD_SUM_MEAN).astype(np.float32)

    starts = range(0, n, _CHUNK)
    if n <= 4 * _CHUNK:
        for lo in starts:
            piece(lo)
    else:                                                # numpy releases the interpreter lock inside its loops
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
            list(pool.map(piece, starts))
    return out


def random_tensor(name: str, req: TensorReq, seed: int, dtype: str = "bfloat16", device: str = "cpu") -> torch.Tensor:
    """One tensor of the manifest; the same values on the host and on a CUDA device."""
    if dtype not in _STORAGE:
        raise ValueError(f"random weights: dtype {dtype!r} is not supported (bfloat16, float32)")
    if req.integer:
        return torch.zeros(req.shape, dtype=torch.int32, device=device)
    std = 0.01 if req.init == "ones" else req.std
    offset = 1.0 if req.init == "ones" else 0.0
    key = tensor_key(seed, name)
    if torch.device(device).type == "cuda":
        from ..csrc import ops
        out = torch.empty(req.shape, dtype=_STORAGE[dtype], device=device)
        return ops.fill_random(out, key, float(_scale(std)), offset)
    n = int(np.prod(req.shape)) if len(req.shape) else 1
    t = torch.from_numpy(hashed_normal(key, n, std, offset)).reshape(tuple(req.shape))
    return t.to(_STORAGE[dtype])


def random_tensors(manifest: Mapping[str, TensorReq], seed: int, dtype: str = "bfloat16",
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Tensors for every entry of the manifest: the values a model folder written by
    ``write_random_model`` with the same seed and storage type holds, wherever they are made."""
    return {name: random_tensor(name, req, seed, dtype, device) for name, req in manifest.items()}


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
