"""Weights by tensor name, checked against what the model's parts ask for.

The reference binds each matrix by name and reports the first missing one
(``"missing tensor X"``, src/model.cpp:29-35; ``"layer i is incomplete"``,
:211-214) without checking shapes.  Here the model's parts state every tensor
they need with its shape; the folder is compared with that list once, and one
error names every missing tensor, every unexpected tensor and every wrong shape.

Storage types: a tensor stored as bfloat16 stays bfloat16, one stored in 32-bit
floating point stays so, float16 is widened to float32 (exact), and integer
tables become int32.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, list_weight_files, read_file


class WeightError(ValueError):
    pass


@dataclass(frozen=True)
class TensorReq:
    """What a part needs of one tensor.  ``init`` tells the random-weights mode
    how to fill it: ``"normal"`` = N(0, std), ``"ones"`` = 1 + N(0, std)."""

    shape: Tuple[int, ...]
    init: str = "normal"
    std: float = 0.02
    integer: bool = False
    optional: bool = False


def _storage_form(name: str, t: torch.Tensor, req: Optional[TensorReq]) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    if t.dtype == torch.int64:
        if t.numel() and (int(t.max()) > 2**31 - 1 or int(t.min()) < -2**31):
            raise WeightError(f"tensor '{name}': 64-bit integer values do not fit int32")
        return t.to(torch.int32)
    raise WeightError(f"tensor '{name}': storage type {t.dtype} is not supported")


def read_model_tensors(model_dir: str) -> Dict[str, torch.Tensor]:
    """Every tensor of the folder in one namespace (several files merge, as in
    the reference's ``SafeTensors::add``, src/gx.h:15-28).  A name that appears
    in two files is an error."""
    files = list(list_weight_files(model_dir))
    if not files:
        raise WeightError(f"{model_dir}: the model folder holds no .safetensors file")
    out: Dict[str, torch.Tensor] = {}
    origin: Dict[str, str] = {}
    for path in files:
        if not os.path.isfile(path):
            raise WeightError(f"{path}: named by the index but not in the folder")
        try:
            part = read_file(path)
        except SafetensorsError as e:
            raise WeightError(str(e)) from None
        for name, t in part.items():
            if name in out:
                raise WeightError(f"tensor '{name}' appears in both {origin[name]} and {os.path.basename(path)}")
            out[name] = t
            origin[name] = os.path.basename(path)
    return out


def check_tensors(tensors: Mapping[str, torch.Tensor], manifest: Mapping[str, TensorReq],
                  ignore_unexpected: Iterable[str] = ()) -> None:
    """One error that lists everything wrong: missing tensors, unexpected
    tensors, wrong shapes, and floating point where an integer table is wanted
    (or the reverse)."""
    ignore = set(ignore_unexpected)
    missing = [n for n, r in manifest.items() if n not in tensors and not r.optional]
    unexpected = [n for n in tensors if n not in manifest and n not in ignore]
    wrong = []
    for n, r in manifest.items():
        if n not in tensors:
            continue
        t = tensors[n]
        if tuple(t.shape) != tuple(r.shape):
            wrong.append(f"{n}: expected {list(r.shape)}, found {list(t.shape)}")
        elif r.integer != (not t.dtype.is_floating_point):
            wrong.append(f"{n}: expected {'an integer' if r.integer else 'a floating-point'} tensor, found {t.dtype}")
    if not (missing or unexpected or wrong):
        return
    lines = ["the checkpoint does not match the configuration:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(sorted(wrong)))
    raise WeightError("\n".join(lines))


def load_checkpoint(model_dir: str, manifest: Mapping[str, TensorReq],
                    ignore_unexpected: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    tensors = read_model_tensors(model_dir)
    check_tensors(tensors, manifest, ignore_unexpected)
    return {n: _storage_form(n, tensors[n], manifest.get(n)) for n in manifest if n in tensors}
