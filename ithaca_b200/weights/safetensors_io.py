"""Reader and writer for the safetensors container.

Format, as the reference reads it (src/gx.cpp:38-55): an 8-byte little-endian
header length ``hl``, a JSON object of ``hl`` bytes whose keys are tensor names
(``__metadata__`` is skipped) with ``dtype``, ``shape`` and ``data_offsets``
relative to byte ``8 + hl``.  The reference rejects ``hl`` beyond the file or
beyond 512 MiB and checks nothing else; this reader also checks that every
tensor lies inside the file, that its byte count matches shape and dtype, and
that no two tensors overlap.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

_MAX_HEADER = 512 << 20

# name -> (torch dtype, bytes per element)
_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path: str) -> Tuple[Dict[str, dict], int, int]:
    """Returns (entries by tensor name, offset of the data section, file size)."""
    size = os.path.getsize(path)
    if size < 8:
        raise SafetensorsError(f"{path}: not a safetensors file (shorter than its 8-byte length field)")
    with open(path, "rb") as f:
        (hl,) = struct.unpack("<Q", f.read(8))
        if hl > size - 8 or hl > _MAX_HEADER:
            raise SafetensorsError(f"{path}: not a safetensors file (header length {hl} does not fit the file of {size} bytes)")
        raw = f.read(hl)
    try:
        header = json.loads(raw.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: bad safetensors header ({e})") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: bad safetensors header (not an object)")
    header.pop("__metadata__", None)
    data_start = 8 + hl
    spans = []
    for name, e in header.items():
        if not isinstance(e, dict) or "dtype" not in e or "shape" not in e or "data_offsets" not in e:
            raise SafetensorsError(f"{path}: bad entry for tensor '{name}'")
        if e["dtype"] not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {e['dtype']} (supported: {', '.join(_DTYPES)})")
        b, en = e["data_offsets"]
        numel = int(np.prod(e["shape"], dtype=np.int64)) if e["shape"] else 1
        want = numel * _DTYPES[e["dtype"]][1]
        if b < 0 or en < b or data_start + en > size:
            raise SafetensorsError(f"{path}: tensor '{name}' lies outside the file (incomplete download?)")
        if en - b != want:
            raise SafetensorsError(f"{path}: tensor '{name}' has {en - b} bytes, but shape {e['shape']} of {e['dtype']} needs {want}")
        spans.append((b, en, name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise SafetensorsError(f"{path}: tensors '{n0}' and '{n1}' overlap")
    return header, data_start, size


def read_file(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one file, as CPU tensors that view a private mapping of
    the file (nothing is copied until a tensor is moved or converted)."""
    header, data_start, _ = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    if not header:
        return out
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    buf = np.frombuffer(mm, dtype=np.uint8)
    for name, e in header.items():
        dt, _ = _DTYPES[e["dtype"]]
        b, en = e["data_offsets"]
        shape = tuple(e["shape"])
        if en == b:
            out[name] = torch.empty(shape, dtype=dt)
            continue
        flat = torch.from_numpy(buf[data_start + b:data_start + en])
        out[name] = flat.view(dt).reshape(shape)
    return out


def write_file(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be written")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def list_weight_files(model_dir: str) -> Iterable[str]:
    """The folder's safetensors files: those the index names if there is one,
    else every ``*.safetensors`` file, in name order."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        files = sorted(set(wm.values()))
    else:
        files = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    return [os.path.join(model_dir, n) for n in files]
