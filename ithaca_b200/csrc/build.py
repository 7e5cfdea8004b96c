"""Compiles the CUDA sources of this folder for sm_100a and loads the result.

The kernel library is a plain shared object with a C interface (no Python or
torch headers, so a file compiles in seconds).  It is built in-tree under
``csrc/_build/`` by ``nvcc`` at the first call that needs it, keyed by a hash of
the sources and flags, and loaded with ``ctypes``.  Head-size-specialised
kernels live in modules of their own that are compiled only for the sizes a
model asks for.  While compiling, a line is printed for each file.

There is no fallback: if the library cannot be built or loaded, an error says
so and nothing runs.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))
_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
_COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
                 "--expt-relaxed-constexpr"]

# The always-needed kernels.  Specialised modules are listed in SPECIALISED.
CORE_SOURCES = ["elementwise.cu", "gemm_simt.cu", "gemm_mma.cu", "gemm_tcgen05.cu", "attention_simt.cu", "sampling.cu"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[ithaca_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = [os.environ.get("IK_NVCC"), os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
             shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelBuildError("nvcc was not found (looked at $IK_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be compiled and there is no other path")


def _build_dir() -> str:
    """In-tree when the tree is writable, else a per-user folder under the
    system's temporary directory."""
    d = os.environ.get("IK_BUILD_DIR") or os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"ithaca_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _hash(sources: Sequence[str], defines: Sequence[str]) -> str:
    """Of every header of the folder, the given sources (listed ones and those they include) and the flags."""
    h = hashlib.sha256()
    for name in sorted(os.listdir(_HERE)):
        if name.endswith((".cuh", ".h")):
            with open(os.path.join(_HERE, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    for s in sources:
        with open(os.path.join(_HERE, s), "rb") as f:
            h.update(s.encode() + b"\0" + f.read())
    h.update(" ".join(list(defines) + _ARCH_FLAGS + _COMMON_FLAGS).encode())
    return h.hexdigest()[:16]


def _run(cmd: List[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise KernelBuildError(f"compiling {what} failed (exit {p.returncode}):\n{' '.join(cmd)}\n{p.stdout}")


def build_library(name: str, sources: Sequence[str], defines: Sequence[str] = (), extra_flags: Sequence[str] = (),
                  libs: Sequence[str] = (), includes: Sequence[str] = ()) -> str:
    """Builds (if needed) and returns the path of ``lib<name>_<hash>.so``.  ``includes``: sources that the
    listed ones include (not compiled on their own, but a change to them is a change to the library)."""
    tag = _hash(list(sources) + list(includes), list(defines) + list(extra_flags))
    out_dir = _build_dir()
    so = os.path.join(out_dir, f"lib{name}_{tag}.so")
    if os.path.isfile(so):
        return so
    nvcc = find_nvcc()
    t0 = time.time()
    _log(f"compiling {name} ({len(sources)} file{'s' if len(sources) != 1 else ''}) for sm_100a into {out_dir}")
    objs: List[str] = []
    work = tempfile.mkdtemp(prefix=f"{name}_", dir=out_dir)

    def one(src: str) -> str:
        obj = os.path.join(work, os.path.splitext(src)[0] + ".o")
        t = time.time()
        _run([nvcc, *_ARCH_FLAGS, *_COMMON_FLAGS, *extra_flags, *[f"-D{d}" for d in defines], "-I", _HERE, "-c",
              os.path.join(_HERE, src), "-o", obj], src)
        _log(f"  {src} done in {time.time() - t:.1f} s")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
            objs = list(ex.map(one, sources))
        tmp = so + f".tmp{os.getpid()}"
        _run([nvcc, *_ARCH_FLAGS, "-shared", "-o", tmp, *objs, *[f"-l{l}" for l in libs]], f"lib{name}")
        os.replace(tmp, so)
        for old in os.listdir(out_dir):                     # builds of earlier versions of these sources
            if old.startswith(f"lib{name}_") and old.endswith(".so") and old != os.path.basename(so):
                try:
                    os.remove(os.path.join(out_dir, old))
                except OSError:
                    pass
    finally:
        shutil.rmtree(work, ignore_errors=True)
    _log(f"{name} ready in {time.time() - t0:.1f} s")
    return so


def load_library(name: str, sources: Sequence[str], defines: Sequence[str] = (), extra_flags: Sequence[str] = (),
                 libs: Sequence[str] = (), includes: Sequence[str] = ()) -> ctypes.CDLL:
    key = name + "|" + ",".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            so = build_library(name, sources, defines, extra_flags, libs, includes)
            try:
                lib = ctypes.CDLL(so)
            except OSError as e:
                raise KernelBuildError(f"{so} could not be loaded: {e}") from None
            _loaded[key] = lib
    return lib


def core() -> ctypes.CDLL:
    return load_library("ithaca_kernels", CORE_SOURCES)


ATTENTION_HEAD_SIZES = (16, 32, 48, 64, 128)     # the sizes the tests and the benchmark use; others compile on demand


PAIRS_SOURCE = "gemm_tcgen05_mc.cu"        # the pair mode of the tcgen05 product: a library of its own, optional


def pairs_available() -> bool:
    return os.path.isfile(os.path.join(_HERE, PAIRS_SOURCE))


def pairs() -> ctypes.CDLL:
    return load_library("ithaca_gemm_pairs", [PAIRS_SOURCE], includes=["gemm_tcgen05.cu"])


def build_all() -> None:
    """Everything that can be compiled ahead of time: the core library, the attention module of
    every usual head size, and the pair mode of the tcgen05 product where its source is there."""
    core()
    for hd in ATTENTION_HEAD_SIZES:
        build_library(f"ithaca_attn_hd{hd}", ["attention_bf16.cu"], defines=[f"IK_HD={hd}"])
    if pairs_available():
        build_library("ithaca_gemm_pairs", [PAIRS_SOURCE], includes=["gemm_tcgen05.cu"])
