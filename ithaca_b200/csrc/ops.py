"""Python side of the kernel library: argument checks, pointers, the current stream.

Every function launches on torch's current CUDA stream and allocates nothing but its
declared outputs.  A non-zero status from the library raises ``KernelError``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_vp, _i, _f, _u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_ulonglong


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32, bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")


_launches = 0


def launch_count() -> int:
    """Kernel-library calls made so far in this process (each is one or two kernel launches)."""
    return _launches


def _check(status: int, what: str, kernels: int = 1) -> None:
    global _launches
    _launches += kernels
    if status == 0:
        return
    if status == -1:
        raise KernelError(f"{what}: bad argument")
    if status == -2:
        raise KernelError(f"{what}: these sizes are not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {status} at launch")


_SIGNATURES = {
    "ik_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _f, _vp, _vp],
    "ik_rmsnorm": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "ik_swiglu": [_vp, _vp, _i, _i, _i, _i, _vp],
    "ik_fill_random": [_vp, _i, _u64, _u64, _f, _f, _vp],
    "ik_device_sm_count": [],
    "ik_copy": [_vp, _vp, _u64, _vp],
    "ik_rope_append": [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "ik_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_gemm_bf16_mma": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_gemm_tcgen05": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "ik_gemm_tcgen05_tile": [_i],
    "ik_gemm_tcgen05_tile_width": [_i, _i],
    "ik_gemm_tcgen05_stream_k_bytes": [],
    "ik_rope_table": [_vp, _vp, _vp, _i, _i, _vp],
    "ik_gemm_qkv_rope_mma": [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "ik_gemm_qkv_rope_tcgen05": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp],
    "ik_attention_simt": [_vp, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp, _vp],
    "ik_argmax": [_vp, _i, _vp, _i, _i, _vp, _vp],
    "ik_argmax_scratch_bytes": [],
    "ik_selftest_wait_expires": [_vp, _vp, _vp, _u64, _vp],
    "ik_gemm_tcgen05_issue_rate": [_i, _i, _i, _vp, _vp, _vp],
    "ik_gemm_tcgen05_take_wait_record": [_vp],
    "ik_sample": [_vp, _i, _vp, _vp, _i, _i, _f, _i, _f, _f, _vp, _i, _u64, _vp, _vp, _vp],
}

_lib = None
_status = {}


# ---------------------------------------------------------------------------------------------
# Per-kernel timing.  The reference times each operation of a forward pass when ITHACA_PROF is set
# (src/model.cpp:1261-1307, src/cuda_tier.cpp:514-527).  Here, while a ``Profile`` is active, every call
# into the kernel library is bracketed by CUDA events; the wrappers below say beforehand how many bytes the call has
# to move and how many floating-point operations it has to do, so that a table can hold each call against the
# device's peaks.  The events keep kernels from overlapping (no early launch), and nothing may be captured into
# a graph meanwhile: it is a tool for looking at a step, not the way a step runs.
class Profile:
    def __init__(self):
        self.records = []            # (label, start event, end event, bytes, flops)

    def __enter__(self):
        global _profile
        if _profile is not None:
            raise KernelError("a kernel profile is already being taken")
        _profile = self
        return self

    def __exit__(self, *exc):
        global _profile, _pending
        _profile, _pending = None, None
        return False

    def rows(self):
        """Per label, in order of first appearance: calls, microseconds, bytes, flops."""
        torch.cuda.synchronize()
        out = {}
        for label, e0, e1, nbytes, flops in self.records:
            r = out.setdefault(label, {"kernel": label, "calls": 0, "us": 0.0, "bytes": 0, "flops": 0})
            r["calls"] += 1
            r["us"] += e0.elapsed_time(e1) * 1e3
            r["bytes"] += nbytes
            r["flops"] += flops
        return list(out.values())


_profile: Optional[Profile] = None
_pending = None                      # (label, bytes, flops) of the library call that comes next


def profiling() -> bool:
    return _profile is not None


def _work(label: str, nbytes: int = 0, flops: int = 0) -> None:
    global _pending
    if _profile is not None:
        _pending = (label, int(nbytes), int(flops))


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


class _TimedLibrary:
    """Stands in for a loaded library while a profile is taken."""

    def __init__(self, library):
        self._library = library

    def __getattr__(self, name):
        fn = getattr(self._library, name)
        if _profile is None or not name.startswith("ik_") or fn.argtypes is None or not fn.argtypes or fn.argtypes[-1] is not _vp:
            return fn                                        # not a launch (no stream argument)

        def call(*args):
            global _pending
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            st = fn(*args)
            e1.record()
            label, nbytes, flops = _pending or (name[3:], 0, 0)
            _pending = None
            _profile.records.append((label, e0, e1, nbytes, flops))
            return st
        return call


def timed(library):
    return _TimedLibrary(library) if _profile is not None else library


def device_status(device) -> torch.Tensor:
    """The int32 status word kernels set when they meet something they refuse to do (an index
    out of range, a wait that ran out); one per device, shared by every runtime on it."""
    key = str(torch.device(device))
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def lib():
    """The loaded kernel library; built on first use.  Raises if that fails."""
    global _lib
    if _lib is None:
        l = build.core()
        for name, sig in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = sig
            fn.restype = _i
        _lib = l
    return timed(_lib)


# ---------------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0, status: Optional[torch.Tensor] = None,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    T, (V, d) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=ids.device)
    _work(f"embed {T}x{d}", T * d * (table.element_size() + 4))
    _check(lib().ik_embed(_ptr(ids), _ptr(table), _code(table), _ptr(out), T, d, V, scale, _ptr(status), _stream()),
           "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows_in: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    d = x.shape[-1]
    if weight.numel() != d:
        raise KernelError(f"rmsnorm: weight has {weight.numel()} elements, rows have {d}")
    rows = x.numel() // d if rows_in is None else rows_in.numel()
    if rows_in is not None:
        _need(rows_in, "rows_in", torch.int32)
    if out is None:
        out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
    _work(f"rmsnorm {rows}x{d}", rows * d * (4 + out.element_size()) + d * 4)
    _check(lib().ik_rmsnorm(_ptr(x), _ptr(rows_in), _ptr(weight), _ptr(out), _code(out), rows, d, eps, _stream()),
           "rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
           interleaved: bool = False) -> torch.Tensor:
    """``interleaved``: gate j and up j sit in columns 2j and 2j + 1 instead of j and ff + j."""
    _need(gate_up, "gate_up", torch.float32)
    T, ff2 = gate_up.shape
    if ff2 % 2:
        raise KernelError("swiglu: the input needs an even number of columns (gate then up)")
    if out is None:
        out = torch.empty((T, ff2 // 2), dtype=out_dtype, device=gate_up.device)
    _work(f"swiglu {T}x{ff2 // 2}", _nbytes(gate_up, out))
    _check(lib().ik_swiglu(_ptr(gate_up), _ptr(out), _code(out), T, ff2 // 2, 1 if interleaved else 0, _stream()), "swiglu")
    return out


def fill_random(out: torch.Tensor, key: int, scale: float, offset: float) -> torch.Tensor:
    """Fills ``out`` with offset + scale * (a centred sum of eight 16-bit hash fields) per flat index; the values are
    the ones ``weights.random_init.hashed_normal`` gives on the host for the same key."""
    _need(out, "out")
    _check(lib().ik_fill_random(_ptr(out), _code(out), out.numel(), key & 0xFFFFFFFFFFFFFFFF, scale, offset, _stream()),
           "fill_random")
    return out


def copy(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """dst = src with this library's streaming copy kernel (sizes a multiple of 16 bytes)."""
    _need(src, "src")
    _need(dst, "dst")
    n = src.numel() * src.element_size()
    if n != dst.numel() * dst.element_size():
        raise KernelError("copy: source and destination differ in size")
    _work(f"copy {n >> 20} MiB", 2 * n)
    _check(lib().ik_copy(_ptr(src), _ptr(dst), n, _stream()), "copy")
    return dst


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                token_seq: torch.Tensor, token_pos: torch.Tensor, table: torch.Tensor,
                inv_freq: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                pairing: int, write_cache: bool, status: Optional[torch.Tensor]) -> None:
    """k_pages / v_pages: [n_pages, n_kv_heads, page_size, head_dim] of one layer."""
    _need(qkv, "qkv", torch.float32)
    _need(q_out, "q_out")
    _need(k_pages, "k_pages")
    _need(v_pages, "v_pages")
    _need(table, "table", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("rope_append: qkv has the wrong width")
    n_pages, nkv, page_size, hd = k_pages.shape
    if nkv != n_kv_heads or hd != head_dim or v_pages.shape != k_pages.shape or v_pages.dtype != k_pages.dtype:
        raise KernelError("rope_append: the pages do not match the head sizes")
    _work(f"rope_append {T}", _nbytes(qkv, q_out) + 2 * T * n_kv_heads * head_dim * k_pages.element_size())
    _check(lib().ik_rope_append(_ptr(qkv), _ptr(q_out), _code(q_out), _ptr(k_pages), _ptr(v_pages), _code(k_pages),
                                _ptr(token_seq), _ptr(token_pos), _ptr(table), table.stride(0), _ptr(inv_freq), T,
                                n_heads, n_kv_heads, head_dim, rotary_dim, pairing, page_size, n_pages,
                                1 if write_cache else 0, _ptr(status), _stream()), "rope_append")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.float32,
              accumulate: bool = False) -> torch.Tensor:
    """out[M, N] (+)= x[M, K] @ w[N, K]^T on the CUDA cores, float accumulation in ascending k."""
    _need(x, "x", contiguous=False)
    _need(w, "w", contiguous=False)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match or rows are not contiguous")
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output to add to")
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _need(out, "out", contiguous=False)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise KernelError("gemm: the output has the wrong shape")
    _work(f"gemm_simt {M}x{N}x{K}", M * K * x.element_size() + N * K * w.element_size() + M * N * out.element_size(), 2 * M * N * K)
    _check(lib().ik_gemm_simt(_ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), M, N, K, x.stride(0),
                              w.stride(0), out.stride(0), 1 if accumulate else 0, _stream()), "gemm_simt")
    return out


def gemm_bf16_mma(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                  accumulate: bool = False, kind: int = 0, swiglu: bool = False) -> Optional[torch.Tensor]:
    """bfloat16 operands, float accumulation on the warp-level tensor-core path.  ``kind``: 0 = by
    M, 1 = the skinny (decode) kernel, 2 = the tiled kernel.  Returns None when the kernels
    do not take these sizes (K not a multiple of 8, unaligned rows).

    ``w`` is a weight: the skinny kernel, launched early, reads its first rows before it waits for the
    kernel before it in the stream, so ``w`` must not be what that kernel writes (``x`` and ``out`` may be)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16, contiguous=False)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match or rows are not contiguous")
    n_out = N // 2 if swiglu else N
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output to add to")
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    _need(out, "out", contiguous=False)
    if out.shape != (M, n_out) or out.stride(1) != 1:
        raise KernelError("gemm: the output has the wrong shape")
    _work(f"gemm_skinny{' +swiglu' if swiglu else ''} {M}x{N}x{K}", 2 * (M * K + N * K) + M * n_out * out.element_size(), 2 * M * N * K)
    st = lib().ik_gemm_bf16_mma(_ptr(x), _ptr(w), _ptr(out), _code(out), M, N, K, x.stride(0), w.stride(0),
                                out.stride(0), 1 if accumulate else 0, kind, 1 if swiglu else 0, _stream())
    if st == -2:
        return None
    _check(st, "gemm_bf16_mma")
    return out


_sm_counts = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once per device)."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = int(lib().ik_device_sm_count())
    return n


_stream_k_scratch = {}


def stream_k_scratch(device) -> torch.Tensor:
    """Scratch of the stream-K product (pieces of tiles and their flags): one per device, zeroed once; the
    kernels leave the flags zero.  Launches that use it must follow one another in one stream."""
    key = str(torch.device(device))
    t = _stream_k_scratch.get(key)
    if t is None:
        t = torch.zeros(lib().ik_gemm_tcgen05_stream_k_bytes() // 4, dtype=torch.float32, device=device)
        _stream_k_scratch[key] = t
    return t


def tcgen05_cluster_fits(M: int, N: int, K: int, n_cl: int) -> bool:
    """Whether the cluster mode of the tcgen05 product takes this shape with ``n_cl`` blocks per tile."""
    tile_m = lib().ik_gemm_tcgen05_tile(M)
    tiles = -(-N // 128) * -(-M // tile_m)
    steps = -(-K // 64)
    most = 4 if tile_m <= 64 else 2 if tile_m <= 128 else 1
    return 2 <= n_cl <= most and tiles * n_cl <= sm_count() and (n_cl - 1) * -(-steps // n_cl) < steps


def tcgen05_splits(M: int, N: int, K: int) -> int:
    """How the tcgen05 product shares out its work: 1 = whole tiles dealt round robin; n > 1 = n slices
    of K and a second kernel that adds them; 0 = stream-K (equal shares of all K steps of all tiles);
    -n = clusters of n blocks per tile, each a slice of K, summed in shared memory (no scratch, one kernel).
    Measured on B200 with 2048 x 2048 .. 28672 x 4096 weights (``bench.py --only products --tokens ...``): with
    fewer tiles than half the SMs, K is sliced: by clusters of 2 or 4 where that busies at least half the SMs (clusters
    of 3 measured far slower), else by a second kernel; stream-K wins when whole tiles would leave more than a
    tenth of the SMs' time unused and there is one token tile of at most 128 tokens (bandwidth-bound); beyond that
    whole tiles win."""
    N_SM = sm_count()
    tile_m = lib().ik_gemm_tcgen05_tile(M)
    tiles_m = -(-M // lib().ik_gemm_tcgen05_tile_width(M, N))
    tiles = -(-N // 128) * tiles_m
    steps = -(-K // 64)
    if 2 * tiles <= N_SM:
        want = max(1, min(N_SM // tiles, steps // 4))
        most = 4 if tile_m <= 64 else 2 if tile_m <= 128 else 1
        n_cl = 4 if want >= 4 and most >= 4 else 2 if want >= 2 and most >= 2 else 0
        if n_cl and 2 * tiles * n_cl >= N_SM and tcgen05_cluster_fits(M, N, K, n_cl):
            return -n_cl
        return want
    rounds = -(-tiles // N_SM)
    if tiles_m == 1 and tile_m <= 128 and tiles / (rounds * N_SM) < 0.9 and tiles * steps >= 8:
        return 0
    return 1


_pairs_lib = None
PAIRS = os.environ.get("IK_PAIRS", "1") != "0"


def pairs_lib():
    """The pair mode of the tcgen05 product (two blocks share one copy of a token tile: less traffic from L2 at
    prefill), a library of its own; None where its source is not there or ``IK_PAIRS=0`` says not to use it."""
    global _pairs_lib
    if _pairs_lib is None:
        if not PAIRS or not build.pairs_available():
            _pairs_lib = False
        else:
            l = build.pairs()
            l.ik_gemm_tcgen05_pairs.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]
            l.ik_gemm_tcgen05_pairs.restype = _i
            l.ik_gemm_qkv_rope_tcgen05_pairs.argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]
            l.ik_gemm_qkv_rope_tcgen05_pairs.restype = _i
            _pairs_lib = l
    return timed(_pairs_lib) if _pairs_lib else None


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                 accumulate: bool = False, splits: Optional[int] = None,
                 status: Optional[torch.Tensor] = None, swiglu: bool = False, pairs: Optional[bool] = None) -> Optional[torch.Tensor]:
    """bfloat16 operands on the tcgen05 tensor cores (TMA-fed, accumulators in TMEM).  Returns None
    when the kernel does not take these sizes (K not a multiple of 8, unaligned rows).

    ``w`` is a weight: launched early, the kernel asks for its first tiles of ``w`` before it waits for the
    kernel before it in the stream, so ``w`` must not be what that kernel writes (``x`` and ``out`` may be)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16, contiguous=False)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match or rows are not contiguous")
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        return None
    n_out = N // 2 if swiglu else N
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output to add to")
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    _need(out, "out", contiguous=False)
    if out.shape != (M, n_out) or out.stride(1) != 1:
        raise KernelError("gemm: the output has the wrong shape")
    if splits is None:
        splits = tcgen05_splits(M, N, K)
    if splits == 1 and M > 256 and pairs is not False:
        pl = pairs_lib()
        if pl is None and pairs:
            raise KernelError("gemm_tcgen05: the pair mode was asked for but its library is not there")
        if pl is not None:
            _work(f"gemm_tcgen05 pairs{' +swiglu' if swiglu else ''} {M}x{N}x{K}", 2 * (M * K + N * K) + M * n_out * out.element_size(), 2 * M * N * K)
            st = pl.ik_gemm_tcgen05_pairs(_ptr(x), _ptr(w), _ptr(out), _code(out), M, N, K, x.stride(0), w.stride(0),
                                          out.stride(0), 1 if accumulate else 0, 1 if swiglu else 0, _ptr(status), _stream())
            if st != -2:
                _check(st, "gemm_tcgen05 (pairs)")
                return out
    partial = (stream_k_scratch(x.device) if splits == 0 else
               torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None)
    _work(f"gemm_tcgen05{' +swiglu' if swiglu else ''} {M}x{N}x{K}", 2 * (M * K + N * K) + M * n_out * out.element_size(), 2 * M * N * K)
    st = lib().ik_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(out), _code(out), _ptr(partial), M, N, K, x.stride(0),
                               w.stride(0), out.stride(0), 1 if accumulate else 0, 1 if swiglu else 0, splits, _ptr(status),
                               _stream())
    if st == -2:
        return None
    _check(st, "gemm_tcgen05", kernels=2 if splits > 1 else 1)
    return out


class RopeStore(ctypes.Structure):
    """Mirror of IkRopeStore (rope_store.cuh): where the fused q/k/v product puts its results."""
    _fields_ = [("q_out", _vp), ("k_pages", _vp), ("v_pages", _vp), ("cos_sin", _vp), ("token_seq", _vp),
                ("token_pos", _vp), ("table", _vp), ("status", _vp), ("table_stride", _i), ("nh", _i), ("nkv", _i),
                ("hd", _i), ("page_size", _i), ("n_pages", _i), ("write_cache", _i)]


def rope_table(token_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[T, half, 2] float: cos and sin of float(pos) * inv_freq, for the fused q/k/v epilogue."""
    _need(token_pos, "token_pos", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    T, half = token_pos.numel(), inv_freq.numel()
    out = torch.empty((T, half, 2), dtype=torch.float32, device=token_pos.device)
    _work(f"rope_table {T}", T * half * 8)
    _check(lib().ik_rope_table(_ptr(token_pos), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rope_table")
    return out


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                  cos_sin: torch.Tensor, token_seq: torch.Tensor, token_pos: torch.Tensor, table: torch.Tensor,
                  n_heads: int, n_kv_heads: int, head_dim: int, write_cache: bool, status: Optional[torch.Tensor],
                  skinny_max: int = 16, splits: Optional[int] = None) -> bool:
    """q, k, v = x W^T with rotary pairs in adjacent rows of W; rotated q to ``q_out``, rotated k and v into
    the pages.  Returns False when the kernels do not take these sizes (the caller then runs the steps apart)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16, contiguous=False)
    _need(q_out, "q_out", torch.bfloat16)
    _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16)
    _need(cos_sin, "cos_sin", torch.float32)
    _need(table, "table", torch.int32)
    M, K = x.shape
    N = w.shape[0]
    n_pages, nkv, page_size, hd = k_pages.shape
    if (N != (n_heads + 2 * n_kv_heads) * head_dim or nkv != n_kv_heads or hd != head_dim or head_dim % 2
            or cos_sin.shape != (M, head_dim // 2, 2) or q_out.shape != (M, n_heads * head_dim)):
        raise KernelError("gemm_qkv_rope: the sizes do not fit together")
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or x.stride(1) != 1 \
            or w.stride(1) != 1:
        return False
    rs = RopeStore(_ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(cos_sin), _ptr(token_seq), _ptr(token_pos),
                   _ptr(table), _ptr(status), table.stride(0), n_heads, n_kv_heads, head_dim, page_size, n_pages,
                   1 if write_cache else 0)
    _work(f"gemm_{'skinny' if M <= skinny_max else 'tcgen05'} +rope+cache {M}x{N}x{K}", 2 * (M * K + N * K + M * N), 2 * M * N * K)
    if M <= skinny_max:
        st = lib().ik_gemm_qkv_rope_mma(_ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), ctypes.byref(rs), _stream())
        kernels = 1
    else:
        if splits is None:
            splits = tcgen05_splits(M, N, K)
        pl = pairs_lib() if splits == 1 and M > 256 else None
        if pl is not None:
            st = pl.ik_gemm_qkv_rope_tcgen05_pairs(_ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), _ptr(status),
                                                   ctypes.byref(rs), _stream())
            if st != -2:
                _check(st, "gemm_qkv_rope (pairs)")
                return True
        partial = (stream_k_scratch(x.device) if splits == 0 else
                   torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None)
        st = lib().ik_gemm_qkv_rope_tcgen05(_ptr(x), _ptr(w), _ptr(partial), M, N, K, x.stride(0), w.stride(0), splits,
                                            _ptr(status), ctypes.byref(rs), _stream())
        kernels = 2 if splits > 1 else 1
    if st == -2:
        return False
    _check(st, "gemm_qkv_rope", kernels=kernels)
    return True


def attention_simt(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, token_seq: torch.Tensor,
                   token_pos: torch.Tensor, table: torch.Tensor, n_heads: int, scale: float, window: int,
                   status: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(q, "q")
    _need(k_pages, "k_pages")
    _need(v_pages, "v_pages")
    _need(table, "table", torch.int32)
    n_pages, nkv, page_size, hd = k_pages.shape
    T = q.shape[0]
    if q.shape[1] != n_heads * hd:
        raise KernelError("attention: q has the wrong width")
    if out is None:
        out = torch.empty_like(q)
    _work(f"attention_simt {T}x{n_heads}", _nbytes(q, out))
    _check(lib().ik_attention_simt(_ptr(q), _code(q), _ptr(k_pages), _ptr(v_pages), _code(k_pages), _ptr(out),
                                   _code(out), _ptr(token_seq), _ptr(token_pos), _ptr(table), table.stride(0), T,
                                   n_heads, nkv, hd, scale, window, page_size, n_pages, _ptr(status), _stream()),
           "attention_simt")
    return out


def wait_records() -> str:
    """Where the first wait of each tensor-core module gave up since the last call (read and cleared): text for an
    error message, empty if none did."""
    found = []
    rec = (ctypes.c_int * 4)()
    takers = [("matrix product", lib().ik_gemm_tcgen05_take_wait_record)]
    from . import attention_bf16
    for hd, m in attention_bf16._modules.items():
        takers.append((f"attention (head size {hd})", m.ik_attn_take_wait_record))
    for name, take in takers:
        if take(rec) == 0 and rec[0] != 0:
            found.append(f"{name}: wait site {rec[0]}, block {rec[1]}, count {rec[2]}, parity {rec[3]}")
    return "; ".join(found)


def selftest_wait_expires(status: torch.Tensor, limit_ns: int = 1_000_000) -> torch.Tensor:
    """Runs the kernel library's check of its bounded waits: waits that nothing satisfies, with a limit of
    ``limit_ns`` (at most 10 ms).  Returns int32 [6]: see gemm_tcgen05.cu."""
    result = torch.full((6,), -1, dtype=torch.int32, device=status.device)
    never = torch.zeros(1, dtype=torch.int32, device=status.device)
    _check(lib().ik_selftest_wait_expires(_ptr(status), _ptr(result), _ptr(never), limit_ns, _stream()), "selftest_wait_expires")
    return result


def tcgen05_issue_rate(n: int, per_commit: int, issuers: int, status: torch.Tensor) -> float:
    """Cycles of the SM clock per tcgen05 product instruction (128 rows, 16 k, ``n`` tokens) when ``issuers`` threads (1 or
    2) issue them back to back, ``per_commit`` between commits, and nothing else runs: what the issuing thread costs.
    With two threads the figure is per thread; together they issue twice as many."""
    out = torch.zeros(2, dtype=torch.int64, device=status.device)
    _check(lib().ik_gemm_tcgen05_issue_rate(n, per_commit, issuers, _ptr(out), _ptr(status), _stream()), "tcgen05_issue_rate")
    cycles, fine = (int(v) for v in out.tolist())
    if not fine:
        raise KernelError("tcgen05_issue_rate: a wait ran out")
    return cycles / (64 * per_commit)


_argmax_scratch = {}


def argmax_scratch(device, fresh: bool = False) -> torch.Tensor:
    """Scratch of the split argmax (counters and per-slice bests), zeroed once; the kernel leaves it as it found
    it.  Launches that share one must follow one another in one stream: by default there is one per (device,
    stream); ``fresh`` makes one for a caller that keeps its own (a captured graph)."""
    if fresh:
        return torch.zeros(lib().ik_argmax_scratch_bytes() // 4, dtype=torch.int32, device=device)
    key = (str(torch.device(device)), _stream())
    t = _argmax_scratch.get(key)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("argmax: no scratch exists for this stream yet and none can be made during a capture; "
                              "pass one made with argmax_scratch(device, fresh=True)")
        t = _argmax_scratch[key] = torch.zeros(lib().ik_argmax_scratch_bytes() // 4, dtype=torch.int32, device=device)
    return t


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of each row's largest value (the lowest index among equals)."""
    _need(logits, "logits", torch.float32, contiguous=False)
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if scratch is None:
        scratch = argmax_scratch(logits.device)
    _work(f"argmax {rows}x{V}", rows * V * 4)
    _check(lib().ik_argmax(_ptr(logits), logits.stride(0), _ptr(out), rows, V, _ptr(scratch), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repetition_penalty: float,
           recent: Optional[torch.Tensor], seed: int, streams: torch.Tensor, counters: torch.Tensor,
           out: Optional[torch.Tensor] = None, work: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "logits", torch.float32, contiguous=False)
    _need(streams, "streams", torch.int32)
    _need(counters, "counters", torch.int32)
    rows, V = logits.shape
    n_recent = 0
    if recent is not None:
        _need(recent, "recent", torch.int32)
        n_recent = recent.shape[1]
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if work is None:
        work = torch.empty((rows, V), dtype=torch.float32, device=logits.device)
    _work(f"sample {rows}x{V}", 3 * rows * V * 4)
    _check(lib().ik_sample(_ptr(logits), logits.stride(0), _ptr(work), _ptr(out), rows, V, temperature, top_k, top_p,
                           repetition_penalty, _ptr(recent), n_recent, seed & 0xFFFFFFFFFFFFFFFF, _ptr(streams),
                           _ptr(counters), _stream()), "sample")
    return out
