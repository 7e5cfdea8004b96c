"""Attention kernels of the bfloat16 path: one compiled module per head size.

``attention_bf16.cu`` is specialised at compile time for a head size; the module for the
size a model has is compiled the first time that model runs a step (a few seconds) and kept
beside the core library.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import build
from . import ops
from .ops import KernelError, _check, _ptr, _stream, sm_count

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_modules: Dict[int, ctypes.CDLL] = {}

DECODE_CHUNK_PAGES = 4        # default: a decode block covers 4 pages = 256 keys; chunks start at multiples of that


def decode_chunk_pages(n_seqs: int, n_heads: int, n_kv_heads: int, max_kv_len: int, page_size: int = 64,
                       n_sm: Optional[int] = None) -> int:
    """Pages per decode block.  Measured on B200 (head size 128, 8 kv heads, contexts 1k-16k, batches 1-64,
    chunks of 2-32 pages): the kernel is fastest with about two blocks per SM in ONE wave, so the pages of a
    sequence are cut into as many chunks as that allows, but into chunks of at least 4 pages (2 when even
    that leaves most SMs idle: set-up and merging per block cost about as much as reading two pages).  With
    more (sequence, kv head) groups than two per SM, or a count that would load the SMs unevenly, there
    are several waves anyway; a long chunk and a short rest then pack best (the short blocks of the last chunk
    start last and fill the tail).  Over 72 measured (batch, context) pairs the chunk picked here is within 1 % of
    the best one's time on average, 13 % at worst."""
    N_SM = n_sm if n_sm is not None else sm_count()
    groups = n_seqs * n_kv_heads * -(-(n_heads // n_kv_heads) // 16)
    pages = max(1, -(-max_kv_len // page_size))
    if groups <= N_SM or groups > 1.5 * N_SM and groups <= 2 * N_SM:
        # (between one and one and a half groups per SM a single wave would give some SMs two blocks and others one)
        n_chunks = max(1, (2 * N_SM) // groups)
        least = 4 if groups * -(-pages // 4) >= 128 else 2
        return min(pages, max(-(-pages // n_chunks), least))
    return -(-pages * 3 // 4) if pages <= 24 else 20


def supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def module(head_dim: int) -> ctypes.CDLL:
    key = head_dim
    m = _modules.get(key)
    if m is None:
        m = build.load_library(f"ithaca_attn_hd{head_dim}", ["attention_bf16.cu"], defines=[f"IK_HD={head_dim}"])
        m.ik_attn_prefill.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp, _vp]
        m.ik_attn_prefill.restype = _i
        m.ik_attn_prefill_tc.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp, _vp]
        m.ik_attn_prefill_tc.restype = _i
        m.ik_attn_decode.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _i, _i, _i, _i,
                                     _vp, _vp]
        m.ik_attn_decode.restype = _i
        m.ik_attn_take_wait_record.argtypes = [_vp]
        m.ik_attn_take_wait_record.restype = _i
        if m.ik_attn_head_dim() != head_dim:
            raise KernelError("the attention module was compiled for another head size")
        _modules[key] = m
    return ops.timed(m)


def prefill(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, cu_seqlens: torch.Tensor,
            kv_lens: torch.Tensor, table: torch.Tensor, n_seqs: int, max_new: int, n_heads: int, scale: float,
            window: int, status: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
            kind: str = "auto", work: Optional[Tuple[int, int]] = None) -> torch.Tensor:
    """``kind``: "tc" = the tcgen05 kernel (head sizes 64 and 128), "mma" = the warp-level kernel,
    "auto" = tcgen05 where it applies."""
    n_pages, nkv, page_size, hd = k_pages.shape
    m = module(hd)
    if out is None:
        out = torch.empty_like(q)
    if kind == "tc" or (kind == "auto" and hd in (64, 128)):
        ops._work(f"attention prefill tcgen05 {q.shape[0]}x{n_heads}", *(work or (0, 0)))
        st = m.ik_attn_prefill_tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(cu_seqlens), _ptr(kv_lens),
                                  _ptr(table), table.stride(0), q.shape[0], n_seqs, max_new, n_heads, nkv, scale, window,
                                  page_size, n_pages, _ptr(status), _stream())
        if st != -2:
            _check(st, "attention prefill (tcgen05)")
            return out
        if kind == "tc":
            raise KernelError("attention prefill (tcgen05): head size or alignment not supported")
    ops._work(f"attention prefill mma {q.shape[0]}x{n_heads}", *(work or (0, 0)))
    _check(m.ik_attn_prefill(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(cu_seqlens), _ptr(kv_lens),
                             _ptr(table), table.stride(0), n_seqs, max_new, n_heads, nkv, scale, window, page_size,
                             n_pages, _ptr(status), _stream()), "attention prefill")
    return out


def decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, kv_lens: torch.Tensor, table: torch.Tensor,
           n_seqs: int, kv_len_bound: int, n_heads: int, scale: float, window: int, status: Optional[torch.Tensor],
           out: Optional[torch.Tensor] = None, chunk_pages: int = DECODE_CHUNK_PAGES, ring_kb: int = 0,
           work: Optional[Tuple[int, int]] = None) -> torch.Tensor:
    """``kv_len_bound``: no sequence of the step is longer than this (it sizes the grid and the
    scratch for the partial results; blocks beyond a sequence's length return at once)."""
    n_pages, nkv, page_size, hd = k_pages.shape
    m = module(hd)
    n_splits = max(1, -(-kv_len_bound // (chunk_pages * page_size)))
    part_o = torch.empty((n_seqs, n_heads, n_splits, hd), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n_seqs, n_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    if out is None:
        out = torch.empty_like(q)
    ops._work(f"attention decode {n_seqs}x{n_heads}", *(work or (0, 0)))
    _check(m.ik_attn_decode(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(part_o), _ptr(part_ml),
                            _ptr(kv_lens), _ptr(table), table.stride(0), n_seqs, n_heads, nkv, scale, window,
                            page_size, n_pages, chunk_pages, n_splits, ring_kb, _ptr(status), _stream()), "attention decode", kernels=2)
    return out


def attend(q, k_pages, v_pages, ctx, table, n_heads: int, scale: float, window: int,
           status) -> Optional[torch.Tensor]:
    """Returns None when no specialised kernel takes these sizes (the caller then uses the
    CUDA-core kernel)."""
    n_pages, nkv, page_size, hd = k_pages.shape
    if k_pages.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or page_size != 64 or not supported(hd):
        return None
    work = None
    if ops.profiling():
        # (query, key) pairs under the causal mask (and the window), from the host's copy of the lengths
        pairs = 0
        for n, end in zip(ctx.host_n_new, ctx.host_kv_lens):
            for p in range(end - n, end):
                pairs += min(p + 1, window) if window else p + 1
        keys = sum(min(e, window + n) if window else e for n, e in zip(ctx.host_n_new, ctx.host_kv_lens))
        work = (2 * q.numel() * 2 + 2 * keys * nkv * hd * 2, 4 * hd * n_heads * pairs)
    if ctx.is_decode:
        # from the bound, not from this step's longest sequence: a captured graph is replayed for other lengths
        chunk = decode_chunk_pages(ctx.n_seqs, n_heads, nkv, ctx.kv_len_bound, page_size)
        return decode(q, k_pages, v_pages, ctx.kv_lens, table, ctx.n_seqs, ctx.kv_len_bound, n_heads, scale, window,
                      status, chunk_pages=chunk, work=work)
    return prefill(q, k_pages, v_pages, ctx.cu_seqlens, ctx.kv_lens, table, ctx.n_seqs, ctx.max_new, n_heads, scale,
                   window, status, work=work)
