"""Looking at a step kernel by kernel, and the device's peaks measured with this library's own kernels.

The reference prints per-operation timers of a forward pass when ``ITHACA_PROF`` / ``ITHACA_GXPROF`` is set
(src/model.cpp:1261-1307, src/cuda_tier.cpp:514-527, src/gx.cpp:302-316) and measures the device's copy bandwidth
and tensor throughput for its hardware report (src/hub.cpp:503-549).  ``profile_step`` is the first: one step of
the engine, run eagerly with CUDA events around every kernel-library call, as a table of time, bytes and
floating-point operations per kernel, held against the peaks.  ``measure_peaks`` is the second.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..csrc import ops


def measure_peaks(device: str = "cuda:0", copy_mib: int = 1024, gemm_n: int = 8192, reps: int = 10) -> Dict[str, float]:
    """``hbm_gbs``: read + write bytes of a copy of ``copy_mib`` MiB (larger than the L2 cache) over its time, the
    best of ``reps``.  ``bf16_tflops``: a bfloat16 product of gemm_n^3 on the tcgen05 kernel, the best of ``reps``.
    Both with this library's kernels, timed with CUDA events."""
    torch.cuda.set_device(device)
    src = torch.empty(copy_mib << 20, dtype=torch.uint8, device=device)
    src.zero_()
    dst = torch.empty_like(src)
    best_copy = float("inf")
    for r in range(reps + 2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ops.copy(src, dst)
        b.record()
        torch.cuda.synchronize()
        if r >= 2:
            best_copy = min(best_copy, a.elapsed_time(b))
    del src, dst
    g = torch.Generator(device=device).manual_seed(1)
    x = (torch.randn((gemm_n, gemm_n), device=device, generator=g) * 0.05).to(torch.bfloat16)
    w = (torch.randn((gemm_n, gemm_n), device=device, generator=g) * 0.05).to(torch.bfloat16)
    y = torch.empty((gemm_n, gemm_n), dtype=torch.bfloat16, device=device)
    status = ops.device_status(device)
    best_gemm = float("inf")
    for r in range(reps + 2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if ops.gemm_tcgen05(x, w, out=y, status=status, splits=1) is None:
            raise ops.KernelError("the tcgen05 product refused the peak measurement's sizes")
        b.record()
        torch.cuda.synchronize()
        if r >= 2:
            best_gemm = min(best_gemm, a.elapsed_time(b))
    return {"hbm_gbs": round(2 * (copy_mib << 20) / (best_copy / 1e3) / 1e9, 1),
            "bf16_tflops": round(2 * gemm_n ** 3 / (best_gemm / 1e3) / 1e12, 1),
            "how": f"own kernels: copy of {copy_mib} MiB (read + write bytes) and a bfloat16 tcgen05 product of {gemm_n}^3, "
                   f"best of {reps}, CUDA events"}


def profile_step(engine, slots: Sequence[int], tokens: Sequence[Sequence[int]], want="last") -> Tuple[Optional[torch.Tensor], List[dict]]:
    """Runs one step like ``Engine.step`` (eagerly, never from a graph) and returns (logits, rows): per kind of
    kernel call and shape, in order of first appearance, the number of calls, their time, and the bytes and
    operations they had to move and do."""
    engine._settle()
    ops.argmax_scratch(engine.runtime.device)             # made now if it is not there yet, not inside the timed calls
    torch.cuda.synchronize()
    with ops.Profile() as prof:
        logits = engine.stepper.step(slots, tokens, want)
        if logits is not None:
            ops.argmax(logits)
    return logits, prof.rows()


def format_table(rows: List[dict], peaks: Optional[Dict[str, float]] = None, title: str = "") -> str:
    """A text table of ``profile_step``'s rows; with ``peaks`` (``hbm_gbs``, ``bf16_tflops``) each row's better
    fraction of a peak is shown."""
    total = sum(r["us"] for r in rows) or 1.0
    lines = []
    if title:
        lines.append(title)
    lines.append(f"{'kernel':<44}{'calls':>6}{'us':>11}{'share':>8}{'GB/s':>9}{'TFLOP/s':>9}{'of peak':>9}")
    for r in rows:
        sec = r["us"] / 1e6
        gbs = r["bytes"] / sec / 1e9 if sec > 0 else 0.0
        tfl = r["flops"] / sec / 1e12 if sec > 0 else 0.0
        frac = ""
        if peaks:
            f = max(gbs / peaks["hbm_gbs"], tfl / peaks["bf16_tflops"])
            frac = f"{f:9.2f}" if r["bytes"] or r["flops"] else ""
        lines.append(f"{r['kernel']:<44}{r['calls']:>6}{r['us']:>11.1f}{r['us'] / total:>8.1%}{gbs:>9.0f}{tfl:>9.1f}{frac}")
    lines.append(f"{'all kernel calls, one after another':<44}{sum(r['calls'] for r in rows):>6}{total:>11.1f}")
    lines.append("(each call timed alone between two events, with the host's gaps between calls: the device clocks lower than "
                 "under a replayed graph, and nothing overlaps; compare shares)")
    return "\n".join(lines)
