"""ik_sample_static, the sampling entry point that allocates no device memory.

Some users of the kernel library cannot allocate: a program that gave the whole device to
its own arena, a loop in which cudaMalloc may not be called because it can stall the device,
a C caller without any tensor allocator.  For them the scratch of the sampling kernel lives
in a fixed device array inside the library.  This test calls that entry point through its
exported C symbol and expects exactly the ids that the ordinary entry point (ik_sample, with
scratch supplied by the caller) returns, on two calls in a row that share the array.

The file is named so that pytest collects it last.
"""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 2 * 1024 * 1024


def static_entry():
    from ithaca_b200.csrc import ops
    fn = ops.lib().ik_sample_static                     # the exported C symbol
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, i, vp, i, i, f, i, f, f, vp, i, ctypes.c_ulonglong, vp, vp, vp]
    fn.restype = i
    return fn, ops


def call_static(fn, logits, temp, top_k, top_p, pen, recent, seed, streams, counters):
    rows, V = logits.shape
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    st = fn(logits.data_ptr(), logits.stride(0), out.data_ptr(), rows, V, temp, top_k, top_p, pen,
            recent.data_ptr() if recent is not None else 0, recent.shape[1] if recent is not None else 0, seed,
            streams.data_ptr(), counters.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return st, out


def case(rows, V, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn((rows, V), generator=g) * 2).to(DEV)
    recent = torch.randint(0, V, (rows, 64), generator=g, dtype=torch.int32)
    recent[:, 40:] = -1
    streams = torch.arange(rows, dtype=torch.int32, device=DEV)
    counters = torch.full((rows,), seed, dtype=torch.int32, device=DEV)
    return logits, recent.to(DEV), streams, counters


def test_static_scratch_gives_the_same_ids_twice_in_a_row():
    fn, ops = static_entry()
    # the second call is smaller than the first: it runs over what the first left in the array
    for rows, V, seed, (temp, top_k, top_p, pen) in [(9, 5003, 1, (0.8, 40, 0.9, 1.1)), (4, 301, 2, (1.3, 100000, 0.7, 1.2)),
                                                    (16, 128256, 3, (0.0, 40, 0.9, 1.1))]:
        logits, recent, streams, counters = case(rows, V, seed)
        want = ops.sample(logits, temp, top_k, top_p, pen, recent, 4321, streams, counters)
        st, got = call_static(fn, logits, temp, top_k, top_p, pen, recent, 4321, streams, counters)
        assert st == 0
        torch.cuda.synchronize()
        assert got.cpu().tolist() == want.cpu().tolist()


def test_the_static_entry_point_takes_no_device_memory():
    """What the entry point is for: between a warmed-up state and the end of a call neither the driver's count of
    free device memory nor torch's own allocator has moved."""
    fn, ops = static_entry()
    logits, recent, streams, counters = case(8, 5003, 7)
    st, _ = call_static(fn, logits, 0.8, 40, 0.9, 1.1, recent, 99, streams, counters)     # first call on the device: set-up
    assert st == 0
    torch.cuda.synchronize()
    out = torch.empty(8, dtype=torch.int32, device=DEV)
    gc.collect()                     # tensors of earlier tests that are still waiting to be collected go now, not in between
    torch.cuda.synchronize()
    count = lambda: torch.cuda.memory_stats()["allocation.all.allocated"]          # allocations torch has ever made
    free0, made0 = torch.cuda.mem_get_info()[0], count()
    for _ in range(3):
        st = fn(logits.data_ptr(), logits.stride(0), out.data_ptr(), 8, 5003, 0.8, 40, 0.9, 1.1, recent.data_ptr(), 64, 99,
                streams.data_ptr(), counters.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert st == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free0, "the driver's free device memory went down during the calls"
    assert count() == made0, "torch's allocator was asked for memory during the calls"


def test_a_request_beyond_the_static_array_is_refused(capfd):
    fn, _ = static_entry()
    rows, V = 17, 128256                                 # 2,180,352 floats > 2,097,152
    assert rows * V > MAX_FLOATS
    logits = torch.zeros((rows, V), device=DEV)
    streams = torch.zeros(rows, dtype=torch.int32, device=DEV)
    st, out = call_static(fn, logits, 0.8, 40, 0.9, 1.0, None, 1, streams, streams)
    torch.cuda.synchronize()
    assert st == -3 and out.cpu().tolist() == [-7] * rows          # nothing was launched
    assert "static array holds 2097152" in capfd.readouterr().err
