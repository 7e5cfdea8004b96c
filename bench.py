"""Decode and prefill throughput of the Llama-3.1-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl reference]
    python bench.py --only decode|prefill|attention|products   one part alone (small cases for profiling)
    python bench.py --only marginal [--batch B]                 what each kernel family costs inside the replayed decode step
    python bench.py --config 1b-unequal|13b-long                the other two workloads alone, through Engine.generate

Prints ONE JSON line.  ``value`` is decoded tokens per second at the given batch with every
sequence's cache filled to the context length; a step is one decode step (forward pass of one
token per sequence plus the greedy pick), replayed from a CUDA graph and timed with CUDA events.
``e2e`` is the same through ``Engine.generate`` (host token ids in, host token ids out, one
upload of the step's description and one read-back of the sampled ids per step).
``prefill`` is one step of 2,048 prompt tokens (the median of five, each timed alone after a
short pause and held against the burst peak; back to back the step takes about a tenth longer
under the power cap).  ``roofline`` divides the bytes a decode step
has to read (every weight once, and the cache of the live sequences) by its time.
``points`` holds decoding at batch 1 and 64 and the two other workloads, each through ``Engine.generate``:
``1b_unequal`` (Llama-3.2-1B shape, 64 prompts of 16 to 2,048 tokens in one prompt step, then 256 decode steps) and
``13b_long`` (Llama-2-13B shape, 8 prompts of 1,024 tokens decoded to 4,096 positions, with the rate near 1,024,
2,048 and 4,096).  Peaks come from MEASURED_PEAKS.json; when that file is absent they are measured here with
this library's own copy and tcgen05 product kernels.
Weights are random (seeded), token ids are seeded-uniform: no dataset, no checkpoint.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_3_1_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                             "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
}
LLAMA_3_2_1B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 16, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True, "torch_dtype": "bfloat16",
}
LLAMA_2_13B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 5120, "num_hidden_layers": 40, "num_attention_heads": 40,
    "num_key_value_heads": 40, "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096 + 64, "tie_word_embeddings": False,
    "torch_dtype": "bfloat16",
}
SHAPES = {"8b": ("Llama-3.1-8B shape", LLAMA_3_1_8B), "1b": ("Llama-3.2-1B shape", LLAMA_3_2_1B),
          "13b": ("Llama-2-13B shape", LLAMA_2_13B)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
E2E_STEPS = 128


def peaks():
    """The roofline's denominators: the driver's measurement if its file is there, else measured now with this
    library's own kernels (the reference measures its device the same way, src/hub.cpp:503-549)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            if all(isinstance(d.get(k), (int, float)) for k in ("hbm_gbs", "bf16_tflops")):
                return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except (OSError, ValueError):
            pass
    from ithaca_b200.engine.profile import measure_peaks
    out = measure_peaks("cuda:0")
    return {"hbm_gbs": out["hbm_gbs"], "bf16_tflops": out["bf16_tflops"], "source": "self-measured"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def fill_cache(eng, slots, length, vocab, seed):
    """Brings every slot to ``length`` positions by real prefill steps of random tokens."""
    import numpy as np
    rng = np.random.default_rng(seed)
    chunk = 2048
    group = max(1, 16384 // chunk)
    for g0 in range(0, len(slots), group):
        part = slots[g0:g0 + group]
        done = 0
        while done < length:
            n = min(chunk, length - done)
            eng.step(part, [rng.integers(0, vocab, size=n).tolist() for _ in part], None)
            done += n


def decode_run(eng, batch, steps, warmup, vocab, context, clocks=None):
    """Times ``steps`` graph-replayed decode steps at ``batch`` sequences whose caches hold
    about ``context`` positions (the last timed step reaches exactly ``context``)."""
    import numpy as np
    import torch
    slots = [eng.alloc_slot() for _ in range(batch)]
    fill_cache(eng, slots, context - steps - warmup - 1, vocab, seed=batch)
    dec = eng._decoder
    rng = np.random.default_rng(1000 + batch)
    toks = [[int(x)] for x in rng.integers(0, vocab, size=batch)]
    dec.step(slots, toks)                                   # captures the graph for this shape
    for _ in range(warmup):
        _, ids = dec.step(slots, toks)
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        _, ids = dec.step(slots, toks)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    info = clocks.stop() if clocks is not None else None
    eng.stepper.check_status()
    launches = dec.launches_last_step
    kv_len = eng.cache.length(slots[0])
    for s in slots:
        eng.free_slot(s)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches_per_step": launches,
            "kv_len": kv_len, "clocks": info}


def e2e_run(eng, batch, steps, vocab, context):
    """The same decode steps through the public entry point: host ids in, host ids out.  Always over the same
    number of steps, whatever --steps says.  The steps right behind the long prompt step run slower (the device
    comes out of the prompt's power draw), so the rate of the first 32 steps is given beside the settled one."""
    import numpy as np
    rng = np.random.default_rng(77)
    prompts = [rng.integers(0, vocab, size=context - steps - 1).tolist() for _ in range(batch)]
    # warm-up over the same lengths: every graph shape the timed run meets exists afterwards
    eng.generate(prompts, max_tokens=steps + 1, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    stamps = []

    def on_token(request, token):
        if request == 0:
            stamps.append(time.perf_counter())
        return True

    out = eng.generate(prompts, max_tokens=steps + 1, temp=0.0, rep_pen=1.0, stop_token_ids=[], on_token=on_token)
    st = eng.last_stats
    assert all(len(o) == steps + 1 for o in out) and len(stamps) == steps + 1
    # the first token of each sequence comes from the prefill step; the decode clock covers the rest
    return {"tok_s": batch * steps / st.decode_seconds, "h2d": eng._decoder.last_upload_bytes, "d2h": batch * 4 + 4,
            "first32_tok_s": batch * 32 / (stamps[32] - stamps[0]),
            "settled_tok_s": batch * (steps - 64) / (stamps[steps] - stamps[64]), "steps": steps}


def unequal_1b_run(pk):
    """Llama-3.2-1B shape: 64 prompts with lengths uniform in 16..2,048 as one prompt step (which the engine runs in
    passes of at most 16,384 tokens), then 256 decode steps, through Engine.generate."""
    import numpy as np
    import torch
    from ithaca_b200 import Engine
    name, cfg = SHAPES["1b"]
    n_req, steps = 64, 256
    rng = np.random.default_rng(4)
    lens = [int(x) for x in rng.integers(16, 2049, size=n_req)]
    vocab = cfg["vocab_size"]
    prompts = [rng.integers(0, vocab, size=n).tolist() for n in lens]
    room = sum(-(-(n + steps + 1) // 64) * 64 for n in lens)
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=room, max_slots=n_req, ctx=2048 + steps + 64)
    opts = dict(max_tokens=steps + 1, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    eng.generate(prompts, **opts)                         # warm-up: the same lengths, so every graph shape exists
    torch.cuda.synchronize()
    out = eng.generate(prompts, **opts)
    st = eng.last_stats
    assert all(len(o) == steps + 1 for o in out) and st.batches == 1
    mean_kv = sum(lens) / n_req + steps / 2
    step_bytes = eng.model.weight_bytes() + eng.cache.bytes_per_token() * mean_kv * n_req
    gbs = step_bytes / (st.decode_seconds / steps) / 1e9
    layer_flops, head_flops = model_flops_per_token(cfg, cfg["num_hidden_layers"])
    attn = sum(4 * cfg["num_attention_heads"] * cfg["head_dim"] * n * (n + 1) / 2 for n in lens) * cfg["num_hidden_layers"]
    pre_flops = layer_flops * sum(lens) + attn + head_flops * n_req
    res = {"model": name, "requests": n_req, "prompt_tokens": sum(lens), "prompt_passes": eng.stepper.max_step_tokens,
           "prefill_tok_s": round(sum(lens) / st.prefill_seconds, 1),
           "prefill_frac": round(pre_flops / st.prefill_seconds / (pk["bf16_tflops"] * 1e12), 4),
           "decode_steps": steps, "decode_tok_s": round(n_req * steps / st.decode_seconds, 1),
           "mean_kv_len": round(mean_kv, 1), "step_gb": round(step_bytes / 1e9, 3), "hbm_frac": round(gbs / pk["hbm_gbs"], 4)}
    del eng
    torch.cuda.empty_cache()
    return res


def long_13b_run(pk):
    """Llama-2-13B shape: 8 prompts of 1,024 tokens, decoded until every sequence holds 4,096 positions, through
    Engine.generate; the rate is taken over 128 steps near 1,024, 2,048 and 4,096 positions from the host's clock
    at each token."""
    import numpy as np
    import torch
    from ithaca_b200 import Engine
    name, cfg = SHAPES["13b"]
    batch, prompt_len, final = 8, 1024, 4096
    steps = final - prompt_len
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(6)
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=batch * (final + 64), max_slots=batch, ctx=final + 64)
    opts = dict(temp=0.0, rep_pen=1.0, stop_token_ids=[])
    # warm-up: a short run at each width of block table the long run will meet, so that its graphs exist
    from ithaca_b200.engine.graph import _bucket
    widths = sorted({_bucket(c) for c in range(prompt_len // 64 + 1, final // 64 + 1)})
    for w in widths:
        n = min(final - 8, max(prompt_len, (w - 1) * 64 + 8))
        eng.generate([rng.integers(0, vocab, size=n).tolist() for _ in range(batch)], max_tokens=4, **opts)
    prompts = [rng.integers(0, vocab, size=prompt_len).tolist() for _ in range(batch)]
    stamps = []

    def on_token(request, token):
        if request == 0:
            stamps.append(time.perf_counter())
        return True

    torch.cuda.synchronize()
    out = eng.generate(prompts, max_tokens=steps + 1, on_token=on_token, **opts)
    st = eng.last_stats
    assert all(len(o) == steps + 1 for o in out) and len(stamps) == steps + 1
    weight_bytes, per_token = eng.model.weight_bytes(), eng.cache.bytes_per_token()
    res = {"model": name, "batch": batch, "prompt_len": prompt_len, "final_len": final,
           "prefill_tok_s": round(batch * prompt_len / st.prefill_seconds, 1),
           "decode_tok_s": round(batch * steps / st.decode_seconds, 1)}
    for label, s0 in (("1024", 0), ("2048", 2048 - prompt_len - 64), ("4096", steps - 128)):
        dt = (stamps[s0 + 128] - stamps[s0]) / 128
        kv = prompt_len + s0 + 64
        res[f"tok_s_at_{label}"] = round(batch / dt, 1)
        res[f"hbm_frac_at_{label}"] = round((weight_bytes + per_token * kv * batch) / dt / 1e9 / pk["hbm_gbs"], 4)
    del eng
    torch.cuda.empty_cache()
    return res


def prefill_run(eng, tokens, vocab, reps=5):
    import numpy as np
    import torch
    rng = np.random.default_rng(5)
    times = []
    for r in range(reps + 1):
        time.sleep(0.3)                                     # each run alone, as a prompt arrives: not in the power state the run before left
        s = eng.alloc_slot()
        ids = rng.integers(0, vocab, size=tokens).tolist()
        ctx = eng.stepper.prepare([s], [ids], "last")
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.model.forward(ctx, eng.cache)
        b.record()
        torch.cuda.synchronize()
        eng.stepper.finish(ctx)
        eng.free_slot(s)
        if r > 0:                                           # the first run is the warm-up
            times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]                   # the median


def products_run(cfg, tokens, reps):
    """A layer's four matrix products alone at ``tokens`` tokens, this library's tcgen05 kernel beside cuBLAS
    (torch.matmul) on the same operands; the weights are rotated through copies larger than L2 together."""
    import torch
    from ithaca_b200.csrc import ops
    dev = "cuda:0"
    d, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = []
    for name, n, k in [("qkv", qkv, d), ("o", d, cfg["num_attention_heads"] * cfg["head_dim"]), ("gate_up", 2 * ff, d), ("down", d, ff)]:
        copies = max(2, min(8, int(300e6 // (n * k * 2)) + 1))
        ws = [torch.randn((n, k), device=dev).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn((tokens, k), device=dev).to(torch.bfloat16)
        y = torch.empty((tokens, n), device=dev, dtype=torch.float32)
        yb = torch.empty((tokens, n), device=dev, dtype=torch.bfloat16)
        row = {"product": name, "rows": n, "k": k}
        for label, fn in [("ours_us", lambda i: ops.gemm_tcgen05(x, ws[i % copies], out=y, status=status)),
                          ("cublas_us", lambda i: torch.matmul(x, ws[i % copies].T, out=yb))]:
            for i in range(3):
                fn(i)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(reps * copies):
                fn(i)
            b.record()
            torch.cuda.synchronize()
            row[label] = round(a.elapsed_time(b) / (reps * copies) * 1e3, 1)
        row["ours_tflops"] = round(2 * tokens * n * k / row["ours_us"] / 1e6, 1)
        row["cublas_tflops"] = round(2 * tokens * n * k / row["cublas_us"] / 1e6, 1)
        out.append(row)
        del ws
    out.append({"status": int(status.item())})
    return out


def products_sweep(cfg, token_counts, reps):
    """A layer's four products at decode-sized token counts: what the dispatcher picks, the warp-level kernel, the
    tcgen05 kernel under each way of sharing out its work (whole tiles, 2 to 8 K slices, stream-K), and cuBLAS.  Each
    variant is captured into a CUDA graph of one call per weight copy (copies larger than L2 together) and the
    graph is replayed, so the figures are device times of back-to-back launches, not of the host's call rate."""
    import torch
    from ithaca_b200.csrc import gemm_bf16, ops
    dev = "cuda:0"
    d, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    status = ops.device_status(dev)
    ops.stream_k_scratch(dev)
    out = []
    for name, n, k in [("qkv", qkv, d), ("o", d, cfg["num_attention_heads"] * cfg["head_dim"]), ("gate_up", 2 * ff, d), ("down", d, ff)]:
        copies = max(2, min(8, int(300e6 // (n * k * 2)) + 1))
        ws = [torch.randn((n, k), device=dev).to(torch.bfloat16) for _ in range(copies)]
        for tokens in token_counts:
            x = torch.randn((tokens, k), device=dev).to(torch.bfloat16)
            y = torch.empty((tokens, n), device=dev, dtype=torch.float32)
            yb = torch.empty((tokens, n), device=dev, dtype=torch.bfloat16)
            variants = {"auto": lambda w: gemm_bf16.gemm(x, w, out=y)}
            if tokens <= 64:
                variants["skinny"] = lambda w: ops.gemm_bf16_mma(x, w, out=y, kind=1)
            for s, label in ((1, "tc_tiles"), (2, "tc_k2"), (4, "tc_k4"), (8, "tc_k8"), (0, "tc_stream_k"),
                             (-2, "tc_cl2"), (-3, "tc_cl3"), (-4, "tc_cl4")):
                if s < 0 and not ops.tcgen05_cluster_fits(tokens, n, k, -s):
                    continue
                variants[label] = (lambda s_: lambda w: ops.gemm_tcgen05(x, w, out=y, status=status, splits=s_))(s)
            variants["cublas"] = lambda w: torch.matmul(x, w.T, out=yb)
            row = {"product": name, "rows": n, "k": k, "tokens": tokens, "picked_splits": ops.tcgen05_splits(tokens, n, k),
                   "picked_skinny": gemm_bf16.takes_skinny(tokens, n, k), "ideal_us": round(n * k * 2 / pk_hbm() / 1e3, 1)}
            for label, fn in variants.items():
                for w in ws[:2]:
                    fn(w)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for w in ws:
                        fn(w)
                g.replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(reps):
                    g.replay()
                b.record()
                torch.cuda.synchronize()
                row[label] = round(a.elapsed_time(b) / (reps * copies) * 1e3, 1)
                del g
            out.append(row)
        del ws
    out.append({"status": int(status.item())})
    return out


def pk_hbm():
    return peaks()["hbm_gbs"]


def attention_run(cfg, reps):
    """The prefill attention kernel alone, on one sequence in a shuffled paged cache: the whole prompt, a chunk
    behind cached tokens, and one query tile per block in front of a long context with two blocks for every SM."""
    import math
    import torch
    from ithaca_b200.csrc import attention_bf16 as A
    dev = "cuda:0"
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    out = []
    for name, heads, kv_heads, kv_len, n_new in [("prompt of 2048", nh, nkv, 2048, 2048), ("2048 behind 6144", nh, nkv, 8192, 2048),
                                                 ("one tile behind 8064, 296 heads", 296, 74, 8192, 128)]:
        g = torch.Generator(device=dev).manual_seed(3)
        n_pages = kv_len // 64
        k = torch.randn((n_pages, kv_heads, 64, hd), device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn((n_pages, kv_heads, 64, hd), device=dev, generator=g).to(torch.bfloat16)
        table = torch.randperm(n_pages, device=dev, generator=g).to(torch.int32).view(1, -1)
        q = torch.randn((n_new, heads * hd), device=dev, generator=g).to(torch.bfloat16)
        cu = torch.tensor([0, n_new], dtype=torch.int32, device=dev)
        lens = torch.tensor([kv_len], dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        res = torch.empty_like(q)
        run = lambda: A.prefill(q, k, v, cu, lens, table, 1, n_new, heads, 1 / math.sqrt(hd), 0, status, out=res)
        for _ in range(2):
            run()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            run()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / reps * 1e3
        pairs = sum(min(kv_len - n_new + i + 1, kv_len) for i in range(n_new))          # (query, key) pairs under the causal mask
        out.append({"case": name, "us": round(us, 1), "tflops": round(4 * hd * heads * pairs / us / 1e6, 1),
                    "status": int(status.item())})
    return out


def marginal_run(eng, cfg, batch, vocab, context, steps=30):
    """What each kernel family costs inside the graph-replayed decode step: the step is captured again with that
    family's launches left out (its results are then wrong, its time is what the rest takes) and the difference to the
    whole step is the family's share, overlap with its neighbours included.  Per layer, in microseconds."""
    import torch
    from ithaca_b200.csrc import attention_bf16, gemm_bf16, ops
    slots = [eng.alloc_slot() for _ in range(batch)]
    fill_cache(eng, slots, context - 100, vocab, seed=1)
    dec, toks, layers = eng._decoder, [[7]] * batch, cfg["num_hidden_layers"]
    d, ff = cfg["hidden_size"], cfg["intermediate_size"]
    keep = dict(rmsnorm=ops.rmsnorm, decode=attention_bf16.decode, gemm=gemm_bf16.gemm, swiglu=gemm_bf16.gemm_swiglu, qkv=ops.gemm_qkv_rope)
    bufs = {}

    def buf(key, shape, dtype, dev):
        if key not in bufs:
            bufs[key] = torch.zeros(shape, dtype=dtype, device=dev)
        return bufs[key]

    def no_norm(x, w, eps, out_dtype, rows_in=None, out=None):
        rows = x.shape[0] if rows_in is None else rows_in.numel()
        return buf(("n", rows, out_dtype), (rows, x.shape[1]), out_dtype, x.device)

    def no_product(rows, cols):
        def f(x, w, out=None, accumulate=False, out_dtype=torch.float32):
            if tuple(w.shape) != (rows, cols):
                return keep["gemm"](x, w, out=out, accumulate=accumulate, out_dtype=out_dtype)
            return out if out is not None else buf(("g", x.shape[0], rows), (x.shape[0], rows), out_dtype, x.device)
        return f

    def timed():
        dec.graphs.clear()
        dec.step(slots, toks)
        for _ in range(5):
            dec.step(slots, toks)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            dec.step(slots, toks)
        b.record()
        torch.cuda.synchronize()
        for s in slots:
            eng.truncate(s, eng.length(s) - steps - 6)          # every variant at the same context
        return a.elapsed_time(b) / steps * 1e3 / layers

    out = {"whole_step": round(timed(), 2)}
    variants = [("norms", ops, "rmsnorm", no_norm),
                ("attention_and_merge", attention_bf16, "decode", lambda q, *a, **k: buf(("a", q.shape), q.shape, q.dtype, q.device)),
                ("o", gemm_bf16, "gemm", no_product(d, cfg["num_attention_heads"] * cfg["head_dim"])),
                ("down", gemm_bf16, "gemm", no_product(d, ff)),
                ("gate_up", gemm_bf16, "gemm_swiglu", lambda x, w, out_dtype=torch.bfloat16: buf(("s", x.shape[0]), (x.shape[0], w.shape[0] // 2), out_dtype, x.device)),
                ("qkv", ops, "gemm_qkv_rope", lambda *a, **k: True)]
    for name, module, attr, stand_in in variants:
        original = getattr(module, attr)
        setattr(module, attr, stand_in)
        try:
            out[name] = round(out["whole_step"] - timed(), 2)
        finally:
            setattr(module, attr, original)
    eng.runtime.status.zero_()
    dec.graphs.clear()
    for s in slots:
        eng.free_slot(s)
    return out


def attempt(run, eng=None):
    """One part of the line: run it, once more if it raises, and if it raises again say so in its place.  The other
    parts of the line stand on their own measurements and are printed all the same."""
    last = None
    for _ in range(2):
        try:
            return run()
        except Exception as e:                             # noqa: BLE001  (whatever it is goes into the line)
            last = e
            import torch
            torch.cuda.synchronize()
            if eng is not None:
                eng.runtime.status.zero_()
                for s in range(eng.cache.max_slots):
                    if eng.cache.table.in_use(s):
                        eng.free_slot(s)
    return {"error": f"{type(last).__name__}: {last}"[:300]}


def model_flops_per_token(cfg, n_layers):
    d, ff, nh, nkv, hd, V = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                             cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"])
    per_layer = 2 * (d * (nh + 2 * nkv) * hd + nh * hd * d + 3 * d * ff)
    return per_layer * n_layers, 2 * d * V


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES),
                    help="layer sizes: 8b is the benchmark's configuration, the others are for comparison")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 decode points and the two other workloads")
    ap.add_argument("--tokens", default=None,
                    help="with --only products: token counts, e.g. 16,32,64: a sweep over the ways the products can run")
    ap.add_argument("--context", type=int, default=None,
                    help="with --only decode / prefill: another context length (decode) or prompt length (prefill) than the default run's")
    ap.add_argument("--config", default=None, choices=["1b-unequal", "13b-long"],
                    help="run one of the other workloads alone and print its figures")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "attention", "products", "marginal", "issue-rate"],
                    help="run one part only and print its figures (for profiling a small case)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "SwankyMan88/ithaca is a Windows-only C++ program (windows.h, nvcuda.dll, build.bat) with no "
                          "Python package or POSIX build: pip cannot install it here and it cannot run on Linux"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this library has no multi-GPU path); --gpus {args.gpus} is not run")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from ithaca_b200 import Engine

    pk = peaks()
    if args.config:
        res = unequal_1b_run(pk) if args.config == "1b-unequal" else long_13b_run(pk)
        print(json.dumps({"config": args.config, "peaks": pk["source"], **res}))
        return 0
    shape_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    if args.only == "issue-rate":
        # what the thread that issues tensor-core products costs: cycles per instruction, one or two issuing threads
        from ithaca_b200.csrc import ops
        status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        rows = [{"tokens": n, "per_commit": per, "issuers": k, "cycles_per_instruction": round(ops.tcgen05_issue_rate(n, per, k, status), 1)}
                for k in (1, 2) for n in (64, 128, 256) for per in (4, 8, 16)]
        print(json.dumps({"only": "issue-rate", "tensor_core_cycles": {"64": 32, "128": 64, "256": 128}, "rows": rows, "status": int(status.item())}))
        return 0
    if args.only == "products" and args.tokens:
        counts = [int(t) for t in args.tokens.split(",")]
        print(json.dumps({"only": "products", "model": shape_name, "sweep": products_sweep(cfg, counts, reps=max(3, min(args.steps, 20)))}))
        return 0
    if args.only == "products":
        print(json.dumps({"only": "products", "model": shape_name, "tokens": PREFILL_TOKENS,
                          "cases": products_run(cfg, PREFILL_TOKENS, reps=max(1, min(args.steps, 5)))}))
        return 0
    if args.only == "attention":
        print(json.dumps({"only": "attention", "model": shape_name, "cases": attention_run(cfg, reps=max(1, min(args.steps, 5)))}))
        return 0
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    vocab = cfg["vocab_size"]
    point_batches = [] if (args.no_points or args.only != "all") else [1, 64]
    # the cache of the largest batch has to fit beside the weights (bounded on purpose: no memory sweep)
    per_token = 2 * 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"]
    point_batches = [b for b in point_batches if b * (CONTEXT + 64) * per_token < 100e9]
    max_b = max([args.batch] + point_batches)
    context = CONTEXT
    if args.context and args.only in ("decode", "prefill"):
        context = args.context
        if args.only == "decode" and args.batch * (context + 64) * per_token > 100e9:
            print(f"bench.py: batch {args.batch} at context {context} needs more than 100 GB of cache; not run")
            return 2
    layer_flops, head_flops = model_flops_per_token(cfg, n_layers)
    held = max(context, PREFILL_TOKENS) + 64
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max_b * held, ctx=held,
                             max_step_tokens=max(16384, context if args.only == "prefill" else 0))

    if args.only == "decode":
        r = decode_run(eng, args.batch, args.steps, args.warmup, vocab, context)
        read = eng.model.weight_bytes() + eng.cache.bytes_per_token() * r["kv_len"] * args.batch
        print(json.dumps({"only": "decode", "batch": args.batch, "context": context, "layers": n_layers,
                          "hbm_frac": round(read / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                          **{k: v for k, v in r.items() if k != "clocks"}}))
        return 0
    if args.only == "marginal":
        r = marginal_run(eng, cfg, args.batch, vocab, CONTEXT)
        print(json.dumps({"only": "marginal", "batch": args.batch, "layers": n_layers, "us_per_layer": r}))
        return 0
    if args.only == "prefill":
        tokens = args.context or PREFILL_TOKENS
        ms = prefill_run(eng, tokens, vocab, reps=max(1, args.steps))
        flops = layer_flops * tokens + head_flops + 4 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * tokens / 2 * n_layers
        print(json.dumps({"only": "prefill", "layers": n_layers, "tokens": tokens, "ms": ms, "tok_s": round(tokens / (ms / 1e3), 1),
                          "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0

    clocks = ClockSampler()
    main_run = decode_run(eng, args.batch, args.steps, args.warmup, vocab, CONTEXT, clocks)
    points = {}
    if point_batches:
        for b in point_batches:
            r = attempt(lambda: decode_run(eng, b, min(args.steps, 32), args.warmup, vocab, CONTEXT), eng)
            if "error" in r:
                points[f"decode_b{b}_error"] = r["error"]
            else:
                points[f"decode_b{b}"] = round(r["tok_s"], 1)
    e2e = attempt(lambda: e2e_run(eng, args.batch, E2E_STEPS, vocab, CONTEXT), eng)
    pre_ms = prefill_run(eng, PREFILL_TOKENS, vocab)

    attn_flops = 4 * cfg["num_attention_heads"] * cfg["head_dim"] * PREFILL_TOKENS * PREFILL_TOKENS / 2 * n_layers
    pre_flops = layer_flops * PREFILL_TOKENS + attn_flops + head_flops
    weight_bytes = eng.model.weight_bytes()
    kv_bytes = eng.cache.bytes_per_token() * main_run["kv_len"] * args.batch
    achieved = (weight_bytes + kv_bytes) / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s @ batch {args.batch}, context 4096 ({shape_name})",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "config": {"model": shape_name, "layers": n_layers, "layers_of_model": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "global_batch": args.batch,
                   "seq_len": CONTEXT, "parallelism": "single GPU", "l2": "inputs larger than L2 (weights + cache)",
                   "cache_page": 64, "peaks": pk["source"]},
        "clocks": main_run["clocks"],
        "e2e": ({"value": round(e2e["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d"],
                 "d2h_bytes_per_step": e2e["d2h"], "steps": e2e["steps"], "first32_tok_s": round(e2e["first32_tok_s"], 1),
                 "settled_tok_s": round(e2e["settled_tok_s"], 1)} if "error" not in e2e else e2e),
        "gpu_launches": main_run["launches_per_step"] * args.steps,
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    if not args.no_points and args.shape == "8b" and not args.layers:
        del eng
        torch.cuda.empty_cache()
        points["1b_unequal"] = attempt(lambda: unequal_1b_run(pk))
        points["13b_long"] = attempt(lambda: long_13b_run(pk))
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
