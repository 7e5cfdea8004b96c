"""Shared helpers of the GPU tests: tolerances, the plain implementation's logits, traces."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Largest |difference| allowed, as a fraction of the largest |reference logit| of the compared block.
# float32: sums of a few hundred float32 products through a few layers stay below 1e-6; 2e-5 leaves
# room for other summation orders and still is a thousand times tighter than anything 16-bit.
# bfloat16: about five roundings to 8 bits of mantissa per layer, each ~2^-9 relative, adding up at
# random through the layers: a few 1e-3 of the logit scale; 2e-2 bounds the worst of thousands of logits.
REL = {"float32": 2e-5, "bfloat16": 2e-2}
# The same engine under different cuttings of the same tokens.
# float32: none at all.  Every sum of that path runs in an order that depends on the position and size of what is
# summed only, never on the step's shape, so two cuttings of the same tokens must give the same bits.
REL_CUT = {"float32": 0.0, "bfloat16": 1e-2}


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.all(np.isfinite(got)), "non-finite logits"
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def plain_logits(cfg, tensors, ids):
    from plain import llama_plain as P
    return P.logits_whole(ids, cfg, tensors).numpy()


def load_plain(model_dir):
    """config.json as a dictionary and the tensors by name, read without the library's loader."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return cfg, tensors


def random_ids(n, vocab, seed):
    g = np.random.default_rng(seed)
    return [int(x) for x in g.integers(0, vocab, size=n)]


def run_trace(model_dir, dtype, out_dir, max_tokens, steps, timeout=900):
    """Runs bin/trace_run on the given steps; returns {step: float32 array [wanted, vocab]}."""
    os.makedirs(out_dir, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                        "--out", out_dir, "--max-tokens", str(max_tokens)], input=text, capture_output=True,
                       text=True, timeout=timeout)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [l.split()[1] for l in done] == [str(s["step"]) for s in steps], p.stdout[-2000:]
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        n_want = sum(len(e.get("want", [])) for e in s["entries"])
        if n_want:
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
        else:
            assert not os.path.exists(path)
    return out


def run_schedule(eng, requests, schedule, truncations=None):
    """Feeds ``requests`` (lists of token ids) through ``eng.step`` as ``schedule`` says: a list of steps, each a
    list of (request, n) = request brings its next n tokens.  ``truncations``: {step index: [(request, keep)]}, done
    before that step; the request's next tokens then follow position ``keep`` (its tokens from there on are fed
    again).  A request gets its slot when it first appears and gives it back after its last token.  Returns the
    logits of every (request, position) as float32 arrays [len(request), vocab] (the last feeding of a position
    counts)."""
    slots, fed, got = {}, {}, {}
    for n, step in enumerate(schedule):
        for r, keep in (truncations or {}).get(n, []):
            eng.truncate(slots[r], keep)
            fed[r] = keep
        for r, _ in step:
            if r not in slots:
                slots[r] = eng.alloc_slot()
                fed[r] = 0
        toks = [requests[r][fed[r]:fed[r] + k] for r, k in step]
        assert all(len(t) == k for t, (_, k) in zip(toks, step)), "the schedule feeds more tokens than a request has"
        lg = eng.step([slots[r] for r, _ in step], toks, "all").cpu().numpy()
        off = 0
        for r, k in step:
            if r not in got:
                got[r] = np.zeros((len(requests[r]), lg.shape[1]), dtype=np.float32)
            got[r][fed[r]:fed[r] + k] = lg[off:off + k]
            off += k
            fed[r] += k
            if fed[r] == len(requests[r]) and not any(r == q for later in schedule[n + 1:] for q, _ in later):
                eng.free_slot(slots.pop(r))
    eng.check_status()
    assert not slots, "the schedule leaves requests unfinished"
    return got
