"""bin/trace_run: the same requests replayed whole, with the last 32 tokens one by one, and in
batches of unequal lengths whose shorter requests end earlier (one batch after another, in a
cache that only holds one batch, so slots and pages are used again), in float32 and bfloat16.
Every (request, position) is compared with the plain implementation."""
import numpy as np
import pytest

from helpers import REL, REL_CUT, load_plain, plain_logits, random_ids, rel_err, run_trace
from tiny import TINY, make_model_dir

pytestmark = pytest.mark.gpu


def rounded(n):
    return -(-n // 64) * 64


def build_trace(requests):
    """Returns (steps, index): index[(mode, request, position)] = (step, row)."""
    steps, index = [], {}
    n = [0]

    def add(entries, end):
        row = 0
        for e in entries:
            for w in e["want"]:
                index[(e["_mode"], e["_req"], e["_pos0"] + w)] = (n[0], row)
                row += 1
        steps.append({"step": n[0], "entries": [{k: v for k, v in e.items() if not k.startswith("_")} for e in entries],
                      "end": end})
        n[0] += 1

    # each request alone and whole
    for r, ids in enumerate(requests):
        add([{"id": f"w{r}", "tokens": ids, "want": list(range(len(ids))), "_mode": "whole", "_req": r, "_pos0": 0}],
            [f"w{r}"])
    # the last 32 tokens one by one
    for r, ids in enumerate(requests):
        if len(ids) <= 33:
            continue
        cut = len(ids) - 32
        add([{"id": f"d{r}", "tokens": ids[:cut], "want": list(range(cut)), "_mode": "last32", "_req": r, "_pos0": 0}], [])
        for t in range(cut, len(ids)):
            add([{"id": f"d{r}", "tokens": [ids[t]], "want": [0], "_mode": "last32", "_req": r, "_pos0": t}],
                [f"d{r}"] if t == len(ids) - 1 else [])
    # batches of unequal lengths; request i of a batch decodes its last (2 + 3i) tokens one by one
    order = list(range(len(requests)))
    for b0 in range(0, len(order), 3):
        batch = order[b0:b0 + 3]
        tails = {r: min(len(requests[r]) - 1, 2 + 3 * i) for i, r in enumerate(batch)}
        add([{"id": f"b{r}", "tokens": requests[r][:len(requests[r]) - tails[r]],
              "want": list(range(len(requests[r]) - tails[r])), "_mode": "batch", "_req": r, "_pos0": 0} for r in batch],
            [f"b{r}" for r in batch if tails[r] == 0])
        pos = {r: len(requests[r]) - tails[r] for r in batch}
        live = [r for r in batch if tails[r] > 0]
        while live:
            ending = [r for r in live if pos[r] == len(requests[r]) - 1]
            add([{"id": f"b{r}", "tokens": [requests[r][pos[r]]], "want": [0], "_mode": "batch", "_req": r,
                  "_pos0": pos[r]} for r in live], [f"b{r}" for r in ending])
            for r in live:
                pos[r] += 1
            live = [r for r in live if r not in ending]
    return steps, index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_whole_one_by_one_and_batched(tmp_path, name, dtype):
    cfg = TINY[name]
    d = make_model_dir(tmp_path, cfg, seed=21)
    pcfg, tensors = load_plain(d)
    maxpos = cfg["max_position_embeddings"]
    lens = [min(l, maxpos) for l in (100, 37, 64, 5, 1, 129, 65)]
    requests = [random_ids(l, cfg["vocab_size"], 300 + i) for i, l in enumerate(lens)]
    steps, index = build_trace(requests)
    # the most that is live at once: the largest batch of three (whole requests and single ones are smaller)
    most = max(sum(rounded(lens[r]) for r in range(b0, min(b0 + 3, len(lens)))) for b0 in range(0, len(lens), 3))
    out = run_trace(d, dtype, str(tmp_path / f"out_{dtype}"), most, steps)
    refs = [plain_logits(pcfg, tensors, ids) for ids in requests]
    seen = set()
    by_mode = {}
    for (mode, r, p), (step, row) in index.items():
        got = out[step][row]
        scale_err = float(np.abs(got - refs[r][p]).max() / np.abs(refs[r]).max())
        assert scale_err <= REL[dtype], (mode, r, p, scale_err)
        by_mode.setdefault((r, p), {})[mode] = got
        seen.add(mode)
    assert seen == {"whole", "last32", "batch"}
    # the same position under the three cuttings
    for (r, p), modes in by_mode.items():
        whole = modes["whole"]
        for mode, got in modes.items():
            assert float(np.abs(got - whole).max() / np.abs(refs[r]).max()) <= REL_CUT[dtype], (mode, r, p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_a_truncation(tmp_path, dtype):
    """A request is fed 70 tokens, cut back to 33 by the trace, fed another tail in two pieces beside a second
    request, and decoded: every logit after the cut belongs to the new sequence."""
    cfg = TINY["B"]
    d = make_model_dir(tmp_path, cfg, seed=22)
    pcfg, tensors = load_plain(d)
    V = cfg["vocab_size"]
    first, tail, other = random_ids(70, V, 400), random_ids(41, V, 401), random_ids(12, V, 402)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": first, "want": [69]}, {"id": "b", "tokens": other[:9], "want": [8]}], "end": []},
        {"step": 1, "truncate": {"a": 33}, "entries": [{"id": "a", "tokens": tail[:30], "want": list(range(30))},
                                                        {"id": "b", "tokens": [other[9]], "want": [0]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": tail[30:40], "want": list(range(10))}, {"id": "b", "tokens": [other[10]], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": [tail[40]], "want": [0]}, {"id": "b", "tokens": [other[11]], "want": [0]}], "end": ["a", "b"]},
    ]
    out = run_trace(d, dtype, str(tmp_path / f"out_{dtype}"), 256, steps)
    ref_first = plain_logits(pcfg, tensors, first)
    ref_new = plain_logits(pcfg, tensors, first[:33] + tail)
    ref_other = plain_logits(pcfg, tensors, other)
    scale = np.abs(ref_new).max()
    assert np.abs(out[0][0] - ref_first[69]).max() / scale <= REL[dtype]
    got_new = np.concatenate([out[1][:30], out[2][:10], out[3][:1]])
    assert np.abs(got_new - ref_new[33:]).max() / scale <= REL[dtype]
    got_other = np.stack([out[0][1], out[1][30], out[2][10], out[3][1]])
    assert np.abs(got_other - ref_other[8:]).max() / np.abs(ref_other).max() <= REL[dtype]
