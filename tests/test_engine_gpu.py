"""The engine against the plain implementation: whole requests, the last tokens one by
one, unequal batches one after another (slots used again), in float32 and bfloat16."""
import numpy as np
import pytest
import torch

from helpers import REL, REL_CUT, load_plain, plain_logits, random_ids, rel_err
from tiny import TINY, make_model_dir

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, cfg in TINY.items():
        d = make_model_dir(root, cfg, seed=11)
        out[name] = (d,) + load_plain(d)
    return out


def engine_for(model_dir, dtype, max_tokens=4096):
    from ithaca_b200 import Engine
    return Engine(model_dir, dtype=dtype, max_tokens=max_tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_request_matches_plain(models, name, dtype):
    d, cfg, tensors = models[name]
    eng = engine_for(d, dtype)
    for n, seed in [(1, 0), (17, 1), (100, 2)]:
        n = min(n, cfg["max_position_embeddings"])
        ids = random_ids(n, cfg["vocab_size"], seed)
        s = eng.alloc_slot()
        got = eng.step([s], [ids], "all").cpu().numpy()
        eng.stepper.check_status()
        eng.free_slot(s)
        assert rel_err(got, plain_logits(cfg, tensors, ids)) <= REL[dtype]
    eng.cache.table.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(models, name, dtype):
    d, cfg, tensors = models[name]
    eng = engine_for(d, dtype)
    n = min(120, cfg["max_position_embeddings"])
    ids = random_ids(n, cfg["vocab_size"], 5)
    ref = plain_logits(cfg, tensors, ids)
    s = eng.alloc_slot()
    rows = [eng.step([s], [ids[:n - 32]], "all").cpu().numpy()]
    for t in range(n - 32, n):
        rows.append(eng.step([s], [[ids[t]]], "last").cpu().numpy())
    eng.stepper.check_status()
    got = np.concatenate(rows, 0)
    assert rel_err(got, ref) <= REL[dtype]
    # the same request whole, on the same engine, in a slot used again
    eng.free_slot(s)
    s2 = eng.alloc_slot()
    whole = eng.step([s2], [ids], "all").cpu().numpy()
    assert rel_err(got, whole) <= REL_CUT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_with_slot_reuse(models, name, dtype):
    """Batches of unequal prompts, then 8 tokens each one by one; shorter requests end
    earlier; three batches one after another through a cache that only fits one."""
    d, cfg, tensors = models[name]
    maxpos = cfg["max_position_embeddings"]
    lens_per_batch = [[5, 9, 17], [1, 7, 33, 64, 100], [64, 2, 65]]
    eng = engine_for(d, dtype, max_tokens=64 * 8)
    seed = 100
    for lens in lens_per_batch:
        lens = [min(l, maxpos - 8) for l in lens]
        extra = [3 + 2 * (i % 3) for i in range(len(lens))]              # decode steps before each request ends
        reqs = [random_ids(l + e, cfg["vocab_size"], seed + i) for i, (l, e) in enumerate(zip(lens, extra))]
        seed += 10
        refs = [plain_logits(cfg, tensors, r) for r in reqs]
        slots = [eng.alloc_slot() for _ in reqs]
        got = [[] for _ in reqs]
        lg = eng.step(slots, [r[:l] for r, l in zip(reqs, lens)], "all").cpu().numpy()
        off = 0
        for i, l in enumerate(lens):
            got[i].append(lg[off:off + l])
            off += l
        live = list(range(len(reqs)))
        pos = list(lens)
        while live:
            lg = eng.step([slots[i] for i in live], [[reqs[i][pos[i]]] for i in live], "last").cpu().numpy()
            nxt = []
            for row, i in enumerate(live):
                got[i].append(lg[row:row + 1])
                pos[i] += 1
                if pos[i] < len(reqs[i]):
                    nxt.append(i)
                else:
                    eng.free_slot(slots[i])
            live = nxt
        eng.stepper.check_status()
        eng.cache.table.check_consistent()
        for i in range(len(reqs)):
            assert rel_err(np.concatenate(got[i], 0), refs[i]) <= REL[dtype], (lens, i)
    assert eng.cache.table.n_slots_in_use() == 0
    assert all(p.n_free == p.n_pages for p in eng.cache.table.pools)
