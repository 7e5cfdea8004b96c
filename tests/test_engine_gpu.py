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


def test_llama_8b_layer_sizes_match_plain():
    """Two layers with the sizes of Llama-3.1-8B (hidden 4096, 32/8 heads of 128, feed-forward 14336,
    llama3 rotary scaling) and a cut vocabulary: every kernel at the sizes the benchmark runs
    (split-K tcgen05 products, deep-unrolled skinny products, head size 128 attention), against the
    plain implementation.  Prompt, then tokens one by one, in a batch of three unequal requests."""
    from ithaca_b200 import Engine
    from ithaca_b200.config import config_from_dict
    from ithaca_b200.engine.model import weight_manifest
    from ithaca_b200.weights import random_tensors
    cfg = {"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 2003, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "rms_norm_eps": 1e-5, "max_position_embeddings": 8192, "tie_word_embeddings": False, "torch_dtype": "bfloat16"}
    tensors = random_tensors(weight_manifest(config_from_dict(cfg)[1].model_spec()), 5, "bfloat16")
    reqs = [random_ids(n, 2003, 60 + n) for n in (40, 21, 70)]
    refs = [plain_logits(cfg, tensors, r) for r in reqs]
    for dtype in ("bfloat16", "float32"):
        eng = Engine.from_random(cfg, 5, dtype=dtype, max_tokens=64 * 64)
        # from_random on the device draws other values than the CPU generator: load the CPU tensors instead
        from ithaca_b200.engine.model import DecoderModel
        eng.model = DecoderModel(eng.model.spec, tensors, eng.runtime)
        eng.stepper.model = eng.model
        slots = [eng.alloc_slot() for _ in reqs]
        cut = [len(r) - 6 for r in reqs]
        lg = eng.step(slots, [r[:c] for r, c in zip(reqs, cut)], "all").cpu().numpy()
        got, off = [], 0
        for c in cut:
            got.append([lg[off:off + c]])
            off += c
        for t in range(6):
            if dtype == "bfloat16":
                lgd, _ = eng._decoder.step(slots, [[r[c + t]] for r, c in zip(reqs, cut)])
            else:
                lgd = eng.step(slots, [[r[c + t]] for r, c in zip(reqs, cut)], "last")
            lgd = lgd.cpu().numpy()
            for i in range(len(reqs)):
                got[i].append(lgd[i:i + 1].copy())
        eng.stepper.check_status()
        for i in range(len(reqs)):
            assert rel_err(np.concatenate(got[i]), refs[i]) <= REL[dtype], (dtype, i)
        # a batch of 40 sequences takes the tcgen05 decode path (more than 16 tokens)
        if dtype == "bfloat16":
            many = [eng.alloc_slot() for _ in range(40)]
            eng.step(many, [reqs[0][:30]] * 40, None)
            lgd, _ = eng._decoder.step(many, [[reqs[0][30]]] * 40)
            lgd = lgd.cpu().numpy()
            assert rel_err(lgd, np.repeat(refs[0][30:31], 40, 0)) <= REL[dtype]
        del eng
        torch.cuda.empty_cache()
