"""Seeded random configurations of the architecture through the engine, against the plain
implementation: sizes the fixed tiny configurations do not have (head sizes from 16 to 256,
groups of 1 to 17 heads, widths that are no multiple of 8, odd vocabularies, windows shorter
and longer than a page), whole, with the last tokens one by one, in an unequal batch whose
requests end one after another, and generated greedily from replayed graphs."""
import numpy as np
import pytest

from helpers import REL, REL_CUT, load_plain, plain_logits, random_ids, rel_err
from tiny import make_model_dir

pytestmark = pytest.mark.gpu


def random_config(seed):
    rng = np.random.default_rng(seed)
    nkv = int(rng.choice([1, 2, 3, 5]))
    scaling = [None, {"rope_type": "linear", "factor": float(rng.choice([2.0, 4.0]))},
               {"rope_type": "llama3", "factor": float(rng.choice([8.0, 32.0])), "low_freq_factor": 1.0,
                "high_freq_factor": 4.0, "original_max_position_embeddings": int(rng.choice([32, 64, 128]))}][int(rng.integers(0, 3))]
    cfg = {"architectures": ["LlamaForCausalLM"],
           "hidden_size": int(rng.choice([64, 72, 136, 200, 264, 66, 68, 100])),
           "num_hidden_layers": int(rng.integers(1, 4)),
           "num_attention_heads": nkv * int(rng.choice([1, 2, 4, 7, 8, 17])),
           "num_key_value_heads": nkv,
           "head_dim": int(rng.choice([16, 48, 64, 80, 128, 160, 256])),
           "intermediate_size": int(rng.choice([96, 172, 328, 130, 77])),
           "vocab_size": int(rng.choice([97, 301, 1003, 2048])),
           "rope_theta": float(rng.choice([10000.0, 500000.0])), "rope_scaling": scaling,
           "rms_norm_eps": float(rng.choice([1e-5, 1e-6, 3e-6])),
           "max_position_embeddings": int(rng.choice([256, 512, 1400])),
           "tie_word_embeddings": bool(rng.integers(0, 2)), "torch_dtype": str(rng.choice(["bfloat16", "float32"]))}
    if rng.integers(0, 2) == 0:
        cfg["sliding_window"] = int(rng.choice([8, 40, 100, 300]))
        cfg["use_sliding_window"] = True
    return cfg


# one configuration by hand: the tcgen05 attention kernel with many tiles of three pages each
NARROW_WINDOW = {"architectures": ["LlamaForCausalLM"], "hidden_size": 72, "num_hidden_layers": 2, "num_attention_heads": 20,
                 "num_key_value_heads": 5, "head_dim": 128, "intermediate_size": 328, "vocab_size": 256, "rope_theta": 10000.0,
                 "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 1400, "tie_word_embeddings": True,
                 "torch_dtype": "bfloat16", "sliding_window": 40, "use_sliding_window": True}


_PLAIN = {}      # case -> what the plain implementation says (computed once for both dtypes)


def plain_side(tmp_path_factory, case):
    if case not in _PLAIN:
        cfg = NARROW_WINDOW if case == "narrow_window" else random_config(case)
        d = make_model_dir(tmp_path_factory.mktemp(f"random_{case}"), cfg, seed=5)
        pcfg, tensors = load_plain(d)
        vocab, maxpos = cfg["vocab_size"], cfg["max_position_embeddings"]
        ids = random_ids(min(1300, maxpos), vocab, 1)
        rng = np.random.default_rng(99)
        lens = [int(x) for x in rng.integers(1, maxpos - 12, size=3)] + [64, 65]
        reqs = [random_ids(l + 6, vocab, 50 + i) for i, l in enumerate(lens)]
        _PLAIN[case] = dict(cfg=cfg, dir=d, ids=ids, ref=plain_logits(pcfg, tensors, ids), lens=lens, reqs=reqs,
                            refs=[plain_logits(pcfg, tensors, r) for r in reqs])
    return _PLAIN[case]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [1, 5, 8, 9, "narrow_window"])
def test_random_configuration(tmp_path_factory, case, dtype):
    from ithaca_b200 import Engine
    side = plain_side(tmp_path_factory, case)
    cfg, d, ids, ref = side["cfg"], side["dir"], side["ids"], side["ref"]
    vocab, maxpos, n = cfg["vocab_size"], cfg["max_position_embeddings"], len(ids)
    eng = Engine(d, dtype=dtype, max_tokens=64 * 120)
    s = eng.alloc_slot()
    whole = eng.step([s], [ids], "all").cpu().numpy()
    eng.free_slot(s)
    assert rel_err(whole, ref) <= REL[dtype]

    s = eng.alloc_slot()
    rows = [eng.step([s], [ids[:n - 32]], "all").cpu().numpy()]
    for t in range(n - 32, n):
        rows.append(eng.step([s], [[ids[t]]], "last").cpu().numpy())
    eng.free_slot(s)
    cut = np.concatenate(rows, 0)
    assert rel_err(cut, ref) <= REL[dtype]
    assert rel_err(cut, whole) <= REL_CUT[dtype]

    lens, reqs, refs = side["lens"], side["reqs"], side["refs"]
    slots = [eng.alloc_slot() for _ in reqs]
    out = eng.step(slots, [r[:l] for r, l in zip(reqs, lens)], "last").cpu().numpy()
    for i in range(len(reqs)):
        assert rel_err(out[i], refs[i][lens[i] - 1]) <= REL[dtype]
    for k in range(6):
        live = list(range(len(reqs)))[k // 2:]                     # the first requests end earlier
        out = eng.step([slots[i] for i in live], [[reqs[i][lens[i] + k]] for i in live], "last").cpu().numpy()
        for j, i in enumerate(live):
            assert rel_err(out[j], refs[i][lens[i] + k]) <= REL[dtype]
    eng.stepper.check_status()
    for sl in slots:
        eng.free_slot(sl)
    eng.cache.table.check_consistent()

    # greedy generation (decode steps replayed from graphs) against the same engine stepped by hand
    prompts = [random_ids(l, vocab, 900 + i) for i, l in enumerate([3, min(70, maxpos - 20), min(129, maxpos - 20)])]
    generated = eng.generate(prompts, max_tokens=10, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    slots = [eng.alloc_slot() for _ in prompts]
    logits = eng.step(slots, prompts, "last")
    by_hand = [[] for _ in prompts]
    for k in range(10):
        nxt = logits.argmax(dim=-1).tolist()
        for i, t in enumerate(nxt):
            by_hand[i].append(int(t))
        if k < 9:
            logits = eng.step(slots, [[t] for t in nxt], "last")
    for sl in slots:
        eng.free_slot(sl)
    assert generated == by_hand
