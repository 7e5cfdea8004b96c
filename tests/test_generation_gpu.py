"""Generation through the Python entry point against the plain implementation: greedy,
sampled with a fixed seed, stop tokens, more requests than slots, long decoding, the first
tokens of a sequence."""
import numpy as np
import pytest
import torch

from helpers import REL, load_plain, plain_logits, random_ids, rel_err
from plain import llama_plain as P
from tiny import TINY, make_model_dir

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen_models")
    return {n: (make_model_dir(root, c, seed=31),) for n, c in TINY.items()}


@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_matches_plain_float32(models, graphs):
    from ithaca_b200 import Engine
    (d,) = models["A"]
    cfg, tensors = load_plain(d)
    eng = Engine(d, dtype="float32", max_tokens=1024, graphs=graphs)
    prompts = [random_ids(n, 256, 40 + n) for n in (5, 9, 17)]
    got = eng.generate(prompts, max_tokens=16, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    want = [P.generate(p, cfg, tensors, 16, repetition_penalty=1.0) for p in prompts]
    assert got == want
    # with the reference's default penalty, and a stop token taken from the plain run
    want_pen = [P.generate(p, cfg, tensors, 16, repetition_penalty=1.1) for p in prompts]
    stop = want_pen[1][5]
    got = eng.generate(prompts, max_tokens=16, stop_token_ids=[stop])
    want = [P.generate(p, cfg, tensors, 16, repetition_penalty=1.1, stop_ids=[stop]) for p in prompts]
    assert got == want and len(got[1]) <= 5
    st = eng.last_stats
    assert st.prompt_tokens == 31 and st.gen_tokens == sum(len(g) for g in got)
    assert eng.cache.table.n_slots_in_use() == 0


def test_sampled_generation_with_a_seed_matches_plain_float32(models):
    """Tiny B: five prompts of lengths 1/7/33/64/100, 24 steps at temperature 0.8, fixed seed;
    three slots only, so the requests run as two batches and slots are used again."""
    from ithaca_b200 import Engine
    (d,) = models["B"]
    cfg, tensors = load_plain(d)
    eng = Engine(d, dtype="float32", max_tokens=64 * 8, max_slots=3)
    prompts = [random_ids(n, 384, 50 + n) for n in (1, 7, 33, 64, 100)]
    opts = dict(max_tokens=24, temp=0.8, top_k=40, top_p=0.9, rep_pen=1.1, seed=1234, stop_token_ids=[])
    got = eng.generate(prompts, **opts)
    want = [P.generate(p, cfg, tensors, 24, temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1, seed=1234,
                       stream=i) for i, p in enumerate(prompts)]
    assert got == want
    assert eng.last_stats.batches == 2
    # a request's tokens do not depend on its batch: alone it gives the same (its stream is its index)
    alone = eng.generate([prompts[0]] * 1, **opts)
    assert alone[0] == got[0]


@pytest.mark.parametrize("name", ["B", "C"])
def test_bfloat16_generation_follows_plain_where_the_choice_is_clear(models, name):
    """bfloat16 logits differ from the plain ones by rounding, so a greedy pick may differ where the
    two largest logits are closer than that.  Teacher-forced on the plain tokens, every position whose
    margin is above the bfloat16 tolerance must be picked alike."""
    from ithaca_b200 import Engine
    (d,) = models[name]
    cfg, tensors = load_plain(d)
    eng = Engine(d, dtype="bfloat16", max_tokens=2048)
    prompt = random_ids(12, cfg["vocab_size"], 77)
    plain = P.generate(prompt, cfg, tensors, 20, repetition_penalty=1.0)
    ids = prompt + plain
    ref = plain_logits(cfg, tensors, ids)
    s = eng.alloc_slot()
    rows = [eng.step([s], [prompt], "last").cpu().numpy()]
    for t in plain[:-1]:
        rows.append(eng.step([s], [[t]], "last").cpu().numpy())
    eng.free_slot(s)
    got = np.concatenate(rows)
    clear = 0
    for i in range(len(plain)):
        r = ref[len(prompt) - 1 + i]
        top2 = np.sort(r)[-2:]
        if top2[1] - top2[0] > 2 * REL["bfloat16"] * np.abs(ref).max():
            clear += 1
            assert int(got[i].argmax()) == plain[i]
    assert clear >= 5, f"only {clear} of {len(plain)} positions have a clear margin: the check says too little"
    out = eng.generate([prompt], max_tokens=20, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    assert len(out[0]) == 20


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_plain_logits(models, dtype):
    """300 tokens decoded one by one after a short prompt (crossing several pages and, for the
    graphs, several block-table widths), compared position by position."""
    from ithaca_b200 import Engine
    (d,) = models["C"]
    cfg, tensors = load_plain(d)
    ids = random_ids(330, cfg["vocab_size"], 88)
    ref = plain_logits(cfg, tensors, ids)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    s = eng.alloc_slot()
    rows = [eng.step([s], [ids[:30]], "all").cpu().numpy()]
    for t in ids[30:]:
        lg, _ = eng._decoder.step([s], [[t]])                      # the graph-replayed decode step
        rows.append(lg.cpu().numpy().copy())
    eng.stepper.check_status()
    assert rel_err(np.concatenate(rows), ref) <= REL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_the_first_tokens_of_a_sequence(models, name, dtype):
    """Positions 0, 1, 2 fed one at a time from an empty slot (a prompt of one token, then decode
    steps at the very start of the first page)."""
    from ithaca_b200 import Engine
    (d,) = models[name]
    cfg, tensors = load_plain(d)
    ids = random_ids(4, cfg["vocab_size"], 3)
    ref = plain_logits(cfg, tensors, ids)
    eng = Engine(d, dtype=dtype, max_tokens=256)
    s = eng.alloc_slot()
    rows = [eng.step([s], [[t]], "last").cpu().numpy() for t in ids]
    assert rel_err(np.concatenate(rows), ref) <= REL[dtype]


def test_step_refuses_what_it_cannot_run(models):
    from ithaca_b200 import Engine
    from ithaca_b200.cache import CacheFull
    from ithaca_b200.engine import StepError
    (d,) = models["A"]
    eng = Engine(d, dtype="float32", max_tokens=192)
    s = eng.alloc_slot()
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([s], [[1, 256]])
    with pytest.raises(StepError, match="not in use"):
        eng.step([s + 1], [[1]])
    with pytest.raises(StepError, match="twice"):
        eng.step([s, s], [[1], [2]])
    with pytest.raises(StepError, match="exceed"):
        eng.step([s], [[1] * 129])
    eng.step([s], [[1] * 100])
    t = eng.alloc_slot()
    with pytest.raises(CacheFull):
        eng.step([t], [[1] * 65])                                   # 2 pages held + 2 needed > 3 in all
    assert eng.cache.length(t) == 0 and eng.cache.length(s) == 100
    eng.step([t], [[1] * 3])                                        # the refusal lost nothing: one page is still there
    eng.cache.table.check_consistent()


def test_command_line(models, tmp_path):
    import os
    import subprocess
    import sys
    from helpers import ROOT
    (d,) = models["A"]
    cfg, tensors = load_plain(d)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ithaca"), "-m", d, "-p", "1,2,3", "-p", "9 8 7 6", "-n", "5",
                        "--dtype", "float32", "--stop-ids", ""], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    got = [[int(x) for x in line.split(",")] for line in p.stdout.strip().splitlines()]
    want = [P.generate(pr, cfg, tensors, 5, repetition_penalty=1.1) for pr in ([1, 2, 3], [9, 8, 7, 6])]
    assert got == want
    assert "[prompt 7 tok @" in p.stderr and "gen 10 tok @" in p.stderr


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("B", "bfloat16")])
def test_a_session_reuses_the_prefix_its_next_prompt_shares(models, name, dtype):
    """Three turns in one slot, beside another request that the engine serves in between.  Turn 2's prompt is turn
    1's prompt, its reply and new tokens: everything up to the reply's last evaluated token is found in the cache.
    Turn 3 changes a token in the middle: the cache is cut back to there.  In float32 every turn's ids equal the
    plain implementation's for the whole prompt; Tiny C (a window) falls back to starting over when the pages it
    would need are gone, with the same ids."""
    from ithaca_b200 import Engine
    (d,) = models[name]
    cfg, tensors = load_plain(d)
    V = cfg["vocab_size"]
    eng = Engine(d, dtype=dtype, max_tokens=64 * 12)
    opts = dict(max_tokens=8, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    with eng.session() as chat:
        p1 = random_ids(40, V, 501)
        r1 = chat.generate(p1, **opts)
        assert chat.reused_last == 0 and len(chat.tokens) == 40 + 7          # the eighth token was sampled, not evaluated
        other = eng.generate([random_ids(9, V, 502)], **opts)                # the engine serves someone else meanwhile
        p2 = p1 + r1 + random_ids(30, V, 503)
        r2 = chat.generate(p2, **opts)
        reused2 = chat.reused_last
        p3 = list(p2)
        p3[55] = (p3[55] + 1) % V
        p3 = p3 + r2[:3]
        r3 = chat.generate(p3, **opts)
        reused3 = chat.reused_last
        assert eng.last_stats.reused_tokens == reused3 and eng.last_stats.prompt_tokens == len(p3) - reused3
        if cfg.get("use_sliding_window"):
            assert reused2 in (0, 47) and reused3 in (0, 55)
        else:
            assert reused2 == 47 and reused3 == 55
        if dtype == "float32":
            for p, r in ((p1, r1), (p2, r2), (p3, r3)):
                assert r == P.generate(p, cfg, tensors, 8, repetition_penalty=1.0)
            assert other[0] == P.generate(random_ids(9, V, 502), cfg, tensors, 8, repetition_penalty=1.0)
        else:
            # bfloat16: the logits behind the reused prefix stay within the 16-bit tolerance of the plain ones
            s = chat.slot
            eng.truncate(s, len(p3) - 1)
            lg = eng.step([s], [[p3[-1]]], "last").cpu().numpy()
            assert rel_err(lg, plain_logits(cfg, tensors, p3)[-1:]) <= REL[dtype]
    eng.check_status()
    assert eng.cache.table.n_slots_in_use() == 0
    eng.cache.table.check_consistent()
