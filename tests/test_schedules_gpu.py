"""Ways of cutting and batching that a caller of the step function may choose, each compared with the plain
implementation position by position, and with the same request run whole on the same engine:

* a mixed step: sequences that go on by one token in the same step as a prompt that starts;
* a prompt fed as several multi-token pieces of unequal size, beside a sequence that goes on by one token;
* a step over the workspace limit, which the engine runs as several passes;
* a sequence cut back to a prefix and fed another tail (across a page boundary, under a window);
* decode batches of 9 to 16 sequences and pieces of 2,048 tokens behind cached ones at the layer sizes of
  Llama-3.1-8B, where the products of one layer go to different kernels.
"""
import numpy as np
import pytest
import torch

from helpers import REL, REL_CUT, load_plain, plain_logits, random_ids, rel_err, run_schedule
from tiny import TINY, make_model_dir

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, cfg in TINY.items():
        d = make_model_dir(root, cfg, seed=31)
        out[name] = (d,) + load_plain(d)
    return out


def whole_logits(eng, ids):
    s = eng.alloc_slot()
    out = eng.step([s], [ids], "all").cpu().numpy()
    eng.free_slot(s)
    return out


def check(eng, cfg, tensors, requests, got, dtype):
    for r, ids in enumerate(requests):
        ref = plain_logits(cfg, tensors, ids)
        assert rel_err(got[r], ref) <= REL[dtype], ("against the plain implementation", r)
        whole = whole_logits(eng, ids)
        err = float(np.abs(got[r] - whole).max() / np.abs(ref).max())
        assert err <= REL_CUT[dtype], ("against the same request whole", r, err)
    eng.cache.table.check_consistent()
    assert eng.cache.table.n_slots_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_step(models, name, dtype):
    """Two sequences are decoding at positions > 0 when a third arrives with its whole prompt in the same step;
    then all three go on by one token; a fourth arrives with a one-token prompt while the others decode."""
    from ithaca_b200 import Engine
    d, cfg, tensors = models[name]
    V = cfg["vocab_size"]
    requests = [random_ids(n, V, 700 + i) for i, n in enumerate((30, 12, 41, 6))]
    schedule = [[(0, 20), (1, 7)], [(0, 1), (1, 1)], [(0, 1), (1, 1), (2, 33)], [(0, 1), (1, 1), (2, 1)],
                [(0, 1), (1, 1), (2, 1), (3, 1)], [(0, 1), (1, 1), (2, 1), (3, 1)], [(3, 4), (0, 5), (2, 5)]]
    eng = Engine(d, dtype=dtype, max_tokens=64 * 8)
    check(eng, cfg, tensors, requests, run_schedule(eng, requests, schedule), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompt_in_pieces_beside_a_decoding_sequence(models, name, dtype):
    """A prompt of 33 + 1 + 36 + 64 + 65 tokens arrives piece by piece (the pieces end before, on and after page
    boundaries, and under Tiny C's window of 40 a piece is longer than the window) while another sequence
    goes on by one token in the same steps."""
    from ithaca_b200 import Engine
    d, cfg, tensors = models[name]
    V, maxpos = cfg["vocab_size"], cfg["max_position_embeddings"]
    pieces = [33, 1, 36, 64, 65] if maxpos >= 256 else [33, 1, 36, 50]
    requests = [random_ids(sum(pieces), V, 810), random_ids(9 + len(pieces), V, 811)]
    schedule = [[(1, 9)]] + [[(0, p), (1, 1)] for p in pieces]
    eng = Engine(d, dtype=dtype, max_tokens=64 * 8)
    check(eng, cfg, tensors, requests, run_schedule(eng, requests, schedule), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_step_over_the_workspace_limit_runs_in_passes(models, name, dtype):
    """With a limit of 24 tokens a step of 17 + 60 + 3 + 29 tokens runs as five passes that cut sequences in the
    middle; rows come back in the caller's order although one request asks for its places out of order."""
    from ithaca_b200 import Engine
    d, cfg, tensors = models[name]
    V = cfg["vocab_size"]
    lens = (17, 60, 3, 29)
    requests = [random_ids(n, V, 900 + i) for i, n in enumerate(lens)]
    eng = Engine(d, dtype=dtype, max_tokens=64 * 8, max_step_tokens=24)
    slots = [eng.alloc_slot() for _ in requests]
    want = [list(range(n)) for n in lens]
    want[1] = want[1][::-1]                                # 59, 58, ..., 0: crosses the passes backwards
    lg = eng.step(slots, requests, want).cpu().numpy()
    assert eng.stepper.passes_last_step == 5
    nxt = eng.step(slots, [[5], [6], [7], [8]], "last").cpu().numpy()     # and the cache is whole afterwards
    eng.check_status()
    for s in slots:
        eng.free_slot(s)
    off = 0
    unlimited = Engine(d, dtype=dtype, max_tokens=64 * 8, max_step_tokens=None)
    for r, ids in enumerate(requests):
        rows = lg[off:off + lens[r]]
        off += lens[r]
        if r == 1:
            rows = rows[::-1]
        ref = plain_logits(cfg, tensors, ids + [5 + r])
        assert rel_err(np.concatenate([rows, nxt[r:r + 1]]), ref) <= REL[dtype], r
        whole = whole_logits(unlimited, ids)
        assert float(np.abs(rows - whole).max() / np.abs(ref).max()) <= REL_CUT[dtype], r
    # nothing has changed when the step is refused: a bad id in the last sequence, found before the first pass
    slots = [eng.alloc_slot() for _ in range(2)]
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.step(slots, [list(range(30)), [1, 2, V]], "last")
    assert eng.length(slots[0]) == 0 and eng.length(slots[1]) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_truncate_then_feed_another_tail(models, name, dtype):
    """100 tokens, cut back to 37, another tail; then cut back to 63, 64 and 65 (before, on and after a page
    boundary) with other tails each time, beside a sequence that decodes; at last back to 0 and a new prompt in
    the same slot.  Every position of every version is compared with the plain implementation of that version."""
    from ithaca_b200 import Engine
    d, cfg, tensors = models[name]
    V = cfg["vocab_size"]
    eng = Engine(d, dtype=dtype, max_tokens=64 * 8)
    base = random_ids(100, V, 1000)
    other = random_ids(40, V, 1001)
    s, o = eng.alloc_slot(), eng.alloc_slot()
    eng.step([s, o], [base, other[:30]], None)
    held = list(base)
    fed_other = 30
    for n, (keep, tail_len) in enumerate([(37, 50), (63, 20), (64, 3), (65, 40), (0, 70)]):
        eng.truncate(s, keep)
        assert eng.length(s) == keep
        tail = random_ids(tail_len, V, 1010 + n)
        held = held[:keep] + tail
        lg = eng.step([s, o], [tail, [other[fed_other]]], "all").cpu().numpy()
        fed_other += 1
        ref = plain_logits(cfg, tensors, held)
        assert rel_err(lg[:tail_len], ref[keep:]) <= REL[dtype], (keep, tail_len)
        # one more token decodes behind the new tail
        lg1 = eng.step([s], [[3]], "last").cpu().numpy()
        held = held + [3]
        assert rel_err(lg1, plain_logits(cfg, tensors, held)[-1:]) <= REL[dtype], (keep, "decode")
    # the sequence beside it never noticed
    lg = eng.step([o], [other[fed_other:]], "all").cpu().numpy()
    assert rel_err(lg, plain_logits(cfg, tensors, other)[fed_other:]) <= REL[dtype]
    with pytest.raises(Exception, match="cannot truncate"):
        eng.truncate(s, eng.length(s) + 1)
    eng.check_status()
    eng.free_slot(s)
    eng.free_slot(o)
    eng.cache.table.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_truncate_under_a_window(models, dtype):
    """Tiny C keeps a window of 40 keys and gives pages back as a sequence grows.  Cutting back is possible while
    the pages the new end looks back to are still held, is refused (with nothing changed) when they are gone, and
    going back to 0 starts the slot again."""
    from ithaca_b200 import Engine
    from ithaca_b200.cache import CacheError
    d, cfg, tensors = models["C"]
    V = cfg["vocab_size"]
    eng = Engine(d, dtype=dtype, max_tokens=64 * 8)
    ids = random_ids(200, V, 1100)
    s = eng.alloc_slot()
    eng.step([s], [ids], None)                     # position 200 looks back to 161: pages 0 and 1 are gone
    with pytest.raises(CacheError, match="released"):
        eng.truncate(s, 150)                       # position 150 would look back to 111, in page 1
    assert eng.length(s) == 200
    eng.truncate(s, 170)                           # looks back to 131: page 2, still held
    tail = random_ids(30, V, 1101)
    lg = eng.step([s], [tail], "all").cpu().numpy()
    ref = plain_logits(cfg, tensors, ids[:170] + tail)
    assert rel_err(lg, ref[170:]) <= REL[dtype]
    eng.truncate(s, 0)
    again = random_ids(90, V, 1102)
    lg = eng.step([s], [again], "all").cpu().numpy()
    assert rel_err(lg, plain_logits(cfg, tensors, again)) <= REL[dtype]
    eng.check_status()
    eng.free_slot(s)
    eng.cache.table.check_consistent()
    assert all(p.n_free == p.n_pages for p in eng.cache.table.pools)


def test_truncate_drops_a_step_launched_ahead(models):
    """Greedy generation launches the next decode step before the host has seen the current one.  A truncation
    right after a generation must not be undone by that step's bookkeeping."""
    from ithaca_b200 import Engine
    d, cfg, tensors = models["B"]
    eng = Engine(d, dtype="bfloat16", max_tokens=64 * 8)
    prompt = random_ids(20, cfg["vocab_size"], 1200)
    s = eng.alloc_slot()
    eng.step([s], [prompt], None)
    tok = 5
    for _ in range(4):                             # decode steps through the graph path, with one launched ahead
        tok = eng._decoder.greedy_step([s], [[tok]])[0]
    eng.truncate(s, 10)
    assert eng.length(s) == 10
    lg = eng.step([s], [prompt[10:15]], "all").cpu().numpy()
    assert rel_err(lg, plain_logits(cfg, tensors, prompt[:15])[10:]) <= REL["bfloat16"]
    eng.free_slot(s)


# --------------------------------------------------------------------------------------------------------------
# the layer sizes of Llama-3.1-8B
# --------------------------------------------------------------------------------------------------------------
CFG_8B_LAYERS = {"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2, "num_attention_heads": 32,
                 "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 2003,
                 "rope_theta": 500000.0,
                 "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                  "original_max_position_embeddings": 8192},
                 "rms_norm_eps": 1e-5, "max_position_embeddings": 8192, "tie_word_embeddings": False, "torch_dtype": "bfloat16"}


@pytest.fixture(scope="module")
def big():
    """The plain side's weights: made on the host by the same generator that makes them on the device."""
    from ithaca_b200.config import config_from_dict
    from ithaca_b200.engine.model import weight_manifest
    from ithaca_b200.weights import random_tensors
    return random_tensors(weight_manifest(config_from_dict(CFG_8B_LAYERS)[1].model_spec()), 5, "bfloat16")


def test_device_made_weights_are_the_host_made_ones(big):
    from ithaca_b200 import Engine
    eng = Engine.from_random(CFG_8B_LAYERS, 5, dtype="bfloat16", max_tokens=64)
    for name in ("model.embed_tokens.weight", "lm_head.weight", "model.layers.1.mlp.down_proj.weight", "model.norm.weight"):
        assert torch.equal(eng.dump_tensor(name), big[name]), name
    assert torch.equal(eng.model.embedding.table.cpu(), big["model.embed_tokens.weight"])
    assert torch.equal(eng.model.head.linear.weight.cpu(), big["lm_head.weight"])
    assert torch.equal(eng.model.layers[1].feed_forward.down.weight.cpu(), big["model.layers.1.mlp.down_proj.weight"])
    assert torch.equal(eng.model.final_norm.weight.cpu(), big["model.norm.weight"].float())
    with pytest.raises(KeyError):
        eng.dump_tensor("no.such.tensor")
    del eng
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_decode_batches_of_9_12_16_at_8b_layer_sizes(big, dtype):
    """With 9 to 16 tokens the small matrices of a layer (q/k/v, output) go to the warp-level kernel with two column
    tiles and the large ones (gate/up, down) to tcgen05; with 17 all go to tcgen05.  Unequal prompts, then five
    tokens one by one, the bfloat16 path through the replayed graphs that generation uses."""
    from ithaca_b200 import Engine
    eng = Engine.from_random(CFG_8B_LAYERS, 5, dtype=dtype, max_tokens=64 * 40)
    for batch in (9, 12, 16, 17):
        lens = [3 + (7 * i) % 23 for i in range(batch)]
        reqs = [random_ids(n + 5, 2003, 2000 + 31 * batch + i) for i, n in enumerate(lens)]
        slots = [eng.alloc_slot() for _ in reqs]
        eng.step(slots, [r[:n] for r, n in zip(reqs, lens)], None)
        rows = []
        for t in range(5):
            toks = [[r[n + t]] for r, n in zip(reqs, lens)]
            if dtype == "bfloat16":
                lg, _ = eng._decoder.step(slots, toks)
            else:
                lg = eng.step(slots, toks, "last")
            rows.append(lg.float().cpu().numpy().copy())
        eng.check_status()
        for s in slots:
            eng.free_slot(s)
        for i in range(0, batch, 4):                       # every fourth request against the plain implementation
            ref = plain_logits(CFG_8B_LAYERS, big, reqs[i])[lens[i]:]
            got = np.stack([rows[t][i] for t in range(5)])
            assert rel_err(got, ref) <= REL[dtype], (batch, i)
    del eng
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_pieces_of_2048_tokens_behind_cached_ones_at_8b_layer_sizes(big, dtype):
    """A sequence is filled as the benchmark fills its caches: pieces of 2,048 tokens, each behind what is cached
    (here 100, then 2,048 behind them, then 150; the float32 path a quarter of that), beside a second sequence that goes on by one
    token per step; then both decode.  The last rows of every piece and the decoded rows are compared."""
    from ithaca_b200 import Engine
    piece = 2048 if dtype == "bfloat16" else 512
    eng = Engine.from_random(CFG_8B_LAYERS, 5, dtype=dtype, max_tokens=64 * 80, max_step_tokens=None)
    long_ids = random_ids(100 + piece + 150 + 3, 2003, 3000)
    side = random_ids(20 + 3 + 3, 2003, 3001)
    s, o = eng.alloc_slot(), eng.alloc_slot()
    eng.step([o], [side[:20]], None)
    got_long, got_side, fed, fed_side = {}, {}, 0, 20
    for n in (100, piece, 150):
        want = [list(range(n - 4, n)), [0]]
        lg = eng.step([s, o], [long_ids[fed:fed + n], [side[fed_side]]], want).cpu().numpy()
        for j in range(4):
            got_long[fed + n - 4 + j] = lg[j]
        got_side[fed_side] = lg[4]
        fed += n
        fed_side += 1
    for t in range(3):
        if dtype == "bfloat16":
            lg, _ = eng._decoder.step([s, o], [[long_ids[fed]], [side[fed_side]]])
        else:
            lg = eng.step([s, o], [[long_ids[fed]], [side[fed_side]]], "last")
        lg = lg.float().cpu().numpy()
        got_long[fed], got_side[fed_side] = lg[0].copy(), lg[1].copy()
        fed += 1
        fed_side += 1
    eng.check_status()
    ref_long = plain_logits(CFG_8B_LAYERS, big, long_ids)
    ref_side = plain_logits(CFG_8B_LAYERS, big, side)
    pos = sorted(got_long)
    assert rel_err(np.stack([got_long[p] for p in pos]), ref_long[pos]) <= REL[dtype]
    pos = sorted(got_side)
    assert rel_err(np.stack([got_side[p] for p in pos]), ref_side[pos]) <= REL[dtype]
    if dtype == "float32":                                  # and bit for bit what the whole sequence gives in one step
        eng.free_slot(s)
        s = eng.alloc_slot()
        pos = sorted(got_long)
        whole = eng.step([s], [long_ids], [pos]).cpu().numpy()
        assert np.array_equal(whole, np.stack([got_long[p] for p in pos]))
    del eng
    torch.cuda.empty_cache()
