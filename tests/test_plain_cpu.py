"""The plain implementation checked against itself: definitions, identities, and the
agreement of its pieces (it is the yardstick of every GPU test, so it gets tests too)."""
import math

import pytest
import torch

from plain import llama_plain as P
from tiny import TINY_A, TINY_B, TINY_C


def tensors_for(cfg, seed=0):
    from ithaca_b200.weights import random_tensors
    from ithaca_b200.config import config_from_dict
    from ithaca_b200.engine.model import weight_manifest
    _, c = config_from_dict(cfg)
    return random_tensors(weight_manifest(c.model_spec()), seed, cfg["torch_dtype"])


def test_rmsnorm_and_silu_definitions():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.rmsnorm(x, torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))
    assert abs(float(P.silu(torch.tensor(1.0, dtype=torch.float64))) - 1 / (1 + math.exp(-1))) < 1e-15


def test_rope_is_a_rotation_and_relative():
    inv = P.rope_inv_freq(16, 10000.0, None)
    assert abs(float(inv[0]) - 1) < 1e-7 and abs(float(inv[7]) - 10000 ** (-14 / 16)) < 1e-9
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 16, generator=g, dtype=torch.float64), torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    for pairing in ("half", "interleaved"):
        r = P.rope(q, torch.tensor([5]), inv, pairing)
        assert abs(float(r.norm() - q.norm())) < 1e-12
        d1 = (P.rope(q, torch.tensor([9]), inv, pairing) * P.rope(k, torch.tensor([4]), inv, pairing)).sum()
        d2 = (P.rope(q, torch.tensor([25]), inv, pairing) * P.rope(k, torch.tensor([20]), inv, pairing)).sum()
        assert abs(float(d1 - d2)) < 1e-5
    assert torch.equal(P.rope(q, torch.tensor([0]), inv), q)


def test_llama3_frequency_scaling_regimes():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = P.rope_inv_freq(32, 500000.0, None).double()
    got = P.rope_inv_freq(32, 500000.0, sc).double()
    wavelen = 2 * math.pi / base
    for i in range(16):
        if wavelen[i] < 64 / 4:
            assert got[i] == base[i]
        elif wavelen[i] > 64 / 1:
            assert abs(got[i] - base[i] / 8) < 1e-9
        else:
            assert base[i] / 8 < got[i] < base[i]
    assert (got[:-1] >= got[1:]).all()
    lin = P.rope_inv_freq(32, 500000.0, {"rope_type": "linear", "factor": 2.0}).double()
    assert torch.allclose(lin, base / 2, rtol=1e-6)


def test_the_librarys_frequency_table_is_the_plain_one():
    from ithaca_b200.parts.position import inverse_frequencies
    for cfg in (TINY_A, TINY_B, TINY_C):
        a = inverse_frequencies(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
        b = P.rope_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"]).numpy()
        assert (abs(a - b) <= 1e-7 * abs(b)).all()


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    T, nh, nkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, generator=g, dtype=torch.float64) for n in (nh, nkv, nkv))
    o = P.attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[6:], v2[6:] = 7.0, -3.0
    assert torch.equal(P.attention(q, k2, v2)[:6], o[:6])                 # later keys never reach earlier queries
    s = (q[4, 3] @ k[:5, 1].T) / math.sqrt(hd)
    assert torch.allclose(o[4, 3], torch.softmax(s, 0) @ v[:5, 1])        # head 3 reads kv head 1
    w = P.attention(q, k, v, window=3)
    s = (q[8, 0] @ k[6:9, 0].T) / math.sqrt(hd)
    assert torch.allclose(w[8, 0], torch.softmax(s, 0) @ v[6:9, 0])
    assert torch.equal(w[:3], o[:3])


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C])
def test_a_prefix_of_a_sequence_has_the_same_logits(cfg):
    w = tensors_for(cfg)
    ids = [int(x) for x in torch.randint(0, cfg["vocab_size"], (24,), generator=torch.Generator().manual_seed(2))]
    full = P.logits_whole(ids, cfg, w)
    part = P.logits_whole(ids[:11], cfg, w)
    assert full.shape == (24, cfg["vocab_size"]) and torch.allclose(full[:11], part, atol=1e-12)
    f32 = P.logits_whole(ids, cfg, w, dtype=torch.float32)
    assert (f32.double() - full).abs().max() < 2e-5 * full.abs().max()


def test_tied_head_uses_the_embedding():
    w = tensors_for(TINY_B)
    assert "lm_head.weight" not in w
    lg = P.logits_whole([1, 2, 3], TINY_B, w)
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"]
    assert torch.equal(lg, P.logits_whole([1, 2, 3], {**TINY_B, "tie_word_embeddings": False}, w2))


def test_sampling_rule():
    lg = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0])
    assert P.sample(lg, 0.0, 40, 0.9, 1.0, [], 0.5) == 1                             # first of equal maxima
    assert P.sample(lg, 0.0, 40, 0.9, 2.0, [1], 0.5) == 3                            # 3.0 / 2 loses to the other 3.0
    assert P.sample(lg, 0.0, 40, 0.9, 2.0, [1, 3, 3], 0.5) == 2                      # penalised once per occurrence
    assert P.sample(torch.tensor([-1.0, -3.0]), 0.0, 40, 0.9, 2.0, [0], 0.5) == 0    # negative logits are multiplied: -2 > -3
    assert {P.sample(lg, 1.0, 1, 1.0, 1.0, [], u / 10 + 0.05) for u in range(10)} == {1}      # top_k = 1
    assert {P.sample(lg, 1.0, 0, 1.0, 1.0, [], u / 10 + 0.05) for u in range(10)} == {1}      # top_k <= 0 is clamped to 1
    assert {P.sample(lg, 1.0, 2, 1.0, 1.0, [], u / 10 + 0.05) for u in range(10)} == {1, 3}
    # top_p: probabilities of the two 3.0s are ~0.39 each; 0.5 needs both, 0.3 only the first
    assert {P.sample(lg, 1.0, 5, 0.5, 1.0, [], u / 10 + 0.05) for u in range(10)} == {1, 3}
    assert {P.sample(lg, 1.0, 5, 0.3, 1.0, [], u / 10 + 0.05) for u in range(10)} == {1}
    counts = [0] * 5
    for n in range(2000):
        counts[P.sample(lg, 1.0, 5, 1.0, 1.0, [], P.philox_uniform(3, 0, n))] += 1
    p = torch.softmax(lg.double(), 0)
    assert all(abs(c / 2000 - float(pi)) < 0.04 for c, pi in zip(counts, p))


def test_philox_stream():
    u = [P.philox_uniform(1, 2, c) for c in range(1000)]
    assert all(0 < x < 1 for x in u) and abs(sum(u) / 1000 - 0.5) < 0.03 and len(set(u)) == 1000
    assert P.philox_uniform(1, 2, 3) == P.philox_uniform(1, 2, 3) != P.philox_uniform(1, 3, 3)
    assert P.philox_uniform(1, 2, 3) != P.philox_uniform(2, 2, 3)


def test_generate_stops_and_penalises():
    w = tensors_for(TINY_A)
    out = P.generate([1, 2, 3], TINY_A, w, 6)
    assert len(out) == 6
    assert P.generate([1, 2, 3], TINY_A, w, 6, stop_ids=[out[2]]) == out[:2]
    pen = P.generate([1, 2, 3], TINY_A, w, 6, repetition_penalty=5.0)
    assert pen[0] == out[0] and len(set(pen)) >= len(set(out))
