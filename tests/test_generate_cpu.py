"""The generation loop's decisions, driven by a scripted backend (no device)."""
import pytest

from ithaca_b200.engine.generate import GenerationOptions, budget_for, generate_loop, next_batch


class FakeBackend:
    """Slots and a page budget like the cache's; 'samples' the next token from a script:
    the token after (request stream, counter) is script[stream][counter]."""

    def __init__(self, script, n_slots=3, n_pages=100, context_length=1000, page=64):
        self.script, self.context_length = script, context_length
        self.n_slots, self.n_pages, self.page = n_slots, n_pages, page
        self.free, self.lengths = list(range(n_slots - 1, -1, -1)), {}
        self.calls, self.slot_history = [], []

    def free_slots(self):
        return len(self.free)

    def room_for(self, lengths, slots=None):
        mine = set(s for s in (slots or []) if s is not None)
        used = sum(-(-l // self.page) for s, l in self.lengths.items() if s not in mine)
        return used + sum(-(-l // self.page) for l in lengths) <= self.n_pages

    def alloc_slot(self):
        s = self.free.pop()
        assert s not in self.lengths
        self.lengths[s] = 0
        self.slot_history.append(s)
        return s

    def free_slot(self, s):
        assert s in self.lengths, "slot freed twice"
        del self.lengths[s]
        self.free.append(s)

    def step_and_sample(self, slots, tokens, streams, counters, recent):
        assert len(set(slots)) == len(slots) and all(s in self.lengths for s in slots)
        self.calls.append(([len(t) for t in tokens], list(streams), list(counters), [list(r) for r in recent]))
        for s, t in zip(slots, tokens):
            self.lengths[s] += len(t)
        return [self.script[st][c] for st, c in zip(streams, counters)]


def test_budget():
    assert budget_for(10, 128, 4096) == 128 and budget_for(4000, 128, 4096) == 96 and budget_for(4096, 5, 4096) == 0


def test_unequal_prompts_stop_tokens_and_early_ends():
    script = {0: [5, 6, 99, 8], 1: [7, 99], 2: [1, 2, 3, 4, 5, 6]}
    be = FakeBackend(script)
    out, st = generate_loop([[1] * 5, [2] * 9, [3] * 17], GenerationOptions(max_tokens=4), be, stop_token_ids=[99])
    assert out == [[5, 6], [7], [1, 2, 3, 4]]
    # one step with all prompts, then one token each for those still running
    assert [c[0] for c in be.calls] == [[5, 9, 17], [1, 1, 1], [1, 1], [1]]
    assert be.calls[1][1] == [0, 1, 2] and be.calls[2][1] == [0, 2] and be.calls[3][1] == [2]
    assert be.calls[2][2] == [2, 2] and be.calls[3][2] == [3]            # counters: tokens generated so far
    assert be.calls[2][3] == [[5, 6], [1, 2]]                            # the ids the penalty covers
    assert st.prompt_tokens == 31 and st.gen_tokens == 7 and st.batches == 1 and st.steps == 4
    assert be.lengths == {} and sorted(be.free) == [0, 1, 2]
    # the last sampled token of request 2 was not evaluated: 17 prompt + 3 steps, not 4
    assert be.calls[-1][0] == [1]


def test_the_stop_token_can_be_kept():
    be = FakeBackend({0: [4, 99, 1]})
    out, _ = generate_loop([[1, 2]], GenerationOptions(max_tokens=5, include_stop=True), be, stop_token_ids=[99])
    assert out == [[4, 99]]
    be = FakeBackend({0: [4, 99, 1, 2, 3]})           # the caller's own (empty) stop list replaces the model's
    out, _ = generate_loop([[1, 2]], GenerationOptions(max_tokens=5, stop_token_ids=[]), be, stop_token_ids=[99])
    assert out == [[4, 99, 1, 2, 3]]


def test_batches_follow_one_another_and_reuse_slots():
    script = {r: [10 + r] * 8 for r in range(7)}
    be = FakeBackend(script, n_slots=3)
    prompts = [[1] * (3 + r) for r in range(7)]
    out, st = generate_loop(prompts, GenerationOptions(max_tokens=2), be)
    assert out == [[10 + r, 10 + r] for r in range(7)]
    assert st.batches == 3 and len(be.slot_history) == 7 and set(be.slot_history) == {0, 1, 2}
    prefill_calls = [c for c in be.calls if max(c[0]) > 1]
    assert [c[1] for c in prefill_calls] == [[0, 1, 2], [3, 4, 5], [6]]


def test_a_batch_is_cut_to_what_the_cache_holds():
    be = FakeBackend({r: [1] * 200 for r in range(4)}, n_slots=4, n_pages=5)
    prompts = [[1] * 60, [1] * 60, [1] * 60, [1] * 60]
    assert next_batch([0, 1, 2, 3], prompts, [100] * 4, be, None) == [0]          # 160 positions = 3 pages each
    assert next_batch([0, 1, 2, 3], prompts, [4] * 4, be, None) == [0, 1, 2, 3]   # 64 each: 4 pages
    assert next_batch([0, 1, 2, 3], prompts, [4] * 4, be, 2) == [0, 1]
    out, st = generate_loop(prompts, GenerationOptions(max_tokens=100), be)
    assert st.batches == 4 and all(len(o) == 100 for o in out)
    with pytest.raises(RuntimeError, match="does not fit"):
        generate_loop([[1] * 400], GenerationOptions(max_tokens=10), FakeBackend({0: [1] * 10}, n_pages=5))


def test_budget_is_cut_by_the_context_and_callback_can_end_a_request():
    be = FakeBackend({0: list(range(100, 200)), 1: list(range(200, 300))}, context_length=12)
    seen = []

    def on_token(req, tok):
        seen.append((req, tok))
        return not (req == 1 and tok == 201)

    out, _ = generate_loop([[1] * 9, [1] * 4], GenerationOptions(max_tokens=50), be, on_token=on_token)
    assert out == [[100, 101, 102], [200, 201]]
    assert (1, 201) in seen
    with pytest.raises(ValueError, match="empty prompt"):
        generate_loop([[]], GenerationOptions(), be)
    with pytest.raises(ValueError, match="longer than the context"):
        generate_loop([[1] * 13], GenerationOptions(), be)


def test_slots_are_freed_when_a_step_fails():
    class Failing(FakeBackend):
        def step_and_sample(self, *a):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().step_and_sample(*a)

    be = Failing({0: [1, 2, 3], 1: [1, 2, 3]})
    with pytest.raises(RuntimeError, match="boom"):
        generate_loop([[1], [2]], GenerationOptions(max_tokens=3), be)
    assert be.lengths == {} and len(be.free) == 3


def test_a_resumed_request_feeds_only_what_its_slot_lacks_and_keeps_the_slot():
    """Request 1 goes on in a slot that already holds 6 of its 9 prompt tokens: the prompt step brings the other
    3, the request decodes like any other, and at the end its slot is still the caller's while the other is freed."""
    be = FakeBackend({0: [5, 6, 7], 1: [8, 9, 10]})
    held = be.alloc_slot()
    be.lengths[held] = 6
    out, st = generate_loop([[1] * 4, [2] * 9], GenerationOptions(max_tokens=3), be, resume=[None, (held, 6)])
    assert out == [[5, 6, 7], [8, 9, 10]]
    assert be.calls[0][0] == [4, 3] and st.prompt_tokens == 7 and st.reused_tokens == 6
    assert list(be.lengths) == [held] and be.lengths[held] == 6 + 3 + 2     # the last sampled token is not evaluated
    with pytest.raises(ValueError, match="cached positions"):
        generate_loop([[2] * 9], GenerationOptions(max_tokens=3), be, resume=[(held, 9)])
    # a held slot needs no free slot: with none free the resumed request still runs, a fresh one has to wait its turn
    be2 = FakeBackend({0: [1, 1], 1: [2, 2]}, n_slots=1)
    h = be2.alloc_slot()
    assert next_batch([0, 1], [[1] * 3, [1] * 3], [2, 2], be2, None, [(h, 0), None]) == [0]


def test_decode_chunk_choice_is_sane():
    """Pages per decode-attention block: between 1 and the sequence's pages, the headline shape keeps its measured
    optimum, and the number of chunks never exceeds what the scratch is sized for."""
    from ithaca_b200.csrc.attention_bf16 import decode_chunk_pages
    assert decode_chunk_pages(8, 32, 8, 4096, n_sm=148) == 16
    assert decode_chunk_pages(1, 32, 8, 4096, n_sm=148) == 4
    for n_seqs in (1, 2, 3, 7, 8, 16, 24, 33, 64, 200):
        for heads, kv in ((32, 8), (4, 4), (6, 2), (40, 40), (64, 1)):
            for length in (1, 63, 64, 65, 700, 4096, 20000):
                pages = -(-length // 64)
                c = decode_chunk_pages(n_seqs, heads, kv, length, n_sm=148)
                assert 1 <= c <= max(pages, 2), (n_seqs, heads, kv, length, c)


def test_which_product_kernel_takes_which_shape():
    from ithaca_b200.csrc.gemm_bf16 import takes_skinny
    assert takes_skinny(1, 128256, 4096) and takes_skinny(8, 28672, 4096)           # up to 8 tokens: always
    assert takes_skinny(12, 6144, 4096) and takes_skinny(16, 4096, 4096)            # small matrices up to 16 tokens
    assert not takes_skinny(9, 28672, 4096) and not takes_skinny(16, 4096, 14336)   # large ones go to tcgen05
    assert not takes_skinny(17, 64, 64)
