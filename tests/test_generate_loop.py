"""Decisions of the generation loop, with a scripted engine instead of a model (no GPU)."""
import pytest

from rocmforge_b200.engine.generate import (CONTEXT_FULL, MAX_TOKENS, STOP_TOKEN, StepEngine, generate)
from rocmforge_b200.sampling import SamplingParams, draw_seed, DEFAULT_SEED


class ScriptedEngine(StepEngine):
    """Next token of a sequence = f(its tokens so far); records every call."""

    def __init__(self, next_token, max_seq_len=1000, max_batch=3, n_slots=3):
        self.next_token = next_token
        self.max_seq_len = max_seq_len
        self.max_batch = max_batch
        self.free = list(range(n_slots))
        self.held = {}                # slot -> tokens so far
        self.calls = []               # (slots, token lists, requests, draws)
        self.freed = []

    def admit(self, prompt_lens, max_new_tokens):
        return min(len(prompt_lens), self.max_batch, len(self.free))

    def alloc_slot(self):
        s = self.free.pop(0)
        self.held[s] = []
        return s

    def free_slot(self, slot):
        assert slot in self.held, "slot freed twice or never held"
        del self.held[slot]
        self.free.append(slot)
        self.free.sort()
        self.freed.append(slot)

    def run(self, slots, tokens, requests, draws, sampling):
        assert len(set(slots)) == len(slots)
        kinds = {len(t) == 1 for t in tokens}
        starts = {len(self.held[s]) == 0 for s in slots}
        assert starts == {True} or (starts == {False} and kinds == {True}), \
            "a step is either all prompts or one token each"
        self.calls.append((list(slots), [list(t) for t in tokens], list(requests), list(draws)))
        out = []
        for s, t in zip(slots, tokens):
            self.held[s] += list(t)
            assert len(self.held[s]) <= self.max_seq_len
            out.append(self.next_token(self.held[s]))
        return out


def count_up(tokens):
    return tokens[-1] + 1


def test_unequal_prompts_stop_tokens_and_early_ends():
    eng = ScriptedEngine(count_up)
    prompts = [[10], [20, 21, 22], [30, 31]]
    res = generate(eng, prompts, max_new_tokens=6, stop_token_ids=[13, 36])
    assert [r.tokens for r in res] == [[11, 12], [23, 24, 25, 26, 27, 28], [32, 33, 34, 35]]
    assert [r.reason for r in res] == [STOP_TOKEN, MAX_TOKENS, STOP_TOKEN]
    assert [r.prompt_len for r in res] == [1, 3, 2]
    # first call: all prompts in one step; then the batch only shrinks
    assert eng.calls[0][1] == prompts
    sizes = [len(c[0]) for c in eng.calls]
    assert sizes == sorted(sizes, reverse=True) and sizes[0] == 3 and sizes[-1] == 1
    # the request with max_tokens never runs its last token through the model
    assert sum(1 for c in eng.calls for r in c[2] if r == 1) == 6
    assert eng.held == {} and sorted(eng.freed) == [0, 1, 2]


def test_a_slot_is_given_back_when_its_sequence_ends():
    eng = ScriptedEngine(count_up)
    generate(eng, [[10], [20]], max_new_tokens=50, stop_token_ids=[12, 25])
    # request 0 ends after 1 token: its slot must be free while request 1 still decodes
    first_free_at = next(i for i, c in enumerate(eng.calls) if len(c[0]) == 1)
    assert first_free_at == 2 and eng.freed[0] == 0


def test_batches_follow_one_another_and_reuse_slots():
    eng = ScriptedEngine(count_up, max_batch=2, n_slots=2)
    prompts = [[i * 10] for i in range(5)]
    res = generate(eng, prompts, max_new_tokens=3)
    assert [r.tokens for r in res] == [[i * 10 + 1, i * 10 + 2, i * 10 + 3] for i in range(5)]
    prefill_calls = [c for c in eng.calls if c[1][0][0] % 10 == 0 and len(c[1][0]) == 1 and c[3][0] == 0]
    assert [c[2] for c in prefill_calls] == [[0, 1], [2, 3], [4]]
    assert all(set(c[0]) <= {0, 1} for c in eng.calls)
    assert eng.held == {}


def test_stop_token_first_and_zero_budget():
    eng = ScriptedEngine(lambda t: 99)
    res = generate(eng, [[1, 2]], max_new_tokens=5, stop_token_ids=[99])
    assert res[0].tokens == [] and res[0].reason == STOP_TOKEN and len(eng.calls) == 1
    eng = ScriptedEngine(count_up)
    res = generate(eng, [[1, 2]], max_new_tokens=0)
    assert res[0].tokens == [] and res[0].reason == MAX_TOKENS and eng.calls == []


def test_context_full():
    eng = ScriptedEngine(count_up, max_seq_len=5)
    res = generate(eng, [[1, 2, 3]], max_new_tokens=10)
    # positions 3 and 4 can still be filled; the third token would need position 5
    assert res[0].tokens == [4, 5] and res[0].reason == CONTEXT_FULL
    assert eng.held == {}


def test_rejects_bad_prompts():
    eng = ScriptedEngine(count_up, max_seq_len=4)
    with pytest.raises(ValueError):
        generate(eng, [[]], max_new_tokens=1)
    with pytest.raises(ValueError):
        generate(eng, [[1, 2, 3, 4, 5]], max_new_tokens=1)
    assert eng.held == {}


def test_slots_are_freed_when_a_step_fails():
    def boom(tokens):
        if len(tokens) > 3:
            raise RuntimeError("device fault")
        return tokens[-1] + 1
    eng = ScriptedEngine(boom)
    with pytest.raises(RuntimeError):
        generate(eng, [[1], [2]], max_new_tokens=10)
    assert eng.held == {}


def test_draws_count_per_request():
    eng = ScriptedEngine(count_up)
    generate(eng, [[10], [20, 21]], max_new_tokens=3, sampling=SamplingParams(temperature=0.7))
    for slots, toks, reqs, draws in eng.calls:
        pass
    assert eng.calls[0][3] == [0, 0] and eng.calls[1][3] == [1, 1] and eng.calls[2][3] == [2, 2]
    assert draw_seed(DEFAULT_SEED, 0, 0) == 0xDEADBEEF + 1          # the reference's first seed
    assert draw_seed(DEFAULT_SEED, 1, 0) != draw_seed(DEFAULT_SEED, 0, 1)


def test_sampling_params_are_checked():
    for bad in (dict(temperature=-1.0), dict(top_p=1.5), dict(top_k=-2)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams().greedy and not SamplingParams(temperature=0.5).greedy
