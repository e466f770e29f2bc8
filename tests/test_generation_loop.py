"""The generation loop's decisions, with a fake engine that computes nothing (no GPU)."""
import pytest

from mdma_b200.engine.generate import (ContextLimitError, FINISH_CONTEXT, FINISH_LENGTH, FINISH_NONFINITE,
                                       FINISH_STOP, Generator, token_budget)
from mdma_b200.sampling import SamplingParams


class FakeEngine:
    """Records what the loop asks for. A sequence's 'logits' are just (slot, length so far)."""

    def __init__(self, max_slots=3, max_context=32, pages=8, page_size=4):
        self.max_slots, self.max_context, self.n_pages, self.page_size = max_slots, max_context, pages, page_size
        self.free = list(range(max_slots))
        self.length = {}
        self.steps = []                 # list of [(slot, tokens)]
        self.released = []

    def acquire(self):
        s = self.free.pop(0)
        self.length[s] = 0
        return s

    def release(self, slot):
        assert slot in self.length, "released a slot that is not held"
        del self.length[slot]
        self.free.append(slot)
        self.released.append(slot)

    def fits(self, sizes):
        return len(sizes) <= self.max_slots and sum(-(-(p + b - 1) // self.page_size) for p, b in sizes) <= self.n_pages

    def step(self, entries):
        self.steps.append([(e.slot, list(e.tokens)) for e in entries])
        out = []
        for e in entries:
            assert list(e.want) == [len(e.tokens) - 1]
            self.length[e.slot] += len(e.tokens)
            assert self.length[e.slot] <= self.max_context
            out.append((e.slot, self.length[e.slot]))
        return out


class ScriptSampler:
    """Token for a row = script[request][step]; flags from `bad`."""

    def __init__(self, script, bad=()):
        self.script, self.bad, self.calls = script, set(bad), []

    def sample(self, logits, params, requests, steps, histories=None):
        self.calls.append((list(requests), list(steps), histories))
        return ([self.script[r][s] for r, s in zip(requests, steps)],
                [1 if (r, s) in self.bad else 0 for r, s in zip(requests, steps)])


def test_budget_rule():
    assert token_budget(5, 8, 128) == (8, False)
    assert token_budget(120, 20, 128) == (9, True)       # 120 + 9 - 1 = 128 rows
    assert token_budget(128, 5, 128) == (1, True)        # the last token is never fed back
    for bad in ((0, 5, 128), (5, 0, 128), (129, 1, 128)):
        with pytest.raises(ContextLimitError):
            token_budget(*bad)


def test_unequal_prompts_early_finishers_and_last_token_not_fed():
    eng = FakeEngine()
    script = {0: [10, 11, 12, 13], 1: [20, 99, 0, 0], 2: [30, 31, 32, 33]}
    gen = Generator(eng, ScriptSampler(script))
    outs = gen.generate([[1, 2, 3], [4], [5, 6]], max_tokens=3, params=SamplingParams.greedy(), stop_ids=[99])
    assert [o.tokens for o in outs] == [[10, 11, 12], [20], [30, 31, 32]]
    assert [o.finish_reason for o in outs] == [FINISH_LENGTH, FINISH_STOP, FINISH_LENGTH]
    # step 0: the three prompts together; step 1: one token each; step 2: the stopped one is gone
    assert eng.steps[0] == [(0, [1, 2, 3]), (1, [4]), (2, [5, 6])]
    assert eng.steps[1] == [(0, [10]), (1, [20]), (2, [30])]
    assert eng.steps[2] == [(0, [11]), (2, [31])]
    assert len(eng.steps) == 3                        # 3 tokens need 2 decode steps
    assert sorted(eng.released) == [0, 1, 2] and eng.length == {}


def test_immediate_stop_and_budget_of_one_make_no_decode_step():
    eng = FakeEngine()
    gen = Generator(eng, ScriptSampler({0: [99], 1: [7]}))
    outs = gen.generate([[1], [2]], max_tokens=1, stop_ids=[99])
    assert [o.tokens for o in outs] == [[], [7]] and len(eng.steps) == 1
    assert outs[0].finish_reason == FINISH_STOP and outs[1].finish_reason == FINISH_LENGTH


def test_context_limit_reason_and_exact_capacity():
    eng = FakeEngine(max_context=6, pages=8)
    gen = Generator(eng, ScriptSampler({0: [5] * 10}))
    outs = gen.generate([[1, 2, 3, 4]], max_tokens=10)
    assert len(outs[0].tokens) == 3 and outs[0].finish_reason == FINISH_CONTEXT    # 4 + 3 - 1 = 6 rows
    with pytest.raises(ContextLimitError):
        gen.generate([[1] * 7], max_tokens=1)


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(max_slots=2, pages=100)
    script = {i: [i + 50] * 4 for i in range(5)}
    gen = Generator(eng, ScriptSampler(script))
    outs = gen.generate([[1], [2, 3], [4], [5], [6]], max_tokens=2)
    assert [o.tokens for o in outs] == [[i + 50] * 2 for i in range(5)]
    prefill_steps = [s for s in eng.steps if any(len(t) > 1 or t[0] < 50 for _, t in s)]
    assert [len(s) for s in prefill_steps] == [2, 2, 1]        # three batches
    assert eng.released.count(0) == 3 and eng.released.count(1) == 2


def test_batches_are_cut_by_cache_pages():
    eng = FakeEngine(max_slots=3, pages=4, page_size=4)
    gen = Generator(eng, ScriptSampler({i: [1] * 8 for i in range(3)}))
    assert gen.plan_batches([(6, 3), (6, 3), (2, 2)]) == [[0, 1], [2]]
    with pytest.raises(ContextLimitError):
        gen.plan_batches([(30, 3)])


def test_nonfinite_logits_end_only_that_sequence():
    eng = FakeEngine()
    gen = Generator(eng, ScriptSampler({0: [1, 2, 3], 1: [4, 5, 6]}, bad={(1, 1)}))
    outs = gen.generate([[1], [2]], max_tokens=3)
    assert outs[0].tokens == [1, 2, 3] and outs[1].tokens == [4]
    assert outs[1].finish_reason == FINISH_NONFINITE


def test_sampler_sees_request_and_step_not_batch_position():
    eng = FakeEngine()
    s = ScriptSampler({0: [99], 1: [5, 6, 7]})
    Generator(eng, s).generate([[1], [2]], max_tokens=3, stop_ids=[99],
                               params=SamplingParams(temperature=0.7, repetition_penalty=1.2, seed=3))
    assert s.calls[0][:2] == ([0, 1], [0, 0])
    assert s.calls[1][:2] == ([1], [1]) and s.calls[2][:2] == ([1], [2])
    assert s.calls[1][2] == [[2, 5]]                  # history = prompt + emitted


def test_slots_are_released_when_a_step_raises():
    eng = FakeEngine()

    def boom(entries):
        raise RuntimeError("kernel failed")
    eng.step = boom
    with pytest.raises(RuntimeError):
        Generator(eng, ScriptSampler({})).generate([[1], [2]], max_tokens=2)
    assert eng.length == {} and sorted(eng.released) == [0, 1]
