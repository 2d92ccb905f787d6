"""The generation loop's decisions, with a fake model: no device needed."""
import pytest

from math_utils_b200.engine.generate import (RequestState, most_positions, plan_batches, run_batch,
                                             take_token)


def test_take_token_rules():
    st = RequestState(0, [1, 2, 3])
    assert take_token(st, 9, {7}, max_tokens=3, context=100) is True and st.produced == [9]
    assert take_token(st, 7, {7}, 3, 100) is False and st.reason == "stop" and st.produced == [9]
    st = RequestState(0, [1, 2, 3])
    assert take_token(st, 4, set(), 2, 100) is True
    assert take_token(st, 5, set(), 2, 100) is False and st.reason == "max_tokens" and st.produced == [4, 5]
    st = RequestState(0, [1, 2, 3])                      # context 5: positions 3 and 4 can still be produced
    assert take_token(st, 4, set(), 10, 5) is True
    assert take_token(st, 5, set(), 10, 5) is False and st.reason == "context" and st.produced == [4, 5]


def test_plan_batches_by_count_and_by_cache_room():
    assert plan_batches([5, 5, 5, 5, 5], 10, 100, max_batch=2, cache_tokens=10 ** 6, page_tokens=64) == \
        [[0, 1], [2, 3], [4]]
    # 60+10-1 = 69 positions -> 128 each; room for three at a time
    assert plan_batches([60] * 7, 10, 100, max_batch=64, cache_tokens=384, page_tokens=64) == \
        [[0, 1, 2], [3, 4, 5], [6]]
    assert most_positions(60, 10, 64) == 64 and most_positions(5, 1, 64) == 5
    with pytest.raises(ValueError, match="cache holds"):
        plan_batches([200], 10, 1000, 4, cache_tokens=128, page_tokens=64)


class FakeModel:
    """Next token = (sum of the sequence so far) % 50; records every step."""

    def __init__(self):
        self.seqs, self.free, self.steps, self.next_slot = {}, [], [], 0

    def acquire(self):
        slot = self.free.pop() if self.free else self.next_slot
        if slot == self.next_slot:
            self.next_slot += 1
        assert slot not in self.seqs
        self.seqs[slot] = []
        return slot

    def release(self, slot):
        del self.seqs[slot]
        self.free.append(slot)

    def step(self, entries):
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        out = []
        for e in entries:
            self.seqs[e.slot].extend(e.tokens)
            assert list(e.want) == [len(e.tokens) - 1]
            out.append(sum(self.seqs[e.slot]) % 50)
        return out

    @staticmethod
    def sample(logits, rows):
        return logits


def expected(prompt, max_tokens, stop, context):
    ids, out = list(prompt), []
    for _ in range(max_tokens):
        if len(ids) >= context:
            break
        t = sum(ids) % 50
        if t in stop:
            break
        out.append(t); ids.append(t)
    return out


def test_batch_of_unequal_prompts_ends_requests_separately():
    m = FakeModel()
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9, 10], [11, 12]]
    states = [RequestState(i, p) for i, p in enumerate(prompts)]
    run_batch(m.step, m.sample, m.acquire, m.release, states, {13, 33}, max_tokens=6, context=9)
    for st, p in zip(states, prompts):
        assert st.produced == expected(p, 6, {13, 33}, 9), st
        assert st.finished
    assert m.seqs == {}                                   # every slot came back
    assert [n for _, n in m.steps[0]] == [3, 1, 6, 2]     # all prompts in the first step
    assert all(n == 1 for step in m.steps[1:] for _, n in step)
    sizes = [len(s) for s in m.steps]
    assert sizes == sorted(sizes, reverse=True) and sizes[-1] < sizes[0]    # the batch thins out
    reasons = {st.reason for st in states}
    assert reasons <= {"stop", "max_tokens", "context"} and len(reasons) >= 2


def test_full_prompt_and_zero_tokens_take_no_slot():
    m = FakeModel()
    states = [RequestState(0, [1] * 9), RequestState(1, [2, 3])]
    run_batch(m.step, m.sample, m.acquire, m.release, states, set(), max_tokens=4, context=9)
    assert states[0].produced == [] and states[0].reason == "context"
    assert states[1].produced == expected([2, 3], 4, set(), 9)
    states = [RequestState(0, [1, 2])]
    run_batch(m.step, m.sample, m.acquire, m.release, states, set(), max_tokens=0, context=9)
    assert states[0].produced == [] and m.seqs == {}


def test_slots_come_back_when_the_model_fails():
    m = FakeModel()

    def bad_step(entries):
        raise RuntimeError("boom")
    with pytest.raises(RuntimeError):
        run_batch(bad_step, m.sample, m.acquire, m.release, [RequestState(0, [1]), RequestState(1, [2])],
                  set(), 3, 10)
    assert m.seqs == {}
