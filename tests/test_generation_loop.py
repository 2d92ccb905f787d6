"""The generation loop's decisions, with a fake model: no device needed."""
import numpy as np
import pytest
import torch

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


# ------------------------------------------------------------------ the loop that runs one step behind the device
class FakeDevice:
    """What the graphed loop drives, without a device: a model whose next token is
    (sum of the tokens its window sees) % 50, keys kept in numbered pages that are found through
    the page lists the host has SENT (not the ones it holds), so a missing hand-over of the
    lists, a page used by two sequences or a step past a sequence's pages shows as a wrong
    token or an assertion.  Sessions behave like ``DecodeSession(pipelined=True)``: samples feed
    the next step on the device, positions come from the host, two steps at most are unread."""

    def __init__(self, cache, window=0, limit=10 ** 9):
        self.cache, self.window, self.limit = cache, window, limit
        self.page = cache.page_tokens
        self.pages = {}                                    # (page number, offset) -> token
        self.steps_launched = 0
        self.most_unread = 0
        self.runtime = type("R", (), {"ops": None, "device": "cpu"})()
        self.graph_safe = True

    def visible(self, table_row, pos):
        first = 0 if self.window <= 0 else max(0, pos - self.window + 1)
        total = 0
        for p in range(first, pos + 1):
            page = int(table_row[p // self.page])
            assert page >= 0, f"position {p} has no page"
            total += self.pages[(page, p % self.page)]
        return total % 50

    def step(self, cache, entries):                        # the eager prompt step
        out = []
        for e in entries:
            start = cache.reserve(e.slot, len(e.tokens))
            row = cache.kv_groups[0].table[e.slot]
            for i, t in enumerate(e.tokens):
                self.pages[(int(row[(start + i) // self.page]), (start + i) % self.page)] = t
            out.append(self.visible(row, start + len(e.tokens) - 1))
            cache.commit(e.slot, len(e.tokens))
        return torch.tensor(out)

    def session(self, n):
        dev = self

        class Session:
            def __init__(self):
                self.tokens, self.unread, self.turn, self.out = [0] * n, [False, False], 0, [None, None]

            def rebind(self, slots, request_ids, draws):
                self.slots, self.table = list(slots), None

            def sync_block_tables(self):
                self.table = dev.cache.kv_groups[0].table[self.slots].copy()

            def start(self, tokens, positions):
                self.tokens, self.unread = list(tokens), [False, False]

            def launch_step(self, positions):
                assert not self.unread[self.turn], "a third step launched with two unread"
                rows_now = dev.cache.kv_groups[0].table[self.slots]
                nxt = []
                for i, (tok, pos) in enumerate(zip(self.tokens, positions)):
                    assert pos < dev.limit, f"member {i} steps at position {pos}: the context ends at {dev.limit}"
                    page = int(self.table[i][pos // dev.page])
                    if page < 0 or page != int(rows_now[i][pos // dev.page]):
                        # only a parked sequence may step without a page of its own: it must not write
                        raise AssertionError(f"member {i} steps at position {pos} without a page it holds")
                    dev.pages[(page, pos % dev.page)] = tok
                    nxt.append(dev.visible(self.table[i], pos))
                self.tokens = nxt
                ticket, self.turn = self.turn, self.turn ^ 1
                self.unread[ticket], self.out[ticket] = True, list(nxt)
                dev.steps_launched += 1
                dev.most_unread = max(dev.most_unread, sum(self.unread))
                return ticket

            def read_step(self, ticket):
                assert self.unread[ticket]
                self.unread[ticket] = False
                return self.out[ticket]

        return Session()


def expected_windowed(prompt, max_tokens, stop, context, window):
    ids, out = list(prompt), []
    for _ in range(max_tokens):
        if len(ids) >= context:
            break
        t = sum(ids if window <= 0 else ids[-window:]) % 50
        if t in stop:
            break
        out.append(t); ids.append(t)
    return out


@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("max_tokens,context,stop", [(40, 200, {13, 33}), (5, 200, set()), (150, 140, {7}), (1, 200, set()),
                                                     (2, 200, set()), (66, 200, {49}),
                                                     (90, 200, {1, 2, 3, 4, 5, 6, 7, 8, 9})])
def test_loop_one_step_behind_the_device(monkeypatch, window, max_tokens, context, stop):
    """``run_batch_graphed`` against the plain recurrence: unequal prompts that cross page borders,
    stop tokens found one step late, ends known in advance, parked requests, the move to a
    smaller graph, batch after batch on the same slots; with a window the loop must not run
    behind."""
    from math_utils_b200.cache import SequenceCache
    from math_utils_b200.engine import decode_session, generate as gen
    from math_utils_b200.parts.base import KVCacheSpec
    from math_utils_b200.sampling import SamplingParams
    all_lens = [1, 63, 64, 65, 127, 30]
    # exactly the pages the first (largest) batch is planned with: a step past a request's planned end finds none
    room = sum(-(-max(most_positions(n, max_tokens, context), 1) // 64) * 64 for n in all_lens)
    cache = SequenceCache([KVCacheSpec(1, 16, window)], room, 200, torch.float32, "cpu", n_slots=6)
    dev = FakeDevice(cache, window, limit=context)
    sessions = {}
    monkeypatch.setattr(decode_session, "session_for",
                        lambda model, c, params, n, pipelined=True: sessions.setdefault(n, dev.session(n)))

    class FakeSampler:
        def __init__(self, *a):
            pass

        def sample(self, logits):
            return logits
    monkeypatch.setattr(gen, "Sampler", FakeSampler)
    rng = np.random.default_rng(max_tokens + context)
    for round_ in range(3):                                # the same slots again and again
        lens = all_lens[: 6 - round_]
        prompts = [rng.integers(0, 50, size=n).tolist() for n in lens]
        states = [RequestState(i, p) for i, p in enumerate(prompts)]
        gen.run_batch_graphed(dev, cache, SamplingParams(temperature=0.0), states, stop, max_tokens, context)
        for st, p in zip(states, prompts):
            assert st.finished
            assert st.produced == expected_windowed(p, max_tokens, stop, context, window), (round_, len(p), st.reason)
        assert cache.slots.n_free == 6 and cache.free_pages(0) == cache.n_pages
    assert dev.most_unread <= (1 if window else 2)
    if max_tokens > 2 and not window:
        assert dev.most_unread == 2                        # the loop did run behind


def test_loop_one_step_behind_on_drawn_cases(monkeypatch):
    """The same comparison on drawn cases: prompt lengths, token budget, context, stop tokens and
    window at random, the cache exactly as large as ``plan_batches`` counts."""
    from math_utils_b200.cache import SequenceCache
    from math_utils_b200.engine import decode_session, generate as gen
    from math_utils_b200.parts.base import KVCacheSpec
    from math_utils_b200.sampling import SamplingParams

    class FakeSampler:
        def __init__(self, *a):
            pass

        def sample(self, logits):
            return logits
    monkeypatch.setattr(gen, "Sampler", FakeSampler)
    rng = np.random.default_rng(2024)
    reasons = set()
    for case in range(60):
        n_req = int(rng.integers(1, 7))
        context = int(rng.integers(2, 200))
        lens = [int(rng.integers(1, context + 1)) for _ in range(n_req)]
        max_tokens = int(rng.choice([0, 1, 2, 3, 17, 64, 65, 300]))
        stop = set(rng.integers(0, 50, size=int(rng.integers(0, 6))).tolist())
        window = int(rng.choice([0, 0, 1, 40, 64, 130]))
        room = sum(-(-max(most_positions(n, max_tokens, context), 1) // 64) * 64 for n in lens)
        cache = SequenceCache([KVCacheSpec(1, 16, window)], room, 200, torch.float32, "cpu", n_slots=n_req)
        dev = FakeDevice(cache, window, limit=context)
        sessions = {}
        monkeypatch.setattr(decode_session, "session_for",
                            lambda model, c, params, n, pipelined=True, dev=dev, sessions=sessions:
                            sessions.setdefault(n, dev.session(n)))
        for round_ in range(2):
            prompts = [rng.integers(0, 50, size=n).tolist() for n in lens]
            states = [RequestState(i, p) for i, p in enumerate(prompts)]
            gen.run_batch_graphed(dev, cache, SamplingParams(temperature=0.0), states, stop, max_tokens, context)
            for st, p in zip(states, prompts):
                assert st.finished
                assert st.produced == expected_windowed(p, max_tokens, stop, context, window), \
                    (case, round_, lens, max_tokens, context, sorted(stop), window, len(p), st.reason)
                reasons.add(st.reason)
            assert cache.slots.n_free == n_req and cache.free_pages(0) == cache.n_pages
        assert dev.most_unread <= (1 if window else 2)
    assert reasons == {"stop", "max_tokens", "context"}


@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("max_tokens,stop", [(5, set()), (40, {13, 33, 7, 21}), (1, set()), (64, {49})])
def test_conversation_on_a_kept_slot(monkeypatch, window, max_tokens, stop):
    """Turn after turn on one slot that the caller keeps (``kept_slots``): after each turn the slot
    holds the earlier turns, the prompt and every emitted token, whether the turn ended on a stop
    token (which the device had already stepped when the host saw it: cut off again), on the token
    budget or on the context (the last token is fed afterwards); the next turn continues from there."""
    from math_utils_b200.cache import SequenceCache
    from math_utils_b200.engine import decode_session, generate as gen
    from math_utils_b200.parts.base import KVCacheSpec
    from math_utils_b200.sampling import SamplingParams
    context = 200
    cache = SequenceCache([KVCacheSpec(1, 16, window)], 256, 200, torch.float32, "cpu", n_slots=1)
    dev = FakeDevice(cache, window, limit=context)
    sessions = {}
    monkeypatch.setattr(decode_session, "session_for",
                        lambda model, c, params, n, pipelined=True: sessions.setdefault(n, dev.session(n)))

    class FakeSampler:
        def __init__(self, *a):
            pass

        def sample(self, logits):
            return logits
    monkeypatch.setattr(gen, "Sampler", FakeSampler)
    rng = np.random.default_rng(max_tokens + window)
    slot = cache.acquire()
    history, reasons = [], set()
    for turn in range(6):
        ids = rng.integers(0, 50, size=int(rng.integers(1, 20))).tolist()
        if len(history) + len(ids) + max_tokens > context:
            break
        state = RequestState(turn, ids, held=len(history))
        gen.run_batch_graphed(dev, cache, SamplingParams(temperature=0.0), [state], stop, max_tokens, context,
                              kept_slots=[slot])
        want = expected_windowed(history + ids, max_tokens, stop, context, window)
        assert state.produced == want, (turn, state.reason)
        history += ids + want
        assert cache.length(slot) == len(history) == state.positions
        assert cache.slots.is_held(slot)
        reasons.add(state.reason)
    assert reasons                                     # at least one turn ran
    cache.release(slot)
    assert cache.free_pages(0) == cache.n_pages


def test_cache_cut_back():
    from math_utils_b200.cache import CacheError, SequenceCache
    from math_utils_b200.parts.base import KVCacheSpec, StateCacheSpec
    cache = SequenceCache([KVCacheSpec(1, 16, 0)], 256, 200, torch.float32, "cpu", n_slots=2)
    slot = cache.acquire()
    cache.reserve(slot, 70); cache.commit(slot, 70)
    held = cache.kv_groups[0].pages_held(slot)
    cache.truncate(slot, 64)
    assert cache.length(slot) == 64 and cache.kv_groups[0].pages_held(slot) == held     # the page stays
    cache.reserve(slot, 3); cache.commit(slot, 3)                                        # and is used again
    assert cache.length(slot) == 67 and cache.kv_groups[0].pages_held(slot) == held
    with pytest.raises(CacheError):
        cache.truncate(slot, 68)
    for spec in (KVCacheSpec(1, 16, 40), StateCacheSpec(8)):
        other = SequenceCache([spec, KVCacheSpec(1, 16, 0)], 256, 200, torch.float32, "cpu", n_slots=1)
        s = other.acquire()
        other.reserve(s, 5); other.commit(s, 5)
        with pytest.raises(CacheError, match="cannot be cut back"):
            other.truncate(s, 4)
        other.truncate(s, 5)                                                             # nothing to cut: allowed
