"""The generation loop above the step function.

For one batch of requests that start together: a slot each, all prompts
(unequal lengths) in one step, a token sampled for each from its last logits,
then one token each per step.  A request ends when it samples a stop token
(which is neither kept nor fed), when it has produced ``max_tokens``, or when
its sequence fills the context; it then leaves the batch and its slot goes
back.  More requests than fit in one batch run as batches one after another.
The single-sequence shape is the reference's: prefill, then
``sample -> stop? -> emit -> forward(one token)`` while ``i < maxTokens`` and
``cache.length < context`` (src/LLM.cpp:688-707; include/ai/LLM.hpp:226-243).

The decisions (how requests are cut into batches, what a sampled token does
to its request) are plain functions of host values, so they are tested
without a device.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling import Sampler, SamplingParams
from .batch import StepEntry


def round_up(n: int, unit: int) -> int:
    return -(-n // unit) * unit


def most_positions(prompt_len: int, max_tokens: int, context: int) -> int:
    """Positions a request can come to hold in the cache: its prompt plus every
    produced token that is fed back (the last one produced never is)."""
    return min(context, prompt_len + max(max_tokens - 1, 0))


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, context: int, max_batch: int,
                 cache_tokens: int, page_tokens: int) -> List[List[int]]:
    """Cuts requests, in order, into batches that fit ``max_batch`` sequences
    and ``cache_tokens`` cache positions (each request rounded up to whole
    pages of its largest possible length)."""
    batches: List[List[int]] = []
    current: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        need = round_up(max(most_positions(n, max_tokens, context), 1), page_tokens)
        if need > cache_tokens:
            raise ValueError(f"request {i} needs {need} cache positions, the cache holds {cache_tokens}")
        if current and (len(current) >= max_batch or used + need > cache_tokens):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


@dataclass
class RequestState:
    index: int                      # place in the caller's list; also keys the sampling stream
    prompt: Sequence[int]
    produced: List[int] = field(default_factory=list)
    finished: bool = False
    reason: str = ""
    held: int = 0                   # positions its slot held before this prompt (a conversation's earlier turns)

    @property
    def positions(self) -> int:
        """Positions the sequence has once everything produced so far is fed."""
        return self.held + len(self.prompt) + len(self.produced)


def take_token(state: RequestState, token: int, stop_ids, max_tokens: int, context: int) -> bool:
    """Applies one sampled token to its request; True if the token is to be
    fed back for another step."""
    if token in stop_ids:
        state.finished, state.reason = True, "stop"
        return False
    state.produced.append(int(token))
    if len(state.produced) >= max_tokens:
        state.finished, state.reason = True, "max_tokens"
        return False
    if state.positions >= context:
        # the reference samples only while cache.length < context (src/LLM.cpp:696)
        state.finished, state.reason = True, "context"
        return False
    return True


def run_batch(step: Callable, sample: Callable, acquire: Callable, release: Callable,
              states: Sequence[RequestState], stop_ids, max_tokens: int, context: int) -> None:
    """One batch from start to end.  ``step(entries) -> logits``,
    ``sample(logits, rows) -> tokens`` (``rows``: indices into ``states``),
    ``acquire() -> slot``, ``release(slot)``."""
    slots = {}
    try:
        live = []
        for k, st in enumerate(states):
            if max_tokens <= 0 or st.held + len(st.prompt) >= context:
                st.finished, st.reason = True, "max_tokens" if max_tokens <= 0 else "context"
                continue
            slots[k] = acquire()
            live.append(k)
        if not live:
            return
        entries = [StepEntry(slots[k], list(states[k].prompt), [len(states[k].prompt) - 1]) for k in live]
        while live:
            logits = step(entries)
            tokens = sample(logits, live)
            fed, entries = [], []
            for k, tok in zip(live, tokens):
                if take_token(states[k], int(tok), stop_ids, max_tokens, context):
                    fed.append(k)
                    entries.append(StepEntry(slots[k], [int(tok)], [0]))
                else:
                    release(slots.pop(k))
            live = fed
    finally:
        for slot in slots.values():
            release(slot)


def run_batch_graphed(model, cache, params: SamplingParams, states: Sequence[RequestState], stop_ids,
                      max_tokens: int, context: int, kept_slots: Optional[Sequence[int]] = None,
                      first_sample: Optional[list] = None) -> None:
    """The same batch as ``run_batch``, with the single-token steps replayed
    from CUDA graphs (``DecodeSession``, pipelined).  The prompts run as one
    eager step.  Then the host stays one step behind the device: each step's
    samples feed the next step on the device, and while the host reads the
    samples of step s, step s + 1 already runs.  A request that samples a stop
    token has by then been stepped once more; that step's sample is dropped and
    its key and value lie past the request's end, in a page the request held
    anyway.  Ends that do not depend on the sample (``max_tokens``, the context)
    are known before the launch, and no such extra step is made.  A finished
    request stays parked in the graph's batch (at its last position, so nothing
    of another sequence is touched) and keeps its slot until the batch has
    halved, when the rest moves to a smaller graph.  With a windowed cache group
    the host does not run behind (pages are given back as a sequence moves on,
    and the page lists on the device must match the step that reads them).

    ``kept_slots``: the slot of each request, taken by the caller, which may
    already hold ``state.held`` positions (a conversation); such slots are not
    given back, and at the end each holds exactly what was fed and emitted (see
    ``settle``)."""
    from .decode_session import session_for
    ops = model.runtime.ops
    slots = {}
    try:
        live = []
        for k, st in enumerate(states):
            if max_tokens <= 0 or st.held + len(st.prompt) >= context:
                st.finished, st.reason = True, "max_tokens" if max_tokens <= 0 else "context"
                continue
            slots[k] = kept_slots[k] if kept_slots is not None else cache.acquire()
            live.append(k)
        if not live:
            return

        def leave(k):
            slot = slots.pop(k)
            if kept_slots is None:
                cache.release(slot)

        sampler = Sampler(params, [states[k].index for k in live], model.runtime.device, ops)
        logits = model.step(cache, [StepEntry(slots[k], list(states[k].prompt), [len(states[k].prompt) - 1])
                                    for k in live])
        tokens = sampler.sample(logits).cpu().tolist()
        if first_sample is not None:
            import time
            first_sample.append(time.perf_counter())       # the prompt step is over: the caller times it apart
        check_kernels(model)
        draws = {k: 1 for k in live}
        feed = {}
        for k, tok in zip(list(live), tokens):
            if take_token(states[k], int(tok), stop_ids, max_tokens, context):
                feed[k] = int(tok)
            else:
                live.remove(k)
                leave(k)
        windowed = any(g.spec.window > 0 for g in cache.kv_groups)
        # steps launched and not yet read: two, unless a step that ran ahead of the news of its sequence's end
        # could not be taken back (pages given back by a window; fixed-size state of a slot that is kept)
        depth = 1 if windowed or (kept_slots is not None and cache.state_groups) else 2
        while live:
            members = list(live)                         # the graph's batch; some may park later
            session = session_for(model, cache, params, len(members))
            run = _GraphedStretch(session, cache, states, slots, members, live, feed, draws, windowed,
                                  stop_ids, max_tokens, context)
            while live and (len(live) * 2 > len(members) or len(members) == 1):
                while run.running and len(run.in_flight) < depth:
                    run.launch()
                run.read()
            while run.in_flight:                         # steps launched before the batch halved or ended
                run.read()
            for k in run.parked:
                leave(k)
        if kept_slots is not None:
            settle(model, cache, states, kept_slots, context)
    finally:
        if kept_slots is None:
            for slot in slots.values():
                cache.release(slot)


def check_kernels(model) -> None:
    """Raises if a kernel gave up one of its bounded waits since the last look; called where the host
    has just waited for the device anyway."""
    ops = model.runtime.ops
    if ops is not None:
        ops.check_status(model.runtime.device)


def settle(model, cache, states: Sequence[RequestState], slots: Sequence[int], context: int) -> None:
    """Leaves every kept slot holding exactly its earlier turns, this prompt and
    every emitted token, as the reference's conversation does (it forwards each
    token it emits, include/ai/LLM.hpp:226-243; a stop token is never fed).  The
    loop above does not feed a request's last token when the end was known in
    advance, and may have stepped a stop token before it saw it: the first is
    fed here with nothing wanted, the second is cut off (its key and value stay
    in the page, past the length, and are overwritten by the next turn)."""
    late = []
    for st, slot in zip(states, slots):
        have, want = cache.length(slot), st.positions
        if have > want:
            cache.truncate(slot, want)
        elif have < want:
            if have != want - 1 or not st.produced:
                raise RuntimeError(f"slot {slot} holds {have} positions, the conversation has {want}")
            late.append(StepEntry(slot, [st.produced[-1]], []))
    if late:
        model.step(cache, late)


class _GraphedStretch:
    """A batch's steps on one graph: from the binding of its live requests
    (``members``) to a session until half of them have ended.  ``live``, ``feed``
    (the token each live request is fed next) and ``draws`` (how far each
    sampling stream has run) are the batch's and are updated in place."""

    def __init__(self, session, cache, states, slots, members, live, feed, draws, windowed, stop_ids,
                 max_tokens, context):
        self.session, self.cache, self.states, self.slots = session, cache, states, slots
        self.live, self.feed, self.draws, self.windowed = live, feed, draws, windowed
        self.stop_ids, self.max_tokens, self.context = stop_ids, max_tokens, context
        self.place = {k: i for i, k in enumerate(members)}
        self.positions = [cache.length(slots[k]) for k in members]     # of each member's next step
        self.stepped_at = list(self.positions)                          # of each member's last launched step
        self.running = list(live)          # stepped for real by the next launch, as far as the host knows
        self.unread = {k: 0 for k in members}                           # launched steps whose samples are unread
        self.in_flight = deque()                                        # (ticket, requests stepped for real)
        self.parked = set()
        self.dirty = True                                               # the page lists on the device are out of date
        session.rebind([slots[k] for k in members], [states[k].index for k in members],
                       [draws[k] for k in members])
        session.start([feed[k] for k in members], self.positions)

    def launch(self) -> None:
        """Launches the next step and works out who goes on after it if no sample
        of an unread step is a stop token."""
        cache, positions, place = self.cache, self.positions, self.place
        for k in self.running:
            if positions[place[k]] % cache.page_tokens == 0:            # the token of this step opens a page
                self.dirty |= cache.reserve_one(self.slots[k])
        if self.dirty:
            self.session.sync_block_tables()
            self.dirty = False
        self.in_flight.append((self.session.launch_step(positions), list(self.running)))
        goes_on = []
        for k in self.running:
            i, st = place[k], self.states[k]
            cache.lengths[self.slots[k]] += 1                           # what commit(slot, 1) does without a window
            self.stepped_at[i] = positions[i]
            self.unread[k] += 1
            made = len(st.produced) + self.unread[k]                    # if none of the unread samples is a stop token
            if made < self.max_tokens and st.held + len(st.prompt) + made < self.context:
                positions[i] += 1
                goes_on.append(k)
            # else this step's sample is its last, whatever it is: it stays where it is
        self.running = goes_on

    def read(self) -> None:
        """Reads the samples of the oldest launched step and applies them to its
        requests."""
        if not self.in_flight:                           # cannot be: a live request is running or has a step unread
            raise RuntimeError("the generation loop has live requests and nothing to wait for")
        ticket, stepped = self.in_flight.popleft()
        tokens = self.session.read_step(ticket)              # raises if a kernel of the step gave up a wait
        for k in stepped:
            self.unread[k] -= 1
            if self.states[k].finished:                  # the step ran ahead of the news of its end
                continue
            if self.windowed:
                self.cache.commit(self.slots[k], 0)
            self.draws[k] += 1
            tok = tokens[self.place[k]]
            if take_token(self.states[k], tok, self.stop_ids, self.max_tokens, self.context):
                self.feed[k] = tok                       # what a smaller graph would go on with
            else:
                self.live.remove(k)
                self.parked.add(k)                       # keeps being stepped at its last position
                if k in self.running:
                    self.running.remove(k)
                    self.positions[self.place[k]] = self.stepped_at[self.place[k]]


def run_requests(model, cache, params: SamplingParams, states: Sequence[RequestState], stop_ids, max_tokens: int,
                 context: int, kept_slots: Optional[Sequence[int]] = None, use_graph: bool = True,
                 timing: Optional[dict] = None, stage_timer=None) -> None:
    """One batch through the loop that fits the model: graph replay where every
    part can be replayed, eager steps otherwise.  Everything that generates
    (``generate``, ``LLM.prompt``, the command line) comes through here.

    ``timing``: a dict that receives ``prompt_s`` (the prompt step up to its
    first sample) and ``decode_s`` (everything after), as the reference times
    them apart (src/LLM.cpp:687-711).  ``stage_timer``: a ``StageTimer`` for
    per-stage device times; the steps then run eagerly."""
    import time
    t0 = time.perf_counter()
    first_sample = []
    if use_graph and stage_timer is None and getattr(model, "graph_safe", True):
        run_batch_graphed(model, cache, params, states, stop_ids, max_tokens, context, kept_slots, first_sample)
    else:
        ops = model.runtime.ops
        sampler = Sampler(params, [s.index for s in states], model.runtime.device, ops)
        n = len(states)

        def step(entries):
            if stage_timer is not None:
                stage_timer.begin(is_prompt=not first_sample)
            return model.step(cache, entries, trace=stage_timer)

        def sample(logits, rows):
            tokens = sampler.sample(logits, None if len(rows) == n else rows).cpu().tolist()
            if not first_sample:
                first_sample.append(time.perf_counter())
            check_kernels(model)
            return tokens

        if kept_slots is None:
            run_batch(step, sample, cache.acquire, cache.release, states, stop_ids, max_tokens, context)
        else:
            taken = iter([slot for st, slot in zip(states, kept_slots)
                          if max_tokens > 0 and st.held + len(st.prompt) < context])
            run_batch(step, sample, lambda: next(taken), lambda slot: None, states, stop_ids, max_tokens, context)
            settle(model, cache, states, kept_slots, context)
    if timing is not None:
        t1 = first_sample[0] if first_sample else time.perf_counter()
        timing["prompt_s"], timing["decode_s"] = t1 - t0, time.perf_counter() - t1


def generate(model, prompts: Sequence[Sequence[int]], max_tokens: int, params: SamplingParams,
             stop_ids: Optional[Sequence[int]] = None, context: Optional[int] = None,
             max_batch: int = 64, cache=None, request_offset: int = 0, use_graph: bool = True) -> List[List[int]]:
    """Generates a continuation for every prompt (lists of token ids)."""
    context = min(context or model.max_positions, model.max_positions)
    stop = frozenset(model.stop_ids if stop_ids is None else stop_ids)
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
        if len(p) > context:
            raise ValueError(f"prompt {i} has {len(p)} tokens, the context holds {context}")
    if cache is None:
        from ..cache import PAGE_TOKENS
        need = sorted((round_up(max(most_positions(len(p), max_tokens, context), 1), PAGE_TOKENS)
                       for p in prompts), reverse=True)
        cache = model.new_cache(max_tokens=max(sum(need[:max_batch]), PAGE_TOKENS), n_slots=max_batch)
    page = cache.page_tokens
    batches = plan_batches([len(p) for p in prompts], max_tokens, context, min(max_batch, cache.n_slots),
                           cache.n_pages * page, page)
    states = [RequestState(i + request_offset, p) for i, p in enumerate(prompts)]
    for batch in batches:
        run_requests(model, cache, params, [states[i] for i in batch], stop, max_tokens, context,
                     use_graph=use_graph)
    return [s.produced for s in states]
