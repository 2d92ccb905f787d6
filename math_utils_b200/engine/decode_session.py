"""Single-token steps of a fixed batch, replayed from one CUDA graph.

Once a batch's prompts are in the cache, every further step has the same
shape: one token per sequence.  A ``DecodeSession`` keeps that step's index
arrays in fixed device buffers, captures the model's forward pass, the
sampling and the hand-over of the sampled tokens to the next step in a CUDA
graph once, and replays it: one launch per step instead of a hundred.  The
kernels are the ones the eager step runs; only the launching differs.

Three ways to drive it:
  * ``feed(tokens, positions)`` then ``launch()`` then ``read_tokens()``: the
    host supplies every step's inputs and reads every step's tokens;
  * ``launch()`` repeatedly: each step's samples are the next step's inputs on
    the device (the sampling kernel hands them over and moves the positions on),
    with no host round trip between steps;
  * ``pipelined``: ``start(tokens)`` once, then ``launch_step(positions)`` and
    ``read_step(ticket)``: the samples feed the next step on the device, the
    host says at which positions every step runs (it alone knows which
    sequences have ended and stay where they are) and reads every step's
    samples, one step behind: while it looks at step s, step s + 1 already
    runs (the generation loop, which has to see stop tokens but should not
    hold the device up).  Neither transfer is in the step's way: the
    positions go to the device on a stream of their own while the step before
    still runs, and the samples come back on another stream while the next
    step runs.  No kernel of a step writes the positions, so a kernel may read
    them before the kernel in front of it has ended (the attention kernels ask
    for their pages that early).
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..sampling import SamplingParams
from .batch import StepContext


class DecodeSession:
    def __init__(self, model, cache, slots: Sequence[int], params: SamplingParams,
                 request_ids: Sequence[int], kv_bound: Optional[int] = None, pipelined: bool = False):
        """``pipelined``: two graphs that take turns, each with device and
        pinned host buffers of its own: for the positions, which a copy stream
        sends ahead of the step, and for the samples and the kernels' status
        word, which another copy stream brings to the host after the step while
        the next step runs.  Without it a launch leaves the inputs alone, and
        each step's samples feed the next on the device."""
        self.model, self.cache = model, cache
        self.pipelined = pipelined
        self.slots = list(slots)
        self.n = len(self.slots)
        self.params = params
        rt = model.runtime
        dev = rt.device
        n = self.n
        self.kv_bound = int(kv_bound or model.max_positions)
        self.tables_shape = [(n, g.max_pages) for g in cache.kv_groups]
        sizes = [n, n, n, n, n] + [a * b for a, b in self.tables_shape]
        offs = np.concatenate([[0], np.cumsum([-(-s // 4) * 4 for s in sizes])]).astype(int)
        self._offs = offs
        self.dev = torch.zeros(int(offs[-1]), dtype=torch.int32, device=dev)
        self.host = torch.zeros(int(offs[-1]), dtype=torch.int32, pin_memory=True)
        h = self.host.numpy()
        h[offs[2]:offs[2] + n] = np.arange(n)            # tok_seq
        h[offs[3]:offs[3] + n] = np.arange(n)            # want_rows: every token's logits
        h[offs[4]:offs[4] + n] = np.asarray(self.slots)
        self.dev.copy_(self.host)

        def part(i, count):
            return self.dev[int(offs[i]): int(offs[i]) + count]

        self.token_ids, self.tok_pos = part(0, n), part(1, n)
        self.block_tables = [part(5 + i, a * b).view(a, b) for i, (a, b) in enumerate(self.tables_shape)]
        self.next_tokens = torch.zeros(n, dtype=torch.int32, device=dev)
        self.next_host = torch.zeros(n, dtype=torch.int32, pin_memory=True)
        self.request_ids = torch.tensor(list(request_ids), dtype=torch.int64, device=dev)
        self.draws = torch.zeros(n, dtype=torch.int32, device=dev)
        self.ctx = StepContext(
            runtime=rt, position=model.assembly.position, n_tokens=n, n_seqs=n,
            token_ids=self.token_ids, tok_pos=self.tok_pos, tok_seq=part(2, n), want_rows=part(3, n),
            block_tables=self.block_tables, seq_slots=part(4, n), slots=self.slots, starts=[0] * n,
            q_lens=[1] * n, max_q_len=1, max_kv_len=self.kv_bound, workspace={})
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._feed_views = None
        self._stream = None
        if pipelined:
            self._turn_graphs = None
            self._turn = 0
            # samples of a turn, and behind them the kernels' status word as that step left it
            self._out_dev = [torch.zeros(n + 1, dtype=torch.int32, device=dev) for _ in range(2)]
            self._out_host = [torch.zeros(n + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._out_stream = torch.cuda.Stream(device=dev)
            self._stepped = [torch.cuda.Event() for _ in range(2)]
            self._done = [torch.cuda.Event() for _ in range(2)]
            self._unread = [False, False]
            self._first_tokens = torch.zeros(n, dtype=torch.int32, pin_memory=True)
            # the positions of a turn's step, sent ahead on a stream of its own
            self._pos_dev = [torch.zeros(n, dtype=torch.int32, device=dev) for _ in range(2)]
            self._pos_host = [torch.zeros(n, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._in_stream = torch.cuda.Stream(device=dev)
            self._sent = [torch.cuda.Event() for _ in range(2)]
            self._turn_ctx = [dataclasses.replace(self.ctx, tok_pos=self._pos_dev[t]) for t in range(2)]
            rt.ops.status_word(dev)                               # exists before any capture asks for it
        self.launches_per_step = 0
        self.logits: Optional[torch.Tensor] = None
        self._tables_host = [None] * len(self.tables_shape)

    def rebind(self, slots: Sequence[int], request_ids: Sequence[int], draws: Sequence[int]) -> None:
        """Gives the session's places to another set of sequences of the same
        number: their slots, their sampling streams and how far those have run."""
        if len(slots) != self.n:
            raise ValueError(f"this session steps {self.n} sequences, got {len(slots)}")
        self.slots = list(slots)
        self.ctx.slots = self.slots
        for ctx in getattr(self, "_turn_ctx", ()):
            ctx.slots = self.slots
        h = self.host.numpy()
        o = int(self._offs[4])
        h[o:o + self.n] = np.asarray(self.slots, dtype=np.int32)
        self.dev[o:o + self.n].copy_(self.host[o:o + self.n], non_blocking=True)
        self.request_ids.copy_(torch.tensor(list(request_ids), dtype=torch.int64), non_blocking=False)
        self.draws.copy_(torch.tensor(list(draws), dtype=torch.int32), non_blocking=False)
        self._tables_host = [None] * len(self.tables_shape)
        self._fed = False

    # ------------------------------------------------------------------ inputs
    def sync_block_tables(self) -> None:
        """Sends the slots' page lists to the device where they changed."""
        offs = self._offs
        h = self.host.numpy()
        for i, g in enumerate(self.cache.kv_groups):
            rows = self.cache.block_table_rows(g.index, self.slots)
            if self._tables_host[i] is None or not np.array_equal(rows, self._tables_host[i]):
                self._tables_host[i] = rows.copy()
                h[offs[5 + i]: offs[5 + i] + rows.size] = rows.reshape(-1)
                self.dev[int(offs[5 + i]): int(offs[5 + i]) + rows.size].copy_(
                    self.host[int(offs[5 + i]): int(offs[5 + i]) + rows.size], non_blocking=True)

    def feed(self, tokens: Sequence[int], positions: Sequence[int]) -> int:
        """This step's token and position of every sequence; returns the bytes
        sent to the device."""
        if self._feed_views is None:
            n, upto = self.n, int(self._offs[1]) + self.n
            h = self.host.numpy()
            self._feed_views = (h[0:n], h[int(self._offs[1]): int(self._offs[1]) + n],
                                self.dev[:upto], self.host[:upto], upto * 4)
        tok_view, pos_view, dev_part, host_part, n_bytes = self._feed_views
        tok_view[:] = tokens
        pos_view[:] = positions
        dev_part.copy_(host_part, non_blocking=True)
        self._fed = True
        return n_bytes

    # ------------------------------------------------ pipelined: one step behind
    def start(self, tokens: Sequence[int], positions: Sequence[int]) -> None:
        """The tokens the first step of these sequences takes (later steps take
        the samples of the step before, on the device) and its positions (where
        the set-up run before a recording writes its keys and values)."""
        # no copy from or to the staging buffers is still under way (a batch that ended with an error may have
        # left steps unread)
        torch.cuda.current_stream().synchronize()
        self._in_stream.synchronize()
        self._out_stream.synchronize()
        self._unread = [False, False]
        self._first_tokens.numpy()[:] = tokens
        self.token_ids.copy_(self._first_tokens, non_blocking=True)
        self._pos_host[self._turn].numpy()[:] = positions
        self.tok_pos.copy_(self._pos_host[self._turn], non_blocking=True)
        self._fed = True

    def launch_step(self, positions: Sequence[int]) -> int:
        """Launches a step at these positions; returns the ticket to read its
        samples with.  At most two steps may be unread at any time."""
        turn = self._turn
        if self._unread[turn]:
            raise RuntimeError("two steps are launched and unread: read the older one first (its buffers come next)")
        if self._turn_graphs is None:
            self.capture()
        ops = self.model.runtime.ops
        # (this turn's buffers are free: the step that last used them has been read)
        self._pos_host[turn].numpy()[:] = positions
        ops.copy_async(self._pos_dev[turn], self._pos_host[turn], stream=self._in_stream)
        self._sent[turn].record(self._in_stream)
        main = torch.cuda.current_stream()
        main.wait_event(self._sent[turn])
        self._unread[turn] = True
        self._turn_graphs[turn].replay()
        self._stepped[turn].record(main)
        self._out_stream.wait_event(self._stepped[turn])
        ops.copy_async(self._out_host[turn], self._out_dev[turn], stream=self._out_stream)
        self._done[turn].record(self._out_stream)
        ops.launch_count += self.launches_per_step
        self._turn = turn ^ 1
        return turn

    def read_step(self, ticket: int) -> List[int]:
        """The samples of the step launched with this ticket (waits for that
        step and the copy of its samples only)."""
        self._done[ticket].synchronize()
        self._unread[ticket] = False
        out = self._out_host[ticket].tolist()
        if out[-1] != 0:
            self.model.runtime.ops.raise_status(self.model.runtime.device, out[-1])
        return out[:-1]

    # ------------------------------------------------------------------- steps
    def _run_once(self, turn: Optional[int] = None) -> None:
        """One step.  With ``turn`` (a recorded step of the pipelined kind) the
        positions are that turn's, which the host sends before every launch
        (the sampling kernel leaves them alone), and the samples and the status
        word go to that turn's buffer."""
        ops = self.model.runtime.ops
        ctx, out, status_to, moves = self.ctx, self.next_tokens, None, self.tok_pos
        if turn is not None:
            ctx, moves = self._turn_ctx[turn], None
            out, status_to = self._out_dev[turn][:self.n], self._out_dev[turn][self.n:]
        logits = self.logits = self.model.forward(ctx, self.cache)
        feed = (self.token_ids, moves, self.kv_bound - 1)            # samples become the next step's inputs
        if self.params.greedy:
            ops.argmax(logits, out=out, feed=feed, status_to=status_to)
        else:
            ops.sample(logits, self.params.temperature, self.params.kept, self.params.seed,
                       self.request_ids, self.draws, out=out, feed=feed, status_to=status_to)

    def capture(self) -> None:
        """Runs the step once eagerly (first-use set-up must not happen inside a
        capture), then records it.  The eager run writes keys and values at the
        current positions and the capture runs nothing, so inputs and counters
        are restored afterwards."""
        if not getattr(self, "_fed", False):
            raise RuntimeError("feed() the real tokens and positions before the first launch: the set-up run "
                               "writes keys and values at the positions it is given")
        ops = self.model.runtime.ops
        saved = (self.token_ids.clone(), self.tok_pos.clone(), self.draws.clone())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._run_once()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self.pipelined:
            self._turn_graphs = [self._record_graph(lambda turn=turn: self._run_once(turn), side)
                                 for turn in range(2)]
        else:
            self.graph = self._record_graph(self._run_once, side)
        self.token_ids.copy_(saved[0]); self.tok_pos.copy_(saved[1]); self.draws.copy_(saved[2])

    def _record_graph(self, body, side: torch.cuda.Stream) -> torch.cuda.CUDAGraph:
        """Records what ``body`` launches on the side stream.  ``torch.cuda.graph`` would do the same
        after a garbage collection and after emptying the allocator's cache, which costs a batch that
        thins out (a smaller graph every time it halves) tens of milliseconds per graph."""
        ops = self.model.runtime.ops
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        # One memory pool for every graph of this model: what a session's recording allocated goes back there
        # when the session is dropped and serves the next recording.  (A pool per graph keeps its memory
        # reserved after the graph is gone: a process that keeps meeting new batch shapes would run out.)
        pool = self.model.__dict__.get("_graph_pool")
        if pool is None:
            # the pool lives as long as a graph recorded into it does: a graph of one small fill, kept with the
            # model, holds it when every session has been dropped (a pool without a graph may not be used again)
            pool = torch.cuda.graph_pool_handle()
            keeper = torch.cuda.CUDAGraph()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                keeper.capture_begin(pool=pool)
                try:
                    held = torch.zeros(16, dtype=torch.int32, device=self.model.runtime.device)
                finally:
                    keeper.capture_end()
            self.model.__dict__["_graph_pool_keeper"] = (keeper, held)
            self.model.__dict__["_graph_pool"] = pool
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph.capture_begin(pool=pool)
            try:
                body()
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)
        self.launches_per_step = ops.launch_count - before
        return graph

    def launch(self) -> None:
        if self.graph is None:
            self.capture()
        self.graph.replay()
        self.model.runtime.ops.launch_count += self.launches_per_step

    def read_tokens(self) -> List[int]:
        """The tokens the last launched step sampled (waits for it)."""
        self.next_host.copy_(self.next_tokens, non_blocking=True)
        if self._stream is None:
            self._stream = torch.cuda.current_stream()
        self._stream.synchronize()
        return self.next_host.tolist()


_SESSIONS_KEPT = 6


def session_for(model, cache, params: SamplingParams, n: int, pipelined: bool = True) -> DecodeSession:
    """A session of ``n`` sequences for this model, cache and sampling rule; the
    last few are kept so that batch after batch replays the same graphs."""
    kept = model.__dict__.setdefault("_decode_sessions", {})
    key = (id(cache), n, params, pipelined)
    session = kept.pop(key, None)
    if session is None or session.cache is not cache:
        session = DecodeSession(model, cache, [0] * n, params, [0] * n, kv_bound=model.max_positions,
                                pipelined=pipelined)
    kept[key] = session                                  # most recently used last
    while len(kept) > _SESSIONS_KEPT:
        kept.pop(next(iter(kept)))
    return session
