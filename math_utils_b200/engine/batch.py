"""One step's batch: which tokens of which sequences run, flattened for the kernels.

Sequences lie one after another in a flat token list.  For token ``t``:
``token_ids[t]``, its absolute position ``tok_pos[t]`` in its sequence, and
``tok_seq[t]``, the index of its sequence within this step.  For each
key/value group, ``block_tables[g][s]`` lists the cache pages of sequence
``s``.  ``want_rows`` are the flat indices of the tokens whose logits are asked
for.  Everything is packed in one int32 buffer that goes to the device in one
copy from pinned memory.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


TILE_QUERIES = 64


@dataclass
class StepEntry:
    """``tokens``: the next tokens of the sequence in ``slot``; ``want``:
    indices into ``tokens`` whose logits are returned (may be empty)."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class PinnedRing:
    """A few pinned host buffers used in turn, so that filling the next step's
    buffer never overwrites one whose copy to the device is still in flight."""

    def __init__(self, depth: int = 4):
        self.depth = depth
        self.buffers: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.turn = 0

    def next(self, n_ints: int) -> torch.Tensor:
        i = self.turn
        self.turn = (self.turn + 1) % self.depth
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.buffers[i]
        if buf is None or buf.numel() < n_ints:
            buf = torch.empty(max(n_ints, 1024), dtype=torch.int32, pin_memory=True)
            self.buffers[i] = buf
        self._last = i
        return buf

    def mark(self) -> None:
        ev = self.events[self._last] or torch.cuda.Event()
        ev.record()
        self.events[self._last] = ev


@dataclass
class StepContext:
    runtime: object
    position: object                      # the model's position-encoding part
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor
    tok_pos: torch.Tensor
    tok_seq: torch.Tensor
    want_rows: Optional[torch.Tensor]
    block_tables: List[torch.Tensor]
    seq_slots: torch.Tensor               # [n_seqs] int32, for parts that keep per-slot state
    slots: List[int]
    starts: List[int]                     # each sequence's length before this step
    q_lens: List[int]
    max_q_len: int
    max_kv_len: int                       # longest sequence after this step
    workspace: dict = field(default_factory=dict)
    q_tiles: Optional[torch.Tensor] = None  # [n, 2] int32: (first flat token, count <= 64) of each query tile
    q_tiles_wide: Optional[torch.Tensor] = None  # the same in tiles of up to 128 queries
    trace: Optional[object] = None          # callable(name, tensor): told every named intermediate result
    tag: str = ""                           # prefix of the names noted now ("h.3." inside layer run 3)

    def note(self, name: str, tensor) -> None:
        """Hands an intermediate result to the step's trace, if there is one.  A
        ``NormedInput`` is computed for the trace; the product that takes it still
        makes its own."""
        if self.trace is not None:
            if hasattr(tensor, "materialize"):
                # (a trace that only keeps time does not look at values: nothing is computed for it)
                tensor = tensor.materialize_copy() if getattr(self.trace, "wants_values", True) else None
            self.trace(self.tag + name, tensor)

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1

    def buffer(self, name: str, shape, dtype, columns=None):
        """An activation buffer of this shape that lives from step to step and is
        shared by every layer that asks under the same name: layers run one after
        another on one stream, so a layer's intermediate results are dead when the
        next layer writes them.  Only the last shape asked for is kept.  With
        ``columns`` (widths that add up to the row) the buffer comes with its
        column blocks as views, made once: ``(buffer, block, block, ...)``."""
        key = ("buffer", name, dtype, columns)
        held = self.workspace.get(key)
        if held is not None and held[0] == shape:
            return held[1]
        numel = 1
        for n in shape:
            numel *= n
        view = self.scratch(name, numel, dtype)[:numel].view(shape)
        if columns is not None:
            edges = [0]
            for w in columns:
                edges.append(edges[-1] + w)
            view = (view,) + tuple(view[:, a:b] for a, b in zip(edges, edges[1:]))
        self.workspace[key] = (shape, view)
        return view

    def scratch(self, name: str, numel: int, dtype=torch.float32) -> torch.Tensor:
        """A reusable device buffer of at least ``numel`` elements."""
        key = (name, dtype)
        buf = self.workspace.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(max(numel, 1), dtype=dtype, device=self.runtime.device)
            self.workspace[key] = buf
        return buf

    def decode_pages(self, page_tokens: int) -> int:
        """Pages per sequence that a single-token step has to cover at most."""
        return max(1, -(-self.max_kv_len // page_tokens))

    def attention_splits(self, n_heads: int, head_dim: int):
        """How single-token steps split each head's keys over warps: enough
        splits to fill the GPU, each of at least 64 keys."""
        if not self.is_decode:
            return 1, 0, None, None
        items = self.n_tokens * n_heads
        by_fill = -(-(8 * self.runtime.ops.sm_count(self.runtime.device)) // items)      # eight warps per SM
        by_keys = max(1, -(-self.max_kv_len // 64))
        n_splits = max(1, min(by_fill, by_keys))
        if n_splits == 1:
            return 1, 0, None, None
        split_keys = -(-self.max_kv_len // n_splits)
        split_keys = -(-split_keys // 32) * 32
        n_splits = -(-self.max_kv_len // split_keys)
        part_o = self.scratch("attn_part_o", items * n_splits * head_dim)
        part_ml = self.scratch("attn_part_ml", items * n_splits * 2)
        return n_splits, split_keys, part_o, part_ml


def build_context(runtime, position, cache, entries: Sequence[StepEntry], starts: Sequence[int],
                  ring: PinnedRing, workspace: dict, trace=None, tokens=None) -> StepContext:
    """Packs the step's index arrays and sends them to the device.  ``tokens``: the entries' tokens as
    integer arrays, if the caller has them already.  Everything here is array arithmetic over the step's
    sequences: the device waits while it runs."""
    if tokens is None:
        tokens = [np.asarray(e.tokens, dtype=np.int64) for e in entries]
    n_seqs = len(entries)
    q_lens = [int(t.shape[0]) for t in tokens]
    lens = np.asarray(q_lens, dtype=np.int64)
    first = np.asarray(starts, dtype=np.int64)                 # each sequence's length before this step
    flat0 = np.cumsum(lens) - lens                             # where each sequence begins in the flat token list
    n_tokens = sum(q_lens)
    slots = [e.slot for e in entries]
    tables = [cache.block_table_rows(g.index, slots) for g in cache.kv_groups]
    want = []
    for s, e in enumerate(entries):
        if len(e.want):
            base, n = int(flat0[s]), q_lens[s]
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"want index {w} is outside the {n} tokens given for slot {e.slot}")
                want.append(base + w)
    n_want = len(want)

    def cut(width):
        """Query tiles of `width` tokens, none across two sequences, those with the most keys first
        (the attention kernels' blocks take them in this order): (first flat token, count) each."""
        found = []
        for base, n, start in zip(flat0.tolist(), q_lens, starts):
            found += [(start + min(o + width, n), base + o, min(width, n - o)) for o in range(0, n, width)]
        found.sort(key=lambda tile: -tile[0])                  # stable: equal ends keep their order
        return np.asarray([tile[1:] for tile in found], dtype=np.int32)

    max_q_len = max(q_lens)
    tiles = wide = None                   # query tiles for the prompt attention kernels
    if max_q_len > 1:
        tiles, wide = cut(TILE_QUERIES), cut(2 * TILE_QUERIES)
    n_tiles, n_wide = (len(tiles), len(wide)) if tiles is not None else (0, 0)
    sizes = [n_tokens, n_tokens, n_tokens, n_want, n_seqs, 2 * n_tiles, 2 * n_wide] + [t.size for t in tables]
    offsets = [0]
    for size in sizes:
        offsets.append(offsets[-1] + -(-size // 4) * 4)       # 16-byte aligned parts
    total = offsets[-1]
    host = ring.next(total)
    h = host.numpy()
    seq_of = np.repeat(np.arange(n_seqs), lens)
    h[offsets[0]: offsets[0] + n_tokens] = tokens[0] if n_seqs == 1 else np.concatenate(tokens)
    h[offsets[1]: offsets[1] + n_tokens] = np.arange(n_tokens) + (first - flat0)[seq_of]
    h[offsets[2]: offsets[2] + n_tokens] = seq_of
    if n_want:
        h[offsets[3]: offsets[3] + n_want] = want
    h[offsets[4]: offsets[4] + n_seqs] = slots
    if n_tiles:
        h[offsets[5]: offsets[5] + 2 * n_tiles] = tiles.reshape(-1)
        h[offsets[6]: offsets[6] + 2 * n_wide] = wide.reshape(-1)
    for i, t in enumerate(tables):
        h[offsets[7 + i]: offsets[7 + i] + t.size] = t.reshape(-1)
    dev = torch.empty(total, dtype=torch.int32, device=runtime.device)
    dev.copy_(host[:total], non_blocking=True)
    ring.mark()

    def part(i, n):
        return dev[int(offsets[i]): int(offsets[i]) + n]

    return StepContext(
        runtime=runtime, position=position, n_tokens=n_tokens, n_seqs=n_seqs,
        token_ids=part(0, n_tokens), tok_pos=part(1, n_tokens), tok_seq=part(2, n_tokens),
        want_rows=part(3, n_want) if n_want else None,
        block_tables=[part(7 + i, t.size).view(t.shape) for i, t in enumerate(tables)],
        seq_slots=part(4, n_seqs),
        q_tiles=part(5, 2 * n_tiles).view(n_tiles, 2) if n_tiles else None,
        q_tiles_wide=part(6, 2 * n_wide).view(n_wide, 2) if n_wide else None,
        slots=slots, starts=list(starts), q_lens=q_lens,
        max_q_len=max_q_len, max_kv_len=max(s + n for s, n in zip(starts, q_lens)),
        workspace=workspace, trace=trace)
