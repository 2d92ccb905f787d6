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
    integer arrays, if the caller has them already."""
    q_lens = [len(e.tokens) for e in entries]
    n_tokens, n_seqs = sum(q_lens), len(entries)
    n_want = sum(len(e.want) for e in entries)
    tables = [cache.block_table_rows(g.index, [e.slot for e in entries]) for g in cache.kv_groups]
    def cut(width):
        """Query tiles of `width` tokens, none across two sequences, those with the most keys first
        (the attention kernels' blocks take them in this order)."""
        found, ends, flat = [], [], 0
        for n, start in zip(q_lens, starts):
            for o in range(0, n, width):
                found.append((flat + o, min(width, n - o)))
                ends.append(start + o + found[-1][1])
            flat += n
        return [found[i] for i in sorted(range(len(found)), key=lambda i: -ends[i])]

    tiles, wide = [], []                  # query tiles for the prompt attention kernels
    if max(q_lens) > 1:
        tiles, wide = cut(TILE_QUERIES), cut(2 * TILE_QUERIES)
    sizes = [n_tokens, n_tokens, n_tokens, n_want, n_seqs, 2 * len(tiles), 2 * len(wide)] + [t.size for t in tables]
    offsets = np.concatenate([[0], np.cumsum([-(-s // 4) * 4 for s in sizes])])   # 16-byte aligned parts
    total = int(offsets[-1])
    host = ring.next(total)
    h = host.numpy()
    o = 0
    flat = 0
    for s, e in enumerate(entries):
        n = q_lens[s]
        h[offsets[0] + flat: offsets[0] + flat + n] = tokens[s] if tokens is not None else np.asarray(e.tokens, dtype=np.int32)
        h[offsets[1] + flat: offsets[1] + flat + n] = np.arange(starts[s], starts[s] + n, dtype=np.int32)
        h[offsets[2] + flat: offsets[2] + flat + n] = s
        for w in e.want:
            if not 0 <= w < n:
                raise ValueError(f"want index {w} is outside the {n} tokens given for slot {e.slot}")
            h[offsets[3] + o] = flat + w
            o += 1
        flat += n
    h[offsets[4]: offsets[4] + n_seqs] = np.asarray([e.slot for e in entries], dtype=np.int32)
    if tiles:
        h[offsets[5]: offsets[5] + 2 * len(tiles)] = np.asarray(tiles, dtype=np.int32).reshape(-1)
        h[offsets[6]: offsets[6] + 2 * len(wide)] = np.asarray(wide, dtype=np.int32).reshape(-1)
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
        q_tiles=part(5, 2 * len(tiles)).view(len(tiles), 2) if tiles else None,
        q_tiles_wide=part(6, 2 * len(wide)).view(len(wide), 2) if wide else None,
        slots=[e.slot for e in entries], starts=list(starts), q_lens=q_lens,
        max_q_len=max(q_lens), max_kv_len=max(s + n for s, n in zip(starts, q_lens)),
        workspace=workspace, trace=trace)
