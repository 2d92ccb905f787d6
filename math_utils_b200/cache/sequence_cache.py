"""The cache: a slot per live sequence, paged keys and values, fixed-size state.

What a sequence holds between steps is kept per *slot*.  A slot is taken when
a request starts and given back when it ends; a later request takes it again.
The reference keeps one ``LocalCache`` per conversation with ``keys[l]`` /
``values[l]`` per layer plus fixed-size ``recurrent[l]`` / ``convWindow[l]``
for mixers with state (include/ai/LocalModel.hpp:1231-1334); here the same
content lives in slots of one arena, so that a batch of sequences can step
together.

Layers are grouped by what their mixer keeps (its ``cache_spec``):
  * a ``KVGroup`` for each distinct (kv heads, head size, window): a pool of
    pages of ``page_tokens`` positions, one page tensor per cache entry (layer
    run), and for each slot the list of pages it holds.  All entries of a group
    share the slot's page list, so a page index means the same positions in
    every layer of the group.  A group with a window gives pages back once no
    later query can see them.
  * a ``StateGroup`` for each distinct state size: ``[n_slots, n_values]``
    float32 per cache entry, zeroed when a slot is taken.

Bookkeeping is host-side and plain Python; storage is torch tensors on the
device given (a CUDA device in the engine, the CPU in bookkeeping tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import KVCacheSpec, StateCacheSpec

PAGE_TOKENS = 64


class CacheError(RuntimeError):
    """Misuse of the cache: an unknown or freed slot, a double free."""


class CacheFull(CacheError):
    """No free slot or page is left for what was asked."""


class SlotAllocator:
    """Hands out slot numbers; a slot is free or held, never both, never twice."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = set()

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} cache slots are held")
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"slot {slot} is not held (freed twice, or never taken)")
        self._held.remove(slot)
        self._free.append(slot)

    def is_held(self, slot: int) -> bool:
        return slot in self._held

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> frozenset:
        return frozenset(self._held)


class PagePool:
    """Free list of page numbers of one group."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = set()

    def take(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} more cache pages are needed, {len(self._free)} of {self.n_pages} are free")
        pages = [self._free.pop() for _ in range(count)]
        self._held.update(pages)
        return pages

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if p not in self._held:
                raise CacheError(f"page {p} is not held (given back twice)")
            self._held.remove(p)
            self._free.append(p)

    @property
    def n_free(self) -> int:
        return len(self._free)


@dataclass
class KVEntryView:
    """What a mixer with a key/value cache gets for one run of its layer."""
    pages: torch.Tensor            # [n_pages, 2, n_kv_heads, page_tokens, head_dim]
    page_tokens: int
    spec: KVCacheSpec
    group: int                     # index into StepContext.block_tables


@dataclass
class StateEntryView:
    """What a mixer with fixed-size state gets: ``values[slot]`` is its state."""
    values: torch.Tensor           # [n_slots, n_values] float32
    spec: StateCacheSpec


class KVGroup:
    def __init__(self, index: int, spec: KVCacheSpec, entries: Sequence[int], n_pages: int, n_slots: int,
                 max_positions: int, page_tokens: int, dtype: torch.dtype, device):
        self.index = index
        self.spec = spec
        self.entries = list(entries)
        self.page_tokens = page_tokens
        self.max_pages = (max_positions + page_tokens - 1) // page_tokens
        self.pool = PagePool(n_pages)
        self.storage: Dict[int, torch.Tensor] = {
            e: torch.zeros((n_pages, 2, spec.n_kv_heads, page_tokens, spec.head_dim), dtype=dtype, device=device)
            for e in self.entries}
        # page number of each page index of each slot; -1 where none is held
        self.table = np.full((n_slots, self.max_pages), -1, dtype=np.int32)

    def first_needed_page(self, length: int) -> int:
        """Index of the oldest page a query at position >= length - 1 can still see."""
        if self.spec.window <= 0 or length <= self.spec.window:
            return 0
        return (length - self.spec.window) // self.page_tokens

    def reserve(self, slot: int, old_len: int, new_len: int) -> None:
        """Pages for positions up to new_len; with a window, drops pages that
        every query from position old_len on has left behind."""
        row = self.table[slot]
        need_upto = (new_len + self.page_tokens - 1) // self.page_tokens
        missing = [i for i in range(need_upto) if row[i] < 0 and i >= self.first_needed_page(old_len + 1)]
        if missing:
            pages = self.pool.take(len(missing))
            for i, p in zip(missing, pages):
                row[i] = p

    def trim(self, slot: int, length: int) -> None:
        """After a step: pages wholly before the window of the next query go back."""
        if self.spec.window <= 0:
            return
        row = self.table[slot]
        upto = self.first_needed_page(length + 1)
        drop = [int(row[i]) for i in range(min(upto, self.max_pages)) if row[i] >= 0]
        if drop:
            for i in range(min(upto, self.max_pages)):
                row[i] = -1
            self.pool.give_back(drop)

    def release(self, slot: int) -> None:
        row = self.table[slot]
        held = [int(p) for p in row if p >= 0]
        row[:] = -1
        self.pool.give_back(held)

    def pages_held(self, slot: int) -> int:
        return int((self.table[slot] >= 0).sum())


class StateGroup:
    def __init__(self, index: int, spec: StateCacheSpec, entries: Sequence[int], n_slots: int, device):
        self.index = index
        self.spec = spec
        self.entries = list(entries)
        self.storage: Dict[int, torch.Tensor] = {
            e: torch.zeros((n_slots, spec.n_values), dtype=torch.float32, device=device) for e in self.entries}

    def clear(self, slot: int) -> None:
        for t in self.storage.values():
            t[slot].zero_()


class SequenceCache:
    """All groups of one model, the slots, and each slot's length.

    ``entry_specs[i]`` is the cache spec of schedule entry ``i`` if that entry
    owns a cache, else ``None``.  ``max_tokens`` is the most positions that live
    sequences hold at any time, each sequence's count rounded up to whole
    pages; it sizes every key/value group.
    """

    def __init__(self, entry_specs: Sequence[Optional[object]], max_tokens: int, max_positions: int,
                 dtype: torch.dtype, device, page_tokens: int = PAGE_TOKENS, n_slots: Optional[int] = None):
        if max_tokens < 1:
            raise CacheError("max_tokens must be at least 1")
        self.page_tokens = page_tokens
        self.max_positions = max_positions
        self.dtype = dtype
        self.device = device
        self.n_pages = (max_tokens + page_tokens - 1) // page_tokens
        self.n_slots = n_slots if n_slots is not None else self.n_pages
        self.slots = SlotAllocator(self.n_slots)
        self.lengths = np.zeros(self.n_slots, dtype=np.int64)
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._entry_view: Dict[int, object] = {}
        by_spec: Dict[object, List[int]] = {}
        for i, spec in enumerate(entry_specs):
            if spec is not None:
                by_spec.setdefault(spec, []).append(i)
        for spec, entries in by_spec.items():
            if isinstance(spec, KVCacheSpec):
                g = KVGroup(len(self.kv_groups), spec, entries, self.n_pages, self.n_slots, max_positions,
                            page_tokens, dtype, device)
                self.kv_groups.append(g)
                for e in entries:
                    self._entry_view[e] = KVEntryView(g.storage[e], page_tokens, spec, g.index)
            elif isinstance(spec, StateCacheSpec):
                g = StateGroup(len(self.state_groups), spec, entries, self.n_slots, device)
                self.state_groups.append(g)
                for e in entries:
                    self._entry_view[e] = StateEntryView(g.storage[e], spec)
            else:
                raise CacheError(f"schedule entry {entries[0]}: unknown cache spec {spec!r}")

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.lengths[slot] = 0
        for g in self.state_groups:
            g.clear(slot)
        return slot

    def release(self, slot: int) -> None:
        self.slots.release(slot)
        for g in self.kv_groups:
            g.release(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        self._check(slot)
        return int(self.lengths[slot])

    def _check(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held")

    # ------------------------------------------------------------------ steps
    def reserve(self, slot: int, n_new: int) -> int:
        """Makes room for ``n_new`` more positions of the slot's sequence;
        returns the length before.  The length itself moves in ``commit``."""
        self._check(slot)
        old = int(self.lengths[slot])
        new = old + n_new
        if new > self.max_positions:
            raise CacheError(f"slot {slot}: {new} positions exceed the model's {self.max_positions}")
        for g in self.kv_groups:
            g.reserve(slot, old, new)
        return old

    def reserve_one(self, slot: int) -> bool:
        """``reserve(slot, 1)`` for the generation loop, which calls it for every
        sequence at every step: True if a page was taken (the block tables on
        the device are then out of date)."""
        old = int(self.lengths[slot])
        if old >= self.max_positions:
            raise CacheError(f"slot {slot}: {old + 1} positions exceed the model's {self.max_positions}")
        took = False
        for g in self.kv_groups:
            if old % self.page_tokens == 0 and g.table[slot, old // self.page_tokens] < 0:
                g.reserve(slot, old, old + 1)
                took = True
        return took

    def commit(self, slot: int, n_new: int) -> None:
        self.lengths[slot] += n_new
        for g in self.kv_groups:
            g.trim(slot, int(self.lengths[slot]))

    def truncate(self, slot: int, length: int) -> None:
        """Forgets the slot's positions from ``length`` on (a step that ran ahead
        of the news that its sequence had ended).  The pages stay with the slot.
        Not for windowed groups, which have given pages back as the sequence
        moved on, nor for fixed-size state, which cannot be wound back."""
        self._check(slot)
        if not 0 <= length <= int(self.lengths[slot]):
            raise CacheError(f"slot {slot} holds {int(self.lengths[slot])} positions, cannot cut it to {length}")
        if length < int(self.lengths[slot]) and (self.state_groups or any(g.spec.window > 0 for g in self.kv_groups)):
            raise CacheError("a cache with a windowed group or with fixed-size state cannot be cut back")
        self.lengths[slot] = length

    def entry(self, index: int):
        """The view of schedule entry ``index``'s cache, or None if it owns none."""
        return self._entry_view.get(index)

    def block_table_rows(self, group: int, slots: Sequence[int]) -> np.ndarray:
        """[len(slots), max_pages] int32 page numbers (0 where no page is held:
        the kernels never read those positions)."""
        rows = self.kv_groups[group].table[list(slots)]
        return np.maximum(rows, 0)

    def free_pages(self, group: int = 0) -> int:
        return self.kv_groups[group].pool.n_free

    def bytes(self) -> int:
        total = 0
        for g in self.kv_groups:
            total += sum(t.numel() * t.element_size() for t in g.storage.values())
        for g in self.state_groups:
            total += sum(t.numel() * t.element_size() for t in g.storage.values())
        return total
