"""How a step is packed for the device: flat tokens, positions, the sequence of each token, wanted rows, query
tiles and page lists.  No device is needed: the arrays are made on the host and the copy goes to a CPU tensor."""
import numpy as np
import pytest
import torch

from math_utils_b200.cache.sequence_cache import SequenceCache
from math_utils_b200.engine.batch import StepEntry, build_context
from math_utils_b200.parts.base import KVCacheSpec


class HostRing:
    """Stands in for the pinned ring: one plain host buffer."""

    def __init__(self):
        self.buffer = torch.zeros(1 << 14, dtype=torch.int32)

    def next(self, n_ints):
        self.buffer.zero_()
        return self.buffer

    def mark(self):
        pass


class HostRuntime:
    device = torch.device("cpu")


def pack(cache, entries):
    starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
    ctx = build_context(HostRuntime, None, cache, entries, starts, HostRing(), {}, None, None)
    for e in entries:
        cache.commit(e.slot, len(e.tokens))
    return ctx


@pytest.fixture
def cache():
    specs = [KVCacheSpec(2, 16, 0), KVCacheSpec(2, 16, 0)]              # two layers, one group
    return SequenceCache(specs, 64 * 12, 640, torch.float32, torch.device("cpu"), n_slots=3)


def test_prompts_of_unequal_lengths_then_single_tokens(cache):
    a, b, c = cache.acquire(), cache.acquire(), cache.acquire()
    ctx = pack(cache, [StepEntry(a, [7, 8, 9], [0, 2]), StepEntry(b, list(range(100, 230)), [129]), StepEntry(c, [5], [])])
    assert (ctx.n_tokens, ctx.n_seqs, ctx.max_q_len, ctx.max_kv_len) == (134, 3, 130, 130)
    assert ctx.q_lens == [3, 130, 1] and ctx.starts == [0, 0, 0] and ctx.slots == [a, b, c]
    assert ctx.token_ids.tolist() == [7, 8, 9] + list(range(100, 230)) + [5]
    assert ctx.tok_pos.tolist() == [0, 1, 2] + list(range(130)) + [0]
    assert ctx.tok_seq.tolist() == [0] * 3 + [1] * 130 + [2]
    assert ctx.want_rows.tolist() == [0, 2, 3 + 129]                       # flat rows, in the order asked for
    assert ctx.seq_slots.tolist() == [a, b, c]
    # tiles of 64 queries: (first flat token, count), the one that ends furthest into its sequence first
    assert ctx.q_tiles.tolist() == [[3 + 128, 2], [3 + 64, 64], [3, 64], [0, 3], [133, 1]]
    assert ctx.q_tiles_wide.tolist() == [[3 + 128, 2], [3, 128], [0, 3], [133, 1]]
    table = ctx.block_tables[0]
    held = [int(table[0, 0]), int(table[2, 0])] + table[1, :3].tolist()  # one page, one page, three pages
    assert table.shape[0] == 3 and len(set(held)) == 5 and all(0 <= p < cache.n_pages for p in held)
    assert not ctx.is_decode

    # then one token each: positions go on from each sequence's own length
    ctx = pack(cache, [StepEntry(b, [1], [0]), StepEntry(a, [2], [0])])
    assert ctx.is_decode and ctx.q_tiles is None and ctx.q_tiles_wide is None
    assert ctx.tok_pos.tolist() == [130, 3] and ctx.tok_seq.tolist() == [0, 1] and ctx.starts == [130, 3]
    assert ctx.want_rows.tolist() == [0, 1] and ctx.max_kv_len == 131
    assert ctx.block_tables[0][0, :3].tolist() == table[1, :3].tolist()     # the same pages, now listed for row 0


def test_a_prompt_continued_at_an_odd_offset(cache):
    a = cache.acquire()
    pack(cache, [StepEntry(a, list(range(70)))])
    ctx = pack(cache, [StepEntry(a, list(range(70, 150)), [79])])
    assert ctx.want_rows.tolist() == [79] and ctx.tok_pos.tolist() == list(range(70, 150)) and ctx.max_kv_len == 150
    assert ctx.q_tiles.tolist() == [[64, 16], [0, 64]] and ctx.q_tiles_wide.tolist() == [[0, 80]]
    ctx = pack(cache, [StepEntry(a, [3])])
    assert ctx.want_rows is None and ctx.tok_pos.tolist() == [150]


def test_a_wanted_place_outside_the_tokens_is_refused(cache):
    a = cache.acquire()
    with pytest.raises(ValueError, match="want index 2"):
        pack(cache, [StepEntry(a, [1, 2], [2])])
