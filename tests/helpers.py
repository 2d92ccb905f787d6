"""Helpers shared by the GPU tests: running the engine in the three ways of
cutting the work, and the error bounds."""
import numpy as np

from math_utils_b200 import StepEntry

# float32 path: absolute bound on logits of order 1 against the float64 plain implementation.
FP32_ABS = 1e-4
# bfloat16 path: weights, activations between kernels and the cache are rounded to 8 bits of
# mantissa (2^-9 relative per rounding), accumulation is float32.  A logit is a sum over the width of
# such products, so its error behaves like noise of some fraction of the row's spread, the same in
# every column; two bounds follow.  The rms of a row's errors must stay below BF16_RMS of the row's
# spread.  The largest error of a row of V such errors lies near sqrt(2 ln V) of their rms (4.7 for
# GPT-2's vocabulary, 3.5 for 512 columns), so it is bounded by that multiple of the rms bound; a
# single wrong column or row stands out far above it.
BF16_RMS = 0.012


def bf16_max_bound(vocab):
    return BF16_RMS * float(np.sqrt(2.0 * np.log(max(vocab, 2))))


# Greedy tokens in bfloat16: where the engine's token is not the plain model's, the plain logits of the
# two must be closer than the noise can bridge.  The difference of two logits' errors has sqrt(2) times
# the rms of one; four of those is a gap that noise crosses less than once in ten thousand draws.
BF16_NEAR_TIE = 4.0 * float(np.sqrt(2.0)) * BF16_RMS


OBSERVED = {"float32": (0.0, ""), "bfloat16 rms": (0.0, ""), "bfloat16 max": (0.0, "")}    # largest error seen, as a fraction of its bound


def _note(kind, used, what):
    if used > OBSERVED[kind][0]:
        OBSERVED[kind] = (used, what)


def check_logits(got, want, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    diff = np.abs(got - want)
    err = diff.max(axis=-1)
    if err.size == 0:
        return
    if dtype == "float32":
        _note("float32", float(err.max() / FP32_ABS), what)
        bad = err > FP32_ABS
        assert not bad.any(), (f"{what}: first wrong row {int(np.argmax(bad))} of {len(err)}, "
                               f"max |diff| {err.max():.3e} (bound {FP32_ABS})")
        return
    spread = np.maximum(want.std(axis=-1), 1e-3)
    rms = np.sqrt((diff ** 2).mean(axis=-1))
    top = bf16_max_bound(want.shape[-1])
    _note("bfloat16 rms", float((rms / (BF16_RMS * spread)).max()), what)
    _note("bfloat16 max", float((err / (top * spread)).max()), what)
    bad = (rms > BF16_RMS * spread) | (err > top * spread)
    assert not bad.any(), (f"{what}: first wrong row {int(np.argmax(bad))} of {len(err)}: rms error "
                           f"{(rms / spread)[np.argmax(bad)]:.4f} of the row's spread (bound {BF16_RMS}), largest "
                           f"{(err / spread)[np.argmax(bad)]:.4f} (bound {top:.4f})")


def run_whole(model, cache, tokens):
    """One request alone, all its tokens in one step, logits everywhere."""
    slot = cache.acquire()
    try:
        out = model.step(cache, [StepEntry(slot, tokens, list(range(len(tokens))))])
        return out.float().cpu().numpy()
    finally:
        cache.release(slot)


def run_tail_one_by_one(model, cache, tokens, tail=32):
    """The prefix in one step, then the last `tail` tokens one at a time."""
    n = len(tokens)
    tail = min(tail, n - 1)
    slot = cache.acquire()
    try:
        head = n - tail
        rows = [model.step(cache, [StepEntry(slot, tokens[:head], list(range(head)))]).float().cpu().numpy()]
        for t in range(head, n):
            rows.append(model.step(cache, [StepEntry(slot, [tokens[t]], [0])]).float().cpu().numpy())
        return np.concatenate(rows, axis=0)
    finally:
        cache.release(slot)


def run_batch(model, cache, requests, prompt_lens):
    """Requests start together: prompts (unequal) in one step, then one token
    each per step; a request leaves when its tokens run out.  Returns the
    logits of every position of every request."""
    slots = [cache.acquire() for _ in requests]
    got = [[] for _ in requests]
    try:
        entries = [StepEntry(s, r[:p], list(range(p))) for s, r, p in zip(slots, requests, prompt_lens)]
        out = model.step(cache, entries).float().cpu().numpy()
        o = 0
        for i, p in enumerate(prompt_lens):
            got[i].append(out[o:o + p])
            o += p
        pos = list(prompt_lens)
        live = [i for i, r in enumerate(requests) if pos[i] < len(r)]
        for i in range(len(requests)):
            if i not in live:
                cache.release(slots[i]); slots[i] = None
        while live:
            entries = [StepEntry(slots[i], [requests[i][pos[i]]], [0]) for i in live]
            out = model.step(cache, entries).float().cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
            still = []
            for i in live:
                if pos[i] < len(requests[i]):
                    still.append(i)
                else:
                    cache.release(slots[i]); slots[i] = None
            live = still
        return [np.concatenate(g, axis=0) for g in got]
    finally:
        for s in slots:
            if s is not None:
                cache.release(s)
