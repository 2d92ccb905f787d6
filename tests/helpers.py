"""Helpers shared by the GPU tests: running the engine in the three ways of
cutting the work, and the error bounds."""
import numpy as np

from math_utils_b200 import StepEntry

# float32 path: absolute bound on logits of order 1 against the float64 plain implementation.
FP32_ABS = 1e-4
# bfloat16 path: bound relative to the spread of the logits of the row.  Weights, activations
# and cache are rounded to 8 bits of mantissa (2^-9 relative per rounding); through a few
# layers that leaves errors of a few percent of a logit's spread, never more.
BF16_REL = 0.04


OBSERVED = {"float32": (0.0, ""), "bfloat16": (0.0, "")}    # the largest error seen so far, as a fraction of its bound


def check_logits(got, want, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - want).max(axis=-1)
    if dtype == "float32":
        bad = err > FP32_ABS
        bound = FP32_ABS
        used = float(err.max() / FP32_ABS) if err.size else 0.0
    else:
        spread = want.std(axis=-1)
        bad = err > BF16_REL * np.maximum(spread, 1e-3)
        bound = f"{BF16_REL} x row spread"
        used = float((err / (BF16_REL * np.maximum(spread, 1e-3))).max()) if err.size else 0.0
    if used > OBSERVED[dtype][0]:
        OBSERVED[dtype] = (used, what)
    assert not bad.any(), (f"{what}: first wrong row {int(np.argmax(bad))} of {len(err)}, "
                           f"max |diff| {err.max():.3e} (bound {bound})")


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
