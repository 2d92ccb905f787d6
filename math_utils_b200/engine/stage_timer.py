"""Per-stage device times of eager steps, for the command line's ``--profile``.

A ``StageTimer`` is handed to ``DecoderModel.step`` as its ``trace``: the step
tells it every named stage as the stage's launches have been issued, and it
records a CUDA event there.  The time between two events is charged to the
later stage's kind (``h.3.qkv`` -> ``qkv``), prompt steps and single-token
steps apart, as the reference's ``LocalProfile`` keeps its stages
(include/ai/LocalModel.hpp:1427-1506; printed by src/LLM.cpp:721-730).
"""
from __future__ import annotations

from collections import OrderedDict

import torch

# what the time up to each note is spent on
STAGE_NAMES = OrderedDict([
    ("embed", "embedding"), ("ln1", "norm 1"), ("qkv", "q | k | v product"), ("attn", "attention"),
    ("res1", "output projection"), ("ln2", "norm 2"), ("act", "feed-forward up"), ("res2", "feed-forward down"),
    ("lnf", "final norm"), ("logits", "output head"),
])


class StageTimer:
    wants_values = False            # the step need not compute anything for this trace's sake

    def __init__(self):
        self.steps = []             # (is_prompt, [(stage kind, event)])
        self._current = None

    def begin(self, is_prompt: bool) -> None:
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        self._current = [("", start)]
        self.steps.append((is_prompt, self._current))

    def __call__(self, name: str, tensor) -> None:
        if self._current is None:
            return
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        self._current.append((name.rsplit(".", 1)[-1], event))

    def totals(self):
        """{stage kind: [seconds in prompt steps, seconds in single-token steps]} (synchronises)."""
        torch.cuda.synchronize()
        out = OrderedDict((k, [0.0, 0.0]) for k in STAGE_NAMES)
        for is_prompt, marks in self.steps:
            for (_, before), (kind, after) in zip(marks, marks[1:]):
                out.setdefault(kind, [0.0, 0.0])[0 if is_prompt else 1] += before.elapsed_time(after) / 1e3
        return out
