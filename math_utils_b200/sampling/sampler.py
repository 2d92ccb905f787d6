"""Greedy and temperature / top-k sampling, on the device.

The rule is the reference's ``sampleTopK`` (include/ai/LocalModel.hpp:3809-3841):
``temperature <= 0`` or ``top_k`` of 0 or 1 is greedy (first maximum wins);
otherwise the ``top_k`` largest logits are kept, softmax at the temperature, and
one uniform draw walks them in descending order.  A negative ``top_k`` keeps the
whole vocabulary (the reference's count is unsigned and has no such value).  Each
request has its own stream of draws keyed by (seed, request index), so a
request's tokens do not depend on which batch it ran in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7          # include/ai/LLM.hpp:76; src/LLM.cpp:222
    top_k: int = 40                   # include/ai/LLM.hpp:77 (the CLI's default is 20, src/LLM.cpp:223)
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or 0 <= self.top_k <= 1

    @property
    def kept(self) -> int:
        """The count the kernel is given: how many of the largest logits stay, 0 for all of them."""
        return max(self.top_k, 0)


class Sampler:
    """Samples one token per row of logits for a fixed set of requests."""

    def __init__(self, params: SamplingParams, request_ids: Sequence[int], device, ops):
        self.params = params
        self.ops = ops
        self.device = device
        self.request_ids = torch.tensor(list(request_ids), dtype=torch.int64, device=device)
        self.draws = torch.zeros(len(request_ids), dtype=torch.int32, device=device)

    def sample(self, logits: torch.Tensor, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
        """``logits`` [n, vocab] float32 for the requests ``rows`` (indices into
        this sampler's requests; all of them if None) -> int32 tokens [n]."""
        if self.params.greedy:
            return self.ops.argmax(logits)
        if rows is None:
            return self.ops.sample(logits, self.params.temperature, self.params.kept, self.params.seed,
                                   self.request_ids, self.draws)
        index = torch.tensor(list(rows), dtype=torch.int64, device=self.device)
        draws = self.draws[index].contiguous()
        out = self.ops.sample(logits, self.params.temperature, self.params.kept, self.params.seed,
                              self.request_ids[index].contiguous(), draws)
        self.draws[index] = draws
        return out
