"""The decoder and its one step function.

``DecoderModel.step(cache, entries)`` runs exactly the tokens it is given: for
each sequence the next tokens after what its cache slot already holds (a whole
prompt, a part of one, or a single token), all sequences of the call as one
batch, and returns the logits at the wanted places.  Per sequence this is the
reference's ``forward(ids, count, startPos, cache, logits)``
(include/ai/LocalModel.hpp:3648-3802); the batch over slots is this library's.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import SequenceCache
from ..config import load_config
from ..weights.loader import load_weights
from .assemble import assemble, collect_tensor_specs
from .batch import PinnedRing, StepEntry, build_context
from .runtime import Runtime


class DecoderModel:
    def __init__(self, plan, tensors, runtime: Runtime, config=None):
        self.plan = plan
        self.config = config
        self.runtime = runtime
        self.assembly = assemble(plan)
        for part in self.assembly.parts():
            part.bind(tensors, runtime)
        if hasattr(self.assembly.head, "attach_embedding"):
            self.assembly.head.attach_embedding(self.assembly.embedding)
        self.vocab_size = plan.vocab_size
        self.max_positions = plan.max_positions
        self.stop_ids = tuple(plan.stop_ids)
        self._ring = PinnedRing()
        self._workspace: dict = {}
        self.weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in self.assembly.parts())

    # ---------------------------------------------------------------- loading
    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", device="cuda:0") -> "DecoderModel":
        """Loads config.json and the weights of a model folder; the class of
        model is chosen by config.json through the registry."""
        runtime = Runtime.create(dtype, device)
        if runtime.device.type != "cuda":
            raise RuntimeError("math_utils_b200 runs on a CUDA device only; there is no CPU path")
        runtime.ops.library()                       # fail now, loudly, if the kernels are missing
        arch, config, plan = load_config(model_dir)
        assembly = assemble(plan)
        specs = collect_tensor_specs(plan, assembly)
        tensors = load_weights(model_dir, specs, runtime.dtype, runtime.device,
                               ignored=plan.ignored_tensors, prefixes=arch.name_prefixes)
        return cls(plan, tensors, runtime, config)

    # ------------------------------------------------------------------ cache
    def cache_specs(self) -> List[Optional[object]]:
        """Per schedule entry: the cache spec of its mixer if the entry owns a
        cache, else None."""
        out = []
        for i, entry in enumerate(self.plan.schedule):
            mixer = self.assembly.layers[entry.layer].mixer
            out.append(mixer.cache_spec() if entry.cache_of == i else None)
        return out

    def new_cache(self, max_tokens: int, n_slots: Optional[int] = None) -> SequenceCache:
        return SequenceCache(self.cache_specs(), max_tokens, self.max_positions, self.runtime.dtype,
                             self.runtime.device, n_slots=n_slots)

    # ------------------------------------------------------------------- step
    def step(self, cache: SequenceCache, entries: Sequence[StepEntry], trace=None) -> Optional[torch.Tensor]:
        """Runs the given tokens; returns float32 logits [wanted, vocab] in the
        order of the entries and of their ``want`` lists, or None if nothing is
        wanted.

        ``trace``: for finding the stage at which a result goes wrong.  A dict
        (filled with name -> float32 host array) or a callable ``(name, tensor)``
        that is told every named intermediate result of the step, all tokens of
        the step as rows: ``embed``, per layer run ``h.N.ln1``, ``h.N.qkv``,
        ``h.N.attn`` (heads merged, before the output projection), ``h.N.res1``,
        ``h.N.ln2``, ``h.N.act`` (the feed-forward's hidden row after the
        activation), ``h.N.res2``, then ``lnf`` and ``logits`` (wanted rows
        only).  The names are those of the reference's ``LocalTrace``
        (include/ai/LocalModel.hpp:1213-1224, filled at 3699-3801) where it has
        them."""
        if isinstance(trace, dict):
            sink = trace

            def trace(name, tensor, sink=sink):
                sink[name] = tensor.detach().float().cpu().numpy().copy()
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        if len({e.slot for e in entries}) != len(entries):
            raise ValueError("a slot appears twice in one step")
        # the tokens once as arrays: checked here, packed for the device by build_context
        tokens = [np.asarray(e.tokens, dtype=np.int64) for e in entries]
        if any(ids.ndim != 1 for ids in tokens):
            raise ValueError("the tokens of an entry are a flat list of ids")
        every = tokens[0] if len(tokens) == 1 else np.concatenate(tokens)
        if int(every.min()) < 0 or int(every.max()) >= self.vocab_size:
            bad = every[(every < 0) | (every >= self.vocab_size)]
            raise ValueError(f"token id {int(bad[0])} is outside the vocabulary of {self.vocab_size}")
        for e, ids in zip(entries, tokens):
            for w in e.want:
                if not 0 <= w < ids.shape[0]:
                    raise ValueError(f"want index {w} is outside the {ids.shape[0]} tokens given for slot {e.slot}")
        starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
        ctx = build_context(self.runtime, self.assembly.position, cache, entries, starts,
                            self._ring, self._workspace, trace, tokens)
        logits = self.forward(ctx, cache)
        for e in entries:
            cache.commit(e.slot, len(e.tokens))
        return logits

    def forward(self, ctx, cache: SequenceCache) -> Optional[torch.Tensor]:
        a = self.assembly
        x = a.embedding.forward(ctx, a.position.embedding_table())
        ctx.note("embed", x)
        for i, entry in enumerate(self.plan.schedule):
            layer = a.layers[entry.layer]
            ctx.tag = f"h.{i}."
            layer.arrangement.forward(x, layer, ctx, cache.entry(entry.cache_of), entry.cache_of == i)
        ctx.tag = ""
        if ctx.want_rows is None:
            return None
        lazy = getattr(a.head, "takes_lazy_norm", False)
        h = a.final_norm.lazy(x, rows=ctx.want_rows) if lazy else a.final_norm.forward(x, rows=ctx.want_rows)
        ctx.note("lnf", h)
        logits = a.head.forward(h)
        ctx.note("logits", logits)
        return logits
