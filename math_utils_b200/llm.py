"""The front door: load a model folder, ask it for tokens.

Shaped after the reference's ``llm::LLM`` and ``llm::Options``
(include/ai/LLM.hpp:72-93, 131-156, 196-245): ``use`` loads a model,
``prompt`` continues the conversation held in the cache, ``once`` is one
self-contained turn, ``reset`` forgets the conversation.  Where the reference
takes and returns text, this library takes and returns token ids (it has no
tokenizer), and it adds ``generate`` for batches of independent requests.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import List, Optional, Sequence

from .engine.generate import generate as _generate
from .engine.generate import RequestState, run_requests
from .engine.model import DecoderModel
from .sampling import SamplingParams


@dataclass
class Options:
    """Names, meanings and defaults of include/ai/LLM.hpp:72-93."""
    context: int = 4096             # cache positions per sequence, clamped to the model's maximum
    max_tokens: int = 512           # most tokens one answer may have
    temperature: float = 0.7        # <= 0: greedy
    top_k: int = 40                 # 0 or 1: greedy; negative: the whole vocabulary
    seed: int = 0
    stateless: bool = False         # every prompt() starts from an empty cache
    dtype: str = "bfloat16"         # "float32": the true 32-bit path
    max_batch: int = 64             # most sequences that step together in generate()
    profile: bool = False           # prompt() keeps per-stage device times (eager steps; see stage_times)


class LLM:
    def __init__(self, model_dir: Optional[str] = None, options: Optional[Options] = None,
                 device: str = "cuda:0", **overrides):
        self.options = replace(options or Options(), **overrides)
        self.device = device
        self.model: Optional[DecoderModel] = None
        self.current = ""
        self._cache = None
        self._batch_cache = None
        self._slot = None
        self._turns = 0
        self.last: dict = {}            # figures of the last prompt(): tokens in and out, seconds, why it ended
        self.stage_times = None         # with options.profile: {stage: [prompt seconds, decode seconds]} of the last prompt()
        if model_dir is not None:
            self.use(model_dir)

    # ----------------------------------------------------------------- model
    def use(self, model_dir: str, options: Optional[Options] = None) -> "LLM":
        """Loads the model of a folder; the one loaded before is dropped first."""
        self.unload()
        if options is not None:
            self.options = options
        self.model = DecoderModel.from_dir(model_dir, dtype=self.options.dtype, device=self.device)
        self.current = model_dir
        return self

    def unload(self) -> None:
        self.model, self._cache, self._slot, self.current, self._turns = None, None, None, "", 0
        self._batch_cache = None

    @property
    def loaded(self) -> bool:
        return self.model is not None

    @property
    def context(self) -> int:
        return min(self.options.context, self.model.max_positions)

    def _params(self, temperature, top_k, seed) -> SamplingParams:
        o = self.options
        return SamplingParams(o.temperature if temperature is None else temperature,
                              o.top_k if top_k is None else top_k, o.seed if seed is None else seed)

    # ------------------------------------------------------------- one talk
    def reset(self) -> None:
        if self._slot is not None:
            self._cache.release(self._slot)
        self._slot, self._turns = None, 0

    def prompt(self, ids: Sequence[int], max_tokens: Optional[int] = None) -> List[int]:
        """Feeds ``ids`` after what the conversation already holds and returns
        the answer's tokens.  When the context would fill, the conversation is
        forgotten first, as the reference does (include/ai/LLM.hpp:214-221).
        Afterwards the cache holds the prompt and every token of the answer
        (the reference forwards each token it emits, include/ai/LLM.hpp:226-243),
        so the next turn continues from there.  The steps run through the same
        loop as ``generate``: a batch of one on a slot that is kept."""
        self._need_model()
        if not ids:
            raise ValueError("the prompt is empty")
        if self.options.stateless:
            self.reset()
        limit = self.context
        max_tokens = self.options.max_tokens if max_tokens is None else max_tokens
        if self._cache is None:
            self._cache = self.model.new_cache(max_tokens=-(-limit // 64) * 64, n_slots=1)
        held = self._cache.length(self._slot) if self._slot is not None else 0
        if held + len(ids) + 8 >= limit:
            self.reset()
            held = 0
        if len(ids) + 8 >= limit:
            raise ValueError("the prompt alone does not fit in the context")
        if self._slot is None:
            self._slot = self._cache.acquire()
        # the conversation so far counts toward the context rule; the turn keys the sampling stream
        state = RequestState(self._turns, list(ids), held=held)
        self._turns += 1
        timing, timer = {}, None
        if self.options.profile:
            from .engine.stage_timer import StageTimer
            timer = StageTimer()
        try:
            run_requests(self.model, self._cache, self._params(None, None, None), [state],
                         frozenset(self.model.stop_ids), max_tokens, limit, kept_slots=[self._slot],
                         timing=timing, stage_timer=timer)
        except Exception:
            self.reset()               # the cache may hold half a turn
            raise
        self.stage_times = timer.totals() if timer is not None else None
        self.last = {"prompt_tokens": len(ids), "produced": len(state.produced), "reason": state.reason,
                     "context_used": self._cache.length(self._slot), "context": limit,
                     "prompt_s": timing.get("prompt_s", 0.0), "decode_s": timing.get("decode_s", 0.0)}
        return state.produced

    def once(self, ids: Sequence[int], max_tokens: Optional[int] = None) -> List[int]:
        """One self-contained turn: nothing before it is seen, nothing of it is kept."""
        self.reset()
        try:
            return self.prompt(ids, max_tokens)
        finally:
            self.reset()

    # --------------------------------------------------------------- batches
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: Optional[int] = None,
                 temperature: Optional[float] = None, top_k: Optional[int] = None,
                 seed: Optional[int] = None, stop_ids: Optional[Sequence[int]] = None,
                 max_batch: Optional[int] = None) -> List[List[int]]:
        """Independent requests, run as batches of unequal prompts; returns the
        produced tokens of each, in order."""
        self._need_model()
        max_tokens = self.options.max_tokens if max_tokens is None else max_tokens
        max_batch = max_batch or self.options.max_batch
        # One cache serves call after call (and with it the recorded graphs of its batch sizes); a
        # call that needs more room than any before gets a larger one.
        from .cache import PAGE_TOKENS
        from .engine.generate import most_positions, round_up
        need = sorted((round_up(max(most_positions(len(p), max_tokens, self.context), 1), PAGE_TOKENS)
                       for p in prompts), reverse=True)
        tokens = max(sum(need[:max_batch]), PAGE_TOKENS)
        held = self._batch_cache
        if held is None or held.n_pages * held.page_tokens < tokens or held.n_slots < min(max_batch, len(prompts)):
            self._batch_cache = None
            self.model.__dict__.pop("_decode_sessions", None)
            held = self._batch_cache = self.model.new_cache(max_tokens=tokens, n_slots=max_batch)
        return _generate(self.model, prompts, max_tokens, self._params(temperature, top_k, seed),
                         stop_ids=stop_ids, context=self.context, max_batch=min(max_batch, held.n_slots), cache=held)

    def _need_model(self) -> None:
        if self.model is None:
            raise RuntimeError("no model loaded: call use(model_dir) first")
