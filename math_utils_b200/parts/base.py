"""What a part is, and the registry of part kinds.

A model is put together from five kinds of parts: ``embedding``, ``position``
(position encoding), ``norm``, ``mixer`` (attention, or anything else that
mixes tokens of a sequence), ``feed_forward``, ``head``; and an
``arrangement`` that wires one layer's norms, mixer and feed-forward around
the residual stream.  A part is built from its ``PartSpec`` alone: it never
learns which model or architecture it is in.

Every part
  * lists the tensors it needs (``tensor_specs``) so the loader can check a
    weight file against the whole model at once;
  * takes them in ``bind`` (already on the device, matrices as ``[out, in]``);
  * a mixer also says what cache it needs (``cache_spec``).

The reference describes the same axes as enums (``NormKind``, ``PosKind``,
``MLPKind``, ``ActKind``, ``LinearLayout``: include/ai/LocalModel.hpp:77-90);
here they are open registries, so a test or a later architecture adds a kind
without touching this package.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Sequence, Tuple

from ..config.base import ConfigError, PartSpec

PART_ROLES = ("embedding", "position", "norm", "mixer", "feed_forward", "head", "arrangement")


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part reads from the weight file.

    ``shape`` is the shape on disk.  ``role`` is ``"matrix"`` (a GEMM operand,
    kept in the compute dtype), ``"table"`` (rows gathered by an index, kept in
    the compute dtype), ``"vector"`` (bias or norm parameter, kept in 32-bit)
    or ``"int_table"`` (kept as int32).  ``transpose`` asks the loader for the
    transposed matrix (files that store ``[in, out]``; the kernels want
    ``[out, in]``, as the reference arranges at load:
    include/ai/LocalModel.hpp:1861-1866).  ``init`` names the random-weights
    rule: ``normal``, ``residual_projection``, ``bias``, ``norm_weight``,
    ``norm_bias``.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    transpose: bool = False
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class KVCacheSpec:
    """A mixer that keeps keys and values of earlier tokens.  ``window`` 0
    keeps all of them; ``window`` w keeps what the last w positions need."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateCacheSpec:
    """A mixer that keeps a fixed number of 32-bit values per sequence,
    whatever the sequence's length; zero when a sequence starts."""
    n_values: int


class Part:
    """Base of all parts.  ``spec.params`` holds sizes and constants,
    ``spec.tensors`` the file names of the part's tensors."""

    # False for a part whose forward pass reads host-side values of the step
    # (``ctx.slots``, ``ctx.q_lens``): such a pass cannot be replayed from a CUDA
    # graph, and generation then launches every step eagerly.
    graph_safe = True

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def tensor_specs(self) -> Sequence[TensorSpec]:
        return ()

    def bind(self, tensors: Mapping[str, Any], runtime) -> None:
        """``tensors``: file name -> device tensor; ``runtime``: dtype, device
        and the kernel namespace (``engine.runtime.Runtime``)."""
        self.runtime = runtime

    def param(self, key: str, default: Any = ...):
        if key in self.spec.params:
            return self.spec.params[key]
        if default is ...:
            raise ConfigError(f"part '{self.spec.kind}' needs parameter '{key}'")
        return default

    def tensor_name(self, role: str) -> str:
        try:
            return self.spec.tensors[role]
        except KeyError:
            raise ConfigError(f"part '{self.spec.kind}' needs a tensor name for '{role}'") from None

    def bias_spec(self, role: str, size: int, init: str = "bias"):
        """The ``TensorSpec`` of a bias vector under the part's ``bias`` parameter:
        true (the default) the file must hold it, ``"if_present"`` it is used when
        the file holds it, false it is never read.  Returns a tuple of zero or one
        specs, to be spliced into ``tensor_specs``."""
        mode = self.param("bias", True)
        if mode is False:
            return ()
        if mode not in (True, "if_present"):
            raise ConfigError(f"part '{self.spec.kind}': parameter 'bias' must be true, false or 'if_present'")
        return (TensorSpec(self.tensor_name(role), (size,), role="vector", init=init, optional=mode != True),)

    def bias_tensor(self, tensors: Mapping[str, Any], role: str):
        """The bound bias of ``role``, or None where the part has none."""
        if self.param("bias", True) is False:
            return None
        return tensors.get(self.tensor_name(role))


class Mixer(Part):
    """Interface of a mixer.

    ``forward(h, residual, ctx, cache, owns_cache)``: ``h`` is ``[T, hidden]``
    in the compute dtype (the normed residual stream of all tokens of the step,
    sequences one after another as ``ctx`` describes); the mixer ADDS its
    result into ``residual`` (``[T, hidden]`` float32) and returns nothing.
    ``cache`` is the view of the cache entry assigned to this run of the layer
    (``None`` if ``cache_spec()`` is ``None``); with ``owns_cache`` false it
    belongs to an earlier layer and is only read.
    """

    takes_lazy_norm = False          # see FeedForward

    def cache_spec(self):
        return None

    def forward(self, h, residual, ctx, cache, owns_cache: bool) -> None:
        raise NotImplementedError


class FeedForward(Part):
    """``forward(h, residual, ctx)``: adds its result into ``residual``.  A
    feed-forward (or mixer) that sets ``takes_lazy_norm`` may be handed a
    ``NormedInput`` (a norm not computed yet) instead of a tensor as ``h`` and
    passes it to its first ``Linear``, which folds the norm into the product
    where it can."""
    takes_lazy_norm = False

    def forward(self, h, residual, ctx) -> None:
        raise NotImplementedError


class Norm(Part):
    """``forward(x, rows=None)``: ``x`` ``[T, hidden]`` float32 -> normed rows in
    the compute dtype; ``rows`` (int32 device tensor) picks rows of ``x``."""

    def forward(self, x, rows=None):
        raise NotImplementedError

    def lazy(self, x, rows=None):
        """The norm as a ``NormedInput`` for a consumer that may fold it into
        its product; a norm that cannot be folded returns the computed tensor."""
        return self.forward(x, rows)


class PositionEncoding(Part):
    """Two hooks, either may do nothing: ``embedding_table()`` is a
    ``[max_positions, hidden]`` table added to the token embedding by absolute
    position, or ``None``; ``rotate(q, k, ctx)`` changes queries and keys in
    place before keys reach the cache."""

    def embedding_table(self):
        return None

    def rotate(self, q, k, ctx) -> None:
        return None


class Embedding(Part):
    """``forward(ctx, position_table)`` -> ``[T, hidden]`` float32 residual."""

    def forward(self, ctx, position_table):
        raise NotImplementedError

    def table(self):
        raise NotImplementedError


class Head(Part):
    """``forward(h)``: ``[n, hidden]`` compute dtype -> ``[n, vocab]`` float32."""

    def forward(self, h):
        raise NotImplementedError


class Arrangement(Part):
    """Wires one layer.  ``forward(x, layer, ctx, cache, owns_cache)`` updates
    the float32 residual stream ``x`` in place; ``layer`` has ``norm1``,
    ``mixer``, ``norm2``, ``feed_forward``."""

    def forward(self, x, layer, ctx, cache, owns_cache: bool) -> None:
        raise NotImplementedError


_PARTS: Dict[Tuple[str, str], Callable[[PartSpec], Part]] = {}


def register_part(role: str, kind: str, factory: Callable[[PartSpec], Part], replace: bool = False) -> None:
    if role not in PART_ROLES:
        raise ValueError(f"unknown part role '{role}'; roles: {', '.join(PART_ROLES)}")
    if (role, kind) in _PARTS and not replace:
        raise ValueError(f"{role} kind '{kind}' is already registered")
    _PARTS[(role, kind)] = factory


def build_part(role: str, spec: PartSpec) -> Part:
    try:
        factory = _PARTS[(role, spec.kind)]
    except KeyError:
        known = sorted(k for r, k in _PARTS if r == role)
        raise ConfigError(f"no {role} of kind '{spec.kind}'; known: {', '.join(known)}") from None
    return factory(spec)


def known_parts(role: Optional[str] = None):
    return sorted((r, k) for r, k in _PARTS if role is None or r == role)
