"""Typed description of a decoder, independent of any one architecture.

An architecture's own configuration class (for instance ``Gpt2Config``) reads
its ``config.json`` keys and turns them into a ``ModelPlan``: which embedding,
position encoding, norm, mixer and feed-forward each layer has, with every
size and constant as a parameter of that part, and in which order the layers
run.  Nothing below the plan knows which architecture it came from.

The reference keeps the same idea as data in ``ArchSpec`` / ``NameMap`` /
``ConfigKeys`` (include/ai/LocalModel.hpp:100-224) and fills a ``LocalConfig``
from JSON through them (include/ai/LocalModel.hpp:750-955).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


_MISSING = object()


class KeyReader:
    """Reads typed values from a config.json mapping and names bad keys."""

    def __init__(self, raw: Mapping[str, Any], where: str = "config.json"):
        if not isinstance(raw, Mapping):
            raise ConfigError(f"{where}: expected a JSON object")
        self.raw = raw
        self.where = where

    def _get(self, key: str, default: Any) -> Any:
        value = self.raw.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: missing key '{key}'")
            return default
        return value

    def integer(self, key: str, default: Any = _MISSING, minimum: int = 1) -> Any:
        value = self._get(key, default)
        if value is default and default is not _MISSING:
            return default
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value == int(value):
                value = int(value)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {value!r}")
        if value < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {value}")
        return value

    def number(self, key: str, default: Any = _MISSING, positive: bool = True) -> Any:
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {value!r}")
        value = float(value)
        if positive and not value > 0.0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {value}")
        return value

    def boolean(self, key: str, default: Any = _MISSING) -> Any:
        value = self._get(key, default)
        if not isinstance(value, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {value!r}")
        return value

    def string(self, key: str, default: Any = _MISSING, choices: Optional[Sequence[str]] = None) -> Any:
        value = self._get(key, default)
        if not isinstance(value, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {value!r}")
        if choices is not None and value not in choices:
            raise ConfigError(
                f"{self.where}: key '{key}' is '{value}', supported: {', '.join(choices)}")
        return value

    def id_list(self, key: str) -> tuple:
        """A token id, a list of them, or nothing (eos_token_id takes all three
        forms; include/ai/LocalModel.hpp:1775-1793)."""
        value = self.raw.get(key)
        if value is None:
            return ()
        if isinstance(value, int) and not isinstance(value, bool):
            return (value,)
        if isinstance(value, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
            return tuple(value)
        raise ConfigError(f"{self.where}: key '{key}' must be an id or a list of ids, got {value!r}")


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered kind and its parameters.

    ``params`` holds every size and constant the part needs; ``tensors`` maps
    the part's own tensor roles (``"weight"``, ``"bias"``, ...) to names in the
    weight file.
    """
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    tensors: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """The parts of one layer and the arrangement that wires them.

    ``extra``: further parts for an arrangement that wants more than the four
    (a third norm, a gate): ``(name, role, PartSpec)`` each, built like the
    others and handed to the arrangement as ``layer.extra[name]``.  The cache
    of a layer is its ``mixer``'s; an extra part keeps no cache."""
    arrangement: str
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    feed_forward: PartSpec
    extra: tuple = ()


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelPlan.layers``; a layer may appear in several
    entries (shared weights).  ``cache_of`` is the schedule index whose mixer
    cache this run uses: its own index (it writes and reads its own) or an
    earlier entry's (it only reads what that entry wrote this step).
    """
    layer: int
    cache_of: int


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    position: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    stop_ids: tuple = ()
    ignored_tensors: tuple = ()      # regular expressions of names a file may hold unused

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for n, layer in enumerate(self.layers):
            names = [item[0] for item in getattr(layer, "extra", ())]
            for item in getattr(layer, "extra", ()):
                if len(item) != 3 or not isinstance(item[2], PartSpec):
                    raise ConfigError(f"layer {n}: an extra part is (name, role, PartSpec), got {item!r}")
            taken = [x for x in names if x in ("norm1", "mixer", "norm2", "feed_forward") or names.count(x) > 1]
            if taken:
                raise ConfigError(f"layer {n}: the extra part name '{taken[0]}' is taken")
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"schedule[{i}] names layer {entry.layer}, model has {len(self.layers)}")
            if not 0 <= entry.cache_of <= i:
                raise ConfigError(f"schedule[{i}] reads the cache of entry {entry.cache_of}, which runs later")
            if entry.cache_of != i and self.schedule[entry.cache_of].cache_of != entry.cache_of:
                raise ConfigError(f"schedule[{i}] reads the cache of entry {entry.cache_of}, which owns none")


def default_schedule(n_layers: int) -> tuple:
    return tuple(ScheduleEntry(layer=i, cache_of=i) for i in range(n_layers))
