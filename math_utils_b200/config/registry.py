"""One registry from an architecture's name to what builds it.

``config.json`` names its architecture twice: ``model_type`` (``"gpt2"``) and
``architectures[0]`` (``"GPT2LMHeadModel"``); either finds the entry.  The
reference dispatches on ``model_type`` alone through ``specRegistry`` /
``specFor`` and answers an unknown type with the list of known ones
(include/ai/LocalModel.hpp:579-602, 1674-1686).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Tuple

from .base import ConfigError, ModelPlan


@dataclass(frozen=True)
class Architecture:
    """``config_class.from_json(raw)`` gives the typed configuration,
    ``.plan()`` of that the model plan; ``name_prefixes`` are prefixes a weight
    file may put before every tensor name."""
    names: Tuple[str, ...]
    config_class: Any
    name_prefixes: Tuple[str, ...] = ("",)


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    for name in arch.names:
        if name in _REGISTRY and not replace:
            raise ValueError(f"architecture name '{name}' is already registered")
        _REGISTRY[name] = arch


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_REGISTRY))


def architecture_for(raw: Mapping[str, Any]) -> Architecture:
    """Looks the architecture up by ``model_type``, then ``architectures``."""
    candidates = []
    if isinstance(raw.get("model_type"), str):
        candidates.append(raw["model_type"])
    archs = raw.get("architectures")
    if isinstance(archs, list):
        candidates.extend(a for a in archs if isinstance(a, str))
    if not candidates:
        raise ConfigError("config.json: neither 'model_type' nor 'architectures' names an architecture")
    for name in candidates:
        if name in _REGISTRY:
            return _REGISTRY[name]
    raise ConfigError(
        f"config.json: unsupported architecture {candidates!r}; known: {', '.join(known_architectures())}")


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def generation_stop_ids(model_dir: str) -> tuple:
    """``eos_token_id`` of the folder's generation_config.json (an id or a list),
    empty if there is no such file or it cannot be read: the reference adds these
    to config.json's own (include/ai/LocalModel.hpp:1788-1792)."""
    from .base import KeyReader
    path = os.path.join(model_dir, "generation_config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except (OSError, json.JSONDecodeError):
        return ()
    if not isinstance(raw, dict):
        return ()
    return KeyReader(raw, "generation_config.json").id_list("eos_token_id")


def load_config(model_dir: str):
    """(architecture entry, typed configuration, plan) of a model folder.  The
    plan's stop ids are config.json's followed by generation_config.json's."""
    raw = read_config_json(model_dir)
    arch = architecture_for(raw)
    config = arch.config_class.from_json(raw)
    plan = config.plan()
    more = tuple(t for t in generation_stop_ids(model_dir) if t not in plan.stop_ids)
    if more:
        plan = dataclasses.replace(plan, stop_ids=tuple(plan.stop_ids) + more)
    return arch, config, plan
