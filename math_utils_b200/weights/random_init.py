"""Random-weights mode: a model folder from a configuration and a seed.

Writes ``config.json`` and ``model.safetensors`` that the ordinary loader
reads back.  Every tensor has its own generator, keyed by the seed and a hash
of the tensor's name (the reference keys per tensor by ``seed ^ FNV1a(name)``
too, include/ai/LocalModel.hpp:1555-1561, 1623-1630), so a tensor's values do
not depend on which other tensors the model has or on the order they are made
in.  Values are drawn in float32 and, for a bfloat16 file, rounded to nearest
even.

The distribution of each tensor comes from its ``init`` rule and the
configuration's ``init_distribution`` (mean, standard deviation).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping

import numpy as np
import torch

from ..config.registry import architecture_for
from .safetensors import write_safetensors

_MASK = (1 << 64) - 1


def fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return h


def splitmix64(x: int) -> int:
    z = (x + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_generator(seed: int, name: str) -> np.random.Generator:
    key = splitmix64((seed & _MASK) ^ fnv1a64(name))
    return np.random.Generator(np.random.Philox(key=key))


def random_tensors(config, plan, seed: int, store_dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    from ..engine.assemble import collect_tensor_specs
    out: Dict[str, torch.Tensor] = {}
    for spec in collect_tensor_specs(plan):
        if spec.name in out:
            continue
        mean, std = config.init_distribution(spec.init)
        rng = tensor_generator(seed, spec.name)
        values = rng.standard_normal(size=spec.shape, dtype=np.float32)
        values = values * np.float32(std) + np.float32(mean)
        if spec.role == "int_table":
            raise ValueError(f"tensor '{spec.name}': no random rule for integer tables")
        out[spec.name] = torch.from_numpy(values).to(store_dtype)
    return out


def write_random_model(model_dir: str, config_json: Mapping[str, Any], seed: int,
                       store_dtype: str = "bfloat16") -> str:
    """Makes ``model_dir`` with config.json and model.safetensors; returns it."""
    dtypes = {"bfloat16": torch.bfloat16, "float32": torch.float32}
    if store_dtype not in dtypes:
        raise ValueError(f"store_dtype must be one of {', '.join(dtypes)}")
    arch = architecture_for(config_json)
    config = arch.config_class.from_json(config_json)
    plan = config.plan()
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_tensors(config, plan, seed, dtypes[store_dtype])
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "random_seed": str(seed)})
    full = dict(config.to_json()) if hasattr(config, "to_json") else dict(config_json)
    for k, v in config_json.items():
        full.setdefault(k, v)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(full, f, indent=2)
    return model_dir
