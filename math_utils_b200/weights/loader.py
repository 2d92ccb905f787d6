"""Weights by tensor name, checked against the whole model at once.

The model's parts list the tensors they need (``TensorSpec``); the loader
finds each by name in ``model.safetensors`` (or the shards that
``model.safetensors.index.json`` names, include/ai/Safetensors.hpp:992-1014),
and raises ONE error that lists every missing tensor, every tensor the model
has no use for, and every wrong shape.  Matrices and gathered tables are kept
in the compute dtype (bfloat16, or float32 on the 32-bit path), vectors
(biases, norm parameters) in float32, integer tables as int32.  A matrix
stored ``[in, out]`` is transposed once here (include/ai/LocalModel.hpp:1861-1866,
1879-1887), so the kernels only ever see ``x @ W^T`` with ``W`` ``[out, in]``.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Iterable, List, Mapping, Sequence

import torch

from ..parts.base import TensorSpec
from .safetensors import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """Missing, unexpected and misshapen tensors of one weight file."""

    def __init__(self, where: str, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.where = where
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)     # (name, found shape, wanted shape)
        self.other = list(other)
        lines = [f"{where}: the weights do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(f)}, wanted {list(w)}" for n, f, w in self.wrong_shape))
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


def open_weight_files(model_dir: str) -> List[SafetensorsFile]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        shards = sorted(set(weight_map.values()))
        if not shards:
            raise SafetensorsError(f"{index}: empty weight_map")
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    return [SafetensorsFile(os.path.join(model_dir, "model.safetensors"))]


def _pick_prefix(names: Iterable[str], specs: Sequence[TensorSpec], prefixes: Sequence[str]) -> str:
    names = set(names)
    best, best_hits = prefixes[0], -1
    for p in prefixes:
        hits = sum(1 for s in specs if p + s.name in names)
        if hits > best_hits:
            best, best_hits = p, hits
    return best


def load_weights(model_dir: str, specs: Sequence[TensorSpec], compute_dtype: torch.dtype,
                 device, ignored: Sequence[str] = (), prefixes: Sequence[str] = ("",)) -> Dict[str, torch.Tensor]:
    """name (without prefix) -> tensor on ``device``, arranged as its spec asks."""
    files = open_weight_files(model_dir)
    try:
        where_of: Dict[str, SafetensorsFile] = {}
        for f in files:
            for n in f.names():
                where_of[n] = f
        prefix = _pick_prefix(where_of, specs, list(prefixes))
        ignore = [re.compile(r) for r in ignored]
        wanted = {}
        for s in specs:
            if s.name in wanted and wanted[s.name] != s:
                # two parts may share one tensor (tied tables) if they agree on it
                if wanted[s.name].shape != s.shape:
                    raise WeightError(model_dir, other=[f"tensor '{s.name}' is asked for with two shapes"])
            wanted.setdefault(s.name, s)

        missing, wrong = [], []
        for name, s in wanted.items():
            f = where_of.get(prefix + name)
            if f is None:
                if not s.optional:
                    missing.append(prefix + name)
                continue
            found = f.tensors[prefix + name].shape
            if tuple(found) != tuple(s.shape):
                wrong.append((prefix + name, found, s.shape))
        unexpected = []
        for n in where_of:
            base = n[len(prefix):] if n.startswith(prefix) else None
            if base is not None and base in wanted:
                continue
            # a name the model never reads may stand with the prefix or without it (a checkpoint that
            # keeps its layers under "transformer." has its tied output copy as plain "lm_head.weight")
            if any(r.fullmatch(c) for r in ignore for c in (base, n) if c is not None):
                continue
            unexpected.append(n)
        if missing or wrong or unexpected:
            raise WeightError(model_dir, sorted(missing), sorted(unexpected), sorted(wrong))

        out: Dict[str, torch.Tensor] = {}
        for name, s in wanted.items():
            f = where_of.get(prefix + name)
            if f is None:
                continue
            out[name] = arrange(f.read(prefix + name), s, compute_dtype, device)
        return out
    finally:
        for f in files:
            f.close()


def arrange(t: torch.Tensor, spec: TensorSpec, compute_dtype: torch.dtype, device) -> torch.Tensor:
    """Moves one tensor to the device in the dtype and orientation of its role."""
    if spec.role == "int_table":
        if t.dtype.is_floating_point:
            raise WeightError(spec.name, other=[f"tensor '{spec.name}' should hold integers, holds {t.dtype}"])
        return t.to(device=device, dtype=torch.int32).contiguous()
    if not t.dtype.is_floating_point:
        raise WeightError(spec.name, other=[f"tensor '{spec.name}' should hold floats, holds {t.dtype}"])
    t = t.to(device)
    if spec.role == "vector":
        return t.to(torch.float32).contiguous()
    if spec.role in ("matrix", "table"):
        t = t.to(compute_dtype)
        if spec.transpose:
            t = t.t()
        return t.contiguous()
    raise ValueError(f"tensor '{spec.name}': unknown role '{spec.role}'")
