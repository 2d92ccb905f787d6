"""From a plan to bound parts: builds every part, lists the tensors they need,
loads them once, and hands each part its tensors."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

from ..config.base import LayerSpec, ModelPlan, PartSpec
from ..parts.base import Arrangement, FeedForward, Mixer, Norm, TensorSpec, build_part


@dataclass
class Layer:
    arrangement: Arrangement
    norm1: Norm
    mixer: Mixer
    norm2: Norm
    feed_forward: FeedForward
    extra: Dict[str, object] = field(default_factory=dict)      # further parts by name (LayerSpec.extra)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward) + tuple(self.extra.values())


def build_layer(spec: LayerSpec) -> Layer:
    extra = {}
    for name, role, part_spec in getattr(spec, "extra", ()):
        part = build_part(role, part_spec)
        if role == "mixer" and part.cache_spec() is not None:
            raise ValueError(f"the extra mixer '{name}' wants a cache of its own: a layer's cache is its mixer's; "
                             "give it a layer of its own in the schedule instead")
        extra[name] = part
    return Layer(
        arrangement=build_part("arrangement", PartSpec(spec.arrangement)),
        norm1=build_part("norm", spec.norm1),
        mixer=build_part("mixer", spec.mixer),
        norm2=build_part("norm", spec.norm2),
        feed_forward=build_part("feed_forward", spec.feed_forward),
        extra=extra,
    )


@dataclass
class Assembly:
    embedding: object
    position: object
    layers: List[Layer]
    final_norm: object
    head: object

    def parts(self):
        out = [self.embedding, self.position]
        for layer in self.layers:
            out.extend(layer.parts())
        out.extend([self.final_norm, self.head])
        return out


def assemble(plan: ModelPlan) -> Assembly:
    plan.validate()
    return Assembly(
        embedding=build_part("embedding", plan.embedding),
        position=build_part("position", plan.position),
        layers=[build_layer(spec) for spec in plan.layers],
        final_norm=build_part("norm", plan.final_norm),
        head=build_part("head", plan.head),
    )


def collect_tensor_specs(plan: ModelPlan, assembly: Assembly = None) -> List[TensorSpec]:
    assembly = assembly or assemble(plan)
    specs: List[TensorSpec] = []
    for part in assembly.parts():
        specs.extend(part.tensor_specs())
    return specs
