"""Position encodings.

``learned_absolute``: a ``[max_positions, hidden]`` table whose row for a
token's absolute position is added to its embedding
(include/ai/LocalModel.hpp:3694-3697); queries and keys are left as they are.
"""
from __future__ import annotations

from ..config.base import PartSpec
from .base import PositionEncoding, TensorSpec, register_part


class LearnedAbsolutePositions(PositionEncoding):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.max_positions = int(self.param("max_positions"))
        self.hidden_size = int(self.param("hidden_size"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.max_positions, self.hidden_size), role="table"),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]

    def embedding_table(self):
        return self.weight


class NoPositions(PositionEncoding):
    """Nothing is added and nothing is rotated."""


register_part("position", "learned_absolute", LearnedAbsolutePositions, replace=True)
register_part("position", "none", NoPositions, replace=True)
