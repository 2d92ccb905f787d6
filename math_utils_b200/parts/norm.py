"""LayerNorm: mean and biased variance of the row in float32, eps inside the
root, weight and bias (include/ai/LocalModel.hpp:1355-1367)."""
from __future__ import annotations

from ..config.base import PartSpec
from .base import Norm, TensorSpec, register_part


class LayerNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.size,), role="vector", init="norm_weight"),
                TensorSpec(self.tensor_name("bias"), (self.size,), role="vector", init="norm_bias"))

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]
        self.bias = tensors[self.tensor_name("bias")]

    def forward(self, x, rows=None):
        return self.runtime.ops.layernorm(x, self.weight, self.bias, self.eps, self.runtime.dtype, rows=rows)

    def lazy(self, x, rows=None):
        """Not computed yet: the product kernels know this norm and make it while they load their rows."""
        return self.runtime.ops.NormedInput(x, self.weight, self.bias, self.eps, self.runtime.dtype, rows=rows)


register_part("norm", "layer_norm", LayerNorm, replace=True)
