"""A matrix product with its epilogue, as the parts use it.

``y = act(x @ W^T + b) (+ residual)`` with ``W`` kept ``[out, in]``.  Which
kernel runs is decided here from the compute dtype and the number of rows:
float32 always takes the CUDA-core kernel (the true 32-bit path); bfloat16
takes the tensor-core kernels where the shape allows them and the CUDA-core
kernel otherwise.  The reference's counterpart is ``Weight`` + ``apply``
(include/ai/LocalModel.hpp:989-1126).
"""
from __future__ import annotations

from typing import Optional

import torch


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], runtime):
        self.weight = weight            # [out, in], compute dtype
        self.bias = bias                # [out] float32 or None
        self.runtime = runtime
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        ops = self.runtime.ops
        if out is None and out_dtype is None:
            out_dtype = torch.float32 if residual is not None else getattr(x, "out_dtype", None) or x.dtype
        return ops.linear(x, self.weight, self.bias, act=act, residual=residual, out=out, out_dtype=out_dtype)
