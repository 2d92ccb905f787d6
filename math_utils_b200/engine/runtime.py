"""What every part is given when it is bound: dtype, device, kernels."""
from __future__ import annotations

from dataclasses import dataclass

import torch

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


_ops = None            # the kernel module, imported when first asked for


@dataclass
class Runtime:
    """``dtype`` is the compute dtype: bfloat16 (the serving path: bfloat16
    weights, activations and cache, float32 accumulation, norms, softmax and
    residual stream) or float32 (everything in true 32-bit, CUDA-core products
    only)."""
    dtype: torch.dtype
    device: torch.device

    @property
    def ops(self):
        global _ops
        if _ops is None:
            from ..csrc import ops
            _ops = ops
        return _ops

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32

    @classmethod
    def create(cls, dtype, device="cuda:0") -> "Runtime":
        if isinstance(dtype, str):
            if dtype not in DTYPES:
                raise ValueError(f"dtype must be one of {', '.join(DTYPES)}, got '{dtype}'")
            dtype = DTYPES[dtype]
        if dtype not in DTYPES.values():
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return cls(dtype=dtype, device=torch.device(device))
