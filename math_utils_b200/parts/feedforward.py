"""Dense two-matrix feed-forward: up projection, activation, down projection
(include/ai/LocalModel.hpp:3767-3774).  The activation is a parameter:
``gelu_new`` (tanh form, include/ai/LocalModel.hpp:1388-1391) or ``gelu``
(erf form).  Parameter ``bias``: true (both biases must be in the file),
``"if_present"`` or false."""
from __future__ import annotations

from ..config.base import ConfigError, PartSpec
from .base import FeedForward, TensorSpec, register_part
from .linear import Linear

ACTIVATIONS = ("gelu_new", "gelu")


class DenseFeedForward(FeedForward):
    takes_lazy_norm = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden_size = int(self.param("hidden_size"))
        self.inner_size = int(self.param("inner_size"))
        self.activation = self.param("activation")
        if self.activation not in ACTIVATIONS:
            raise ConfigError(f"dense_ffn: activation '{self.activation}' is not one of {', '.join(ACTIVATIONS)}")
        self.in_out = self.param("weight_layout", "out_in") == "in_out"

    def _matrix(self, role, out_f, in_f, init):
        shape = (in_f, out_f) if self.in_out else (out_f, in_f)
        return TensorSpec(self.tensor_name(role), shape, role="matrix", transpose=self.in_out, init=init)

    def tensor_specs(self):
        d, i = self.hidden_size, self.inner_size
        return ((self._matrix("up_weight", i, d, "normal"),) + self.bias_spec("up_bias", i)
                + (self._matrix("down_weight", d, i, "residual_projection"),) + self.bias_spec("down_bias", d))

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.up = Linear(tensors[self.tensor_name("up_weight")], self.bias_tensor(tensors, "up_bias"), runtime)
        self.down = Linear(tensors[self.tensor_name("down_weight")], self.bias_tensor(tensors, "down_bias"), runtime)

    def forward(self, h, residual, ctx) -> None:
        hidden = None if ctx is None else ctx.buffer("feed_forward.hidden", (ctx.n_tokens, self.inner_size),
                                                     self.runtime.dtype)
        u = self.up(h, act=self.activation, out=hidden)
        if ctx is not None:
            ctx.note("act", u)
        self.down(u, residual=residual, out=residual)


register_part("feed_forward", "dense_ffn", DenseFeedForward, replace=True)
