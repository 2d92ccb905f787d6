"""Token embedding: a row of the table per token, plus the position table's
row when the position encoding has one; the result is the float32 residual
stream (include/ai/LocalModel.hpp:3686-3697)."""
from __future__ import annotations

from ..config.base import PartSpec
from .base import Embedding, Head, TensorSpec, register_part


class TokenEmbedding(Embedding):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self.param("vocab_size"))
        self.hidden_size = int(self.param("hidden_size"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.vocab_size, self.hidden_size), role="table"),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]

    def table(self):
        return self.weight

    def forward(self, ctx, position_table):
        return self.runtime.ops.embed(ctx.token_ids, ctx.tok_pos, self.weight, position_table)


class TiedHead(Head):
    """Logits = h @ table^T with the token table itself, no bias
    (include/ai/LocalModel.hpp:1938-1940, 3796-3799)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self.param("vocab_size"))
        self.hidden_size = int(self.param("hidden_size"))
        self.linear = None

    def attach_embedding(self, embedding: Embedding) -> None:
        from .linear import Linear
        table = embedding.table()
        if tuple(table.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError("the tied head and the token table disagree on their sizes")
        self.linear = Linear(table, None, self.runtime)

    takes_lazy_norm = True

    def forward(self, h):
        import torch
        return self.linear(h, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("head", "tied_head", TiedHead, replace=True)
