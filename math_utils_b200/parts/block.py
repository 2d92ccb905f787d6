"""Arrangements: how a layer's parts sit around the residual stream.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(include/ai/LocalModel.hpp:3705-3782).  The residual stream stays float32;
mixer and feed-forward add into it in their last product's epilogue.
"""
from __future__ import annotations

from .base import Arrangement, register_part


class PreNormBlock(Arrangement):
    def forward(self, x, layer, ctx, cache, owns_cache: bool) -> None:
        h = layer.norm1.lazy(x) if layer.mixer.takes_lazy_norm else layer.norm1.forward(x)
        ctx.note("ln1", h)
        layer.mixer.forward(h, x, ctx, cache, owns_cache)
        ctx.note("res1", x)
        h = layer.norm2.lazy(x) if layer.feed_forward.takes_lazy_norm else layer.norm2.forward(x)
        ctx.note("ln2", h)
        layer.feed_forward.forward(h, x, ctx)
        ctx.note("res2", x)


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)
