"""Causal self-attention over the paged cache.

Parameters: ``hidden_size, n_heads, n_kv_heads, head_dim, softmax_scale,
window`` (0: every earlier key) and ``weight_layout`` (``in_out`` for files
that store ``[in, out]``).  One fused q|k|v projection, keys and values
appended to the layer's cache pages, attention of each new token over the keys
up to its own position, output projection added into the residual stream
(include/ai/LocalModel.hpp:2577-2669; include/ai/Kernels.hpp:132-168).
Head h reads kv head h // (n_heads / n_kv_heads).
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import KVCacheSpec, Mixer, TensorSpec, register_part
from .linear import Linear


class CausalSelfAttention(Mixer):
    takes_lazy_norm = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden_size = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.n_kv_heads = int(self.param("n_kv_heads", self.n_heads))
        self.head_dim = int(self.param("head_dim"))
        self.scale = float(self.param("softmax_scale"))
        self.window = int(self.param("window", 0))
        self.in_out = self.param("weight_layout", "out_in") == "in_out"
        if self.n_heads % self.n_kv_heads != 0:
            raise ConfigError(f"causal_attention: {self.n_heads} heads do not split over {self.n_kv_heads} kv heads")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ConfigError(f"causal_attention: head_dim {self.head_dim} is not a multiple of 16 in [16, 256]")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim

    def _matrix(self, role, out_f, in_f, init):
        shape = (in_f, out_f) if self.in_out else (out_f, in_f)
        return TensorSpec(self.tensor_name(role), shape, role="matrix", transpose=self.in_out, init=init)

    def tensor_specs(self):
        qkv = self.q_width + 2 * self.kv_width
        return (self._matrix("qkv_weight", qkv, self.hidden_size, "normal"),
                TensorSpec(self.tensor_name("qkv_bias"), (qkv,), role="vector", init="bias"),
                self._matrix("out_weight", self.hidden_size, self.q_width, "residual_projection"),
                TensorSpec(self.tensor_name("out_bias"), (self.hidden_size,), role="vector", init="bias"))

    def cache_spec(self):
        return KVCacheSpec(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.qkv = Linear(tensors[self.tensor_name("qkv_weight")], tensors[self.tensor_name("qkv_bias")], runtime)
        self.out = Linear(tensors[self.tensor_name("out_weight")], tensors[self.tensor_name("out_bias")], runtime)

    def forward(self, h, residual, ctx, cache, owns_cache: bool) -> None:
        ops = self.runtime.ops
        qkv, q, k, v = ctx.buffer("attention.qkv", (ctx.n_tokens, self.q_width + 2 * self.kv_width),
                                  self.runtime.dtype, columns=(self.q_width, self.kv_width, self.kv_width))
        self.qkv(h, out=qkv)
        ctx.position.rotate(q, k, ctx)
        table = ctx.block_tables[cache.group]
        attn = ctx.buffer("attention.out", (ctx.n_tokens, self.q_width), qkv.dtype)
        if ctx.is_decode and cache.page_tokens == 64:
            # one launch: append this token's key and value, attend page by page, merge
            ops.attention_decode(q, k if owns_cache else None, v if owns_cache else None, attn, cache.pages,
                                 table, cache.page_tokens, ctx.tok_pos, None, self.n_heads,
                                 self.n_kv_heads, self.head_dim, self.scale, self.window,
                                 ctx.decode_pages(cache.page_tokens))
        else:
            if ctx.q_tiles_wide is not None and ops.prefill_tc_ok(q, attn, self.head_dim, cache.page_tokens):
                # the append and the attention from one call into the library
                ops.attention_prefill_tc(q, attn, cache.pages, table, cache.page_tokens, ctx.tok_pos, ctx.tok_seq,
                                         ctx.q_tiles_wide, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                         self.window, k_new=k if owns_cache else None,
                                         v_new=v if owns_cache else None, append_tiles=ctx.q_tiles)
                self.out(attn, residual=residual, out=residual)
                return
            if owns_cache:
                ops.kv_append(k, v, ctx.tok_pos, ctx.tok_seq, table, cache.page_tokens,
                              self.n_kv_heads, self.head_dim, cache.pages, tiles=ctx.q_tiles)
            if ctx.q_tiles is not None and ops.prefill_ok(q, self.head_dim, cache.page_tokens):
                ops.attention_prefill(q, attn, cache.pages, table, cache.page_tokens, ctx.tok_pos, ctx.tok_seq,
                                      ctx.q_tiles, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                      self.window)
                self.out(attn, residual=residual, out=residual)
                return
            n_splits, split_keys, part_o, part_ml = ctx.attention_splits(self.n_heads, self.head_dim)
            ops.attention(q, attn, cache.pages, table, cache.page_tokens, ctx.tok_pos, ctx.tok_seq,
                          self.n_heads, self.n_kv_heads, self.head_dim, self.scale, self.window,
                          n_splits, split_keys, part_o, part_ml)
        self.out(attn, residual=residual, out=residual)


register_part("mixer", "causal_attention", CausalSelfAttention, replace=True)
