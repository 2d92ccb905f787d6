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
        if not 1 <= self.head_dim <= 256:
            raise ConfigError(f"causal_attention: head_dim {self.head_dim} is outside [1, 256]")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim

    def _matrix(self, role, out_f, in_f, init):
        shape = (in_f, out_f) if self.in_out else (out_f, in_f)
        return TensorSpec(self.tensor_name(role), shape, role="matrix", transpose=self.in_out, init=init)

    def tensor_specs(self):
        qkv = self.q_width + 2 * self.kv_width
        return ((self._matrix("qkv_weight", qkv, self.hidden_size, "normal"),) + self.bias_spec("qkv_bias", qkv)
                + (self._matrix("out_weight", self.hidden_size, self.q_width, "residual_projection"),)
                + self.bias_spec("out_bias", self.hidden_size))

    def cache_spec(self):
        return KVCacheSpec(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.qkv = Linear(tensors[self.tensor_name("qkv_weight")], self.bias_tensor(tensors, "qkv_bias"), runtime)
        self.out = Linear(tensors[self.tensor_name("out_weight")], self.bias_tensor(tensors, "out_bias"), runtime)

    def forward(self, h, residual, ctx, cache, owns_cache: bool) -> None:
        qkv, q, k, v = ctx.buffer("attention.qkv", (ctx.n_tokens, self.q_width + 2 * self.kv_width),
                                  self.runtime.dtype, columns=(self.q_width, self.kv_width, self.kv_width))
        self.qkv(h, out=qkv)
        ctx.position.rotate(q, k, ctx)
        ctx.note("qkv", qkv)
        attn = ctx.buffer("attention.out", (ctx.n_tokens, self.q_width), qkv.dtype)
        self.attend(q, k if owns_cache else None, v if owns_cache else None, attn, ctx, cache)
        ctx.note("attn", attn)
        self.out(attn, residual=residual, out=residual)

    def attend(self, q, k_new, v_new, attn, ctx, cache) -> None:
        """Appends the step's keys and values (if given) to the cache pages and
        writes each token's attention over the keys up to its own position,
        through the kernel that fits the step and the sizes."""
        ops = self.runtime.ops
        table = ctx.block_tables[cache.group]
        page = cache.page_tokens
        sizes = (self.n_heads, self.n_kv_heads, self.head_dim, self.scale, self.window)
        if ctx.is_decode and page == 64 and ops.decode_ok(self.head_dim):
            # one launch: append this token's key and value, attend page by page, merge
            ops.attention_decode(q, k_new, v_new, attn, cache.pages, table, page, ctx.tok_pos, None, *sizes,
                                 ctx.decode_pages(page))
            return
        if ctx.q_tiles_wide is not None and ops.prefill_tc_ok(q, attn, self.head_dim, page):
            # the append and the attention from one call into the library
            ops.attention_prefill_tc(q, attn, cache.pages, table, page, ctx.tok_pos, ctx.tok_seq, ctx.q_tiles_wide,
                                     *sizes, k_new=k_new, v_new=v_new, append_tiles=ctx.q_tiles)
            return
        if k_new is not None:
            ops.kv_append(k_new, v_new, ctx.tok_pos, ctx.tok_seq, table, page, self.n_kv_heads, self.head_dim,
                          cache.pages, tiles=ctx.q_tiles)
        if ctx.q_tiles is not None and ops.prefill_ok(q, self.head_dim, page):
            ops.attention_prefill(q, attn, cache.pages, table, page, ctx.tok_pos, ctx.tok_seq, ctx.q_tiles, *sizes)
            return
        n_splits, split_keys, part_o, part_ml = ctx.attention_splits(self.n_heads, self.head_dim)
        ops.attention(q, attn, cache.pages, table, page, ctx.tok_pos, ctx.tok_seq, *sizes,
                      n_splits, split_keys, part_o, part_ml)


register_part("mixer", "causal_attention", CausalSelfAttention, replace=True)
