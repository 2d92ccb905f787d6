"""Arrangements: how a layer's parts sit around the residual stream.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(include/ai/LocalModel.hpp:3705-3782).  The residual stream stays float32;
mixer and feed-forward add into it in their last product's epilogue.

A prompt step of a layer whose parts are this package's own LayerNorm, causal
attention and two-matrix feed-forward, in bfloat16 at the sizes the tcgen05
kernels take, goes to the library as ONE call that issues the layer's eight
launches (``ops.prompt_layer``): the same kernels through the same entry
points, without the host spending longer on the calls than the device on the
kernels.  Every other layer, step and precision goes part by part.
"""
from __future__ import annotations

import torch

from .attention import CausalSelfAttention
from .base import Arrangement, PositionEncoding, register_part
from .feedforward import DenseFeedForward
from .norm import LayerNorm


class PreNormBlock(Arrangement):
    def forward(self, x, layer, ctx, cache, owns_cache: bool) -> None:
        if ctx.trace is None and not ctx.is_decode and self._whole_layer(x, layer, ctx, cache, owns_cache):
            return
        h = layer.norm1.lazy(x) if layer.mixer.takes_lazy_norm else layer.norm1.forward(x)
        ctx.note("ln1", h)
        layer.mixer.forward(h, x, ctx, cache, owns_cache)
        ctx.note("res1", x)
        h = layer.norm2.lazy(x) if layer.feed_forward.takes_lazy_norm else layer.norm2.forward(x)
        ctx.note("ln2", h)
        layer.feed_forward.forward(h, x, ctx)
        ctx.note("res2", x)

    # ------------------------------------------------------------ the layer as one call
    def _whole_layer(self, x, layer, ctx, cache, owns_cache: bool) -> bool:
        """Runs the layer through ``ops.prompt_layer`` if it is the kind that call is for; False if not."""
        args = getattr(layer, "_prompt_args", None)
        if args is None:
            args = layer._prompt_args = self._layer_args(layer)
        if args is False:
            return False
        mixer, ff = layer.mixer, layer.feed_forward
        rt = mixer.runtime
        ops = rt.ops
        n = ctx.n_tokens
        if (n <= 64 or ctx.q_tiles_wide is None or cache is None or cache.page_tokens != 64
                or type(ctx.position).rotate is not PositionEncoding.rotate
                or x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != mixer.hidden_size):
            return False
        width = mixer.q_width + 2 * mixer.kv_width
        qkv = ctx.buffer("attention.qkv", (n, width), rt.dtype, columns=(mixer.q_width, mixer.kv_width, mixer.kv_width))[0]
        attn = ctx.buffer("attention.out", (n, mixer.q_width), rt.dtype)
        inner = ctx.buffer("feed_forward.hidden", (n, ff.inner_size), rt.dtype)
        normed = ops.scratch("layernorm_out", x.device, n * mixer.hidden_size, torch.bfloat16)
        table = ctx.block_tables[cache.group]
        args.x, args.normed, args.qkv, args.attn, args.inner_buf = (x.data_ptr(), normed.data_ptr(), qkv.data_ptr(),
                                                                    attn.data_ptr(), inner.data_ptr())
        args.tok_pos, args.tok_seq, args.block_table = ctx.tok_pos.data_ptr(), ctx.tok_seq.data_ptr(), table.data_ptr()
        args.tiles_wide, args.tiles = ctx.q_tiles_wide.data_ptr(), ctx.q_tiles.data_ptr()
        args.n_tiles_wide, args.n_tiles = ctx.q_tiles_wide.shape[0], ctx.q_tiles.shape[0]
        args.status = ops.status_word(x.device).data_ptr()
        args.kv_pages, args.n_cache_pages = cache.pages.data_ptr(), cache.pages.shape[0]
        args.max_pages, args.page_tokens = table.shape[1], cache.page_tokens
        args.n_tokens, args.owns_cache = n, int(owns_cache)
        ops.prompt_layer(args)
        return True

    @staticmethod
    def _layer_args(layer):
        """The part of the call's arguments that never changes (weights, sizes), or False for a layer
        that is not made of this package's LayerNorm, causal attention and two-matrix feed-forward in
        bfloat16 at sizes the tcgen05 kernels take."""
        n1, mixer, n2, ff = layer.norm1, layer.mixer, layer.norm2, layer.feed_forward
        if not (type(n1) is LayerNorm and type(n2) is LayerNorm and type(mixer) is CausalSelfAttention
                and type(ff) is DenseFeedForward):
            return False
        rt = mixer.runtime
        if rt.dtype != torch.bfloat16 or not rt.ops.PREFILL_TC or mixer.head_dim != 64:
            return False
        weights = (mixer.qkv.weight, mixer.out.weight, ff.up.weight, ff.down.weight)
        if any(w.dtype != torch.bfloat16 or w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16 or w.shape[1] % 8
               for w in weights):
            return False
        if (mixer.q_width + 2 * mixer.kv_width) % 8 or mixer.q_width % 8 or ff.inner_size % 8 or mixer.hidden_size % 8:
            return False
        ops = rt.ops
        a = ops.PromptLayerArgs()
        ptr = lambda t: None if t is None else t.data_ptr()
        a.ln1_gamma, a.ln1_beta, a.eps1 = ptr(n1.weight), ptr(n1.bias), n1.eps
        a.ln2_gamma, a.ln2_beta, a.eps2 = ptr(n2.weight), ptr(n2.bias), n2.eps
        a.qkv_weight, a.qkv_bias, a.ld_qkv_weight = ptr(mixer.qkv.weight), ptr(mixer.qkv.bias), mixer.qkv.weight.stride(0)
        a.out_weight, a.out_bias, a.ld_out_weight = ptr(mixer.out.weight), ptr(mixer.out.bias), mixer.out.weight.stride(0)
        a.up_weight, a.up_bias, a.ld_up_weight = ptr(ff.up.weight), ptr(ff.up.bias), ff.up.weight.stride(0)
        a.down_weight, a.down_bias, a.ld_down_weight = ptr(ff.down.weight), ptr(ff.down.bias), ff.down.weight.stride(0)
        a.hidden, a.inner, a.act = mixer.hidden_size, ff.inner_size, ops.ACT_CODES[ff.activation]
        a.n_heads, a.n_kv_heads, a.head_dim = mixer.n_heads, mixer.n_kv_heads, mixer.head_dim
        a.scale, a.window = mixer.scale, mixer.window
        return a


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)
