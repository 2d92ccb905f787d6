"""GPT-2's configuration: its own config.json keys, typed, and its plan.

Keys read: ``n_layer, n_embd, n_head, n_inner, vocab_size, n_positions,
layer_norm_epsilon, activation_function, scale_attn_by_inverse_layer_idx,
scale_attn_weights, tie_word_embeddings, initializer_range, eos_token_id``.
The reference reads the first six through ``gpt2Spec``'s key table
(include/ai/LocalModel.hpp:542-550, 755-774) and fixes the feed-forward width
at four times the model width (include/ai/LocalModel.hpp:767-768) and the
activation at tanh-GELU (include/ai/LocalModel.hpp:538); here ``n_inner`` and
``activation_function`` are honoured, and so is
``scale_attn_by_inverse_layer_idx`` (an extra 1/(layer index + 1) on the
attention scores).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .base import (ConfigError, KeyReader, LayerSpec, ModelPlan, PartSpec,
                   default_schedule)

ACTIVATIONS = ("gelu_new", "gelu")


@dataclass(frozen=True)
class Gpt2Config:
    n_layer: int
    n_embd: int
    n_head: int
    vocab_size: int
    n_positions: int
    n_inner: Optional[int] = None            # None: 4 * n_embd
    layer_norm_epsilon: float = 1e-5
    activation_function: str = "gelu_new"
    scale_attn_weights: bool = True
    scale_attn_by_inverse_layer_idx: bool = False
    tie_word_embeddings: bool = True
    initializer_range: float = 0.02
    eos_token_ids: tuple = ()

    model_type = "gpt2"
    architecture = "GPT2LMHeadModel"

    def __post_init__(self):
        if self.n_embd % self.n_head != 0:
            raise ConfigError(
                f"config.json: n_embd ({self.n_embd}) is not a multiple of n_head ({self.n_head})")
        if self.activation_function not in ACTIVATIONS:
            raise ConfigError(
                f"config.json: key 'activation_function' is '{self.activation_function}', "
                f"supported: {', '.join(ACTIVATIONS)}")
        if not self.tie_word_embeddings:
            raise ConfigError("config.json: key 'tie_word_embeddings' false is not supported for gpt2 "
                              "(the output matrix is the token table)")

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "Gpt2Config":
        r = KeyReader(raw)
        for key in ("add_cross_attention",):
            if raw.get(key):
                raise ConfigError(f"config.json: key '{key}' true is not supported")
        return cls(
            n_layer=r.integer("n_layer"),
            n_embd=r.integer("n_embd"),
            n_head=r.integer("n_head"),
            vocab_size=r.integer("vocab_size"),
            n_positions=r.integer("n_positions"),
            n_inner=r.integer("n_inner", default=None),
            layer_norm_epsilon=r.number("layer_norm_epsilon", default=1e-5),
            activation_function=r.string("activation_function", default="gelu_new", choices=ACTIVATIONS),
            scale_attn_weights=r.boolean("scale_attn_weights", default=True),
            scale_attn_by_inverse_layer_idx=r.boolean("scale_attn_by_inverse_layer_idx", default=False),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=True),
            initializer_range=r.number("initializer_range", default=0.02),
            eos_token_ids=r.id_list("eos_token_id"),
        )

    def to_json(self) -> dict:
        out = {
            "model_type": self.model_type,
            "architectures": [self.architecture],
            "n_layer": self.n_layer, "n_embd": self.n_embd, "n_head": self.n_head,
            "n_inner": self.n_inner, "vocab_size": self.vocab_size,
            "n_positions": self.n_positions,
            "layer_norm_epsilon": self.layer_norm_epsilon,
            "activation_function": self.activation_function,
            "scale_attn_weights": self.scale_attn_weights,
            "scale_attn_by_inverse_layer_idx": self.scale_attn_by_inverse_layer_idx,
            "tie_word_embeddings": self.tie_word_embeddings,
            "initializer_range": self.initializer_range,
        }
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def init_distribution(self, rule: str):
        """(mean, standard deviation) of a random-weights rule.  Matrices, tables
        and biases N(0, r) with r = initializer_range; both output projections
        into the residual stream N(0, r / sqrt(2 n_layer)); norm weights
        1 + N(0, r), norm biases N(0, r), so that no parameter is a no-op."""
        r = self.initializer_range
        rules = {
            "normal": (0.0, r), "bias": (0.0, r), "norm_bias": (0.0, r),
            "norm_weight": (1.0, r),
            "residual_projection": (0.0, r / math.sqrt(2.0 * self.n_layer)),
        }
        if rule not in rules:
            raise ConfigError(f"no random-weights rule '{rule}'")
        return rules[rule]

    # ------------------------------------------------------------------ plan
    def plan(self) -> ModelPlan:
        """Every layer: LayerNorm -> causal attention -> LayerNorm -> two-matrix
        feed-forward, pre-norm residual (include/ai/LocalModel.hpp:3705-3782)."""
        d, h, dh = self.n_embd, self.n_head, self.head_dim
        layers = []
        for i in range(self.n_layer):
            scale = 1.0 / math.sqrt(dh) if self.scale_attn_weights else 1.0
            if self.scale_attn_by_inverse_layer_idx:
                scale /= float(i + 1)
            p = f"h.{i}"
            norm = lambda n: PartSpec("layer_norm", {"size": d, "eps": self.layer_norm_epsilon},
                                      {"weight": f"{p}.{n}.weight", "bias": f"{p}.{n}.bias"})
            mixer = PartSpec(
                "causal_attention",
                {"hidden_size": d, "n_heads": h, "n_kv_heads": h, "head_dim": dh,
                 "softmax_scale": scale, "window": 0, "weight_layout": "in_out"},
                {"qkv_weight": f"{p}.attn.c_attn.weight", "qkv_bias": f"{p}.attn.c_attn.bias",
                 "out_weight": f"{p}.attn.c_proj.weight", "out_bias": f"{p}.attn.c_proj.bias"})
            ffn = PartSpec(
                "dense_ffn",
                {"hidden_size": d, "inner_size": self.inner, "activation": self.activation_function,
                 "weight_layout": "in_out"},
                {"up_weight": f"{p}.mlp.c_fc.weight", "up_bias": f"{p}.mlp.c_fc.bias",
                 "down_weight": f"{p}.mlp.c_proj.weight", "down_bias": f"{p}.mlp.c_proj.bias"})
            layers.append(LayerSpec("pre_norm", norm("ln_1"), mixer, norm("ln_2"), ffn))
        plan = ModelPlan(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=d,
            max_positions=self.n_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": d},
                               {"weight": "wte.weight"}),
            position=PartSpec("learned_absolute", {"max_positions": self.n_positions, "hidden_size": d},
                              {"weight": "wpe.weight"}),
            layers=tuple(layers),
            schedule=default_schedule(self.n_layer),
            final_norm=PartSpec("layer_norm", {"size": d, "eps": self.layer_norm_epsilon},
                                {"weight": "ln_f.weight", "bias": "ln_f.bias"}),
            head=PartSpec("tied_head", {"vocab_size": self.vocab_size, "hidden_size": d}, {}),
            stop_ids=self.eos_token_ids,
            # the checkpoint's causal-mask buffers and a tied output copy are never read
            ignored_tensors=(r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias", r"lm_head\.weight"),
        )
        plan.validate()
        return plan
