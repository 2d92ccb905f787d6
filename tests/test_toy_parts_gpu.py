"""More toy parts, defined here and registered from outside the package: a rotary
position encoding (through the ``rotate`` hook), a feed-forward with routing
over experts, grouped heads, a windowed layer next to a full one (two cache
groups in one model) and a layer whose projections have no bias.  None of these is a model of anyone's; they show that the
part interfaces carry more than GPT-2."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import check_logits, run_batch, run_tail_one_by_one, run_whole
from math_utils_b200 import DecoderModel, LLM, Options, register_architecture, write_random_model
from math_utils_b200.config import Architecture, LayerSpec, ModelPlan, PartSpec, default_schedule
from math_utils_b200.parts import (Arrangement, Embedding, FeedForward, Linear, PositionEncoding, TensorSpec,
                                   register_part)

pytestmark = pytest.mark.gpu


class ToyRotary(PositionEncoding):
    """Rotates pairs (2i, 2i+1) of every head of q and k by position * base^(-2i/head_dim);
    angles in float32.  Nothing is added to the embedding."""

    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(self.param("head_dim"))
        self.base = float(self.param("base"))

    def rotate(self, q, k, ctx):
        half = self.head_dim // 2
        inv = self.base ** (-torch.arange(half, device=q.device, dtype=torch.float32) * 2.0 / self.head_dim)
        ang = ctx.tok_pos.float()[:, None] * inv[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        for t in (q, k):
            v = t.float().reshape(t.shape[0], -1, half, 2)
            a, b = v[..., 0], v[..., 1]
            out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).reshape(t.shape[0], -1)
            t.copy_(out.to(t.dtype))


class ToyRoutedFeedForward(FeedForward):
    """Each token goes to the one expert its router logit (float32) is largest for; the
    expert is a gelu_new two-matrix feed-forward.  Every expert runs on all tokens and a
    mask picks: a toy, not a fast path."""
    takes_lazy_norm = False

    def __init__(self, spec):
        super().__init__(spec)
        self.d, self.inner, self.n = (int(self.param(k)) for k in ("hidden_size", "inner_size", "n_experts"))

    def tensor_specs(self):
        t = self.spec.tensors
        specs = [TensorSpec(t["router"], (self.n, self.d), role="matrix")]
        for e in range(self.n):
            specs += [TensorSpec(t["up"].format(e=e), (self.inner, self.d)),
                      TensorSpec(t["up_bias"].format(e=e), (self.inner,), role="vector", init="bias"),
                      TensorSpec(t["down"].format(e=e), (self.d, self.inner), init="residual_projection"),
                      TensorSpec(t["down_bias"].format(e=e), (self.d,), role="vector", init="bias")]
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        t = self.spec.tensors
        self.router = tensors[t["router"]]
        self.experts = [(Linear(tensors[t["up"].format(e=e)], tensors[t["up_bias"].format(e=e)], runtime),
                         Linear(tensors[t["down"].format(e=e)], tensors[t["down_bias"].format(e=e)], runtime))
                        for e in range(self.n)]

    def forward(self, h, residual, ctx):
        choice = torch.argmax(h.float() @ self.router.float().t(), dim=-1)
        for e, (up, down) in enumerate(self.experts):
            y = down(up(h, act="gelu_new"), out_dtype=torch.float32)
            residual += y * (choice == e)[:, None]


class ToyEmbedding(Embedding):
    """A token table looked up with torch's own indexing: recorded single-token steps ask nothing of an
    embedding beyond ``forward``."""

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (int(self.param("vocab_size")), int(self.param("hidden_size"))),
                           role="table"),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]

    def table(self):
        return self.weight

    def forward(self, ctx, position_table):
        assert position_table is None
        return self.weight[ctx.token_ids.long()].float()


class ToyConfig2:
    def __init__(self, raw):
        self.raw = dict(raw)

    @classmethod
    def from_json(cls, raw):
        return cls(raw)

    def to_json(self):
        return dict(self.raw)

    def init_distribution(self, rule):
        return {"norm_weight": (1.0, 0.05)}.get(rule, (0.0, 0.08))

    def plan(self):
        r = self.raw
        d, heads, kv_heads, dh = r["width"], r["heads"], r["kv_heads"], r["head_dim"]

        def norm(name):
            return PartSpec("layer_norm", {"size": d, "eps": 1e-5}, {"weight": name + ".w", "bias": name + ".b"})

        def attn(i, window):
            if i == 1:              # the second layer's projections have no bias: no names, nothing in the file
                return PartSpec("causal_attention",
                                {"hidden_size": d, "n_heads": heads, "n_kv_heads": kv_heads, "head_dim": dh,
                                 "softmax_scale": dh ** -0.5, "window": window, "bias": False},
                                {"qkv_weight": f"l{i}.qkv.w", "out_weight": f"l{i}.o.w"})
            return PartSpec("causal_attention",
                            {"hidden_size": d, "n_heads": heads, "n_kv_heads": kv_heads, "head_dim": dh,
                             "softmax_scale": dh ** -0.5, "window": window},
                            {"qkv_weight": f"l{i}.qkv.w", "qkv_bias": f"l{i}.qkv.b",
                             "out_weight": f"l{i}.o.w", "out_bias": f"l{i}.o.b"})

        routed = PartSpec("toy_routed_ffn", {"hidden_size": d, "inner_size": r["inner"], "n_experts": r["experts"]},
                          {"router": "l0.router", "up": "l0.e{e}.up.w", "up_bias": "l0.e{e}.up.b",
                           "down": "l0.e{e}.down.w", "down_bias": "l0.e{e}.down.b"})
        dense = PartSpec("dense_ffn", {"hidden_size": d, "inner_size": r["inner"], "activation": "gelu", "bias": False},
                         {"up_weight": "l1.up.w", "down_weight": "l1.down.w"})
        layers = (LayerSpec("pre_norm", norm("l0.n1"), attn(0, r["window"]), norm("l0.n2"), routed),
                  LayerSpec("pre_norm", norm("l1.n1"), attn(1, 0), norm("l1.n2"), dense))
        return ModelPlan("ToyModel2", r["vocab"], d, r["positions"],
                         PartSpec("toy_embedding", {"vocab_size": r["vocab"], "hidden_size": d}, {"weight": "emb"}),
                         PartSpec("toy_rotary", {"head_dim": dh, "base": r["base"]}),
                         layers, default_schedule(2), norm("final"),
                         PartSpec("tied_head", {"vocab_size": r["vocab"], "hidden_size": d}))


def toy2_plain(ids, r, w):
    d, heads, kv_heads, dh = r["width"], r["heads"], r["kv_heads"], r["head_dim"]
    n = len(ids)
    x = w["emb"][ids]
    half = dh // 2
    inv = r["base"] ** (-np.arange(half) * 2.0 / dh)
    ang = np.arange(n)[:, None] * inv[None, :]

    def rotate(t):
        v = t.reshape(n, -1, half, 2)
        a, b = v[..., 0], v[..., 1]
        c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        return np.stack((a * c - b * s, a * s + b * c), axis=-1).reshape(n, -1)

    for i, window in ((0, r["window"]), (1, 0)):
        p = f"l{i}"
        h = plain_gpt2.layer_norm(x, w[p + ".n1.w"], w[p + ".n1.b"], 1e-5)
        qkv = h @ w[p + ".qkv.w"].T + (w[p + ".qkv.b"] if i == 0 else 0.0)
        qw, kw = heads * dh, kv_heads * dh
        q, k, v = rotate(qkv[:, :qw]), rotate(qkv[:, qw:qw + kw]), qkv[:, qw + kw:]
        a = plain_gpt2.causal_attention(q, k, v, heads, kv_heads, dh ** -0.5, window)
        x = x + a @ w[p + ".o.w"].T + (w[p + ".o.b"] if i == 0 else 0.0)
        h = plain_gpt2.layer_norm(x, w[p + ".n2.w"], w[p + ".n2.b"], 1e-5)
        if i == 0:
            choice = np.argmax(h @ w["l0.router"].T, axis=-1)
            y = np.zeros_like(x)
            for e in range(r["experts"]):
                u = plain_gpt2.gelu_new(h @ w[f"l0.e{e}.up.w"].T + w[f"l0.e{e}.up.b"])
                y += (u @ w[f"l0.e{e}.down.w"].T + w[f"l0.e{e}.down.b"]) * (choice == e)[:, None]
            x = x + y
        else:
            x = x + plain_gpt2.gelu_erf(h @ w["l1.up.w"].T) @ w["l1.down.w"].T
    return plain_gpt2.layer_norm(x, w["final.w"], w["final.b"], 1e-5) @ w["emb"].T


@pytest.fixture(scope="module")
def toy2(tmp_path_factory):
    register_part("position", "toy_rotary", ToyRotary, replace=True)
    register_part("embedding", "toy_embedding", ToyEmbedding, replace=True)
    register_part("feed_forward", "toy_routed_ffn", ToyRoutedFeedForward, replace=True)
    register_architecture(Architecture(names=("toy2", "ToyModel2"), config_class=ToyConfig2), replace=True)
    raw = {"model_type": "toy2", "width": 80, "heads": 4, "kv_heads": 2, "head_dim": 16, "inner": 136, "experts": 3,
           "vocab": 301, "positions": 200, "window": 50, "base": 100.0}
    d = tmp_path_factory.mktemp("toy2")
    write_random_model(str(d), raw, seed=5)
    return str(d), raw


def test_toy_model_with_rotary_routing_groups_and_window(toy2):
    """float32 only: a token near a routing tie may go to another expert in bfloat16, which is
    a property of routing, not a fault."""
    folder, raw = toy2
    model = DecoderModel.from_dir(folder, dtype="float32")
    cache = model.new_cache(max_tokens=1024, n_slots=4)
    assert [g.spec.window for g in cache.kv_groups] == [50, 0]          # the windowed layer has storage of its own
    w = plain_gpt2.read_safetensors(folder + "/model.safetensors")
    assert "l0.qkv.b" in w and not any(n.startswith("l1.") and n.endswith(".b") and ".n" not in n for n in w)
    rng = np.random.default_rng(2)
    reqs = [rng.integers(0, raw["vocab"], size=n).tolist() for n in (200, 70, 129, 3)]
    want = [toy2_plain(r, raw, w) for r in reqs]
    check_logits(run_whole(model, cache, reqs[0]), want[0], "float32", "toy2 whole")
    check_logits(run_tail_one_by_one(model, cache, reqs[0], 64), want[0], "float32", "toy2 tail")
    for round_ in range(2):
        got = run_batch(model, cache, reqs, [120, 69, 64, 1])
        for g, wnt in zip(got, want):
            check_logits(g, wnt, "float32", f"toy2 batch {round_}")
    assert cache.slots.n_free == 4 and cache.free_pages(0) == cache.n_pages and cache.free_pages(1) == cache.n_pages
    # the windowed group gave pages back while the long request ran: it never needs more than two
    slot = cache.acquire()
    from math_utils_b200 import StepEntry
    model.step(cache, [StepEntry(slot, reqs[0][:150])])
    assert cache.kv_groups[0].pages_held(slot) <= 2 and cache.kv_groups[1].pages_held(slot) == 3
    cache.release(slot)


def test_toy_model_generates_through_the_front_door(toy2):
    folder, raw = toy2
    llm = LLM(folder, Options(dtype="float32", temperature=0.0))
    w = plain_gpt2.read_safetensors(folder + "/model.safetensors")
    prompts = [[5, 9, 200], [17] * 40]
    got = llm.generate(prompts, max_tokens=12, stop_ids=[])
    for p, g in zip(prompts, got):
        ids = list(p)
        for tok in g:
            assert tok == int(np.argmax(toy2_plain(ids, raw, w)[-1]))
            ids.append(tok)


# ------------------------------------------------------------------ a layer with a part beyond the four
class ToySandwich(Arrangement):
    """x += mixer(norm1(x)); x += norm3(feed_forward(norm2(x))): a third norm, on the feed-forward's way back
    into the residual stream, which the layer carries as an extra part."""

    def forward(self, x, layer, ctx, cache, owns_cache):
        layer.mixer.forward(layer.norm1.forward(x), x, ctx, cache, owns_cache)
        branch = torch.zeros_like(x)
        layer.feed_forward.forward(layer.norm2.forward(x), branch, ctx)
        x += layer.extra["norm3"].forward(branch).float()


class ToyConfig3:
    def __init__(self, raw):
        self.raw = dict(raw)

    @classmethod
    def from_json(cls, raw):
        return cls(raw)

    def to_json(self):
        return dict(self.raw)

    def init_distribution(self, rule):
        return {"norm_weight": (1.0, 0.05)}.get(rule, (0.0, 0.1))

    def plan(self):
        r = self.raw
        d, heads = r["width"], r["heads"]

        def norm(name):
            return PartSpec("layer_norm", {"size": d, "eps": 1e-5}, {"weight": name + ".w", "bias": name + ".b"})

        attn = PartSpec("causal_attention", {"hidden_size": d, "n_heads": heads, "n_kv_heads": heads, "head_dim": d // heads,
                                             "softmax_scale": (d // heads) ** -0.5, "window": 0},
                        {"qkv_weight": "qkv.w", "qkv_bias": "qkv.b", "out_weight": "o.w", "out_bias": "o.b"})
        ffn = PartSpec("dense_ffn", {"hidden_size": d, "inner_size": r["inner"], "activation": "gelu_new"},
                       {"up_weight": "up.w", "up_bias": "up.b", "down_weight": "down.w", "down_bias": "down.b"})
        layer = LayerSpec("toy_sandwich", norm("n1"), attn, norm("n2"), ffn, extra=(("norm3", "norm", norm("n3")),))
        return ModelPlan("ToyModel3", r["vocab"], d, r["positions"],
                         PartSpec("token_embedding", {"vocab_size": r["vocab"], "hidden_size": d}, {"weight": "emb"}),
                         PartSpec("learned_absolute", {"max_positions": r["positions"], "hidden_size": d}, {"weight": "pos"}),
                         (layer,), default_schedule(1), norm("final"),
                         PartSpec("tied_head", {"vocab_size": r["vocab"], "hidden_size": d}))


def test_layer_with_an_extra_part(tmp_path):
    """A third norm in a layer: declared in the plan's LayerSpec, built, loaded and handed to the arrangement by
    name, with no change to the package."""
    register_part("arrangement", "toy_sandwich", ToySandwich, replace=True)
    register_architecture(Architecture(names=("toy3", "ToyModel3"), config_class=ToyConfig3), replace=True)
    raw = {"model_type": "toy3", "width": 48, "heads": 3, "inner": 72, "vocab": 97, "positions": 90}
    write_random_model(str(tmp_path), raw, seed=9)
    w = plain_gpt2.read_safetensors(str(tmp_path / "model.safetensors"))
    assert "n3.w" in w and "n3.b" in w

    def plain(ids):
        n = len(ids)
        x = w["emb"][ids] + w["pos"][:n]
        h = plain_gpt2.layer_norm(x, w["n1.w"], w["n1.b"], 1e-5)
        qkv = h @ w["qkv.w"].T + w["qkv.b"]
        a = plain_gpt2.causal_attention(qkv[:, :48], qkv[:, 48:96], qkv[:, 96:], 3, 3, 16 ** -0.5, 0)
        x = x + a @ w["o.w"].T + w["o.b"]
        h = plain_gpt2.layer_norm(x, w["n2.w"], w["n2.b"], 1e-5)
        y = plain_gpt2.gelu_new(h @ w["up.w"].T + w["up.b"]) @ w["down.w"].T + w["down.b"]
        x = x + plain_gpt2.layer_norm(y, w["n3.w"], w["n3.b"], 1e-5)
        return plain_gpt2.layer_norm(x, w["final.w"], w["final.b"], 1e-5) @ w["emb"].T

    model = DecoderModel.from_dir(str(tmp_path), dtype="float32")
    cache = model.new_cache(max_tokens=256, n_slots=3)
    rng = np.random.default_rng(4)
    reqs = [rng.integers(0, 97, size=n).tolist() for n in (70, 9, 33)]
    check_logits(run_whole(model, cache, reqs[0]), plain(reqs[0]), "float32", "toy3 whole")
    check_logits(run_tail_one_by_one(model, cache, reqs[0], 20), plain(reqs[0]), "float32", "toy3 tail")
    for g, r in zip(run_batch(model, cache, reqs, [40, 9, 1]), reqs):
        check_logits(g, plain(r), "float32", "toy3 batch")
