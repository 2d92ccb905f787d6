"""Each part alone, and a toy architecture defined here, outside the package:
a mixer with state of its own, a layer that runs twice, a layer that reads
another layer's cache.  Nothing of the package is changed to run it."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import check_logits, run_batch, run_tail_one_by_one, run_whole
from math_utils_b200 import DecoderModel, StepEntry, register_architecture, write_random_model
from math_utils_b200.cache import SequenceCache
from math_utils_b200.config import (Architecture, ConfigError, LayerSpec, ModelPlan, PartSpec,
                                    ScheduleEntry)
from math_utils_b200.engine.batch import PinnedRing, build_context
from math_utils_b200.engine.runtime import Runtime
from math_utils_b200.parts import Mixer, StateCacheSpec, TensorSpec, build_part, register_part

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


from test_kernels_gpu import assert_close


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to("cuda", dtype)


def context_for(runtime, cache, entries, position=None):
    starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
    position = position or build_part("position", PartSpec("none"))
    return build_context(runtime, position, cache, entries, starts, PinnedRing(), {})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    rt = Runtime.create(dtype)
    rng = np.random.default_rng(0)
    part = build_part("norm", PartSpec("layer_norm", {"size": 200, "eps": 1e-4}, {"weight": "g", "bias": "b"}))
    assert [s.shape for s in part.tensor_specs()] == [(200,), (200,)]
    g, b = rng.standard_normal(200), rng.standard_normal(200)
    part.bind({"g": dev(g), "b": dev(b)}, rt)
    x = rng.standard_normal((9, 200)) * 2 + 1
    got = part.forward(dev(x)).float().cpu().numpy()
    assert_close(got, plain_gpt2.layer_norm(x.astype(np.float32).astype(np.float64), g, b, 1e-4), dtype, "norm part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("activation,layout", [("gelu_new", "in_out"), ("gelu", "out_in")])
def test_feed_forward_part(activation, layout, dtype):
    rt = Runtime.create(dtype)
    rng = np.random.default_rng(1)
    d, inner = 72, 200
    spec = PartSpec("dense_ffn", {"hidden_size": d, "inner_size": inner, "activation": activation,
                                  "weight_layout": layout},
                    {"up_weight": "u", "up_bias": "ub", "down_weight": "dn", "down_bias": "db"})
    part = build_part("feed_forward", spec)
    shapes = {s.name: s for s in part.tensor_specs()}
    assert shapes["u"].shape == ((d, inner) if layout == "in_out" else (inner, d))
    assert shapes["u"].transpose == (layout == "in_out") and shapes["dn"].init == "residual_projection"
    wu = dev(rng.standard_normal((inner, d)) / math.sqrt(d), DT[dtype])
    wd = dev(rng.standard_normal((d, inner)) / math.sqrt(inner), DT[dtype])
    ub, db = rng.standard_normal(inner), rng.standard_normal(d)
    part.bind({"u": wu, "ub": dev(ub), "dn": wd, "db": dev(db)}, rt)
    h = dev(rng.standard_normal((7, d)), DT[dtype])
    x0 = rng.standard_normal((7, d))
    x = dev(x0)
    part.forward(h, x, None)
    hh = h.double().cpu().numpy()
    u = plain_gpt2.ACTIVATIONS[activation](hh @ wu.double().cpu().numpy().T + ub)
    want = x0.astype(np.float32).astype(np.float64) + u @ wd.double().cpu().numpy().T + db
    assert_close(x.cpu().numpy(), want, dtype, "feed-forward part")
    with pytest.raises(ConfigError, match="activation"):
        build_part("feed_forward", PartSpec("dense_ffn", dict(spec.params, activation="relu"), spec.tensors))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [(4, 4, 16, 0), (6, 2, 32, 0), (3, 1, 48, 50)])
def test_attention_part(n_heads, n_kv_heads, head_dim, window, dtype):
    """Two sequences of unequal length as one step, then one more token each;
    grouped heads and a window, which GPT-2 itself never asks for."""
    rt = Runtime.create(dtype)
    rng = np.random.default_rng(2)
    d = 80
    qw, kvw = n_heads * head_dim, n_kv_heads * head_dim
    scale = 0.9 / math.sqrt(head_dim)
    spec = PartSpec("causal_attention",
                    {"hidden_size": d, "n_heads": n_heads, "n_kv_heads": n_kv_heads, "head_dim": head_dim,
                     "softmax_scale": scale, "window": window},
                    {"qkv_weight": "w", "qkv_bias": "b", "out_weight": "ow", "out_bias": "ob"})
    part = build_part("mixer", spec)
    assert part.cache_spec().window == window and part.cache_spec().n_kv_heads == n_kv_heads
    w = dev(rng.standard_normal((qw + 2 * kvw, d)) / math.sqrt(d), DT[dtype])
    ow = dev(rng.standard_normal((d, qw)) / math.sqrt(qw), DT[dtype])
    b, ob = rng.standard_normal(qw + 2 * kvw), rng.standard_normal(d)
    part.bind({"w": w, "b": dev(b), "ow": ow, "ob": dev(ob)}, rt)
    cache = SequenceCache([part.cache_spec()], 512, 200, DT[dtype], "cuda")
    lens = [70, 9]
    hs = [rng.standard_normal((n + 1, d)) for n in lens]
    slots = [cache.acquire() for _ in lens]

    def plain(hfull):
        hq = dev(hfull, DT[dtype]).double().cpu().numpy()
        qkv = hq @ w.double().cpu().numpy().T + b
        if dtype == "bfloat16":
            qkv = dev(qkv, DT[dtype]).double().cpu().numpy()
        a = plain_gpt2.causal_attention(qkv[:, :qw], qkv[:, qw:qw + kvw], qkv[:, qw + kvw:], n_heads, n_kv_heads,
                                        scale, window)
        return a @ ow.double().cpu().numpy().T + ob

    entries = [StepEntry(s, [0] * n) for s, n in zip(slots, lens)]
    ctx = context_for(rt, cache, entries)
    h = dev(np.concatenate([x[:n] for x, n in zip(hs, lens)]), DT[dtype])
    x = torch.zeros((sum(lens), d), device="cuda")
    part.forward(h, x, ctx, cache.entry(0), True)
    for e in entries:
        cache.commit(e.slot, len(e.tokens))
    want = np.concatenate([plain(full)[:n] for full, n in zip(hs, lens)])
    assert_close(x.cpu().numpy(), want, dtype, "attention part, prompts")
    entries = [StepEntry(s, [0]) for s in slots]
    ctx = context_for(rt, cache, entries)
    h = dev(np.stack([x[n] for x, n in zip(hs, lens)]), DT[dtype])
    x = torch.zeros((2, d), device="cuda")
    part.forward(h, x, ctx, cache.entry(0), True)
    want = np.stack([plain(full)[n] for full, n in zip(hs, lens)])
    assert_close(x.cpu().numpy(), want, dtype, "attention part, one token each")


def test_embedding_position_and_head_parts():
    rt = Runtime.create("float32")
    rng = np.random.default_rng(3)
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 50, "hidden_size": 24}, {"weight": "e"}))
    pos = build_part("position", PartSpec("learned_absolute", {"max_positions": 30, "hidden_size": 24}, {"weight": "p"}))
    head = build_part("head", PartSpec("tied_head", {"vocab_size": 50, "hidden_size": 24}))
    e, p = rng.standard_normal((50, 24)), rng.standard_normal((30, 24))
    emb.bind({"e": dev(e)}, rt); pos.bind({"p": dev(p)}, rt); head.bind({}, rt)
    head.attach_embedding(emb)
    cache = SequenceCache([], 64, 30, torch.float32, "cuda")
    s = cache.acquire()
    cache.reserve(s, 4); cache.commit(s, 4)                      # the sequence already holds 4 tokens
    ctx = context_for(rt, cache, [StepEntry(s, [7, 49, 0])], position=pos)
    x = emb.forward(ctx, pos.embedding_table()).cpu().numpy()
    assert np.allclose(x, (e[[7, 49, 0]] + p[[4, 5, 6]]).astype(np.float32), atol=1e-6)
    logits = head.forward(dev(x)).cpu().numpy()
    assert_close(logits, x.astype(np.float64) @ e.astype(np.float32).astype(np.float64).T, "float32", "tied head")


# ------------------------------------------------------------------ a toy architecture
class RunningMeanMixer(Mixer):
    """Output at a token = gain * mean of the inputs of all tokens so far.
    Keeps a fixed-size state per sequence: the running sum and the count."""
    graph_safe = False          # walks the step's sequences on the host

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("gain"), (self.hidden,), role="vector", init="norm_weight"),)

    def cache_spec(self):
        return StateCacheSpec(self.hidden + 1)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.gain = tensors[self.tensor_name("gain")]

    def forward(self, h, residual, ctx, cache, owns_cache):
        o = 0
        for slot, n in zip(ctx.slots, ctx.q_lens):
            state = cache.values[slot]
            sums = state[:self.hidden] + torch.cumsum(h[o:o + n].float(), dim=0)
            counts = state[self.hidden] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
            residual[o:o + n] += self.gain * sums / counts[:, None]
            if owns_cache:
                state[:self.hidden] = sums[-1]
                state[self.hidden] = counts[-1]
            o += n


class ToyConfig:
    """Three layers: attention, running-mean mixer, attention that reads layer
    0's keys and values; layer 0 runs a second time at the end."""

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
        d, v, p, heads = self.raw["width"], self.raw["vocab"], self.raw["positions"], self.raw["heads"]
        dh = d // heads

        def norm(name):
            return PartSpec("layer_norm", {"size": d, "eps": 1e-5}, {"weight": name + ".w", "bias": name + ".b"})

        def attn(i, kv_heads):
            return PartSpec("causal_attention", {"hidden_size": d, "n_heads": heads, "n_kv_heads": kv_heads,
                                                 "head_dim": dh, "softmax_scale": dh ** -0.5},
                            {"qkv_weight": f"l{i}.qkv.w", "qkv_bias": f"l{i}.qkv.b",
                             "out_weight": f"l{i}.o.w", "out_bias": f"l{i}.o.b"})

        def ffn(i, act):
            return PartSpec("dense_ffn", {"hidden_size": d, "inner_size": 2 * d + 8, "activation": act},
                            {"up_weight": f"l{i}.up.w", "up_bias": f"l{i}.up.b",
                             "down_weight": f"l{i}.down.w", "down_bias": f"l{i}.down.b"})

        mixers = [attn(0, heads), PartSpec("toy_running_mean", {"hidden_size": d}, {"gain": "l1.gain"}), attn(2, heads)]
        layers = tuple(LayerSpec("pre_norm", norm(f"l{i}.n1"), mixers[i], norm(f"l{i}.n2"),
                                 ffn(i, "gelu" if i == 1 else "gelu_new")) for i in range(3))
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 0), ScheduleEntry(0, 3))
        return ModelPlan("ToyModel", v, d, p,
                         PartSpec("token_embedding", {"vocab_size": v, "hidden_size": d}, {"weight": "emb"}),
                         PartSpec("learned_absolute", {"max_positions": p, "hidden_size": d}, {"weight": "pos"}),
                         layers, schedule, norm("final"), PartSpec("tied_head", {"vocab_size": v, "hidden_size": d}))


def toy_plain(ids, raw, w):
    """The toy model, whole sequence, in float64 NumPy."""
    d, heads = raw["width"], raw["heads"]
    x = w["emb"][ids] + w["pos"][:len(ids)]
    kv0 = None
    for layer, cache_of in ((0, "own"), (1, None), (2, "layer0"), (0, "own")):
        p = f"l{layer}"
        h = plain_gpt2.layer_norm(x, w[p + ".n1.w"], w[p + ".n1.b"], 1e-5)
        if layer == 1:
            x = x + w["l1.gain"] * np.cumsum(h, axis=0) / np.arange(1, len(ids) + 1)[:, None]
        else:
            qkv = h @ w[p + ".qkv.w"].T + w[p + ".qkv.b"]
            q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
            if layer == 0 and kv0 is None:
                kv0 = (k, v)
            if cache_of == "layer0":
                k, v = kv0
            a = plain_gpt2.causal_attention(q, k, v, heads, heads, (d // heads) ** -0.5)
            x = x + a @ w[p + ".o.w"].T + w[p + ".o.b"]
        h = plain_gpt2.layer_norm(x, w[p + ".n2.w"], w[p + ".n2.b"], 1e-5)
        act = plain_gpt2.gelu_erf if layer == 1 else plain_gpt2.gelu_new
        x = x + act(h @ w[p + ".up.w"].T + w[p + ".up.b"]) @ w[p + ".down.w"].T + w[p + ".down.b"]
    return plain_gpt2.layer_norm(x, w["final.w"], w["final.b"], 1e-5) @ w["emb"].T


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    register_part("mixer", "toy_running_mean", RunningMeanMixer, replace=True)
    register_architecture(Architecture(names=("toy", "ToyModel"), config_class=ToyConfig), replace=True)
    raw = {"model_type": "toy", "width": 48, "heads": 3, "vocab": 211, "positions": 150}
    d = tmp_path_factory.mktemp("toy")
    write_random_model(str(d), raw, seed=77)
    return str(d), raw


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_with_state_shared_cache_and_repeated_layer(toy_dir, dtype):
    folder, raw = toy_dir
    model = DecoderModel.from_dir(folder, dtype=dtype)
    cache = model.new_cache(max_tokens=512, n_slots=4)
    assert len(cache.kv_groups) == 1 and cache.kv_groups[0].entries == [0, 3]      # entry 2 borrows entry 0's
    assert len(cache.state_groups) == 1 and cache.state_groups[0].entries == [1]
    w = plain_gpt2.read_safetensors(folder + "/model.safetensors")
    rng = np.random.default_rng(8)
    reqs = [rng.integers(0, raw["vocab"], size=n).tolist() for n in (150, 33, 70, 5)]
    want = [toy_plain(r, raw, w) for r in reqs]
    for r, wnt in zip(reqs, want):
        check_logits(run_whole(model, cache, r), wnt, dtype, "toy whole")
    check_logits(run_tail_one_by_one(model, cache, reqs[0], 32), want[0], dtype, "toy tail")
    for round_ in range(2):             # the second round reuses slots whose state must start at zero
        got = run_batch(model, cache, reqs, [100, 33 - 1, 7, 2])
        for g, wnt in zip(got, want):
            check_logits(g, wnt, dtype, f"toy batch {round_}")
    assert cache.slots.n_free == 4
