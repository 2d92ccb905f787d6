"""The engine against the plain implementation, in 32-bit and in bfloat16:
each request alone and whole, with its last tokens one by one, and in batches
of unequal lengths one after another so that slots and pages are used again."""
import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import check_logits, run_batch, run_tail_one_by_one, run_whole
from math_utils_b200 import DecoderModel

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def requests_for(cfg, seed, lengths):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


@pytest.fixture(scope="module")
def engines(model_dirs):
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = DecoderModel.from_dir(model_dirs[name], dtype=dtype)
        return cache[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def plain_logits(plain_models):
    memo = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in memo:
            cfg, w = plain_models[name]
            memo[key] = plain_gpt2.forward(list(tokens), cfg, w)
        return memo[key]
    return get


LENGTHS = {"tiny_a": [5, 17, 32, 128, 70], "tiny_b": [1, 2, 9, 40, 63, 80], "tiny_c": [3, 64, 65, 150]}
NAMES = ["tiny_a", "tiny_b", "tiny_c"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests(name, dtype, engines, plain_models, plain_logits):
    model = engines(name, dtype)
    cfg = plain_models[name][0]
    cache = model.new_cache(max_tokens=256)
    for tokens in requests_for(cfg, 1, LENGTHS[name]):
        got = run_whole(model, cache, tokens)
        check_logits(got, plain_logits(name, tokens), dtype, f"{name} whole n={len(tokens)}")
    assert cache.slots.n_free == cache.n_slots and cache.free_pages() == cache.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_tokens_one_by_one(name, dtype, engines, plain_models, plain_logits):
    model = engines(name, dtype)
    cfg = plain_models[name][0]
    cache = model.new_cache(max_tokens=256)
    for tokens in requests_for(cfg, 2, LENGTHS[name][2:]):
        got = run_tail_one_by_one(model, cache, tokens, tail=32)
        check_logits(got, plain_logits(name, tokens), dtype, f"{name} tail n={len(tokens)}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_reuse_slots(name, dtype, engines, plain_models, plain_logits):
    model = engines(name, dtype)
    cfg = plain_models[name][0]
    top = cfg["n_positions"]
    # room for one batch only, so the second batch must take the first one's slots and pages
    totals_a = [top, 40, 66, 7]
    cache = model.new_cache(max_tokens=sum(-(-t // 64) * 64 for t in totals_a), n_slots=4)
    for round_, totals in enumerate([totals_a, [33, top, 12, 64], [top - 1, 3, 65, 20]]):
        reqs = requests_for(cfg, 10 + round_, totals)
        prompts = [max(1, min(t - 1, p)) for t, p in zip(totals, [17, 5, 64, 2])]
        got = run_batch(model, cache, reqs, prompts)
        for i, (g, r) in enumerate(zip(got, reqs)):
            check_logits(g, plain_logits(name, r), dtype, f"{name} batch {round_} request {i}")
        assert cache.slots.n_free == 4 and cache.free_pages() == cache.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
def test_split_prompt_equals_whole(dtype, engines, plain_models, plain_logits):
    """A prompt fed in two parts (the second starts at a filled cache)."""
    from math_utils_b200 import StepEntry
    name = "tiny_b"
    model = engines(name, dtype)
    tokens = requests_for(plain_models[name][0], 5, [71])[0]
    cache = model.new_cache(max_tokens=128)
    slot = cache.acquire()
    a = model.step(cache, [StepEntry(slot, tokens[:30], list(range(30)))]).cpu().numpy()
    b = model.step(cache, [StepEntry(slot, tokens[30:], list(range(41)))]).cpu().numpy()
    cache.release(slot)
    check_logits(np.concatenate([a, b]), plain_logits(name, tokens), dtype, "split prompt")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_one_token(dtype, engines, plain_models, plain_logits):
    """The first tokens of a sequence and a long run of single-token steps."""
    name = "tiny_a"
    model = engines(name, dtype)
    tokens = requests_for(plain_models[name][0], 6, [128])[0]
    cache = model.new_cache(max_tokens=128)
    got = run_tail_one_by_one(model, cache, tokens, tail=127)
    check_logits(got, plain_logits(name, tokens), dtype, "decode from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_stage_trace_matches_plain(dtype, engines, plain_models):
    """``step(..., trace=...)`` hands out every stage by name; each is held against the plain
    model's stage of the same name, for a prompt and for a single-token step after it, so a wrong
    logit can be followed back to the first stage that is off."""
    from math_utils_b200 import StepEntry
    name = "tiny_b"
    cfg, w = plain_models[name]
    model = engines(name, dtype)
    tokens = requests_for(cfg, 8, [41])[0]
    want = {}
    plain_gpt2.forward(tokens, cfg, w, trace=want)
    cache = model.new_cache(max_tokens=128)
    slot = cache.acquire()
    got_prompt, got_step = {}, {}
    model.step(cache, [StepEntry(slot, tokens[:40], [39])], trace=got_prompt)
    model.step(cache, [StepEntry(slot, tokens[40:], [0])], trace=got_step)
    cache.release(slot)
    names = ["embed"] + [f"h.{i}.{s}" for i in range(cfg["n_layer"])
                         for s in ("ln1", "qkv", "attn", "res1", "ln2", "act", "res2")] + ["lnf", "logits"]
    assert list(got_prompt) == names and list(got_step) == names          # in the order they are computed
    for n in names:
        full = want[n]
        for got, rows in ((got_prompt[n], full[:40] if n not in ("lnf", "logits") else full[39:40]),
                          (got_step[n], full[40:41])):
            assert got.shape == rows.shape, n
            scale = max(float(np.abs(rows).max()), 1.0)
            bound = 1e-4 * scale if dtype == "float32" else 0.03 * scale
            assert np.abs(got - rows).max() < bound, (n, float(np.abs(got - rows).max()), scale)
    # the trace changes nothing
    slot = cache.acquire()
    a = model.step(cache, [StepEntry(slot, tokens[:40], [39])]).cpu().numpy()
    cache.release(slot)
    assert np.array_equal(a, got_prompt["logits"])


def test_step_refuses_what_it_cannot_run(engines, plain_models):
    """A token outside the vocabulary, a wanted place outside the tokens given, a slot named twice: each is an
    error before anything runs, and the cache holds what it held."""
    from math_utils_b200 import StepEntry
    cfg, _ = plain_models["tiny_a"]
    model = engines("tiny_a", "float32")
    cache = model.new_cache(max_tokens=256, n_slots=3)
    a, b = cache.acquire(), cache.acquire()
    model.step(cache, [StepEntry(a, [1, 2, 3])])
    free = cache.free_pages(0)
    with pytest.raises(ValueError, match=f"token id {cfg['vocab_size']} is outside the vocabulary"):
        model.step(cache, [StepEntry(a, [4]), StepEntry(b, [1, cfg["vocab_size"], 2])])
    with pytest.raises(ValueError, match="token id -1 is outside"):
        model.step(cache, [StepEntry(b, [-1])])
    with pytest.raises(ValueError, match="twice"):
        model.step(cache, [StepEntry(a, [4]), StepEntry(a, [5])])
    with pytest.raises(ValueError, match="flat list"):
        model.step(cache, [StepEntry(b, [[1, 2], [3, 4]])])
    with pytest.raises(ValueError, match="want index 3"):
        model.step(cache, [StepEntry(b, [1, 2, 3], [3])])
    assert cache.length(a) == 3 and cache.length(b) == 0 and cache.free_pages(0) == free
    out = model.step(cache, [StepEntry(b, [1, 2, 3], [2])])          # the slot still works
    assert out.shape == (1, cfg["vocab_size"]) and cache.length(b) == 3
    cache.release(a); cache.release(b)
    assert cache.slots.n_free == 3 and cache.free_pages(0) == cache.n_pages
