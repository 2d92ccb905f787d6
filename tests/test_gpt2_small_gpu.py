"""GPT-2 small's sizes (12 layers, width 768, 12 heads, vocabulary 50257) with
random weights: the engine against the plain implementation, whole and with
the last tokens one by one, in 32-bit and in bfloat16, and a batch of unequal
prompts.  The width, the vocabulary (odd, so rows of logits are not 16-byte
aligned) and the depth are the ones the benchmark runs at."""
import numpy as np
import pytest

import plain_gpt2
from helpers import BF16_NEAR_TIE, check_logits, run_batch, run_tail_one_by_one
from math_utils_b200 import DecoderModel, write_random_model

pytestmark = pytest.mark.gpu

SMALL = {"model_type": "gpt2", "n_layer": 12, "n_embd": 768, "n_head": 12, "n_inner": 3072,
         "activation_function": "gelu_new", "vocab_size": 50257, "n_positions": 1024,
         "layer_norm_epsilon": 1e-5, "initializer_range": 0.05}


@pytest.fixture(scope="module")
def small(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("gpt2_small"))
    write_random_model(folder, SMALL, seed=2024)
    cfg, weights = plain_gpt2.read_model(folder)
    rng = np.random.default_rng(0)
    requests = [rng.integers(0, 50257, size=n).tolist() for n in (150, 70, 33)]
    want = [plain_gpt2.forward(r, cfg, weights) for r in requests]
    return folder, requests, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpt2_small_sizes(small, dtype):
    folder, requests, want = small
    model = DecoderModel.from_dir(folder, dtype=dtype)
    cache = model.new_cache(max_tokens=512, n_slots=4)
    got = run_tail_one_by_one(model, cache, requests[0], tail=32)
    check_logits(got, want[0], dtype, "prefix whole, last 32 one by one")
    got = run_batch(model, cache, requests, [110, 69, 5])
    for i, (g, w) in enumerate(zip(got, want)):
        check_logits(g, w, dtype, f"batch request {i}")
    assert cache.slots.n_free == 4 and cache.free_pages() == cache.n_pages


def test_overlapped_launches_change_no_bit(small):
    """Kernels launched with programmatic stream serialization start while the
    kernel before them drains; nothing a predecessor writes may be read before
    the dependency wait.  The same prompt step, single-token steps and graphed
    generation with the overlap off and on must agree to the bit."""
    import torch
    from math_utils_b200 import LLM, Options, StepEntry
    from math_utils_b200.csrc import ops
    folder, requests, _ = small
    results = []
    try:
        for overlapped in (False, True):
            ops.set_pdl(overlapped)
            model = DecoderModel.from_dir(folder, dtype="bfloat16")
            cache = model.new_cache(max_tokens=1024, n_slots=4)
            slots = [cache.acquire() for _ in requests]
            logits = [model.step(cache, [StepEntry(s, r[:-8], [len(r) - 9]) for s, r in zip(slots, requests)]).clone()]
            for k in range(8, 0, -1):
                logits.append(model.step(cache, [StepEntry(s, [r[-k]], [0]) for s, r in zip(slots, requests)]).clone())
            llm = LLM(folder, Options(dtype="bfloat16", temperature=0.0))
            tokens = llm.generate([r[:40] for r in requests], max_tokens=12, stop_ids=[])
            results.append((torch.cat(logits), tokens))
            ops.check_status()
    finally:
        ops.set_pdl(True)
    assert torch.equal(results[0][0], results[1][0])
    assert results[0][1] == results[1][1]


# ------------------------------------------------------------------ the schedules the benchmark runs
# GPT-2 small's layer sizes with two layers (the float64 plain model stays affordable): batches of 24,
# 40 and 64 sequences, prompts of 300 to 900 tokens in one step, then single-token steps; the paths a
# batch of 17 to 64 takes (norm as its own launch, few-rows products with 4 to 8 row tiles and the cut
# over a cluster, the tcgen05 product inside a recorded graph, the 2-warp ring of the attention) and
# contexts of many pages are reached by nothing smaller.
WIDE = dict(SMALL, n_layer=2)
N_DECODE = 26


def tokens_near_plain(plain_rows, tokens, what):
    """Greedy tokens against the plain logits of the same history: each must be the plain argmax, or
    within bfloat16's noise of it (a near tie that the other precision may resolve the other way)."""
    for i, (row, tok) in enumerate(zip(plain_rows, tokens)):
        best = int(np.argmax(row))
        if tok != best:
            gap = (row[best] - row[tok]) / row.std()
            assert gap < BF16_NEAR_TIE, f"{what}: token {i} is {tok}, plain says {best} ({gap:.4f} of the spread apart)"


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("gpt2_wide"))
    write_random_model(folder, WIDE, seed=77)
    cfg, weights = plain_gpt2.read_model(folder)
    rng = np.random.default_rng(5)
    prompt_lens = rng.integers(300, 901, size=64).tolist()
    prompt_lens[3], prompt_lens[40] = 900, 300
    # a request has its prompt and the tokens its single-token steps are fed; some end early
    totals = [p + (N_DECODE if i % 5 else 7 + i % 11) for i, p in enumerate(prompt_lens)]
    requests = [rng.integers(0, 50257, size=n).tolist() for n in totals]
    memo = {}

    def plain_rows(i, first, tokens=None):
        """Plain logits of request i (or of `tokens`) at positions first.."""
        ids = requests[i] if tokens is None else tokens
        key = (i, first, tuple(ids[-40:]), len(ids))
        if key not in memo:
            memo[key] = plain_gpt2.forward(ids, cfg, weights, rows=list(range(first, len(ids))))
        return memo[key]
    return folder, cfg, requests, prompt_lens, plain_rows


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("members", [range(3, 4), range(38, 41), range(0, 24), range(24, 64), range(0, 64)],
                         ids=["b1", "b3", "b24", "b40", "b64"])
def test_wide_batches_step_by_step(wide, members, dtype):
    """Prompts in one step, then one token each through ``model.step``; logits of each prompt's last
    position and of every single-token step against the plain model; shorter requests end early; the
    same slots and pages serve a second batch."""
    folder, cfg, requests, prompt_lens, plain_rows = wide
    if dtype == "float32" and len(members) > 24:
        pytest.skip("the 32-bit path at this size is covered by the batch of 24")
    from math_utils_b200 import StepEntry
    from math_utils_b200.csrc import ops
    model = DecoderModel.from_dir(folder, dtype=dtype)
    members = list(members)
    cache = model.new_cache(max_tokens=sum(-(-len(requests[i]) // 64) * 64 for i in members), n_slots=len(members))
    for round_ in range(2):
        order = members if round_ == 0 else members[::-1]
        slots = {i: cache.acquire() for i in order}
        pos = {i: prompt_lens[i] for i in order}
        out = model.step(cache, [StepEntry(slots[i], requests[i][:pos[i]], [pos[i] - 1]) for i in order])
        got = {i: [row] for i, row in zip(order, out.float().cpu().numpy())}
        live = list(order)
        while live:
            out = model.step(cache, [StepEntry(slots[i], [requests[i][pos[i]]], [0]) for i in live])
            for i, row in zip(live, out.float().cpu().numpy()):
                got[i].append(row)
                pos[i] += 1
            for i in [i for i in live if pos[i] >= len(requests[i])]:
                cache.release(slots.pop(i))
                live.remove(i)
        ops.check_status()
        for i in order:
            check_logits(np.stack(got[i]), plain_rows(i, prompt_lens[i] - 1), dtype, f"round {round_} request {i}")
        assert cache.slots.n_free == len(members) and cache.free_pages() == cache.n_pages


@pytest.mark.parametrize("members", [range(3, 4), range(38, 41), range(0, 24), range(24, 64), range(0, 64)],
                         ids=["b1", "b3", "b24", "b40", "b64"])
def test_wide_batches_generate(wide, members):
    """The same batches through ``LLM.generate`` (graph replay, the host one step behind): greedy tokens
    against the plain model fed the same history, requests of unequal budgets, twice on one cache."""
    folder, cfg, requests, prompt_lens, plain_rows = wide
    from math_utils_b200 import LLM, Options
    llm = LLM(folder, Options(dtype="bfloat16", temperature=0.0, max_batch=64))
    members = list(members)
    prompts = [requests[i][:prompt_lens[i]] for i in members]
    first = llm.generate(prompts, max_tokens=N_DECODE, stop_ids=[])
    again = llm.generate(prompts, max_tokens=N_DECODE, stop_ids=[])
    assert first == again                                    # same slots, pages and graphs, same tokens
    for i, p, g in zip(members, prompts, first):
        assert len(g) == N_DECODE
        rows = plain_rows(i, len(p) - 1, p + g[:-1])
        tokens_near_plain(rows, g, f"request {i}")
    # a stop token ends some requests early: what they produced is a prefix of the free run
    stop = {first[0][5]} | ({first[1][9]} if len(first) > 1 else set())
    cut = llm.generate(prompts, max_tokens=N_DECODE, stop_ids=sorted(stop))
    for g, f in zip(cut, first):
        n = next((k for k, t in enumerate(f) if t in stop), len(f))
        assert g == f[:n]
    assert len(cut[0]) <= 5 and (len(cut) == 1 or len(cut[1]) <= 9)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_thousand_tokens(wide, dtype):
    """One request that fills 16 pages: the prefix whole, the last 32 tokens one by one."""
    folder, cfg, requests, prompt_lens, plain_rows = wide
    rng = np.random.default_rng(9)
    tokens = rng.integers(0, 50257, size=1000).tolist()
    model = DecoderModel.from_dir(folder, dtype=dtype)
    cache = model.new_cache(max_tokens=1024, n_slots=1)
    got = run_tail_one_by_one(model, cache, tokens, tail=32)
    _, weights = plain_gpt2.read_model(folder)
    check_logits(got[-40:], plain_gpt2.forward(tokens, cfg, weights, rows=list(range(960, 1000))), dtype,
                 "1,000 tokens, the last 40 positions")


# GPT-2 XL's ragged sizes in one layer: width 1,600 (no multiple of 128), 25 heads, inner 6,400
XL_LAYER = {"model_type": "gpt2", "n_layer": 1, "n_embd": 1600, "n_head": 25, "n_inner": 6400,
            "activation_function": "gelu_new", "vocab_size": 50257, "n_positions": 1024,
            "layer_norm_epsilon": 1e-5, "initializer_range": 0.04}


@pytest.mark.parametrize("batch", [5, 40])
def test_xl_sizes_in_a_batch(tmp_path_factory, batch):
    folder = str(tmp_path_factory.mktemp("gpt2_xl_layer"))
    write_random_model(folder, XL_LAYER, seed=3)
    cfg, weights = plain_gpt2.read_model(folder)
    rng = np.random.default_rng(batch)
    prompt_lens = rng.integers(20, 200, size=batch).tolist()
    requests = [rng.integers(0, 50257, size=p + 9).tolist() for p in prompt_lens]
    model = DecoderModel.from_dir(folder, dtype="bfloat16")
    cache = model.new_cache(max_tokens=batch * 256, n_slots=batch)
    got = run_batch(model, cache, requests, prompt_lens)
    for i, (g, r, p) in enumerate(zip(got, requests, prompt_lens)):
        want = plain_gpt2.forward(r, cfg, weights, rows=list(range(p - 1, len(r))))
        check_logits(g[p - 1:], want, "bfloat16", f"request {i}")
    from math_utils_b200 import LLM, Options
    llm = LLM(folder, Options(dtype="bfloat16", temperature=0.0, max_batch=64))
    prompts = [r[:p] for r, p in zip(requests, prompt_lens)]
    out = llm.generate(prompts, max_tokens=8, stop_ids=[])
    for i in range(0, batch, 7):
        rows = plain_gpt2.forward(prompts[i] + out[i][:-1], cfg, weights,
                                  rows=list(range(prompt_lens[i] - 1, prompt_lens[i] + 7)))
        tokens_near_plain(rows, out[i], f"request {i}")
