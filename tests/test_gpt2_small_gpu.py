"""GPT-2 small's sizes (12 layers, width 768, 12 heads, vocabulary 50257) with
random weights: the engine against the plain implementation, whole and with
the last tokens one by one, in 32-bit and in bfloat16, and a batch of unequal
prompts.  The width, the vocabulary (odd, so rows of logits are not 16-byte
aligned) and the depth are the ones the benchmark runs at."""
import numpy as np
import pytest

import plain_gpt2
from helpers import check_logits, run_batch, run_tail_one_by_one
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
