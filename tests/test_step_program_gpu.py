"""The single-token step recorded as one program for the persistent step
kernel (csrc/decode_program.cu) against the same step launched kernel by
kernel: same logits, same tokens, with sequences of unequal length whose pages
lie anywhere in the cache."""
import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import check_logits
from math_utils_b200 import DecoderModel, StepEntry
from math_utils_b200.engine.decode_session import DecodeSession
from math_utils_b200.sampling import SamplingParams

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_recorded_step_matches_plain_and_launched_step(name, model_dirs, plain_models):
    cfg, w = plain_models[name]
    model = DecoderModel.from_dir(model_dirs[name], dtype="bfloat16")
    rng = np.random.default_rng(3)
    top = cfg["n_positions"]
    lens = [top - 9, 1, 33, 64, 65][:5]
    reqs = [rng.integers(0, cfg["vocab_size"], size=n + 6).tolist() for n in lens]
    cache = model.new_cache(max_tokens=5 * 128 + 128, n_slots=6)
    spare = cache.acquire()                                   # shifts the others' pages away from zero
    model.step(cache, [StepEntry(spare, [1] * 70)])
    slots = [cache.acquire() for _ in reqs]
    model.step(cache, [StepEntry(s, r[:n]) for s, r, n in zip(slots, reqs, lens)])
    params = SamplingParams(temperature=0.0)
    session = DecodeSession(model, cache, slots, params, list(range(len(slots))), use_program=True)
    for step in range(6):
        for s in slots:
            cache.reserve(s, 1)
        session.sync_block_tables()
        session.feed([r[n + step] for r, n in zip(reqs, lens)], [n + step for n in lens])
        session.launch()
        tokens = session.read_tokens()
        assert session.program is not None and len(session.program.ops) == 2 + 5 * cfg["n_layer"]
        got = session.logits.float().cpu().numpy()
        want = np.stack([plain_gpt2.forward(r[:n + step + 1], cfg, w)[-1] for r, n in zip(reqs, lens)])
        check_logits(got, want, "bfloat16", f"{name} recorded step {step}")
        assert tokens == [int(np.argmax(g)) for g in got]
        for s in slots:
            cache.commit(s, 1)
    from math_utils_b200.csrc import ops
    ops.check_status()


def test_unrecordable_step_falls_back(model_dirs):
    """float32 has no recorded form: the session keeps launching kernel by kernel."""
    model = DecoderModel.from_dir(model_dirs["tiny_a"], dtype="float32")
    cache = model.new_cache(max_tokens=128, n_slots=1)
    slot = cache.acquire()
    model.step(cache, [StepEntry(slot, [5, 6, 7])])
    session = DecodeSession(model, cache, [slot], SamplingParams(temperature=0.0), [0], use_program=True)
    cache.reserve(slot, 1)
    session.sync_block_tables()
    session.feed([9], [3])
    session.launch()
    assert session.program is None and len(session.read_tokens()) == 1
