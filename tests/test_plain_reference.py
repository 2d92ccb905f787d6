"""The plain implementation against logits made by the reference's own code
(tests/golden/make_golden.py: its NumPy oracle and its C++ LocalModel), and
against itself where the reference has nothing to say."""
import os

import numpy as np
import pytest

import plain_gpt2
from golden import make_golden

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("k,name", list(enumerate(make_golden.GOLDEN_CONFIGS)))
def test_plain_matches_reference_code(k, name):
    cfg = make_golden.GOLDEN_CONFIGS[name]
    weights = {n: w.astype(np.float64) for n, w in make_golden.make_weights(cfg, seed=1234 + k).items()}
    ids = make_golden.GOLDEN_IDS[name]
    logits = plain_gpt2.forward(ids, cfg, weights)
    stored = np.load(os.path.join(GOLDEN, name + ".npz"))
    # the reference computes in float32: a few 1e-6 of rounding on logits of order 1
    assert np.abs(logits - stored["oracle"]).max() < 2e-5
    rows = stored["local_model_rows"]
    assert np.abs(logits[rows] - stored["local_model_whole"]).max() < 2e-5
    assert np.abs(logits[rows] - stored["local_model_stepwise"]).max() < 2e-5


def test_plain_matches_the_oracle_on_the_options_the_decoder_lacks():
    """n_inner = 320, erf GELU, scale_attn_by_inverse_layer_idx, eps 1e-6 (the second tiny test configuration):
    the reference's NumPy oracle run in float64 with its activation exchanged for the erf form and the
    layer-index scaling folded into the query weights (tests/golden/make_golden.py says how)."""
    cfg = make_golden.GOLDEN_C
    weights = {n: w.astype(np.float64) for n, w in make_golden.make_weights(cfg, seed=1236).items()}
    logits = plain_gpt2.forward(make_golden.GOLDEN_C_IDS, cfg, weights)
    stored = np.load(os.path.join(GOLDEN, "golden_c.npz"))
    assert np.abs(logits[stored["rows"]] - stored["oracle_rows"]).max() < 1e-9
    # and each of the three options moves the logits, so the comparison pins them
    for change in ({"activation_function": "gelu_new"}, {"scale_attn_by_inverse_layer_idx": False}):
        other = plain_gpt2.forward(make_golden.GOLDEN_C_IDS, dict(cfg, **change), weights)
        assert np.abs(other[stored["rows"]] - stored["oracle_rows"]).max() > 1e-5, change


def test_inverse_layer_scaling_is_identity_for_one_layer():
    cfg = dict(make_golden.GOLDEN_CONFIGS["golden_a"], n_layer=1)
    w = {n: a.astype(np.float64) for n, a in make_golden.make_weights(cfg, seed=5).items()}
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    a = plain_gpt2.forward(ids, cfg, w)
    b = plain_gpt2.forward(ids, dict(cfg, scale_attn_by_inverse_layer_idx=True), w)
    assert np.array_equal(a, b)
    cfg2 = dict(make_golden.GOLDEN_CONFIGS["golden_a"])
    w2 = {n: x.astype(np.float64) for n, x in make_golden.make_weights(cfg2, seed=5).items()}
    c = plain_gpt2.forward(ids, cfg2, w2)
    d = plain_gpt2.forward(ids, dict(cfg2, scale_attn_by_inverse_layer_idx=True), w2)
    assert np.abs(c - d).max() > 1e-4          # with two layers the flag matters


def test_erf_gelu_differs_from_tanh_gelu_slightly():
    x = np.linspace(-4, 4, 101)
    diff = np.abs(plain_gpt2.gelu_erf(x) - plain_gpt2.gelu_new(x)).max()
    assert 1e-5 < diff < 2e-3
    assert abs(plain_gpt2.gelu_erf(np.array([1.0]))[0] - 0.8413447460685429) < 1e-12


def test_attention_window_and_groups():
    rng = np.random.default_rng(0)
    T, H, Hkv, dh = 9, 4, 2, 16
    q = rng.standard_normal((T, H * dh))
    k = rng.standard_normal((T, Hkv * dh))
    v = rng.standard_normal((T, Hkv * dh))
    full = plain_gpt2.causal_attention(q, k, v, H, Hkv, 0.25)
    wide = plain_gpt2.causal_attention(q, k, v, H, Hkv, 0.25, window=T + 3)
    assert np.allclose(full, wide)
    one = plain_gpt2.causal_attention(q, k, v, H, Hkv, 0.25, window=1)
    for h in range(H):                           # a window of one sees only the token's own value
        assert np.allclose(one[:, h * dh:(h + 1) * dh], v[:, (h // 2) * dh:(h // 2 + 1) * dh])


def test_attention_forms_agree():
    """Query by query (include/ai/Kernels.hpp:132-161) and the masked score matrix
    (include/ai/GPT2.hpp:261-271) are the same attention, window or not."""
    rng = np.random.default_rng(5)
    T, H, Hkv, dh = 37, 6, 2, 10
    q, k, v = (rng.standard_normal((T, n * dh)) for n in (H, Hkv, Hkv))
    for window in (0, 1, 9, 50):
        a = plain_gpt2.causal_attention(q, k, v, H, Hkv, 0.3, window)
        b = plain_gpt2.causal_attention_masked(q, k, v, H, Hkv, 0.3, window)
        assert np.abs(a - b).max() < 1e-12, window


def test_sampling_rules():
    row = np.array([0.1, 2.0, 2.0, -1.0, 1.5], dtype=np.float32)
    assert plain_gpt2.argmax(row) == 1                      # first maximum wins
    assert plain_gpt2.sample_top_k(row, 0.0, 0, 0.7)[0] == 1
    assert plain_gpt2.sample_top_k(row, 1.0, 1, 0.7)[0] == 1
    assert plain_gpt2.sample_top_k(row, 1.0, 2, 0.0)[0] == 1       # walk starts at the best, lower index first
    assert plain_gpt2.sample_top_k(row, 1.0, 2, 0.999)[0] == 2
    assert plain_gpt2.sample_top_k(row, 1.0, -1, 0.999999)[0] == 3  # the smallest comes last
    assert plain_gpt2.sample_top_k(row, 1.0, 0, 0.999999)[0] == 1   # a count of 0 is greedy, as the reference's
    u = [plain_gpt2.uniform_draw(1, 2, n) for n in range(1000)]
    assert 0.0 <= min(u) and max(u) < 1.0 and 0.45 < float(np.mean(u)) < 0.55
    assert plain_gpt2.uniform_draw(1, 2, 3) != plain_gpt2.uniform_draw(1, 3, 3)
