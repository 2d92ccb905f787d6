"""Shared test set-up: the ``gpu`` marker, tiny configurations, model folders."""
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)

# Two tiny GPT-2 configurations that differ in every size and option.
TINY_A = {
    "model_type": "gpt2", "architectures": ["GPT2LMHeadModel"],
    "n_layer": 2, "n_embd": 64, "n_head": 4, "n_inner": 256, "activation_function": "gelu_new",
    "vocab_size": 512, "n_positions": 128, "layer_norm_epsilon": 1e-5,
    "scale_attn_by_inverse_layer_idx": False, "eos_token_id": 7,
}
TINY_B = {
    "model_type": "gpt2", "architectures": ["GPT2LMHeadModel"],
    "n_layer": 3, "n_embd": 96, "n_head": 3, "n_inner": 320, "activation_function": "gelu",
    "vocab_size": 1031, "n_positions": 80, "layer_norm_epsilon": 1e-6,
    "scale_attn_by_inverse_layer_idx": True, "eos_token_id": [11, 500],
}
# head size 20: no multiple of 16, which GPT-2's config.json allows (n_embd / n_head)
TINY_C = {
    "model_type": "gpt2", "architectures": ["GPT2LMHeadModel"],
    "n_layer": 2, "n_embd": 100, "n_head": 5, "activation_function": "gelu_new",
    "vocab_size": 333, "n_positions": 150, "layer_norm_epsilon": 1e-5,
}
TINY = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors, random weights."""
    from math_utils_b200.weights import write_random_model
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        d = tmp_path_factory.mktemp(name)
        # a larger spread than the default 0.02 so that logits differ visibly between tokens
        write_random_model(str(d), dict(cfg, initializer_range=0.08), seed=100 + i)
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    import plain_gpt2
    return {name: plain_gpt2.read_model(d) for name, d in model_dirs.items()}


def pytest_terminal_summary(terminalreporter):
    """How much of their bounds the logit comparisons used: a bound that is never approached pins little."""
    try:
        import helpers
    except ImportError:
        return
    for dtype, (used, what) in helpers.OBSERVED.items():
        if used > 0.0:
            terminalreporter.write_line(f"logits, {dtype}: largest error was {used:.2f} of its bound ({what})")
