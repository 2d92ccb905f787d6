"""Makes the golden logits under tests/golden/ from the reference's own code.

Run once, by hand, on a machine that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

Two statements of GPT-2 in the reference are run on tiny random models made by
``make_weights`` below (plain NumPy, seeded):
  * the NumPy oracle ``tools/gpt2_oracle.py`` (``forward``), imported;
  * the C++ decoder ``ai::LocalModel`` (include/ai/LocalModel.hpp), compiled
    with g++ against the reference's headers from the small driver
    ``local_model_probe.cpp`` beside this script, whole prompt and token by token.
The reference's C++ decoder fixes the feed-forward width at four times the
model width and the tanh GELU and does not know ``scale_attn_by_inverse_layer_idx``
(include/ai/LocalModel.hpp:538, 547, 767-768), so ``golden_a`` and ``golden_b`` keep
to what it has.  ``golden_c`` pins the other options (``n_inner`` = 320, erf GELU,
the layer-index scaling, eps 1e-6: the second tiny test configuration) on the
reference's NumPy oracle, which takes any feed-forward width as it is: its one
activation function is exchanged for the erf form for that run (``math.erf``; the
oracle has only the tanh form, tools/gpt2_oracle.py:221-227), and the scaling
1 / (layer + 1) of the scores is folded into the query columns of ``c_attn``
(weight and bias), which is the same arithmetic since the scores are linear in the
queries.  Everything else of that run (embedding, norms, masking, softmax, head
split, projections, the tied head) is the oracle's own code.
``tests/test_plain_reference.py`` rebuilds the same weights and checks the plain
implementation against the stored logits.
"""
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

GOLDEN_CONFIGS = {
    "golden_a": {"model_type": "gpt2", "n_layer": 2, "n_embd": 64, "n_head": 4, "vocab_size": 512,
                 "n_positions": 128, "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new"},
    "golden_b": {"model_type": "gpt2", "n_layer": 3, "n_embd": 96, "n_head": 3, "vocab_size": 1031,
                 "n_positions": 80, "layer_norm_epsilon": 1e-6, "activation_function": "gelu_new"},
}
# the second tiny test configuration, every option the C++ decoder lacks switched on; oracle only
GOLDEN_C = {"model_type": "gpt2", "n_layer": 3, "n_embd": 96, "n_head": 3, "n_inner": 320, "vocab_size": 1031,
            "n_positions": 80, "layer_norm_epsilon": 1e-6, "activation_function": "gelu",
            "scale_attn_by_inverse_layer_idx": True}
GOLDEN_C_IDS = [7, 1030, 512, 0, 33, 33, 900, 4, 250, 77, 1000, 640, 12, 81, 300, 2, 45, 999, 731, 8, 64, 100, 410, 29, 650,
                3, 5, 6, 1, 18, 200, 515, 940]

GOLDEN_IDS = {
    "golden_a": [5, 17, 3, 250, 511, 0, 42, 42, 99, 310, 7, 128, 64, 200, 1, 2, 3],
    "golden_b": [1030, 0, 517, 33, 900, 12, 12, 640, 77, 1000, 5, 81, 300, 2, 45, 999, 731, 8, 64, 100,
                 410, 29, 650, 3],
}


def LOCAL_MODEL_ROWS(n):
    return [0, 1, n // 2, n - 2, n - 1]


def make_weights(cfg, seed):
    """name -> float32 array, GPT-2's tensor names and on-disk ([in, out]) shapes."""
    rng = np.random.default_rng(seed)
    d, v, p, n = cfg["n_embd"], cfg["vocab_size"], cfg["n_positions"], cfg["n_layer"]
    inner = cfg.get("n_inner") or 4 * d

    def normal(*shape, mean=0.0, std=0.08):
        return (rng.standard_normal(shape) * std + mean).astype(np.float32)

    w = {"wte.weight": normal(v, d), "wpe.weight": normal(p, d),
         "ln_f.weight": normal(d, mean=1.0), "ln_f.bias": normal(d)}
    for i in range(n):
        h = f"h.{i}"
        w[h + ".ln_1.weight"] = normal(d, mean=1.0)
        w[h + ".ln_1.bias"] = normal(d)
        w[h + ".attn.c_attn.weight"] = normal(d, 3 * d)
        w[h + ".attn.c_attn.bias"] = normal(3 * d)
        w[h + ".attn.c_proj.weight"] = normal(d, d)
        w[h + ".attn.c_proj.bias"] = normal(d)
        w[h + ".ln_2.weight"] = normal(d, mean=1.0)
        w[h + ".ln_2.bias"] = normal(d)
        w[h + ".mlp.c_fc.weight"] = normal(d, inner)
        w[h + ".mlp.c_fc.bias"] = normal(inner)
        w[h + ".mlp.c_proj.weight"] = normal(inner, d)
        w[h + ".mlp.c_proj.bias"] = normal(d)
    return w


def write_f32_safetensors(path, weights):
    header, offset = {}, 0
    for name in sorted(weights):
        n = weights[name].nbytes
        header[name] = {"dtype": "F32", "shape": list(weights[name].shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in sorted(weights):
            f.write(np.ascontiguousarray(weights[name]).tobytes())


def write_model_dir(folder, cfg, weights):
    """config.json, F32 weights and the dummy byte-level tokenizer files that
    LocalModel::load insists on (include/ai/LocalModel.hpp:1724, 1800-1817)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_f32_safetensors(os.path.join(folder, "model.safetensors"), weights)
    sys.path.insert(0, os.path.join(REFERENCE, "tools"))
    import gpt2_oracle
    symbols = list(gpt2_oracle.bytes_to_unicode().values())
    vocab = {s: i for i, s in enumerate(symbols)}
    vocab[symbols[0] + symbols[1]] = len(vocab)
    with open(os.path.join(folder, "vocab.json"), "w", encoding="utf-8") as f:
        json.dump(vocab, f, ensure_ascii=False)
    with open(os.path.join(folder, "merges.txt"), "w", encoding="utf-8") as f:
        f.write("#version: 0.2\n" + symbols[0] + " " + symbols[1] + "\n")


def run_oracle(cfg, weights, ids):
    sys.path.insert(0, os.path.join(REFERENCE, "tools"))
    import gpt2_oracle
    return np.asarray(gpt2_oracle.forward(list(ids), weights, cfg, gpt2_oracle.Dumper(None)), dtype=np.float32)


def run_oracle_with_options(cfg, weights, ids):
    """The oracle on a configuration with erf GELU and the layer-index scaling: see the top of the file."""
    import math
    sys.path.insert(0, os.path.join(REFERENCE, "tools"))
    import gpt2_oracle
    d = cfg["n_embd"]
    w = {n: a.astype(np.float64) for n, a in weights.items()}
    if cfg.get("scale_attn_by_inverse_layer_idx"):
        for i in range(cfg["n_layer"]):
            w[f"h.{i}.attn.c_attn.weight"][:, :d] /= float(i + 1)
            w[f"h.{i}.attn.c_attn.bias"][:d] /= float(i + 1)
    kept = gpt2_oracle.gelu_new
    if cfg.get("activation_function") == "gelu":
        erf = np.vectorize(math.erf, otypes=[np.float64])
        gpt2_oracle.gelu_new = lambda x: 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))
    try:
        return np.asarray(gpt2_oracle.forward(list(ids), w, cfg, gpt2_oracle.Dumper(None)), dtype=np.float64)
    finally:
        gpt2_oracle.gelu_new = kept


def run_local_model(folder, ids, vocab):
    """Compiles the probe against the reference's headers and runs it: logits
    of every position, once from whole-prompt calls and once token by token."""
    exe = os.path.join(tempfile.gettempdir(), "local_model_probe")
    if not os.path.exists(exe):
        cmd = ["g++", "-std=c++2b", "-O2", "-w", "-I", os.path.join(REFERENCE, "include"),
               os.path.join(HERE, "local_model_probe.cpp"), os.path.join(REFERENCE, "src", "gpu", "Stub.cpp"),
               "-lpthread", "-o", exe]
        subprocess.run(cmd, check=True)
    out = os.path.join(folder, "probe_out.bin")
    subprocess.run([exe, folder, out] + [str(i) for i in ids], check=True)
    both = np.fromfile(out, dtype=np.float32).reshape(2, len(ids), vocab)
    return both[0], both[1]


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py PATH_TO_A_CHECKOUT_OF_hday200202/math-utils")
    REFERENCE = sys.argv[1]
    with_cpp = os.path.exists(os.path.join(HERE, "local_model_probe.cpp"))
    for k, (name, cfg) in enumerate(GOLDEN_CONFIGS.items()):
        weights = make_weights(cfg, seed=1234 + k)
        ids = GOLDEN_IDS[name]
        arrays = {"oracle": run_oracle(cfg, weights, ids)}
        if with_cpp:
            folder = tempfile.mkdtemp(prefix=name)
            write_model_dir(folder, cfg, weights)
            whole, stepwise = run_local_model(folder, ids, cfg["vocab_size"])
            rows = LOCAL_MODEL_ROWS(len(ids))          # a few rows keep the files small
            arrays["local_model_rows"] = np.asarray(rows)
            arrays["local_model_whole"] = whole[rows]
            arrays["local_model_stepwise"] = stepwise[rows]
            print(name, "LocalModel vs oracle, all rows:", float(np.abs(whole - arrays["oracle"]).max()),
                  float(np.abs(stepwise - arrays["oracle"]).max()))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
        print(name, {k2: v.shape for k2, v in arrays.items()})
    weights = make_weights(GOLDEN_C, seed=1236)
    logits = run_oracle_with_options(GOLDEN_C, weights, GOLDEN_C_IDS)
    rows = [0, 1, 16, 31, 32]                          # a few rows keep the file small
    np.savez_compressed(os.path.join(HERE, "golden_c.npz"), rows=np.asarray(rows), oracle_rows=logits[rows])
    print("golden_c", logits.shape, "rows", rows)
else:
    REFERENCE = os.environ.get("MATH_UTILS_REFERENCE", "")      # only needed to regenerate the files
