"""A plain, slow GPT-2: whole sequences, no cache, one function per part.

Written from the reference's formulas (file:line beside each function, paths
within the reference project) and from nothing of the package under test: it
has its own safetensors reader, its own config reading and its own sampling.
The engine's logits are compared with this.  It computes in float64 unless
asked otherwise, so what it returns is the exact value up to ~1e-12.

It rests on the formulas; ``tests/golden/`` anchors it once on the reference's
own code (see ``tests/golden/make_golden.py``).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

_MASK = (1 << 64) - 1


# --------------------------------------------------------------------- files
def read_safetensors(path, dtype=np.float64):
    """name -> ndarray.  Header: u64 LE length, JSON, payload
    (include/ai/Safetensors.hpp:389-485; tools/gpt2_oracle.py:56-84)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        payload = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        raw = np.frombuffer(payload, dtype=np.uint8, count=e - b, offset=b)
        kind = meta["dtype"]
        if kind == "BF16":
            # bfloat16 is the high half of a float32 (tools/gpt2_oracle.py:71-75)
            arr = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif kind == "F32":
            arr = raw.view(np.float32)
        elif kind == "F16":
            arr = raw.view(np.float16)
        elif kind == "F64":
            arr = raw.view(np.float64)
        else:
            raise ValueError(f"{name}: dtype {kind}")
        out[name] = arr.reshape(meta["shape"]).astype(dtype)
    return out


def read_model(model_dir, dtype=np.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"), dtype)
    return cfg, weights


# --------------------------------------------------------------------- parts
def embed(ids, start, wte, wpe):
    """x[t] = wte[id_t] + wpe[start + t]
    (include/ai/LocalModel.hpp:3686-3697; include/ai/GPT2.hpp:305-310)."""
    ids = np.asarray(ids)
    pos = start + np.arange(len(ids))
    assert pos.max(initial=0) < wpe.shape[0], "position beyond n_positions"
    return wte[ids] + wpe[pos]


def layer_norm(x, weight, bias, eps):
    """Biased variance, eps inside the root
    (include/ai/LocalModel.hpp:1355-1367; include/ai/Tensor.hpp:344-375)."""
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * weight + bias


def gelu_new(x):
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
    (include/ai/LocalModel.hpp:1388-1391; include/ai/Tensor.hpp:301-316)."""
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def gelu_erf(x):
    """0.5 x (1 + erf(x / sqrt 2)): the exact form that ``activation_function``
    "gelu" names.  The reference has only the tanh form."""
    try:
        from scipy.special import erf
    except ImportError:                                        # pragma: no cover
        erf = np.vectorize(math.erf, otypes=[x.dtype])
    return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))


ACTIVATIONS = {"gelu_new": gelu_new, "gelu": gelu_erf}


def softmax(s):
    """Max-subtracted (include/ai/Kernels.hpp:145-158; include/ai/Tensor.hpp:319-341)."""
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def linear_in_out(x, weight, bias):
    """Conv1D: weight is stored [in, out], so x @ W + b, no transpose
    (include/ai/GPT2.hpp:253; tools/gpt2_oracle.py:248)."""
    return x @ weight + bias


def causal_attention(q, k, v, n_heads, n_kv_heads, scale, window=0, start=0):
    """q [T, H*dh]; k, v [start+T, Hkv*dh].  Query t is at absolute position
    start+t and sees keys first..position, first = position+1-window when a
    window is set (include/ai/Kernels.hpp:132-161); head h reads kv head
    h // (H / Hkv) (include/ai/Kernels.hpp:143)."""
    T = q.shape[0]
    dh = q.shape[1] // n_heads
    out = np.zeros_like(q)
    group = n_heads // n_kv_heads
    for h in range(n_heads):
        kv = h // group
        qh = q[:, h * dh:(h + 1) * dh]
        kh = k[:, kv * dh:(kv + 1) * dh]
        vh = v[:, kv * dh:(kv + 1) * dh]
        for t in range(T):
            p = start + t
            first = p + 1 - window if (window and p + 1 > window) else 0
            s = (kh[first:p + 1] @ qh[t]) * scale
            w = softmax(s)
            out[t, h * dh:(h + 1) * dh] = w @ vh[first:p + 1]
    return out


def causal_attention_masked(q, k, v, n_heads, n_kv_heads, scale, window=0):
    """The same attention in the reference's other form: the whole [T, T] score
    matrix of a head, everything a query may not see filled with -1e10 before
    the softmax (include/ai/GPT2.hpp:261-271; tools/gpt2_oracle.py:258-267; in
    float64 the filled entries weigh exactly nothing, exp underflows to 0).  No
    loop over queries, so long sequences stay affordable."""
    T = q.shape[0]
    dh = q.shape[1] // n_heads
    out = np.zeros_like(q)
    group = n_heads // n_kv_heads
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    hidden = j > i
    if window:
        hidden = hidden | (j < i + 1 - window)
    for h in range(n_heads):
        kv = h // group
        s = (q[:, h * dh:(h + 1) * dh] @ k[:, kv * dh:(kv + 1) * dh].T) * scale
        s = np.where(hidden, -1e10, s)
        out[:, h * dh:(h + 1) * dh] = softmax(s) @ v[:, kv * dh:(kv + 1) * dh]
    return out


def attention_block(h, w, prefix, cfg, layer, trace=None, masked=False):
    """c_attn, split into q|k|v by columns, heads, c_proj
    (include/ai/LocalModel.hpp:2130-2145, 2604-2667; include/ai/GPT2.hpp:248-276)."""
    d = cfg["n_embd"]
    n_head = cfg["n_head"]
    qkv = linear_in_out(h, w[prefix + ".attn.c_attn.weight"], w[prefix + ".attn.c_attn.bias"])
    if trace is not None:
        trace[prefix + ".qkv"] = qkv.copy()
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    scale = 1.0
    if cfg.get("scale_attn_weights", True):
        scale = 1.0 / math.sqrt(d // n_head)                    # include/ai/Kernels.hpp:136
    if cfg.get("scale_attn_by_inverse_layer_idx", False):
        scale = scale / float(layer + 1)
    attend = causal_attention_masked if masked else causal_attention
    a = attend(q, k, v, n_head, n_head, scale)
    if trace is not None:
        trace[prefix + ".attn"] = a.copy()
    return linear_in_out(a, w[prefix + ".attn.c_proj.weight"], w[prefix + ".attn.c_proj.bias"])


def feed_forward(h, w, prefix, cfg, trace=None):
    """c_fc, activation, c_proj (include/ai/LocalModel.hpp:3767-3774;
    include/ai/GPT2.hpp:279-290)."""
    act = ACTIVATIONS[cfg.get("activation_function", "gelu_new")]
    u = act(linear_in_out(h, w[prefix + ".mlp.c_fc.weight"], w[prefix + ".mlp.c_fc.bias"]))
    if trace is not None:
        trace[prefix + ".act"] = u.copy()
    return linear_in_out(u, w[prefix + ".mlp.c_proj.weight"], w[prefix + ".mlp.c_proj.bias"])


def forward(ids, cfg, w, trace=None, rows=None, masked=None):
    """Logits [len(ids), vocab] of one whole sequence
    (include/ai/LocalModel.hpp:3648-3802; include/ai/GPT2.hpp:300-339;
    tools/gpt2_oracle.py:285-321).  ``rows``: only these positions' logits (the
    reference computes the last row only, include/ai/LocalModel.hpp:3788-3799).
    ``masked``: attention in the masked-matrix form instead of query by query
    (default: for sequences of more than 200 tokens).  ``trace``: a dict that
    receives every stage by the reference's names (include/ai/LocalModel.hpp:
    3699-3801): embed, h.N.ln1, h.N.qkv, h.N.attn, h.N.res1, h.N.ln2, h.N.act,
    h.N.res2, lnf, logits."""
    eps = cfg.get("layer_norm_epsilon", 1e-5)
    masked = len(ids) > 200 if masked is None else masked
    x = embed(ids, 0, w["wte.weight"], w["wpe.weight"])
    if trace is not None:
        trace["embed"] = x.copy()
    for i in range(cfg["n_layer"]):
        p = f"h.{i}"
        h = layer_norm(x, w[p + ".ln_1.weight"], w[p + ".ln_1.bias"], eps)
        if trace is not None:
            trace[p + ".ln1"] = h.copy()
        x = x + attention_block(h, w, p, cfg, i, trace, masked)
        if trace is not None:
            trace[p + ".res1"] = x.copy()
        h = layer_norm(x, w[p + ".ln_2.weight"], w[p + ".ln_2.bias"], eps)
        if trace is not None:
            trace[p + ".ln2"] = h.copy()
        x = x + feed_forward(h, w, p, cfg, trace)
        if trace is not None:
            trace[p + ".res2"] = x.copy()
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    x = layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], eps)
    logits = x @ w["wte.weight"].T                             # tied head, no bias
    if trace is not None:
        trace["lnf"], trace["logits"] = x.copy(), logits.copy()
    return logits


# ------------------------------------------------------------------ sampling
def argmax(row):
    """First maximum wins (include/ai/LocalModel.hpp:3809-3813)."""
    best = 0
    for i in range(1, len(row)):
        if row[i] > row[best]:
            best = i
    return best


def splitmix64(x):
    """include/math/Random.hpp:79-84 (the seeding mixer of the reference's RNG)."""
    z = (x + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_draw(seed, request, n):
    """The n-th uniform of a request's own stream, in [0, 1): 53 high bits as in
    include/math/Random.hpp:27.  The stream is keyed by (seed, request) so a
    request's tokens do not depend on its place in a batch."""
    key = splitmix64((seed & _MASK) ^ ((request * 0x9E3779B97F4A7C15) & _MASK))
    x = splitmix64((key + n * 0xD1B54A32D192ED03) & _MASK)
    return (x >> 11) * 2.0 ** -53


def sample_top_k(row, temperature, top_k, u):
    """include/ai/LocalModel.hpp:3815-3841: greedy when temperature <= 0 or
    top_k <= 1 (the reference's count is unsigned; a negative top_k here keeps
    all, which the reference cannot ask for); else keep the top_k largest,
    p = exp(l/T - best/T),
    pick = u * sum p, walk in descending order subtracting p until <= 0.  Ties
    are ordered by index.  Returns (token, distance of pick to the nearest
    boundary relative to the total), so a test can tell a rounding-level
    disagreement from a real one."""
    row = np.asarray(row, dtype=np.float32)
    if temperature <= 0.0 or 0 <= top_k <= 1:
        return argmax(row), 1.0
    n = len(row)
    keep = n if top_k < 0 else min(top_k, n)
    order = sorted(range(n), key=lambda i: (-float(row[i]), i))[:keep]
    t = np.float32(temperature)
    best = row[order[0]] / t
    probs = np.exp((row[order] / t - best).astype(np.float32)).astype(np.float64)
    total = probs.sum()
    pick = u * total
    cum = np.cumsum(probs)
    idx = int(np.searchsorted(cum, pick, side="left"))
    idx = min(idx, keep - 1)
    margin = float(np.min(np.abs(cum - pick)) / total)
    return order[idx], margin


def generate(prompt, cfg, w, max_new_tokens, temperature=0.0, top_k=0, seed=0, request=0,
             stop_ids=(), context=None):
    """Prefill, then sample / stop? / feed, as src/LLM.cpp:688-707: the
    stop token is neither kept nor fed, and generation ends when the context is
    full.  Re-runs the whole sequence for each token (include/ai/GPT2.hpp:396-412)."""
    limit = min(context or cfg["n_positions"], cfg["n_positions"])
    ids = list(prompt)
    out = []
    for n in range(max_new_tokens):
        if len(ids) >= limit:                   # "cache.length < context" fails
            break
        logits = forward(ids, cfg, w)[-1]
        tok, _ = sample_top_k(logits, temperature, top_k, uniform_draw(seed, request, n))
        if tok in stop_ids:
            break
        out.append(int(tok))
        ids.append(int(tok))
    return out
