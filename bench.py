"""Measures decode and prefill throughput of math_utils_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --config medium|xl          # BASELINE.json's fourth and fifth workloads
    python bench.py --only decode|prefill [--layers N] [--batch B]     # a small case for a profiler
    python bench.py --only marginal [--batch B]    # each kernel class's share of the recorded decode step

A "step" is one decode step of the whole batch.  The default run has the layer
sizes of GPT-2 small (BASELINE.json's third configuration) with seeded random
weights in bfloat16, a batch of 8 sequences with 512-token random prompts and a
context of 1,024.  One JSON line is printed:
  value       decoded tokens per second: K single-token steps of the batch, timed on
              the device with CUDA events, driven through the calls the generation
              loop itself makes (a recorded graph per step, each step's samples
              feeding the next on the device, the host reading one step behind);
              ``config.ctx_first`` / ``ctx_last`` say which cache lengths they cover;
  checked     the first tokens of every sequence from the recorded graph equal those
              of eager steps on a second cache (the run stops otherwise);
  e2e         the same through the Python entry point ``LLM.generate``: host token
              lists in, host token lists out;
  prefill     one step of 2 x 1,024 prompt tokens (``host_ms``: the host's share);
  roofline    bytes a decode step must read (every weight once, the live cache)
              over its time, against the measured copy bandwidth;
  points      decode tokens per second at batch 1 and 64 over the same window;
  full_run    batch 1, 8 and 64 from 512-token prompts all the way to 1,024.
Inputs of a step (247 MB of weights plus the cache) are larger than the 126 MB
L2, so no flush is needed between iterations.
"""
import argparse
import json
import os
import re
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}      # an earlier measurement on this pool
SIZE_KEYS = ("n_layer", "n_embd", "n_head", "n_inner", "vocab_size", "n_positions")
DEFAULT_SIZES = {
    "small": {"n_layer": 12, "n_embd": 768, "n_head": 12, "n_inner": 3072, "vocab_size": 50257, "n_positions": 1024},
    "medium": {"n_layer": 24, "n_embd": 1024, "n_head": 16, "n_inner": 4096, "vocab_size": 50257, "n_positions": 1024},
    "xl": {"n_layer": 48, "n_embd": 1600, "n_head": 25, "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024},
}
BASELINE_INDEX = {"small": 2, "medium": 3, "xl": 4}
PROMPT_LEN, CONTEXT, PREFILL_SEQS = 512, 1024, 2
METRIC = "decode tok/s, GPT-2 small, batch 8, 512-token prompts, context 1024"


def baseline_config(name="small"):
    """The sizes of one of BASELINE.json's GPT-2 configurations, as it states them."""
    cfg = dict(DEFAULT_SIZES[name])
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            text = json.load(f)["configs"][BASELINE_INDEX[name]]
        for key in SIZE_KEYS:
            m = re.search(key + r"=(\d+)", text)
            if m:
                cfg[key] = int(m.group(1))
    except (OSError, KeyError, IndexError, ValueError):
        pass
    cfg.update(model_type="gpt2", architectures=["GPT2LMHeadModel"], layer_norm_epsilon=1e-5,
               activation_function="gelu_new")
    return cfg


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
        except (OSError, KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        reasons = sorted({n for s in self.samples for n, v in zip(self.NAMES, s[2:]) if v == "Active"})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def matrix_bytes(cfg, bytes_per=2):
    """Every matrix a decode step reads once: the layers' four products and the tied head."""
    d, i, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    return (cfg["n_layer"] * (3 * d * d + d * d + 2 * d * i) + v * d) * bytes_per


def cache_bytes_per_position(cfg, bytes_per=2):
    return 2 * cfg["n_layer"] * cfg["n_embd"] * bytes_per


def prefill_flops(cfg, seq_lens, n_logit_rows):
    d, i, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    tokens = sum(seq_lens)
    linear = 2.0 * tokens * cfg["n_layer"] * (3 * d * d + d * d + 2 * d * i)
    attention = sum(4.0 * d * (n * (n + 1) / 2) for n in seq_lens) * cfg["n_layer"]      # QK^T and PV, causal half
    return linear + attention + 2.0 * n_logit_rows * v * d


def load_random(cfg, seed=0, **options):
    """An ``LLM`` on seeded random weights of this configuration."""
    from math_utils_b200 import LLM, Options, write_random_model
    with tempfile.TemporaryDirectory(prefix="mu_b200_bench_") as folder:
        write_random_model(folder, cfg, seed=seed)
        llm = LLM(folder, Options(dtype="bfloat16", **options))
    llm.model.stop_ids = ()
    return llm


def eager_tokens(model, prompts, n_steps, params):
    """The first tokens of every sequence from eager steps on a cache of their own: what a recorded
    graph must reproduce."""
    from math_utils_b200 import StepEntry
    from math_utils_b200.sampling import Sampler
    n = len(prompts)
    cache = model.new_cache(max_tokens=n * (-(-(len(prompts[0]) + n_steps + 1) // 64) * 64), n_slots=n)
    slots = [cache.acquire() for _ in prompts]
    sampler = Sampler(params, list(range(n)), model.runtime.device, model.runtime.ops)
    logits = model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    tokens = [sampler.sample(logits).cpu().tolist()]
    for _ in range(n_steps):
        logits = model.step(cache, [StepEntry(s, [t], [0]) for s, t in zip(slots, tokens[-1])])
        tokens.append(sampler.sample(logits).cpu().tolist())
    return tokens


def time_decode(model, prompts, steps, warmup, params, check_steps=4):
    """Device time of ``steps`` single-token steps of one batch, through the calls the generation loop
    makes (``session_for`` / ``rebind`` / ``start`` / ``launch_step`` / ``read_step``: two steps
    launched, the host reading the older one).  Returns a dict: seconds, launches inside the timed
    region, the cache lengths of the first and the last timed step, and whether the graph's first
    tokens matched eager steps."""
    import torch
    from math_utils_b200 import StepEntry
    from math_utils_b200.engine.decode_session import session_for
    from math_utils_b200.sampling import Sampler
    ops = model.runtime.ops
    n, prompt_len = len(prompts), len(prompts[0])
    if prompt_len + warmup + steps > CONTEXT:
        raise SystemExit(f"{warmup} + {steps} steps after {prompt_len}-token prompts do not fit the context of {CONTEXT}")
    cache = model.new_cache(max_tokens=n * CONTEXT, n_slots=n)
    slots = [cache.acquire() for _ in prompts]
    logits = model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = Sampler(params, list(range(n)), model.runtime.device, ops).sample(logits).cpu().tolist()
    for s in slots:                      # every page the run can need, so no host work between launches
        cache.reserve(s, CONTEXT - cache.length(s))
    session = session_for(model, cache, params, n)
    session.rebind(slots, list(range(n)), [1] * n)
    session.sync_block_tables()
    positions = [prompt_len] * n
    session.start(first, positions)
    seen = [first]
    tickets = []

    def run(count, keep):
        for _ in range(count):
            if len(tickets) == 2:
                tokens = session.read_step(tickets.pop(0))
                if keep:
                    seen.append(tokens)
            tickets.append(session.launch_step(positions))
            for i in range(n):
                positions[i] += 1

    run(warmup, keep=True)
    while tickets:
        seen.append(session.read_step(tickets.pop(0)))
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = ops.launch_count
    ctx_first = positions[0] + 1                          # the cache length the first timed step attends over
    start.record()
    run(steps, keep=False)
    end.record()
    while tickets:
        session.read_step(tickets.pop(0))
    torch.cuda.synchronize()
    ops.check_status(model.runtime.device)
    result = {"seconds": start.elapsed_time(end) / 1e3, "launches": ops.launch_count - before,
              "ctx_first": ctx_first, "ctx_last": positions[0], "checked": None}
    result["mean_ctx"] = (result["ctx_first"] + result["ctx_last"]) / 2.0
    for s in slots:
        cache.release(s)
    if check_steps:
        k = min(check_steps, warmup)
        want = eager_tokens(model, prompts, k, params)
        result["checked"] = seen[:k + 1] == want[:k + 1]
        if not result["checked"]:
            raise SystemExit(f"bench: the recorded graph's tokens differ from eager steps at batch {n}: "
                             f"{seen[:k + 1]} vs {want[:k + 1]}")
    return result


def time_prefill(model, prompts, repeats=5, warmup=3):
    """Median device time and host time of one step over these prompts (milliseconds)."""
    import torch
    from math_utils_b200 import StepEntry
    cache = model.new_cache(max_tokens=sum(-(-len(p) // 64) * 64 for p in prompts), n_slots=len(prompts))
    device_ms, host_ms = [], []
    for it in range(warmup + repeats):
        slots = [cache.acquire() for _ in prompts]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        start.record()
        model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        end.record()
        t1 = time.perf_counter()                          # every launch is issued; the device may still run
        torch.cuda.synchronize()
        if it >= warmup:
            device_ms.append(start.elapsed_time(end))
            host_ms.append((t1 - t0) * 1e3)
        for s in slots:
            cache.release(s)
    model.runtime.ops.check_status(model.runtime.device)
    return statistics.median(device_ms), statistics.median(host_ms)


def run_ours(args):
    import numpy as np
    import torch
    from math_utils_b200.sampling import SamplingParams

    cfg = baseline_config("small")
    pk = peaks()
    rng = np.random.default_rng(0)

    def prompts(n, length):
        return [rng.integers(0, cfg["vocab_size"], size=length).tolist() for _ in range(n)]

    llm = load_random(cfg, temperature=0.0, context=CONTEXT, max_batch=64)
    model = llm.model
    greedy = SamplingParams(temperature=0.0)
    steps, warmup, batch = args.steps, max(args.warmup, 4), args.batch
    weights = matrix_bytes(cfg)
    per_pos = cache_bytes_per_position(cfg)

    def run_steps(run):
        return run["ctx_last"] - run["ctx_first"] + 1

    def hbm(batch_, run):
        bytes_ = weights + batch_ * run["mean_ctx"] * per_pos
        return bytes_ / (run["seconds"] / run_steps(run)) / 1e9

    clocks = ClockSampler()
    clocks.start()
    # --- decode, device-timed (the headline value) ---
    head = time_decode(model, prompts(batch, PROMPT_LEN), steps, warmup, greedy)
    value = batch * steps / head["seconds"]
    achieved = hbm(batch, head)

    # --- decode, end to end through LLM.generate ---
    e2e_prompts = prompts(batch, PROMPT_LEN)
    # the same call once untimed: it sizes the cache the entry point keeps and records the graph
    llm.generate(e2e_prompts, max_tokens=steps + 1, stop_ids=[], max_batch=batch)
    torch.cuda.synchronize(); t0 = time.perf_counter()
    llm.generate(e2e_prompts, max_tokens=1, stop_ids=[], max_batch=batch)
    torch.cuda.synchronize(); t1 = time.perf_counter()
    out = llm.generate(e2e_prompts, max_tokens=steps + 1, stop_ids=[], max_batch=batch)
    torch.cuda.synchronize(); t2 = time.perf_counter()
    if not all(len(o) == steps + 1 for o in out):
        raise SystemExit("bench: LLM.generate returned the wrong number of tokens")
    e2e = batch * steps / max((t2 - t1) - (t1 - t0), 1e-9)

    # --- prefill: one step of 2 x 1,024 tokens ---
    pre_ms, pre_host_ms = time_prefill(model, prompts(PREFILL_SEQS, CONTEXT))
    pre_tokens = PREFILL_SEQS * CONTEXT
    pre_flops = prefill_flops(cfg, [CONTEXT] * PREFILL_SEQS, PREFILL_SEQS)

    # --- other batch sizes over the same window, then every batch size all the way to the full context ---
    points = {}
    for b in (1, 64):
        r = time_decode(model, prompts(b, PROMPT_LEN), steps, warmup, greedy)
        points[f"decode_b{b}"] = round(b * steps / r["seconds"], 1)
    full = {}
    full_steps = CONTEXT - 1 - PROMPT_LEN - 4              # the last step leaves the cache one short of the context
    for b in (1, 8, 64):
        r = time_decode(model, prompts(b, PROMPT_LEN), full_steps, 4, greedy, check_steps=0)
        full[f"decode_b{b}"] = round(b * full_steps / r["seconds"], 1)
        full[f"hbm_frac_b{b}"] = round(hbm(b, r) / pk["hbm_gbs"], 4)
        full["ctx_first"], full["ctx_last"] = r["ctx_first"], r["ctx_last"]
    clock_record = clocks.stop()                           # sampled over every timed part of this record

    line = {
        "metric": METRIC,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(head["seconds"] / steps * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random token ids, seeded random weights)",
        "impl": "ours", "checked": bool(head["checked"]),
        "config": {"model": "gpt2-small", "n_layer": cfg["n_layer"], "n_layer_run": cfg["n_layer"],
                   "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "head_dim": cfg["n_embd"] // cfg["n_head"],
                   "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"],
                   "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                   "ctx_first": head["ctx_first"], "ctx_last": head["ctx_last"], "parallelism": "none",
                   "sampling": "greedy", "decode": "cuda graph replay, host one step behind",
                   "l2": "inputs larger than L2 (weights 247 MB + cache per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": batch * 4,
                "d2h_bytes_per_step": batch * 4 + 4},
        "gpu_launches": head["launches"],
        "prefill": {"value": round(pre_tokens / (pre_ms / 1e3), 1), "tokens": pre_tokens, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                    "host_ms": round(pre_host_ms, 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "full_run": full,
        "clocks": clock_record,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_workload(args):
    """BASELINE.json's fourth (GPT-2 medium: 16 prompts of 1 to 900 tokens, one prompt step, decoded to
    1,024 at temperature 1.0) or fifth (GPT-2 XL: 64 prompts of 128 tokens, greedy to a full cache)
    workload through ``LLM.generate``, prompt step and decoding timed apart as the reference's own
    report does (src/LLM.cpp:687-738).  One JSON line; not the contract's bench record."""
    import numpy as np
    import torch
    name = args.config
    cfg = baseline_config(name)
    if args.layers:
        cfg["n_layer"] = args.layers
    pk = peaks()
    rng = np.random.default_rng(1)
    if name == "medium":
        lens = rng.integers(1, 901, size=16).tolist()
        options = {"temperature": 1.0, "top_k": -1, "seed": 5}
    else:
        lens = [128] * 64
        options = {"temperature": 0.0}
    n = len(lens)
    prompts = [rng.integers(0, cfg["vocab_size"], size=k).tolist() for k in lens]
    t_load = time.perf_counter()
    llm = load_random(cfg, context=CONTEXT, max_batch=n, max_tokens=CONTEXT, **options)
    load_s = time.perf_counter() - t_load
    budget = args.tokens or CONTEXT                         # every request runs until its cache is full
    # the same tokens from eager steps and from the recorded graphs, on the first steps
    few = llm.generate(prompts, max_tokens=4, stop_ids=[], max_batch=n)
    from math_utils_b200.engine.generate import generate as plain_loop
    eager = plain_loop(llm.model, prompts, 4, llm._params(None, None, None), stop_ids=[], context=CONTEXT,
                       max_batch=n, use_graph=False)
    if few != eager:
        raise SystemExit(f"bench: graph replay and eager steps disagree on {name}: {few[:2]} vs {eager[:2]}")
    clocks = ClockSampler()
    clocks.start()
    llm.generate(prompts, max_tokens=budget, stop_ids=[], max_batch=n)          # records the graphs, sizes the cache
    torch.cuda.synchronize(); t0 = time.perf_counter()
    llm.generate(prompts, max_tokens=1, stop_ids=[], max_batch=n)               # the prompt step and one sample
    torch.cuda.synchronize(); t1 = time.perf_counter()
    out = llm.generate(prompts, max_tokens=budget, stop_ids=[], max_batch=n)
    torch.cuda.synchronize(); t2 = time.perf_counter()
    clock_record = clocks.stop()
    prompt_s = t1 - t0
    decode_s = max((t2 - t1) - prompt_s, 1e-9)
    produced = [len(o) for o in out]
    if produced != [min(budget, CONTEXT - k) for k in lens]:
        raise SystemExit(f"bench: {name} produced {produced}")
    decoded = sum(produced) - n                             # tokens that came from single-token steps
    n_steps = max(produced) - 1
    # bytes a step must read: every matrix once, and the cache of the requests still running
    weights, per_pos = matrix_bytes(cfg), cache_bytes_per_position(cfg)
    cache_bytes = 0.0
    for k, made in zip(lens, produced):
        cache_bytes += sum((k + j) * per_pos for j in range(1, made))          # the step that feeds token j attends over k + j
    total_bytes = n_steps * weights + cache_bytes
    achieved = total_bytes / decode_s / 1e9
    print(json.dumps({
        "workload": name, "impl": "ours", "dtype": "bf16", "checked": True,
        "data": "synthetic (seeded random token ids, seeded random weights)",
        "config": {"n_layer": cfg["n_layer"], "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"],
                   "vocab_size": cfg["vocab_size"], "batch": n, "prompt_tokens": sum(lens), "context": CONTEXT,
                   "sampling": "temperature 1.0" if name == "medium" else "greedy", "peaks": pk["source"]},
        "load_s": round(load_s, 2),
        "prompt": {"tokens": sum(lens), "s": round(prompt_s, 4), "tok_s": round(sum(lens) / prompt_s, 1)},
        "decode": {"tokens": decoded, "steps": n_steps, "s": round(decode_s, 4), "tok_s": round(decoded / decode_s, 1),
                   "ms_per_step": round(decode_s / max(n_steps, 1) * 1e3, 4),
                   "mean_bytes_per_step": round(total_bytes / max(n_steps, 1) / 1e6, 1), "unit": "MB"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clock_record}), flush=True)
    return 0


def run_part(args):
    """One part of the measurement on its own, optionally with fewer layers: a
    small case for a profiler.  Prints a short JSON line; not a bench record."""
    import numpy as np
    from math_utils_b200.sampling import SamplingParams
    cfg = baseline_config("small")
    if args.layers:
        cfg["n_layer"] = args.layers
    rng = np.random.default_rng(0)
    llm = load_random(cfg, temperature=0.0, context=CONTEXT)
    model = llm.model
    if args.only == "decode":
        prompts = [rng.integers(0, cfg["vocab_size"], size=args.prompt_len).tolist() for _ in range(args.batch)]
        r = time_decode(model, prompts, args.steps, max(args.warmup, 2), SamplingParams(temperature=0.0), check_steps=0)
        print(json.dumps({"part": "decode", "batch": args.batch, "layers": cfg["n_layer"], "steps": args.steps,
                          "ctx_first": r["ctx_first"], "ctx_last": r["ctx_last"],
                          "ms_per_step": round(r["seconds"] / args.steps * 1e3, 4), "launches": r["launches"]}))
    else:
        pre = [rng.integers(0, cfg["vocab_size"], size=CONTEXT).tolist() for _ in range(PREFILL_SEQS)]
        ms, host_ms = time_prefill(model, pre, repeats=args.steps, warmup=args.warmup)
        print(json.dumps({"part": "prefill", "tokens": PREFILL_SEQS * CONTEXT, "layers": cfg["n_layer"],
                          "ms": round(ms, 4), "host_ms": round(host_ms, 4)}))
    return 0


def run_marginal(args):
    """What each class of launches costs INSIDE the recorded, overlapped single-token step: the step is
    recorded again with that class left out (its outputs are then stale, which no timing cares about), and
    the difference to the whole step is the class's share.  A profiler serialises the launches and cannot
    say this.  Prints one JSON line; not a bench record."""
    import numpy as np
    import torch
    from math_utils_b200.csrc import ops
    from math_utils_b200.sampling import SamplingParams
    cfg = baseline_config(args.config)             # --config medium|xl: that model's layer sizes
    if args.layers:
        cfg["n_layer"] = args.layers
    llm = load_random(cfg, temperature=0.0, context=CONTEXT, max_batch=64)
    model = llm.model
    rng = np.random.default_rng(0)
    greedy = SamplingParams(temperature=0.0)
    real = {k: getattr(ops, k) for k in ("linear", "attention_decode", "argmax")}

    def linear_without(shapes):
        def linear(x, weight, bias=None, act=None, residual=None, out=None, out_dtype=None):
            if tuple(weight.shape) in shapes:
                rows = x.n_rows if isinstance(x, ops.NormedInput) else x.shape[0]
                return out if out is not None else torch.empty((rows, weight.shape[0]), dtype=out_dtype or weight.dtype,
                                                               device=weight.device)
            return real["linear"](x, weight, bias, act=act, residual=residual, out=out, out_dtype=out_dtype)
        return linear

    d, i, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    variants = {
        "whole step": {},
        "attention": {"attention_decode": lambda q, k_new, v_new, out, *a, **kw: out},
        "norm + q|k|v": {"linear": linear_without({(3 * d, d)})},
        "out-proj": {"linear": linear_without({(d, d)})},
        "norm + FC": {"linear": linear_without({(i, d)})},
        "proj": {"linear": linear_without({(d, i)})},
        "head": {"linear": linear_without({(v, d)})},
        "argmax": {"argmax": lambda logits, out=None, **kw: out if out is not None else real["argmax"](logits)},
    }
    prompts = [rng.integers(0, v, size=PROMPT_LEN).tolist() for _ in range(args.batch)]
    times = {}
    try:
        for name, patch in variants.items():
            for key, fn in real.items():
                setattr(ops, key, fn)
            for key, fn in patch.items():
                setattr(ops, key, fn)
            model.__dict__.pop("_decode_sessions", None)
            r = time_decode(model, prompts, args.steps, max(args.warmup, 4), greedy, check_steps=0)
            times[name] = r["seconds"] / args.steps * 1e6
    finally:
        for key, fn in real.items():
            setattr(ops, key, fn)
    whole = times.pop("whole step")
    print(json.dumps({"part": "marginal", "config": args.config, "batch": args.batch, "layers": cfg["n_layer"], "step_us": round(whole, 1),
                      "marginal_us": {k: round(whole - t, 1) for k, t in times.items()},
                      "per_layer_us": {k: round((whole - t) / cfg["n_layer"], 2) for k, t in times.items()
                                       if k not in ("head", "argmax")}}))
    return 0


# ------------------------------------------------------------------------------------------ the reference arm
REF_DIR = os.path.join(ROOT, "baseline", "_ref")          # --reference-dir names another checkout
REF_DRIVER = os.path.join(ROOT, "baseline", "reference_arm.cpp")


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def write_reference_folder(folder, cfg, seed):
    """The seeded model of ``run_ours`` as a folder the reference loads: float32 weights, and the dummy
    byte-level tokenizer files its loader insists on (include/ai/LocalModel.hpp:1724, 1800-1817), made
    with the reference's own ``bytes_to_unicode`` (tools/gpt2_oracle.py)."""
    from math_utils_b200 import write_random_model
    write_random_model(folder, cfg, seed=seed, store_dtype="float32")
    sys.path.insert(0, os.path.join(REF_DIR, "tools"))
    import gpt2_oracle
    symbols = list(gpt2_oracle.bytes_to_unicode().values())
    vocab = {s: i for i, s in enumerate(symbols)}
    vocab[symbols[0] + symbols[1]] = len(vocab)
    with open(os.path.join(folder, "vocab.json"), "w", encoding="utf-8") as f:
        json.dump(vocab, f, ensure_ascii=False)
    with open(os.path.join(folder, "merges.txt"), "w", encoding="utf-8") as f:
        f.write("#version: 0.2\n" + symbols[0] + " " + symbols[1] + "\n")


def run_reference(args):
    """The unmodified reference (a C++ header library: ``pip install`` has nothing to install) compiled
    here with g++ from a checkout under baseline/_ref, driven through its own
    ``ai::LocalModel::load`` / ``forward`` / ``sampleTopK`` on the CPU: it has no CUDA path and no
    batch, so the batch's sequences run one after another."""
    import numpy as np
    global REF_DIR
    if args.reference_dir:
        REF_DIR = os.path.abspath(args.reference_dir)
    header = os.path.join(REF_DIR, "include", "ai", "LocalModel.hpp")
    stub = os.path.join(REF_DIR, "src", "gpu", "Stub.cpp")
    if not (os.path.exists(header) and os.path.exists(stub) and os.path.exists(REF_DRIVER)):
        return unavailable(f"no checkout of hday200202/math-utils under {os.path.relpath(REF_DIR, ROOT)} (a C++ header "
                           "library that pip cannot install: it has no setup.py or pyproject.toml)")
    gxx = shutil.which("g++")
    if not gxx:
        return unavailable("g++ was not found; the reference is C++ and has to be compiled")
    cfg = baseline_config("small")
    steps, warmup, batch = args.steps, max(args.warmup, 3), args.batch
    rng = np.random.default_rng(0)
    with tempfile.TemporaryDirectory(prefix="mu_b200_ref_") as work:
        exe = os.path.join(work, "reference_arm")
        build = subprocess.run([gxx, "-std=c++2b", "-O3", "-march=native", "-w", "-I", os.path.join(REF_DIR, "include"),
                                REF_DRIVER, stub, "-lpthread", "-o", exe], capture_output=True, text=True)
        if build.returncode != 0:
            return unavailable("the reference did not compile here: " + build.stderr.strip().splitlines()[-1][:200])
        folder = os.path.join(work, "model")
        os.makedirs(folder)
        write_reference_folder(folder, cfg, seed=0)
        n_ids = batch * PROMPT_LEN + PREFILL_SEQS * CONTEXT
        ids_file = os.path.join(work, "ids.txt")
        with open(ids_file, "w") as f:
            f.write(" ".join(str(int(t)) for t in rng.integers(0, cfg["vocab_size"], size=n_ids)))
        run = subprocess.run([exe, folder, ids_file, str(batch), str(PROMPT_LEN), str(warmup), str(steps),
                              str(CONTEXT), str(PREFILL_SEQS), str(CONTEXT)], capture_output=True, text=True)
        if run.returncode != 0:
            return unavailable("the reference's run failed: " + (run.stderr.strip().splitlines() or ["no message"])[-1][:200])
        r = json.loads(run.stdout.strip().splitlines()[-1])
    value = r["decode_tokens"] / r["decode_seconds"]
    pre_flops = prefill_flops(cfg, [CONTEXT] * PREFILL_SEQS, PREFILL_SEQS)
    print(json.dumps({
        "metric": METRIC, "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        # a "step" of the batch: the reference steps its sequences one at a time, so their times add up
        "ms_per_step": round(r["decode_seconds"] / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32 (CPU)", "data": "synthetic (seeded random token ids, seeded random weights)",
        "impl": "reference",
        "config": {"model": "gpt2-small", "n_layer": cfg["n_layer"], "n_embd": cfg["n_embd"], "n_head": cfg["n_head"],
                   "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"],
                   "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "parallelism": "none",
                   "sampling": "greedy", "how": "ai::LocalModel on the CPU, sequences one after another",
                   "cpu_threads": r["threads"]},
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "prefill": {"value": round(r["prefill_tokens"] / r["prefill_seconds"], 1), "tokens": r["prefill_tokens"],
                    "ms": round(r["prefill_seconds"] * 1e3, 1),
                    "gflops": round(pre_flops / r["prefill_seconds"] / 1e9, 1)},
    }), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="small", choices=["small", "medium", "xl"],
                    help="medium / xl: BASELINE.json's fourth / fifth workload through LLM.generate")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "marginal"],
                    help="run one part only and print a short line (decode / prefill: a small case for a profiler; "
                         "marginal: what each class of launches costs inside the recorded single-token step)")
    ap.add_argument("--layers", type=int, default=0, help="with --only or --config: fewer layers than the model has")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="with --only decode: tokens per prompt")
    ap.add_argument("--reference-dir", default="", help="with --impl reference: a checkout other than baseline/_ref")
    ap.add_argument("--tokens", type=int, default=0, help="with --config: fewer tokens per request than fill the context")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library has no multi-GPU path (asked for {args.gpus})",
              flush=True)
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.only == "marginal":
        return run_marginal(args)
    if args.config != "small":
        return run_workload(args)
    if args.only != "all":
        return run_part(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
