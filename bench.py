"""Measures decode and prefill throughput of math_utils_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run has the layer
sizes of GPT-2 small (BASELINE.json's third configuration) with seeded random
weights in bfloat16, a batch of 8 sequences with 512-token random prompts and a
context of 1,024.  One JSON line is printed:
  value       decoded tokens per second, timed on the device with CUDA events
              around K graph replays (each step's samples feed the next step
              on the device);
  e2e         the same through the Python entry point ``LLM.generate``: host
              token lists in, host token lists out; every step's positions are
              copied to the device from pinned memory (the host decides which
              sequences move on) and its samples read back, the host reading
              one step behind the device;
  prefill     one step of 2 x 1,024 prompt tokens;
  roofline    bytes a decode step must read (every weight once, the live cache)
              over its time, against the measured copy bandwidth;
  points      decode tokens per second at batch 1 and 64.
Inputs of a step (247 MB of weights plus the cache) are larger than the 126 MB
L2, so no flush is needed between iterations.
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}      # an earlier measurement on this pool
GPT2_SMALL = {"n_layer": 12, "n_embd": 768, "n_head": 12, "n_inner": 3072, "vocab_size": 50257,
              "n_positions": 1024, "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new"}
PROMPT_LEN, CONTEXT, PREFILL_SEQS = 512, 1024, 2


def baseline_config():
    """GPT-2 small's sizes as BASELINE.json's third configuration states them."""
    cfg = dict(GPT2_SMALL)
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            text = json.load(f)["configs"][2]
        for key in ("n_layer", "n_embd", "n_head", "n_inner", "vocab_size", "n_positions"):
            m = re.search(key + r"=(\d+)", text)
            if m:
                cfg[key] = int(m.group(1))
    except (OSError, KeyError, IndexError, ValueError):
        pass
    cfg.update(model_type="gpt2", architectures=["GPT2LMHeadModel"])
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


def matrix_bytes(cfg, n_layers, bytes_per=2):
    d, i, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    return (n_layers * (3 * d * d + d * d + 2 * d * i) + v * d) * bytes_per


def prefill_flops(cfg, n_layers, seq_lens, n_logit_rows):
    d, i, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    tokens = sum(seq_lens)
    linear = 2.0 * tokens * n_layers * (3 * d * d + d * d + 2 * d * i)
    attention = sum(4.0 * d * (n * (n + 1) / 2) for n in seq_lens) * n_layers      # QK^T and PV, causal half
    return linear + attention + 2.0 * n_logit_rows * v * d


def time_decode(model, prompts, steps, warmup, params):
    """Device time of `steps` graph-replayed decode steps of one batch; returns
    (seconds, launches inside the timed region, mean cached length while timed)."""
    import torch
    from math_utils_b200 import StepEntry
    from math_utils_b200.engine.decode_session import DecodeSession
    from math_utils_b200.sampling import Sampler
    ops = model.runtime.ops
    n = len(prompts)
    cache = model.new_cache(max_tokens=n * CONTEXT, n_slots=n)
    slots = [cache.acquire() for _ in prompts]
    logits = model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = Sampler(params, list(range(n)), model.runtime.device, ops).sample(logits).cpu().tolist()
    for s in slots:                      # every page the run can need, so no host work between replays
        cache.reserve(s, CONTEXT - cache.length(s))
    session = DecodeSession(model, cache, slots, params, list(range(n)), kv_bound=CONTEXT)
    session.sync_block_tables()
    session.feed(first, [len(p) for p in prompts])
    session.capture()
    for _ in range(warmup):
        session.launch()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = ops.launch_count
    start.record()
    for _ in range(steps):
        session.launch()
    end.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(end) / 1e3
    launches = ops.launch_count - before
    first_len = len(prompts[0]) + warmup
    mean_len = sum(min(first_len + k + 1, CONTEXT) for k in range(steps)) / steps
    del session
    return seconds, launches, mean_len


def run_ours(args):
    import numpy as np
    import torch
    from math_utils_b200 import LLM, Options, StepEntry, write_random_model
    from math_utils_b200.sampling import SamplingParams

    cfg = baseline_config()
    n_layers_full = cfg["n_layer"]
    pk = peaks()
    rng = np.random.default_rng(0)

    def prompts(n, length):
        return [rng.integers(0, cfg["vocab_size"], size=length).tolist() for _ in range(n)]

    with tempfile.TemporaryDirectory(prefix="mu_b200_bench_") as folder:
        write_random_model(folder, cfg, seed=0)
        llm = LLM(folder, Options(dtype="bfloat16", temperature=0.0, context=CONTEXT, max_batch=64))
    model = llm.model
    model.stop_ids = ()
    greedy = SamplingParams(temperature=0.0)
    steps, warmup, batch = args.steps, max(args.warmup, 3), args.batch

    clocks = ClockSampler()
    clocks.start()
    # --- decode, device-timed (the headline value) ---
    seconds, launches, mean_len = time_decode(model, prompts(batch, PROMPT_LEN), steps, warmup, greedy)
    value = batch * steps / seconds
    kv_bytes_per_pos = 2 * n_layers_full * cfg["n_embd"] * 2
    step_bytes = matrix_bytes(cfg, n_layers_full) + batch * mean_len * kv_bytes_per_pos
    achieved = step_bytes / (seconds / steps) / 1e9

    # --- decode, end to end through LLM.generate ---
    e2e_prompts = prompts(batch, PROMPT_LEN)
    # the same call once untimed: it sizes the cache the entry point keeps and records the graph
    llm.generate(e2e_prompts, max_tokens=steps + 1, stop_ids=[], max_batch=batch)
    torch.cuda.synchronize(); t0 = time.perf_counter()
    llm.generate(e2e_prompts, max_tokens=1, stop_ids=[], max_batch=batch)
    torch.cuda.synchronize(); t1 = time.perf_counter()
    out = llm.generate(e2e_prompts, max_tokens=steps + 1, stop_ids=[], max_batch=batch)
    torch.cuda.synchronize(); t2 = time.perf_counter()
    assert all(len(o) == steps + 1 for o in out)
    e2e = batch * steps / max((t2 - t1) - (t1 - t0), 1e-9)
    clock_record = clocks.stop()

    # --- prefill: one step of 2 x 1,024 tokens ---
    pre = prompts(PREFILL_SEQS, CONTEXT)
    cache = model.new_cache(max_tokens=PREFILL_SEQS * CONTEXT, n_slots=PREFILL_SEQS)
    times = []
    for it in range(3 + 5):
        slots = [cache.acquire() for _ in pre]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, pre)])
        end.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(start.elapsed_time(end))
        for s in slots:
            cache.release(s)
    pre_ms = statistics.median(times)
    pre_tokens = PREFILL_SEQS * CONTEXT
    pre_flops = prefill_flops(cfg, n_layers_full, [CONTEXT] * PREFILL_SEQS, PREFILL_SEQS)
    del cache

    # --- other batch sizes ---
    points = {}
    for b in (1, 64):
        k = min(steps, 256)
        s_b, _, _ = time_decode(model, prompts(b, PROMPT_LEN), k, warmup, greedy)
        points[f"decode_b{b}"] = round(b * k / s_b, 1)

    line = {
        "metric": "decode tok/s, GPT-2 small, batch 8, 512-token prompts, context 1024",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(seconds / steps * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random token ids, seeded random weights)",
        "impl": "ours",
        "config": {"model": "gpt2-small", "n_layer": n_layers_full, "n_layer_run": n_layers_full,
                   "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "head_dim": cfg["n_embd"] // cfg["n_head"],
                   "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"],
                   "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "parallelism": "none",
                   "sampling": "greedy", "decode": "cuda graph replay",
                   "l2": "inputs larger than L2 (weights 247 MB + cache per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": batch * 4,
                "d2h_bytes_per_step": batch * 4},
        "gpu_launches": launches,
        "prefill": {"value": round(pre_tokens / (pre_ms / 1e3), 1), "tokens": pre_tokens, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_record,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_part(args):
    """One part of the measurement on its own, optionally with fewer layers: a
    small case for a profiler.  Prints a short JSON line; not a bench record."""
    import numpy as np
    import torch
    from math_utils_b200 import LLM, Options, StepEntry, write_random_model
    from math_utils_b200.sampling import SamplingParams
    cfg = baseline_config()
    if args.layers:
        cfg["n_layer"] = args.layers
    rng = np.random.default_rng(0)
    with tempfile.TemporaryDirectory(prefix="mu_b200_bench_") as folder:
        write_random_model(folder, cfg, seed=0)
        llm = LLM(folder, Options(dtype="bfloat16", temperature=0.0, context=CONTEXT))
    model = llm.model
    model.stop_ids = ()
    if args.only == "decode":
        prompts = [rng.integers(0, cfg["vocab_size"], size=PROMPT_LEN).tolist() for _ in range(args.batch)]
        seconds, launches, _ = time_decode(model, prompts, args.steps, args.warmup, SamplingParams(temperature=0.0))
        print(json.dumps({"part": "decode", "batch": args.batch, "layers": cfg["n_layer"], "steps": args.steps,
                          "ms_per_step": round(seconds / args.steps * 1e3, 4), "launches": launches}))
    else:
        pre = [rng.integers(0, cfg["vocab_size"], size=CONTEXT).tolist() for _ in range(PREFILL_SEQS)]
        cache = model.new_cache(max_tokens=PREFILL_SEQS * CONTEXT, n_slots=PREFILL_SEQS)
        times = []
        for it in range(args.warmup + args.steps):
            slots = [cache.acquire() for _ in pre]
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            model.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, pre)])
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
            for s in slots:
                cache.release(s)
        print(json.dumps({"part": "prefill", "tokens": PREFILL_SEQS * CONTEXT, "layers": cfg["n_layer"],
                          "ms": round(statistics.median(times[args.warmup:]), 4)}))
    return 0


def run_reference(args):
    # The reference is a header-only C++ project with a makefile and no Python packaging, so an
    # offline `pip install --target baseline/_ref` of its checkout has nothing to install.
    print(json.dumps({"impl": "reference",
                      "unavailable": "hday200202/math-utils is a C++ header library without setup.py or "
                                     "pyproject.toml: pip cannot install it offline, and it has no CUDA path"}),
          flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only and print a short line (for profiling a small case)")
    ap.add_argument("--layers", type=int, default=0, help="with --only: fewer layers than the model has")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library has no multi-GPU path (asked for {args.gpus})",
              flush=True)
        return 2
    if args.only != "all":
        return run_part(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
