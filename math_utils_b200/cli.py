"""Command line, in the manner of the reference's ``src/LLM.cpp``.

    llm <model-dir> [--tokens N] [--temp F] [--topk N] [--seed N] [--ctx N]
        [--prompt IDS] [--random] [--config FILE] [--fp32] [--stop IDS] [--profile] [--load-only]

Option names, meanings and defaults are the reference's (src/LLM.cpp:88-128,
215-282): ``--tokens`` 256, ``--temp`` 0.7, ``--topk`` 20, ``--seed`` 0,
``--ctx`` 4096 (clamped to the model), ``--prompt`` for one shot, else a read
loop with ``/reset``, ``/stats`` and ``/quit``; ``--random`` runs the topology
with invented weights, reproducible with ``--seed``.  Prompts are token ids
separated by commas or spaces, since this library carries no tokenizer, and
answers are printed as ids.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import tempfile
import time
from typing import List

USAGE_NOTE = "prompts are token ids, e.g. --prompt '464,3139,286'"


def parse_ids(text: str) -> List[int]:
    parts = [p for p in re.split(r"[,\s]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise ValueError(f"expected token ids separated by commas or spaces, got '{text}'") from None


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="llm", description="GPT-2 generation on one B200. " + USAGE_NOTE)
    ap.add_argument("model_dir", nargs="?", help="a folder holding config.json and model.safetensors")
    ap.add_argument("--model", dest="model_opt", help="same as the positional model folder")
    ap.add_argument("--tokens", type=int, default=256, help="most new tokens per answer")
    ap.add_argument("--temp", type=float, default=0.7, help="temperature; 0 is greedy")
    ap.add_argument("--topk", type=int, default=20, help="keep the k likeliest tokens; 0 or 1 is greedy, a negative number keeps all")
    ap.add_argument("--seed", type=int, default=0, help="seed of sampling and of --random weights")
    ap.add_argument("--ctx", type=int, default=4096, help="cache positions, clamped to the model's maximum")
    ap.add_argument("--prompt", help="one shot: answer these token ids and exit")
    ap.add_argument("--random", action="store_true",
                    help="run the topology of config.json with invented weights (see --config)")
    ap.add_argument("--config", help="with --random: a config.json to invent weights for")
    ap.add_argument("--fp32", action="store_true", help="the true 32-bit path instead of bfloat16")
    ap.add_argument("--stop", help="stop token ids (default: eos_token_id of config.json)")
    ap.add_argument("--profile", action="store_true",
                    help="print load time and, per answer, prompt and generation rates and per-stage device times "
                         "(steps then run one by one instead of from recorded graphs)")
    ap.add_argument("--load-only", action="store_true", help="load, report, and exit")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    model_dir = args.model_dir or args.model_opt
    tmp = None
    if args.random:
        from .weights import write_random_model
        config_path = args.config or (os.path.join(model_dir, "config.json") if model_dir else None)
        if not config_path:
            print("--random needs a model folder or --config FILE to take the topology from", file=sys.stderr)
            return 1
        with open(config_path, "r", encoding="utf-8") as f:
            config_json = json.load(f)
        tmp = tempfile.TemporaryDirectory(prefix="llm_random_")
        model_dir = write_random_model(tmp.name, config_json, seed=args.seed)
        print(f"(random weights for {config_path}, seed {args.seed})")
    if not model_dir:
        build_parser().print_usage()
        return 1

    from .llm import LLM, Options
    t0 = time.time()
    llm = LLM(model_dir, Options(context=args.ctx, max_tokens=args.tokens, temperature=args.temp,
                                 top_k=args.topk, seed=args.seed, dtype="float32" if args.fp32 else "bfloat16",
                                 profile=args.profile))
    if args.stop is not None:
        llm.model.stop_ids = tuple(parse_ids(args.stop))
    load_s = time.time() - t0
    if args.profile or args.load_only:
        print(f"loaded {model_dir}: {llm.model.weight_bytes / 1e6:.1f} MB of weights in {load_s:.2f}s, "
              f"context {llm.context}")
    if args.load_only:
        return 0

    def run(ids: List[int]) -> None:
        out = llm.prompt(ids)
        print(" ".join(str(t) for t in out), flush=True)

    def stats() -> None:
        """Prompt and generation apart, as the reference reports them (src/LLM.cpp:716-730)."""
        last = llm.last
        if not last:
            return
        made = max(last["produced"] - 1, 0)               # the first token comes out of the prompt step
        print(f"  prompt {last['prompt_tokens']} tok in {last['prompt_s']:.4f}s "
              f"({last['prompt_tokens'] / max(last['prompt_s'], 1e-9):.1f} tok/s)   "
              f"generated {made} tok in {last['decode_s']:.4f}s ({made / max(last['decode_s'], 1e-9):.1f} tok/s)   "
              f"context {last['context_used']}/{last['context']}")
        if llm.stage_times:
            from .engine.stage_timer import STAGE_NAMES
            print("  stage                              prompt(s)   decode(s)")
            for kind, (prompt_s, decode_s) in llm.stage_times.items():
                if prompt_s or decode_s:
                    print(f"  {STAGE_NAMES.get(kind, kind):<33} {prompt_s:9.4f}   {decode_s:9.4f}")

    if args.prompt is not None:
        run(parse_ids(args.prompt))
        if args.profile:
            stats()
        return 0
    print("token ids per line; /reset forgets the conversation, /stats, /quit")
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        if line in ("/quit", "/exit"):
            break
        if line == "/reset":
            llm.reset(); print("(conversation reset)"); continue
        if line == "/stats":
            stats(); continue
        try:
            run(parse_ids(line))
        except ValueError as e:
            print(f"error: {e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
