"""Generation through the Python entry point and the command line, and trace replay
as a program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_gpt2
from conftest import ROOT
from helpers import check_logits

pytestmark = pytest.mark.gpu


def prompts_for(cfg, seed, lengths):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


def same_or_near_tie(model_cfg, weights, prompt, got, want, stop, context):
    """Greedy tokens must agree; where they first differ the plain logits of the
    two candidates must be within rounding of each other (a near tie that the
    other precision may resolve the other way), and the comparison ends there."""
    for i, (g, w) in enumerate(zip(got, want)):
        if g != w:
            logits = plain_gpt2.forward(list(prompt) + want[:i], model_cfg, weights)[-1]
            assert abs(logits[g] - logits[w]) < 2e-2 * logits.std(), (i, g, w)
            return
    assert len(got) == len(want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,context", [("tiny_a", [5, 17, 32], None), ("tiny_b", [1, 2, 9, 40, 63], 80)])
def test_greedy_generation_matches_plain(name, lengths, context, dtype, model_dirs, plain_models):
    from math_utils_b200 import LLM, Options
    cfg, w = plain_models[name]
    llm = LLM(model_dirs[name], Options(dtype=dtype, temperature=0.0, max_batch=3))
    prompts = prompts_for(cfg, 21, lengths)
    n_new = 16 if name == "tiny_a" else 80
    got = llm.generate(prompts, max_tokens=n_new, stop_ids=[])
    for p, g in zip(prompts, got):
        want = plain_gpt2.generate(p, cfg, w, n_new, context=context)
        assert len(g) == min(n_new, cfg["n_positions"] - len(p))
        if dtype == "float32":
            assert g == want
        else:
            same_or_near_tie(cfg, w, p, g, want, (), context)


def test_stop_tokens_end_requests_early(model_dirs, plain_models):
    from math_utils_b200 import LLM, Options
    cfg, w = plain_models["tiny_a"]
    llm = LLM(model_dirs["tiny_a"], Options(dtype="float32", temperature=0.0))
    prompts = prompts_for(cfg, 22, [4, 9, 30, 2])
    free_run = llm.generate(prompts, max_tokens=24, stop_ids=[])
    stop = {free_run[0][3], free_run[2][10]}                 # tokens that do come up
    got = llm.generate(prompts, max_tokens=24, stop_ids=sorted(stop))
    for p, g, f in zip(prompts, got, free_run):
        cut = next((i for i, t in enumerate(f) if t in stop), len(f))
        assert g == f[:cut] and g == plain_gpt2.generate(p, cfg, w, 24, stop_ids=stop)
    assert len(got[0]) <= 3 and len(got[2]) <= 10
    assert llm.model.stop_ids == (7,)                        # eos_token_id of config.json is the default


def test_temperature_sampling_is_seeded_per_request(model_dirs, plain_models):
    from math_utils_b200 import LLM, Options
    cfg, w = plain_models["tiny_b"]
    llm = LLM(model_dirs["tiny_b"], Options(dtype="float32", temperature=0.8, top_k=-1, seed=3))
    prompts = prompts_for(cfg, 23, [1, 2, 9, 40, 63])
    a = llm.generate(prompts, max_tokens=12, stop_ids=[])
    b = llm.generate(prompts, max_tokens=12, stop_ids=[], max_batch=2)      # other batches, same streams
    c = llm.generate(prompts, max_tokens=12, stop_ids=[], seed=4)
    assert a == b and a != c
    for i, (p, g) in enumerate(zip(prompts, a)):
        assert len(g) == 12
        # every draw against the plain sampler fed the same history and the same uniform: the same
        # token, unless the draw falls within float32 rounding of a boundary between two tokens
        for n, tok in enumerate(g):
            logits = plain_gpt2.forward(p + g[:n], cfg, w)[-1]
            want, margin = plain_gpt2.sample_top_k(logits, 0.8, -1, plain_gpt2.uniform_draw(3, i, n))
            assert tok == want or margin < 1e-5, (i, n, tok, want, margin)


def test_conversation_keeps_its_cache(model_dirs, plain_models):
    from math_utils_b200 import LLM, Options
    cfg, w = plain_models["tiny_a"]
    llm = LLM(model_dirs["tiny_a"], Options(dtype="float32", temperature=0.0, max_tokens=5))
    llm.model.stop_ids = ()
    first = llm.prompt([3, 1, 4])
    second = llm.prompt([1, 5])
    # the second turn continues the first: prompt, the whole answer, new ids (include/ai/LLM.hpp:226-243)
    history = [3, 1, 4] + first + [1, 5]
    assert second == plain_gpt2.generate(history, cfg, w, 5)
    third = llm.prompt([9])
    assert third == plain_gpt2.generate(history + second + [9], cfg, w, 5)
    assert llm.once([3, 1, 4]) == first
    llm.reset()
    assert llm.prompt([3, 1, 4]) == first


def test_new_batch_shapes_do_not_pile_up_memory(model_dirs):
    """Every new (cache, batch size, sampling rule) records graphs of its own and the oldest are dropped: what
    they held must serve the next recordings (one memory pool for all of a model's graphs), not stay reserved
    by the allocator until the device is full."""
    import torch
    from math_utils_b200 import LLM, Options
    from math_utils_b200.engine.generate import generate
    from math_utils_b200.sampling import SamplingParams
    llm = LLM(model_dirs["tiny_b"], Options(dtype="bfloat16", temperature=0.0))
    rng = np.random.default_rng(0)
    vocab = llm.model.vocab_size

    def some_calls(first_seed, count):
        for seed in range(first_seed, first_seed + count):
            n = int(rng.integers(1, 7))
            prompts = [rng.integers(0, vocab, size=int(rng.integers(1, 30))).tolist() for _ in range(n)]
            generate(llm.model, prompts, 5, SamplingParams(temperature=0.9, top_k=-1, seed=seed), stop_ids=[])

    some_calls(0, 30)                                   # more than the sessions that are kept: the first are gone
    torch.cuda.synchronize()
    before = torch.cuda.memory_reserved()
    some_calls(100, 60)
    torch.cuda.synchronize()
    assert llm.model.__dict__.get("_graph_pool") is not None
    assert torch.cuda.memory_reserved() - before < 64 * 2 ** 20, "recorded graphs that were dropped keep their memory"
    # with every session gone the pool must still take the next recording
    llm.model.__dict__.pop("_decode_sessions")
    import gc
    gc.collect()
    some_calls(500, 3)


def test_a_given_up_wait_stops_generation(model_dirs, monkeypatch):
    """Kernels with bounded waits report a wait that ran out through a status word.  The word is set by
    hand here (nothing faults): the loop must raise where it next reads samples, give its slots back,
    and work again afterwards."""
    import torch
    from math_utils_b200 import LLM, Options
    from math_utils_b200.csrc import ops
    from math_utils_b200.engine import generate as gen
    llm = LLM(model_dirs["tiny_a"], Options(dtype="bfloat16", temperature=0.0))
    prompts = [[5, 6, 7], [8] * 20]
    want = llm.generate(prompts, max_tokens=10, stop_ids=[])
    word = ops.status_word(torch.device("cuda:0"))
    word.fill_(4)
    with pytest.raises(ops.KernelError, match="single-token attention"):      # seen right after the prompt step
        llm.generate(prompts, max_tokens=10, stop_ids=[])
    assert int(word.item()) == 0
    # seen by the loop that reads one step behind: the word travels with each step's samples
    real_check = gen.check_kernels
    monkeypatch.setattr(gen, "check_kernels", lambda model: None)
    word.fill_(2)
    with pytest.raises(ops.KernelError, match="tensor cores"):
        llm.generate(prompts, max_tokens=10, stop_ids=[])
    monkeypatch.setattr(gen, "check_kernels", real_check)
    cache = llm._batch_cache
    assert cache.slots.n_free == cache.n_slots and cache.free_pages() == cache.n_pages
    assert llm.generate(prompts, max_tokens=10, stop_ids=[]) == want


def test_command_line(model_dirs, plain_models, tmp_path):
    cfg, w = plain_models["tiny_a"]
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llm"), model_dirs["tiny_a"], "--prompt",
                          "5,17,3", "--tokens", "6", "--temp", "0", "--fp32", "--stop", ""],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr
    got = [int(t) for t in out.stdout.strip().splitlines()[-1].split()]
    assert got == plain_gpt2.generate([5, 17, 3], cfg, w, 6)
    # --profile: the same tokens from eager steps, prompt and generation rates apart, a table of stages
    prof = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llm"), model_dirs["tiny_a"], "--prompt",
                           "5,17,3", "--tokens", "6", "--temp", "0", "--fp32", "--stop", "", "--profile"],
                          capture_output=True, text=True, env=env, timeout=600)
    assert prof.returncode == 0, prof.stderr
    lines = prof.stdout.strip().splitlines()
    tokens_line = next(l for l in lines if l and all(p.isdigit() for p in l.split()))
    assert [int(t) for t in tokens_line.split()] == got
    assert any(l.strip().startswith("prompt 3 tok in") and "generated 5 tok in" in l and "context 9/" in l for l in lines), lines
    assert any("attention" in l for l in lines) and any("output head" in l for l in lines)
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(cfg))
    out = subprocess.run([sys.executable, "-m", "math_utils_b200", "--random", "--config", str(cfg_file),
                          "--seed", "9", "--prompt", "1 2 3", "--tokens", "4", "--topk", "1"],
                         capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert out.returncode == 0, out.stderr
    # the invented weights are those of write_random_model with the same seed: the plain model reads them
    from math_utils_b200 import write_random_model
    folder = write_random_model(str(tmp_path / "same_seed"), cfg, seed=9)
    cfg9, w9 = plain_gpt2.read_model(folder)
    got = [int(t) for t in out.stdout.strip().splitlines()[-1].split()]
    want = plain_gpt2.generate([1, 2, 3], cfg9, w9, 4, stop_ids=cfg9.get("eos_token_id", ()) if isinstance(
        cfg9.get("eos_token_id", ()), (list, tuple)) else (cfg9["eos_token_id"],))
    same_or_near_tie(cfg9, w9, [1, 2, 3], got, want, (), None)


def replay(model_dir, dtype, steps, out_dir, max_tokens):
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", str(max_tokens)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(dtype, model_dirs, plain_models, tmp_path):
    """Unequal batch, requests that end early, a second batch in the freed room."""
    name = "tiny_b"
    cfg, w = plain_models[name]
    vocab = cfg["vocab_size"]
    reqs = {rid: r for rid, r in zip("abcdef", prompts_for(cfg, 31, [80, 20, 66, 41, 80, 9]))}
    steps, wanted = [], {}

    def batch(ids, prompt_lens, step0):
        step = step0
        pos = dict(zip(ids, prompt_lens))
        entries = [{"id": i, "tokens": reqs[i][:pos[i]], "want": list(range(pos[i]))} for i in ids]
        live = list(ids)
        while live:
            ends = [e["id"] for e in entries if pos[e["id"]] >= len(reqs[e["id"]])]
            steps.append({"step": step, "entries": entries, "end": ends})
            wanted[step] = [(e["id"], pos[e["id"]] - len(e["tokens"]) + k) for e in entries for k in e["want"]]
            live = [i for i in live if i not in ends]
            entries = [{"id": i, "tokens": [reqs[i][pos[i]]], "want": [0]} for i in live]
            for i in live:
                pos[i] += 1
            step += 1
        return step

    nxt = batch(["a", "b", "c"], [50, 19, 64], 0)
    batch(["d", "e", "f"], [1, 79, 9], nxt)
    out_dir = str(tmp_path / f"out_{dtype}")
    # a, b, c hold at most 128 + 64 + 128 positions; so do d, e, f
    replay(model_dirs[name], dtype, steps, out_dir, max_tokens=320)
    plain = {rid: plain_gpt2.forward(r, cfg, w) for rid, r in reqs.items()}
    with open(os.path.join(out_dir, "manifest.json")) as f:
        manifest = json.load(f)
    assert [m["name"] for m in manifest] == [f"{s['step']}.f32" for s in steps]
    assert all(m["shape"] == [len(wanted[s["step"]]), vocab] for m, s in zip(manifest, steps))
    for s in steps:
        got = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(-1, vocab)
        want = np.stack([plain[rid][p] for rid, p in wanted[s["step"]]])
        check_logits(got, want, dtype, f"replay step {s['step']}")
