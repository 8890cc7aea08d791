"""Generation through the Python entry point and the command line: greedy equals the plain model's greedy
loop, temperature sampling is reproducible and independent of the batch, requests that do not fit wait."""

import json
import re
import os
import subprocess
import sys

import pytest
import torch

import tiny
from models_util import model_folder, plain_weights
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def prompts_for(name, lengths, seed=7):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, tiny.CONFIGS[name][0]["vocab_size"], (n,), generator=g).tolist() for n in lengths]


@pytest.mark.parametrize("name,lengths", [("A", (5, 17, 33)), ("B", (1, 31, 64, 130)), ("C", (3, 40, 70))])
def test_greedy_generation_equals_plain(name, lengths):
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = tiny.CONFIGS[name]
    folder = model_folder(name)
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=page, num_pages=40, max_batch_tokens=24)
    prompts = prompts_for(name, lengths)
    got = engine.generate(prompts, max_new_tokens=8, ignore_eos=True)
    w = plain_weights(folder, "float32")
    assert got == [plain.greedy_generate(w, raw, p, 8) for p in prompts]
    assert engine.manager.free_pages() == [40] * len(engine.manager.groups)
    engine.manager.check_invariants()


@pytest.mark.parametrize("name", ["A", "C"])
def test_bfloat16_greedy_generation_close_to_plain(name):
    """bfloat16 may pick another token where two logits are within rounding; every pick must still be
    (nearly) the best token of the plain model given the same history.  (C: the decode steps run the fused
    kernels: norm on the GEMM's token operand, rotation and cache write, SiLU-mul and the residual sum on its
    output tile.)"""
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = tiny.CONFIGS[name]
    folder = model_folder(name)
    engine = Engine.from_pretrained(folder, dtype="bfloat16", page_size=page, num_pages=40)
    prompts = prompts_for(name, (5, 17, 33))
    got = engine.generate(prompts, max_new_tokens=8, ignore_eos=True)
    w = plain_weights(folder, "bfloat16")
    for prompt, out in zip(prompts, got):
        ids = list(prompt)
        for token in out:
            logits = plain.forward_logits(w, raw, ids)[-1]
            assert float(logits.max() - logits[token]) <= 3e-2
            ids.append(token)


def test_eos_stops_and_limit_stops():
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = tiny.CONFIGS["A"]
    folder = model_folder("A")
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=page, num_pages=40)
    prompt = prompts_for("A", (9,))[0]
    free_run = engine.generate([prompt], max_new_tokens=12, ignore_eos=True)[0]
    engine.eos_token_ids = (free_run[4],)
    stopped = engine.generate([prompt], max_new_tokens=12)[0]
    first = free_run.index(free_run[4])
    assert stopped == free_run[:first + 1]


def test_temperature_sampling_reproducible_and_batch_independent():
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.sampling.sampler import SamplingParams
    raw, page = tiny.CONFIGS["B"]
    folder = model_folder("B")
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=page, num_pages=64, max_batch_tokens=24)
    prompts = prompts_for("B", (1, 31, 64, 130))
    a = engine.generate(prompts, max_new_tokens=10, temperature=0.8, seed=1234, ignore_eos=True)
    b = engine.generate(prompts, max_new_tokens=10, temperature=0.8, seed=1234, ignore_eos=True)
    assert a == b
    assert a != engine.generate(prompts, max_new_tokens=10, temperature=0.8, seed=99, ignore_eos=True)
    # the same request alone (same seed and stream) draws the same tokens
    scheduler = engine.new_scheduler()
    alone = scheduler.submit("solo", prompts[2], 10, sampling=SamplingParams(0.8, 1234, stream=2), ignore_eos=True)
    while scheduler.has_work():
        scheduler.step()
    assert alone.output_ids == a[2]
    # and each draw is the plain inverse-CDF pick for the plain logits (up to ties at rounding level)
    w = plain_weights(folder, "float32")
    ids = list(prompts[1])
    for step, token in enumerate(a[1]):
        logits = plain.forward_logits(w, raw, ids)[-1]
        u = plain.uniform_from_key(1234, 1, step)
        cdf = plain.temperature_cdf(logits, 0.8)
        lo = float(cdf[token - 1]) if token else 0.0
        assert lo - 1e-4 <= u <= float(cdf[token]) + 1e-4
        ids.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rounds_queued_ahead_choose_the_same_tokens(dtype):
    """The scheduler queues a round before it has read the tokens of the one before (they reach the next round's
    embedding on the device).  Round by round or ahead: the same tokens, also across an EOS, whose speculative
    successor is dropped."""
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = tiny.CONFIGS["B"]
    engine = Engine.from_pretrained(model_folder("B"), dtype=dtype, page_size=page, num_pages=64, max_batch_tokens=40)
    prompts = prompts_for("B", (3, 50, 64, 21), seed=11)
    free_run = engine.generate(prompts, max_new_tokens=20, temperature=0.7, seed=5, ignore_eos=True)
    eos = free_run[1][6]
    results = {}
    for ahead in (False, True):
        scheduler = engine.new_scheduler(lookahead=ahead, eos_token_ids=(eos,))
        from ampere_kv_engine_b200.sampling.sampler import SamplingParams
        requests = [scheduler.submit(i, p, 20, sampling=SamplingParams(0.7, 5, stream=i)) for i, p in enumerate(prompts)]
        while scheduler.has_work():
            scheduler.step()
        results[ahead] = [r.output_ids for r in requests]
        assert all(r.stop_reason in ("eos", "length") for r in requests)
        if ahead:
            assert scheduler.dropped_tokens >= 1
        assert engine.manager.free_pages() == [64] * len(engine.manager.groups)
    assert results[True] == results[False]
    for run, full in zip(results[True], free_run):
        cut = full.index(eos) + 1 if eos in full else len(full)
        assert run == full[:cut]


def test_requests_wait_for_pages_and_all_finish():
    """Pages for two requests at a time only: the others wait in arrival order; all finish with the tokens they
    get when run alone; every page comes back."""
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = tiny.CONFIGS["A"]
    folder = model_folder("A")
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=page, num_pages=8, max_batch_tokens=16)
    prompts = prompts_for("A", (40, 33, 20, 45, 9))
    together = engine.generate(prompts, max_new_tokens=6, ignore_eos=True)
    alone = [engine.generate([p], max_new_tokens=6, ignore_eos=True)[0] for p in prompts]
    assert together == alone
    assert engine.manager.free_pages() == [8]


@pytest.mark.parametrize("name", ["A", "B"])
def test_preempted_requests_are_recomputed_to_the_same_tokens(name):
    """Optimistic admission with too few pages for everybody's outputs: the newest request gives its pages back,
    waits and is recomputed over its prompt and the tokens it already has; rounds are queued ahead meanwhile.
    Everybody ends with the tokens they get alone, no page is lost, and the window's released pages (B) take part."""
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = tiny.CONFIGS[name]
    lengths = (30, 22, 41, 12)
    new_tokens = 40
    need = [(n + new_tokens + page - 1) // page for n in lengths]
    pool = max(need) + sum(need) // 3
    engine = Engine.from_pretrained(model_folder(name), dtype="float32", page_size=page, num_pages=pool,
                                    max_batch_tokens=32)
    prompts = prompts_for(name, lengths, seed=3)
    alone = [engine.generate([p], max_new_tokens=new_tokens, ignore_eos=True)[0] for p in prompts]
    for ahead in (False, True):
        scheduler = engine.new_scheduler(admission="optimistic", lookahead=ahead)
        requests = [scheduler.submit(i, p, new_tokens, ignore_eos=True) for i, p in enumerate(prompts)]
        rounds = 0
        while scheduler.has_work():
            scheduler.step()
            rounds += 1
            assert rounds < 2000
        assert [r.output_ids for r in requests] == alone
        assert all(r.stop_reason == "length" for r in requests)
        assert scheduler.preemptions >= 1
        engine.manager.check_invariants()
        assert engine.manager.free_pages() == [pool] * len(engine.manager.groups)


def test_command_line_generate(tmp_path):
    folder = model_folder("A")
    prompt = prompts_for("A", (12,))[0]
    ids_file = tmp_path / "prompt.json"
    ids_file.write_text(json.dumps(prompt))
    cmd = [sys.executable, "-m", "ampere_kv_engine_b200.runner", "--model", folder, "--mode", "generate",
           "--cache", "paged", "--kv-dtype", "fp32", "--dtype", "float32", "--prompt-ids", str(ids_file),
           "--max-new-tokens", "5", "--ignore-eos"]
    proc = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("generated_token_ids = ")][0]
    got = json.loads(line.split(" = ", 1)[1])
    w = plain_weights(folder, "float32")
    assert got == plain.greedy_generate(w, tiny.CONFIGS["A"][0], prompt, 5)


def test_command_line_random_config_and_check_mode(tmp_path):
    """``--random-config`` builds seeded random weights without a model folder, ``--prompt-len`` makes a seeded
    prompt, and the default mode (check) compares the bfloat16 run with the float32 path step by step."""
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(tiny.config("C")))
    cmd = [sys.executable, "-m", "ampere_kv_engine_b200.runner", "--random-config", str(config_file), "--random-seed", "4",
           "--prompt-len", "37", "--max-new-tokens", "6", "--ignore-eos", "--num-pages", "16"]
    proc = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert "prompt_tokens=37" in proc.stdout and "mode=check" in proc.stdout
    line = [l for l in proc.stdout.splitlines() if l.startswith("generated_token_ids = ")][0]
    assert len(json.loads(line.split(" = ", 1)[1])) == 6
    check = [l for l in proc.stdout.splitlines() if l.startswith("check: ")][0]
    found = re.fullmatch(r"check: (\d+)/(\d+) steps pick the same token as the float32 path; "
                         r"largest logit difference ([0-9.e+-]+)", check)
    assert found, check
    agree, steps, worst = int(found.group(1)), int(found.group(2)), float(found.group(3))
    # random weights leave near-ties between the best tokens, so a step or two may pick the neighbour; the logits
    # themselves must agree to bfloat16 rounding
    assert steps == 6 and agree >= 4 and 0.0 < worst < 3e-2, check
    # neither a folder nor a configuration: refused with the two ways named
    proc = subprocess.run([sys.executable, "-m", "ampere_kv_engine_b200.runner", "--mode", "generate"], cwd=ROOT,
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "--model DIR or --random-config FILE" in proc.stderr
