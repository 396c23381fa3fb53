"""Generation through the Python entry point and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from helpers import CONFIGS, make_engine, model_dir, plain_model, random_tokens  # noqa: E402
from plain import qwen3_plain as P  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# Weights with a wider spread than N(0, 0.02) separate the top logits well, so
# that the greedy token is the same in float32 whatever the order of the sums.
STD = 0.08


def test_greedy_generation_matches_the_plain_loop_config_a():
    """BASELINE's tiny workload A: 3 prompts of 5/11/17 tokens, 8 greedy steps."""
    eng = make_engine("A", "float32", std=STD)
    cfg, w = plain_model("A", std=STD)
    prompts = [random_tokens(512, n, 60 + n) for n in (5, 11, 17)]
    out = wick.generate(eng, prompts, wick.GenOptions(max_tokens=8, sampler=wick.SamplerConfig.greedy()))
    for p, r in zip(prompts, out):
        assert r.tokens == P.greedy(cfg, w, p, 8) and r.finish == "length" and r.prompt_tokens == len(p)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_with_stop_tokens_and_more_requests_than_a_batch_holds(dtype):
    eng = make_engine("B", dtype, std=STD, max_tokens=64 * 6)
    cfg, w = plain_model("B", std=STD)
    prompts = [random_tokens(1000, n, 70 + n) for n in (1, 7, 30, 64, 3, 12, 40)]
    free = [P.greedy(cfg, w, p, 10) for p in prompts]
    stop = free[1][4]
    want = [P.greedy(cfg, w, p, 10, stop=(stop,)) for p in prompts]
    out = wick.generate(eng, prompts, wick.GenOptions(max_tokens=10, sampler=wick.SamplerConfig.greedy(),
                                                      stop_token_ids=[stop], max_batch=3))
    if dtype == "float32":
        assert [r.tokens for r in out] == want
        assert out[1].finish == "stop" and len(out[1].tokens) <= 4
    else:
        # bfloat16 may pick another of two close candidates; the first tokens agree
        assert sum(r.tokens[:2] == w_[:2] for r, w_ in zip(out, want)) >= len(want) - 1
    eng.cache.check()
    assert eng.cache.pages.n_held == 0


def test_temperature_sampling_given_the_engines_logits():
    """BASELINE's tiny workload B: prompts 1/7/30/64, 12 steps at temperature 0.8
    with a fixed seed.  The tokens must be the ones the plain sampler draws from
    the logits the engine produced (the sampler is tested apart from the model)."""
    eng = make_engine("B", "float32", std=STD)
    prompts = [random_tokens(1000, n, 80 + n) for n in (1, 7, 30, 64)]
    for cfg in (wick.SamplerConfig(temperature=0.8, seed=1234),
                wick.SamplerConfig(temperature=0.8, top_k=0, top_p=1.0, seed=1234),
                wick.SamplerConfig(temperature=1.1, top_k=20, top_p=0.8, min_p=0.05, repetition_penalty=1.3, seed=5)):
        out = wick.generate(eng, prompts, wick.GenOptions(max_tokens=12, sampler=cfg))
        for p, r in zip(prompts, out):
            assert len(r.tokens) == 12
            rng = P.PlainRng(cfg.seed)
            slot = eng.open_seq()
            seq = list(p)
            logits = eng.step([slot], [seq])[0].cpu()
            for t in r.tokens:
                want = P.sample_plain(logits.numpy(), seq, temperature=cfg.temperature, top_k=cfg.top_k,
                                      top_p=cfg.top_p, min_p=cfg.min_p, repetition_penalty=cfg.repetition_penalty,
                                      rng=rng)
                assert t == want
                seq.append(t)
                logits = eng.step([slot], [[t]])[0].cpu()
            eng.close_seq(slot)


def test_sampling_alone_and_in_a_batch_gives_the_same_tokens():
    eng = make_engine("A", "float32", std=STD)
    prompts = [random_tokens(512, n, 90 + n) for n in (4, 9, 2)]
    opts = wick.GenOptions(max_tokens=6, sampler=wick.SamplerConfig(temperature=0.9, seed=42))
    together = wick.generate(eng, prompts, opts)
    alone = [wick.generate(eng, [p], opts)[0] for p in prompts]
    assert [r.tokens for r in together] == [r.tokens for r in alone]


def test_command_line_run_and_errors(tmp_path):
    d = model_dir("A", std=STD)
    cfg, w = plain_model("A", std=STD)
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "wick")]
    r = subprocess.run(cmd + ["run", d, "--ids", "5,17,3", "--ids", "9,9", "-n", "5", "-t", "0", "-q", "f32"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
    assert lines == [P.greedy(cfg, w, [5, 17, 3], 5), P.greedy(cfg, w, [9, 9], 5)]
    assert "wick: " in r.stderr and "2 layers" in r.stderr and "generated at" in r.stderr and "Length" in r.stderr
    r = subprocess.run(cmd + ["run", str(tmp_path / "nowhere"), "--ids", "1"], capture_output=True, text=True, env=env)
    assert r.returncode == 1 and r.stderr.startswith("wick: ") and "config.json" in r.stderr
    r = subprocess.run(cmd + ["run", d, "--bogus"], capture_output=True, text=True, env=env)
    assert r.returncode == 2 and "unknown option --bogus" in r.stderr
    r = subprocess.run(cmd + ["bench", d, "--prompt-len", "16", "-n", "4", "--batch", "2", "-q", "bf16"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "tok/s" in r.stdout and "ms/step" in r.stdout, r.stderr
