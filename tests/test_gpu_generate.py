"""Generation through the Python entry point and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from helpers import (BF16_REL, CONFIGS, assert_logits_close, make_engine, model_dir, plain_model,  # noqa: E402
                     random_tokens)
from plain import qwen3_plain as P  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# Weights with a wider spread than N(0, 0.02) separate the top logits well, so
# that the greedy token is the same in float32 whatever the order of the sums.
STD = 0.08


def test_greedy_generation_matches_the_plain_loop_config_a():
    """The tiny workload A: 3 prompts of 5/11/17 tokens, 8 greedy steps."""
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
        # bfloat16 may pick another of two close candidates.  Every token it did pick must be
        # one the plain implementation rates within the bfloat16 tolerance of its best, at the
        # position where it was picked; and the engine's own logits along the generated
        # sequence (fed again, one token at a time) must match the plain ones.
        for p, r in zip(prompts, out):
            seq = list(p) + r.tokens
            ref = P.forward(cfg, w, seq) if len(seq) > len(p) else None
            slot = eng.open_seq()
            got = [eng.step([slot], [list(p)]).clone()] + [eng.step([slot], [[t]]).clone() for t in r.tokens[:-1]]
            eng.close_seq(slot)
            for i, t in enumerate(r.tokens):
                row = ref[len(p) - 1 + i]
                assert row[t] >= row.max() - BF16_REL * row.abs().max(), f"token {i} of prompt {len(p)}"
                assert int(got[i][0].argmax()) == t or got[i][0][t] >= got[i][0].max() - 1e-3 * got[i][0].abs().max()
            if r.tokens:
                assert_logits_close(torch.cat(got), ref[len(p) - 1:len(p) - 1 + len(r.tokens)], dtype, "generated positions")
            assert r.finish in ("stop", "length") and (r.finish == "length") == (len(r.tokens) == 10)
            assert stop not in r.tokens
    eng.cache.check()
    assert eng.cache.pages.n_held == 0


def test_temperature_sampling_given_the_engines_logits():
    """The tiny workload B: prompts 1/7/30/64, 12 steps at temperature 0.8
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


SAMPLERS = [wick.SamplerConfig.greedy(),
            wick.SamplerConfig(temperature=0.8, seed=1234),
            wick.SamplerConfig(temperature=0.9, top_k=0, top_p=1.0, seed=77),
            wick.SamplerConfig(temperature=1.1, top_k=20, top_p=0.8, min_p=0.05, repetition_penalty=1.3, seed=5)]


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("D", "bfloat16"), ("R", "bfloat16")])
def test_a_batch_stepped_on_the_device_gives_the_tokens_of_the_stepwise_loop(name, dtype):
    """The generation loop over a batch that is advanced on the device (sampled token, length,
    finished flag, generators and seen tokens stay there; the host reads one step behind)
    against the same loop taking one step at a time with the sampler on the host side: same
    tokens and endings for every way of sampling, with stop tokens, with requests that end at
    different times and with more requests than one batch holds.  (R has a vocabulary beyond
    the selection kernel's 1,024 candidates: the draw over all tokens.)"""
    vocab = CONFIGS[name]["vocab_size"]
    eng = make_engine(name, dtype, std=STD, max_tokens=64 * 12)
    prompts = [random_tokens(vocab, n, 300 + n) for n in (3, 70, 1, 18, 40, 9, 2)]
    for k, cfg in enumerate(SAMPLERS):
        base = wick.GenOptions(max_tokens=9, sampler=cfg, max_batch=4)
        free = wick.generate(eng, prompts, base, sampler_factory=wick.Sampler)
        stop = [free[1].tokens[3], free[4].tokens[0]]
        opts = wick.GenOptions(max_tokens=9, sampler=cfg, max_batch=4, stop_token_ids=stop)
        want = wick.generate(eng, prompts, opts, sampler_factory=wick.Sampler)
        runs = []
        begin = eng.begin_run
        eng.begin_run = lambda *a, **kw: runs.append(begin(*a, **kw)) or runs[-1]
        try:
            got = wick.generate(eng, prompts, opts)
        finally:
            del eng.begin_run
        assert [(r.tokens, r.finish) for r in got] == [(r.tokens, r.finish) for r in want], f"sampler {k}"
        assert any(r.finish == "stop" for r in got) and any(r.finish == "length" for r in got)
        assert len(runs) == 2, "two batches"
        # a description goes to the device when the batch's composition changes, not every step
        assert all(r.uploads <= 5 for r in runs), [r.uploads for r in runs]
        eng.cache.check()
        assert eng.cache.pages.n_held == 0 and eng.cache.slots.n_held == 0


@pytest.mark.parametrize("graphs", [True, False])
def test_steady_decoding_uploads_nothing(graphs):
    eng = make_engine("D", "bfloat16", std=STD, max_tokens=64 * 16, use_graphs=graphs)
    prompts = [random_tokens(640, n, 500 + n) for n in (30, 5, 11)]
    runs = []
    begin = eng.begin_run
    eng.begin_run = lambda *a, **kw: runs.append(begin(*a, **kw)) or runs[-1]
    out = wick.generate(eng, prompts, wick.GenOptions(max_tokens=40, sampler=wick.SamplerConfig.greedy()))
    assert all(len(r.tokens) == 40 for r in out)
    assert runs[0].uploads == 1, "39 decode steps of one composition: one description"
    cfg, w = plain_model("D", std=STD)
    for p, r in zip(prompts, out):
        ref = P.forward(cfg, w, list(p) + r.tokens)
        for i, t in enumerate(r.tokens):
            row = ref[len(p) - 1 + i]
            assert row[t] >= row.max() - BF16_REL * row.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_models_own_stop_tokens_end_a_sequence(dtype):
    """Config B names two end-of-sequence ids (7 and 9).  A prompt whose greedy continuation
    under the plain implementation reaches one of them: the entry point and the command line
    must stop there without being told any stop token."""
    cfg, w = plain_model("B", std=STD)
    p = random_tokens(1000, 4, 9058)             # (found by a search over seeds: reaches token 9 at its ninth token)
    toks = P.greedy(cfg, w, p, 12)
    assert any(t in (7, 9) for t in toks[1:]), "the prompt no longer reaches an end-of-sequence id: search again"
    cut = next(i for i, t in enumerate(toks) if t in (7, 9))
    want = P.greedy(cfg, w, p, 12, stop=(7, 9))
    assert want == toks[:cut]
    eng = make_engine("B", dtype, std=STD)
    out = wick.generate(eng, [p], wick.GenOptions(max_tokens=12, sampler=wick.SamplerConfig.greedy()))[0]
    if dtype == "float32":
        assert out.tokens == want and out.finish == "stop"
        env = dict(os.environ, PYTHONPATH=ROOT)
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "wick"), "run", model_dir("B", std=STD), "--ids",
                            ",".join(map(str, p)), "-n", "12", "-t", "0", "-q", "f32"], capture_output=True, text=True,
                           env=env, timeout=600)
        assert r.returncode == 0, r.stderr
        assert json.loads(r.stdout.strip().splitlines()[0]) == want and "Stop" in r.stderr
    else:
        assert 7 not in out.tokens and 9 not in out.tokens
        assert out.finish == "stop" or len(out.tokens) == 12


def test_a_shrinking_batch_that_ends_soon_keeps_its_captured_step():
    """Five requests that end at different times: the batch shrinks from 5 (a captured step of
    8) to 1, but all of them end within 64 steps, so no smaller step is captured on the way:
    one captured step serves the whole batch.  A generation that goes on for long captures the
    step of its own size."""
    eng = make_engine("D", "bfloat16", std=STD, max_tokens=64 * 40)
    prompts = [random_tokens(640, n, 800 + n) for n in (12, 5, 30, 7, 3)]
    base = wick.GenOptions(max_tokens=30, sampler=wick.SamplerConfig.greedy())
    free = wick.generate(eng, prompts, base, sampler_factory=wick.Sampler)
    stops = [free[0].tokens[3], free[1].tokens[8], free[3].tokens[14]]
    opts = wick.GenOptions(max_tokens=30, sampler=wick.SamplerConfig.greedy(), stop_token_ids=stops)
    want = wick.generate(eng, prompts, opts, sampler_factory=wick.Sampler)
    eng2 = make_engine("D", "bfloat16", std=STD, max_tokens=64 * 40, use_graphs=True)
    got = wick.generate(eng2, prompts, opts)
    assert [(r.tokens, r.finish) for r in got] == [(r.tokens, r.finish) for r in want]
    assert len({len(r.tokens) for r in got}) > 2, "the requests end at different times"
    captured = sorted(k for k, g in eng2._graphs.items() if g.graph is not None)
    assert captured == [(8, 8)], captured
    long = wick.generate(eng2, [prompts[0]], wick.GenOptions(max_tokens=200, sampler=wick.SamplerConfig.greedy()))
    assert len(long[0].tokens) == 200 and (1, 8) in {k for k, g in eng2._graphs.items() if g.graph is not None}


def test_warm_up_captures_what_generation_would():
    """Engine.warm_up captures the decode steps and the short prompt steps ahead of time;
    a generation within those sizes then captures nothing more, and gives what it gives on an
    engine that was not warmed up."""
    eng = make_engine("D", "bfloat16", std=STD, max_tokens=64 * 40, use_graphs=True)
    n = eng.warm_up(max_batch=5, context=300, prompt_tokens=128)
    decode = sorted(k for k, g in eng._graphs.items() if g.graph is not None)
    assert decode == [(1, 8), (2, 8), (4, 8), (8, 8)], decode
    assert sorted(eng._prompt_graphs) == [(t, b + 1, b + 1) for t in (64, 128) for b in (1, 2, 4, 8)]
    assert n == len(decode) + len(eng._prompt_graphs)
    assert eng.warm_up(max_batch=5, context=300, prompt_tokens=128) == 0
    eng.cache.check()
    prompts = [random_tokens(640, k, 900 + k) for k in (12, 5, 30, 7, 3)]
    opts = wick.GenOptions(max_tokens=20, sampler=wick.SamplerConfig.greedy())
    got = wick.generate(eng, prompts, opts)
    assert sorted(k for k, g in eng._graphs.items() if g.graph is not None) == decode and len(eng._prompt_graphs) == 8
    cold = make_engine("D", "bfloat16", std=STD, max_tokens=64 * 40, use_graphs=True)
    want = wick.generate(cold, prompts, opts)
    assert [(r.tokens, r.finish) for r in got] == [(r.tokens, r.finish) for r in want]
    off = make_engine("D", "bfloat16", std=STD, max_tokens=64 * 40, use_graphs=False)
    assert off.warm_up(max_batch=5) == 0
