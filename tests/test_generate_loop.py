"""The generation loop's decisions, against a scripted engine (no GPU)."""
import pytest
import torch

from wick_b200.cache import Cache
from wick_b200.engine.generate import GenOptions, generate, plan_batch
from wick_b200.parts.base import CacheNeed
from wick_b200.sampling.sampler import SamplerConfig


class ScriptedEngine:
    """Logits that make greedy sampling emit, for a sequence whose last fed token
    is t, the token (t + 1) % vocab.  Records every step."""

    def __init__(self, vocab=50, max_tokens=64 * 16, max_seqs=None, max_position=None):
        self.vocab = vocab
        self.cache = Cache([CacheNeed("paged_kv", kv_heads=1, head_dim=16)], max_tokens=max_tokens,
                           dtype=torch.float32, device="cpu", allocate=False, max_seqs=max_seqs,
                           max_position=max_position)
        self.steps = []
        self.opened, self.closed = [], []

    def open_seq(self):
        s = self.cache.open_seq()
        self.opened.append(s)
        return s

    def close_seq(self, s):
        self.closed.append(s)
        self.cache.close_seq(s)

    def step(self, slots, tokens, want):
        self.steps.append((list(slots), [list(t) for t in tokens]))
        for s, t in zip(slots, tokens):
            self.cache.reserve(s, self.cache.length(s) + len(t))
            self.cache.advance(s, len(t))
        out = torch.full((len(slots), self.vocab), -1.0)
        for i, t in enumerate(tokens):
            out[i, (t[-1] + 1) % self.vocab] = 1.0
        return out


class CpuGreedy:
    def __init__(self, cfg, n):
        pass

    def sample(self, logits, seq_ids, histories=None):
        return logits.argmax(-1).tolist()


def run(engine, prompts, **kw):
    opts = GenOptions(sampler=SamplerConfig.greedy(), **kw)
    return generate(engine, prompts, opts, sampler_factory=CpuGreedy)


def test_unequal_prompts_one_prefill_then_one_token_each():
    e = ScriptedEngine()
    res = run(e, [[1, 2, 3], [10], [20, 21]], max_tokens=4)
    assert [r.tokens for r in res] == [[4, 5, 6, 7], [11, 12, 13, 14], [22, 23, 24, 25]]
    assert [r.finish for r in res] == ["length"] * 3 and [r.prompt_tokens for r in res] == [3, 1, 2]
    assert e.steps[0][1] == [[1, 2, 3], [10], [20, 21]], "all prompts run in one step"
    assert all(len(t) == 1 for _, toks in e.steps[1:] for t in toks)
    assert len(e.steps) == 4, "no step runs after the last token (engine.rs:204-206)"
    e.cache.check()
    assert e.cache.slots.n_held == 0 and e.cache.pages.n_held == 0


def test_stop_token_ends_a_sequence_early_and_is_neither_returned_nor_fed():
    e = ScriptedEngine()
    res = run(e, [[1], [30]], max_tokens=8, stop_token_ids=[4])
    assert res[0].tokens == [2, 3] and res[0].finish == "stop"
    assert res[1].tokens == list(range(31, 39)) and res[1].finish == "length"
    fed = [t for _, toks in e.steps for seq in toks for t in seq]
    assert 4 not in fed
    # after the first sequence stopped the batch shrank to one sequence
    assert [len(s) for s, _ in e.steps] == [2, 2, 2, 1, 1, 1, 1, 1]
    assert e.closed[0] == e.opened[0], "a finished sequence gives its slot back at once"


def test_stop_token_as_first_sample_gives_an_empty_result():
    e = ScriptedEngine()
    res = run(e, [[3]], max_tokens=5, stop_token_ids=[4])
    assert res[0].tokens == [] and res[0].finish == "stop" and len(e.steps) == 1


def test_limit_is_clamped_to_the_context():
    e = ScriptedEngine()
    res = run(e, [[1, 2, 3, 4, 5, 6]], max_tokens=100, context=10)
    assert len(res[0].tokens) == 4 and res[0].finish == "length"    # engine.rs:169-170
    res = run(e, [[1, 2, 3]], max_tokens=0)
    assert res[0].tokens == [] and res[0].finish == "length"
    assert e.cache.slots.n_held == 0


def test_errors_for_empty_and_overlong_prompts():
    e = ScriptedEngine()
    with pytest.raises(ValueError, match="empty prompt"):
        run(e, [[1], []])
    with pytest.raises(ValueError, match="prompt is 12 tokens, context is 8"):
        run(e, [list(range(12))], context=8)
    e2 = ScriptedEngine(max_position=6)
    with pytest.raises(ValueError, match="context is 6"):
        run(e2, [list(range(7))])


def test_batches_follow_one_another_and_reuse_slots():
    e = ScriptedEngine(max_seqs=4)
    prompts = [[i] for i in range(10)]
    res = run(e, prompts, max_tokens=3, max_batch=4)
    assert [r.tokens for r in res] == [[i + 1, i + 2, i + 3] for i in range(10)]
    starts = [s for s, toks in e.steps if len(toks[0]) == 1 and toks[0][0] < 10 and toks[0][0] == prompts[toks[0][0]][0]]
    first_steps = [i for i, (s, toks) in enumerate(e.steps) if i % 3 == 0]
    assert [len(e.steps[i][0]) for i in first_steps] == [4, 4, 2]
    assert set(e.opened) == {1, 2, 3, 4} and len(e.opened) == 10, "slots are used again by later batches"
    e.cache.check()
    assert e.cache.slots.n_held == 0 and e.cache.pages.n_held == 0


def test_batch_size_is_bounded_by_free_pages():
    e = ScriptedEngine(max_tokens=64 * 4)
    res = run(e, [[1] * 60, [2] * 60, [3] * 60], max_tokens=10)     # 70 tokens -> 2 pages each
    assert [len(s) for s, _ in e.steps][:1] == [2]
    assert all(len(r.tokens) == 10 for r in res)
    with pytest.raises(RuntimeError, match="needs 5 cache pages"):
        run(e, [[1] * 300], max_tokens=10)


def test_plan_batch_takes_a_prefix_of_the_queue():
    lens, lim = [10, 100, 10, 10], [10, 100, 10, 10]
    assert plan_batch([0, 1, 2, 3], lens, lim, free_pages=10, free_slots=8, max_batch=8) == [0, 1, 2, 3]
    assert plan_batch([0, 1, 2, 3], lens, lim, free_pages=4, free_slots=8, max_batch=8) == [0]
    assert plan_batch([0, 1, 2, 3], lens, lim, free_pages=10, free_slots=2, max_batch=8) == [0, 1]
    assert plan_batch([2, 3], lens, lim, free_pages=10, free_slots=8, max_batch=1) == [2]
    assert plan_batch([1], lens, lim, free_pages=3, free_slots=8, max_batch=8) == []


def test_on_step_sees_who_is_still_running():
    e = ScriptedEngine()
    seen = []
    generate(e, [[1], [30]], GenOptions(max_tokens=3, sampler=SamplerConfig.greedy(), stop_token_ids=[3]),
             sampler_factory=CpuGreedy, on_step=lambda n, live: seen.append((n, list(live))))
    assert seen == [(1, [0, 1]), (2, [1]), (3, [])]
