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


class LaggingRun:
    """A batch stepped one step ahead of what the loop has read, the way the device-side
    run is: ``launch`` feeds every sequence the token sampled for it last, a sequence that
    sampled a stop token or reached its limit is frozen (it keeps its token and its place),
    and the loop sees a step's tokens only when it collects them."""
    depth = 1

    def __init__(self, engine, opts, stops, n):
        self.e, self.stops = engine, set(stops)
        self.next, self.made, self.limit, self.frozen = {}, {}, {}, {}
        self.queue = []
        self.launches = []

    def _sample(self, slots, logits):
        out = []
        for s, row in zip(slots, logits):
            tok = int(row.argmax())
            out.append(tok)
            if self.frozen[s]:
                continue
            self.made[s] += 1
            self.next[s] = tok
            if tok in self.stops or self.made[s] >= self.limit[s]:
                self.frozen[s] = True
        self.queue.append(out)

    def start(self, slots, prompts, limits):
        for s, l in zip(slots, limits):
            self.made[s], self.limit[s], self.frozen[s] = 0, l, False
        self._sample(slots, self.e.step(list(slots), [list(p) for p in prompts], None))

    def launch(self, slots):
        self.launches.append(list(slots))
        live = [s for s in slots if not self.frozen[s]]
        logits = torch.full((len(slots), self.e.vocab), -1.0)
        if live:
            got = self.e.step(live, [[self.next[s]] for s in live], None)
            for s, row in zip(live, got):
                logits[slots.index(s)] = row
        self._sample(slots, logits)

    def collect(self):
        return self.queue.pop(0)


def test_a_run_one_step_ahead_gives_the_same_results():
    prompts = [[1], [30], [40, 41], [7]]
    kw = dict(max_tokens=6, stop_token_ids=[4, 44])
    want = run(ScriptedEngine(), prompts, **kw)
    e = ScriptedEngine()
    runs = []

    def factory(engine, opts, stops, n):
        runs.append(LaggingRun(engine, opts, stops, n))
        return runs[-1]

    got = generate(e, prompts, GenOptions(sampler=SamplerConfig.greedy(), **kw), run_factory=factory)
    assert [(r.tokens, r.finish) for r in got] == [(r.tokens, r.finish) for r in want]
    assert got[0].tokens == [2, 3] and got[0].finish == "stop" and got[2].tokens == [42, 43]
    fed = [t for _, toks in e.steps[1:] for seq in toks for t in seq]
    assert 4 not in fed and 44 not in fed, "a stop token is never fed, not even in the step launched ahead"
    # sequence 0 stops at its third token: the step launched before the loop read that token
    # still carries its slot (frozen), the one after does not
    slot0 = e.opened[0]
    assert [slot0 in l for l in runs[0].launches] == [True, True, True, False, False]
    e.cache.check()
    assert e.cache.slots.n_held == 0 and e.cache.pages.n_held == 0


def test_a_run_ahead_launches_nothing_beyond_the_length_limits():
    e = ScriptedEngine()
    runs = []
    res = generate(e, [[1, 2, 3], [10]], GenOptions(sampler=SamplerConfig.greedy(), max_tokens=4),
                   run_factory=lambda eng, o, st, n: runs.append(LaggingRun(eng, o, st, n)) or runs[-1])
    assert [r.tokens for r in res] == [[4, 5, 6, 7], [11, 12, 13, 14]]
    assert len(runs[0].launches) == 3 and len(e.steps) == 4, "no step runs after the last token"


def test_stop_tokens_of_the_model_end_a_sequence_without_being_asked_for():
    e = ScriptedEngine()
    e.spec = type("Spec", (), {"stop_token_ids": (5,)})()
    res = run(e, [[1], [30]], max_tokens=8)
    assert res[0].tokens == [2, 3, 4] and res[0].finish == "stop" and res[1].finish == "length"
    res = run(e, [[1]], max_tokens=8, stop_token_ids=[3])
    assert res[0].tokens == [2] and res[0].finish == "stop", "the caller's stop tokens are added to the model's"


def test_kernel_status_is_checked_when_a_batch_has_drained():
    e = ScriptedEngine()
    calls = []
    e.check_kernels = lambda: calls.append(1)
    run(e, [[i] for i in range(5)], max_tokens=2, max_batch=2)
    assert len(calls) == 3, "once per batch"
