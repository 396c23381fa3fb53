"""The host side of sampling against the plain sampler and wick's own unit tests (no GPU)."""
import numpy as np
import pytest

from wick_b200.sampling.sampler import Rng, SamplerConfig, pick_from_sorted
from plain import qwen3_plain as P


def test_defaults_are_the_reference_ones():
    c = SamplerConfig()
    assert (c.temperature, c.top_k, c.top_p, c.min_p, c.repetition_penalty, c.seed) == (0.7, 40, 0.9, 0.0, 1.0, 0x5EED)
    assert SamplerConfig.greedy().temperature == 0.0       # sampler.rs:16-25


def test_generator_matches_the_plain_one_and_known_values():
    # splitmix64(0) first output is a published constant of the algorithm
    z = (0 + 0x9E3779B97F4A7C15) & ((1 << 64) - 1)
    x = z
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & ((1 << 64) - 1)
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & ((1 << 64) - 1)
    assert Rng(0).s[0] == x ^ (x >> 31) == 0xE220A8397B1DCDAF
    for seed in (0, 1, 0x5EED, 2**63 + 5):
        a, b = Rng(seed), P.PlainRng(seed)
        assert [a.next_u64() for _ in range(50)] == [b.next_u64() for _ in range(50)]
        u = [a.next_f32() for _ in range(1000)]
        assert all(0.0 <= v < 1.0 for v in u) and abs(np.mean(u) - 0.5) < 0.05
        assert u[:20] == [float(b.next_f32()) for _ in range(20)]


def _sorted_candidates(logits, k):
    order = sorted(range(len(logits)), key=lambda i: (-float(logits[i]), i))[:k]
    return np.array([logits[i] for i in order], dtype=np.float32), np.array(order, dtype=np.int32)


@pytest.mark.parametrize("cfg", [
    SamplerConfig(),                                                   # the reference's defaults
    SamplerConfig(temperature=0.8, top_k=0, top_p=1.0),
    SamplerConfig(temperature=1.3, top_k=5, top_p=0.5, min_p=0.1),
    SamplerConfig(temperature=0.3, top_k=100, top_p=0.95, min_p=0.02, seed=99),
    SamplerConfig(temperature=1.0, top_k=1),
])
def test_candidate_cuts_and_draw_match_the_plain_sampler(cfg):
    rs = np.random.RandomState(1)
    a, b = Rng(cfg.seed), P.PlainRng(cfg.seed)
    for trial in range(200):
        logits = (rs.randn(300) * 3).astype(np.float32)
        k = len(logits) if cfg.top_k == 0 else min(cfg.top_k, len(logits))
        vals, idx = _sorted_candidates(logits, k)
        got = pick_from_sorted(vals, idx, cfg, a)
        want = P.sample_plain(logits, [], temperature=cfg.temperature, top_k=cfg.top_k, top_p=cfg.top_p,
                              min_p=cfg.min_p, repetition_penalty=1.0, rng=b)
        assert got == want, trial


def test_reference_unit_cases():
    # sampler.rs:150-162 (greedy, repetition penalty, top_k = 1)
    logits = [0.0, 3.0, 1.0, 2.9]
    assert P.argmax_first(logits) == 1
    assert P.sample_plain(logits, [1], temperature=0.0, top_k=40, top_p=0.9, min_p=0.0, repetition_penalty=1.5,
                          rng=P.PlainRng(1)) == 3
    r = Rng(0x5EED)
    cfg = SamplerConfig(temperature=1.0, top_k=1)
    for _ in range(50):
        v, i = _sorted_candidates(logits, 1)
        assert pick_from_sorted(v, i, cfg, r) == 1


def test_draws_follow_the_distribution():
    # sampler.rs:164-172: probabilities 1/4 and 3/4, 20000 draws, within 0.02
    cfg = SamplerConfig(temperature=1.0, top_k=0, top_p=1.0)
    r = Rng(cfg.seed)
    logits = np.array([0.0, np.log(3.0)], dtype=np.float32)
    v, i = _sorted_candidates(logits, 2)
    ones = sum(pick_from_sorted(v, i, cfg, r) == 1 for _ in range(20000))
    assert abs(ones / 20000 - 0.75) < 0.02


def test_argmax_first_takes_the_first_maximum_and_ignores_nan():
    assert P.argmax_first([1.0, 5.0, 5.0, 2.0]) == 1
    assert P.argmax_first([1.0, float("nan"), 0.5]) == 0
    assert P.argmax_first([float("-inf")] * 3) == 0
