"""Properties of the plain implementation itself (no GPU)."""
import math

import torch

from helpers import plain_model, random_tokens
from plain import qwen3_plain as P


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]])
    w = torch.tensor([1.0, 2.0, 1.0, 1.0])
    out = P.rms_norm(x, w, 0.0)
    s = 1.0 / math.sqrt((9 + 16) / 4)
    assert torch.allclose(out, torch.tensor([[3 * s, 8 * s, 0.0, 0.0]]))


def test_rope_is_a_rotation_of_half_split_pairs():
    inv = P.rope_inv_freq(10000.0, 8)
    assert inv.dtype == torch.float32 and inv[0] == 1.0 and abs(inv[1].item() - 10000 ** -0.25) < 1e-7
    x = torch.randn(5, 3, 8)
    y = P.rope(x, torch.arange(5), inv)
    assert torch.allclose(y[0], x[0]), "position 0 is the identity"
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    a, b, th = x[2, 1, 1], x[2, 1, 5], 2 * inv[1]
    assert abs(y[2, 1, 1] - (a * math.cos(th) - b * math.sin(th))) < 1e-5
    assert abs(y[2, 1, 5] - (b * math.cos(th) + a * math.sin(th))) < 1e-5


def test_attention_is_causal_and_groups_heads():
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = P.causal_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0
    assert torch.allclose(P.causal_attention(q, k2, v2)[:4], out[:4])
    # one dominant key: the output is its value
    q[5, 0] = 50 * k[2, 0] / k[2, 0].norm() ** 2 * math.sqrt(8) * 10
    out = P.causal_attention(q, k, v)
    assert torch.allclose(out[5, 0], v[2, 0], atol=1e-3)


def test_logits_at_a_position_do_not_depend_on_later_tokens():
    cfg, w = plain_model("B")
    t = random_tokens(cfg["vocab"], 40, 1)
    full = P.forward(cfg, w, t)
    assert torch.allclose(P.forward(cfg, w, t[:17]), full[:17], atol=1e-6)
    assert (P.forward(cfg, w, t, dtype=torch.float64) - full).abs().max() < 1e-5


def test_schedule_variants():
    cfg, w = plain_model("A")
    t = random_tokens(cfg["vocab"], 12, 2)
    base = P.forward(cfg, w, t)
    assert torch.equal(P.forward(cfg, w, t, schedule=[(0, None), (1, None)]), base)
    twice = P.forward(cfg, w, t, schedule=[(0, None), (1, None), (1, None)])
    shared = P.forward(cfg, w, t, schedule=[(0, None), (1, 0)])
    assert not torch.allclose(twice, base) and not torch.allclose(shared, base)


def test_greedy_stops_on_a_stop_token():
    cfg, w = plain_model("A")
    free = P.greedy(cfg, w, [3, 4, 5], 6)
    assert len(free) == 6
    k = max(i for i in range(6) if free[i] not in free[:i])     # last token that appears for the first time
    assert P.greedy(cfg, w, [3, 4, 5], 6, stop=(free[k],)) == free[:k]
