#!/usr/bin/env python3
"""Writes ``plain_tiny.json`` beside this file: the plain implementation's logits
and greedy continuation for two tiny Qwen3 models whose weights this script makes
itself (numpy's seeded legacy generator, so the values do not depend on any
library's version), plus, where wick's source tree is at hand, how far the plain
implementation is from the logits that wick's repository records for its own tiny
fixture (tests/fixtures/tiny/qwen3-qknorm-f32/expected.json; wick's
tests/tiny_models.rs:58-113 checks its engine against the same file).

wick is a Rust program and no Rust toolchain is installed here, so wick's own
model code could not be run; the recorded logits of its fixture are the nearest
thing to it, and everything else rests on the formulas that
``tests/plain/qwen3_plain.py`` cites.

    python tests/golden/make_golden.py [--fixture DIR]

``tests/test_plain_golden.py`` recomputes the values and compares.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from plain import qwen3_plain as P  # noqa: E402

CONFIGS = {
    "g1": dict(hidden_size=48, num_attention_heads=3, num_key_value_heads=1, head_dim=16, intermediate_size=80,
               num_hidden_layers=2, vocab_size=97, max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-6,
               tie_word_embeddings=True),
    "g2": dict(hidden_size=40, num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=56,
               num_hidden_layers=3, vocab_size=131, max_position_embeddings=64, rope_theta=500000.0, rms_norm_eps=1e-5,
               tie_word_embeddings=False),
}
TOKENS = {"g1": [5, 17, 3, 96, 0, 41, 41, 8, 60, 2, 33], "g2": [130, 1, 77, 12, 9, 9, 54]}
GREEDY_NEW = 6


def make_weights(cfg: dict, seed: int):
    """Every tensor a Qwen3 checkpoint names (wick src/model.rs:95-173), float32."""
    rs = np.random.RandomState(seed)
    H, hd, I, V = cfg["hidden_size"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    w = {}

    def mat(name, r, c, std=0.08):
        w[name] = torch.from_numpy((rs.standard_normal((r, c)) * std).astype(np.float32))

    def vec(name, n):
        w[name] = torch.from_numpy((1.0 + 0.2 * rs.standard_normal(n)).astype(np.float32))

    mat("model.embed_tokens.weight", V, H, 0.5)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        vec(p + "input_layernorm.weight", H)
        mat(p + "self_attn.q_proj.weight", nh * hd, H)
        mat(p + "self_attn.k_proj.weight", nkv * hd, H)
        mat(p + "self_attn.v_proj.weight", nkv * hd, H)
        mat(p + "self_attn.o_proj.weight", H, nh * hd)
        vec(p + "self_attn.q_norm.weight", hd)
        vec(p + "self_attn.k_norm.weight", hd)
        vec(p + "post_attention_layernorm.weight", H)
        mat(p + "mlp.gate_proj.weight", I, H)
        mat(p + "mlp.up_proj.weight", I, H)
        mat(p + "mlp.down_proj.weight", H, I)
    vec("model.norm.weight", H)
    if not cfg["tie_word_embeddings"]:
        mat("lm_head.weight", V, H, 0.3)
    return w


def compute(fixture: str) -> dict:
    out = {"models": {}}
    for i, (name, j) in enumerate(sorted(CONFIGS.items())):
        cfg = P.plain_config(j)
        w = make_weights(j, 1234 + i)
        logits = P.forward(cfg, w, TOKENS[name])
        out["models"][name] = {
            "tokens": TOKENS[name],
            "logits_last": [round(float(v), 6) for v in logits[-1]],
            "logits_row_sums": [round(float(v), 5) for v in logits.double().sum(1)],
            "greedy": P.greedy(cfg, w, TOKENS[name], GREEDY_NEW),
        }
    if os.path.isdir(fixture):
        cfg, w = P.read_model_dir(fixture)
        exp = json.load(open(os.path.join(fixture, "expected.json")))
        got = P.forward(cfg, w, exp["tokens"])
        out["wick_fixture"] = {
            "what": "max |plain - recorded| over the logits wick records for tests/fixtures/tiny/qwen3-qknorm-f32",
            "max_abs_diff": float((got - torch.tensor(exp["logits"])).abs().max()),
            "greedy_equal": P.greedy(cfg, w, exp["greedy_prompt"], len(exp["greedy"])) == exp["greedy"],
        }
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--fixture", default=os.environ.get("WICK_REFERENCE_FIXTURE", ""))
    args = ap.parse_args()
    res = compute(args.fixture)
    with open(os.path.join(HERE, "plain_tiny.json"), "w") as f:
        json.dump(res, f, indent=1)
        f.write("\n")
    print(json.dumps({k: (v if k != "models" else list(v)) for k, v in res.items()}))
