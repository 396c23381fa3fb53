"""The plain implementation against the logits that wick's repository records
for its tiny Qwen3 model (made by wick's scripts/make_tiny.py with transformers
in float32; checked by wick's tests/tiny_models.rs:58-71 to 1e-3 and the greedy
continuation in :97-113).  The fixture is read where wick's source tree is at
hand and the test is skipped elsewhere."""
import json
import os

import pytest
import torch

from plain import qwen3_plain as P

# wick's source tree is looked for beside this repository unless the variable names it.
_BESIDE = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
FIXTURE = os.environ.get("WICK_REFERENCE_FIXTURE", os.path.join(_BESIDE, "tests", "fixtures", "tiny", "qwen3-qknorm-f32"))
needs_fixture = pytest.mark.skipif(not os.path.isdir(FIXTURE), reason="wick's fixture is not on this machine")


@needs_fixture
def test_plain_matches_recorded_logits():
    cfg, w = P.read_model_dir(FIXTURE)
    exp = json.load(open(os.path.join(FIXTURE, "expected.json")))
    got = P.forward(cfg, w, exp["tokens"])
    want = torch.tensor(exp["logits"])
    assert got.shape == want.shape
    # The recorded values are rounded to 1e-6; wick itself reports 4.7e-5 on a real model.
    assert (got - want).abs().max().item() < 2e-5
    got64 = P.forward(cfg, w, exp["tokens"], dtype=torch.float64)
    assert (got64 - want).abs().max().item() < 2e-5


@needs_fixture
def test_plain_greedy_matches_recorded_tokens():
    cfg, w = P.read_model_dir(FIXTURE)
    exp = json.load(open(os.path.join(FIXTURE, "expected.json")))
    assert P.greedy(cfg, w, exp["greedy_prompt"], len(exp["greedy"])) == exp["greedy"]
