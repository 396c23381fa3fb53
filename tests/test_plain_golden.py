"""The plain implementation against the values committed under tests/golden
(made by tests/golden/make_golden.py, which also records how far the plain
implementation was from wick's own recorded fixture logits when it was run
beside wick's source tree)."""
import importlib.util
import json
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _golden_module():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_plain_reproduces_committed_values():
    want = json.load(open(os.path.join(HERE, "golden", "plain_tiny.json")))
    got = _golden_module().compute("")
    assert set(got["models"]) == set(want["models"])
    for name, w in want["models"].items():
        g = got["models"][name]
        assert g["tokens"] == w["tokens"]
        assert g["greedy"] == w["greedy"], name
        assert (torch.tensor(g["logits_last"]) - torch.tensor(w["logits_last"])).abs().max() < 2e-5, name
        assert (torch.tensor(g["logits_row_sums"]) - torch.tensor(w["logits_row_sums"])).abs().max() < 2e-4, name


def test_recorded_distance_to_wicks_fixture_is_small():
    want = json.load(open(os.path.join(HERE, "golden", "plain_tiny.json")))
    rec = want["wick_fixture"]
    assert rec["max_abs_diff"] < 2e-5 and rec["greedy_equal"] is True
