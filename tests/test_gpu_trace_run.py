"""bin/trace_run driven as a user would: the same requests replayed whole, with
the last 32 tokens one by one, and in batches of unequal lengths whose requests
end at different steps with slots used again, in float32 and bfloat16, all
compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from helpers import CONFIGS, assert_logits_close, model_dir, plain_logits, random_tokens  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, name, dtype, out_dir, max_tokens):
        self.out = str(out_dir)
        self.vocab = CONFIGS[name]["vocab_size"]
        self.proc = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir(name), "--dtype", dtype,
             "--out", self.out, "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.n = 0

    def step(self, entries, end=()):
        rec = {"step": self.n, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.n}", f"trace_run said {line!r}"
        path = os.path.join(self.out, f"{self.n}.f32")
        wanted = sum(len(e["want"]) for e in entries)
        self.n += 1
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        a = np.fromfile(path, dtype="<f4")
        assert a.size == wanted * self.vocab
        return torch.from_numpy(a.reshape(wanted, self.vocab))

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=120) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_three_cuttings_of_the_same_requests(name, dtype, tmp_path):
    vocab = CONFIGS[name]["vocab_size"]
    reqs = {f"r{i}": random_tokens(vocab, n, 200 + i) for i, n in enumerate((40, 33, 97, 150, 64))}
    refs = {k: plain_logits(name, v) for k, v in reqs.items()}
    # enough for the largest batch below: 150 + 97 + 64 tokens, each rounded up to 64
    rp = Replay(name, dtype, tmp_path, max_tokens=192 + 128 + 64)

    # 1. each request alone and whole
    for k, toks in reqs.items():
        got = rp.step([{"id": k + "w", "tokens": toks, "want": list(range(len(toks)))}], end=[k + "w"])
        assert_logits_close(got, refs[k], dtype, f"{k} whole")

    # 2. the last 32 tokens one by one
    for k, toks in list(reqs.items())[:3]:
        head = len(toks) - 32
        got = [rp.step([{"id": k + "d", "tokens": toks[:head], "want": [head - 1]}])]
        for i in range(head, len(toks)):
            got.append(rp.step([{"id": k + "d", "tokens": [toks[i]], "want": [0]}],
                               end=[k + "d"] if i == len(toks) - 1 else []))
        assert_logits_close(torch.cat(got), refs[k][head - 1:], dtype, f"{k} last 32 one by one")

    # 3. batches of unequal lengths; shorter requests end earlier; two batches in
    #    a row so that slots and pages are used again
    for batch in (["r0", "r1", "r2"], ["r3", "r2", "r4"]):
        dec = {k: 4 + 3 * j for j, k in enumerate(batch)}
        pre = {k: len(reqs[k]) - dec[k] for k in batch}
        got = rp.step([{"id": k, "tokens": reqs[k][:pre[k]], "want": [0, pre[k] - 1]} for k in batch])
        for j, k in enumerate(batch):
            assert_logits_close(got[2 * j:2 * j + 2], refs[k][[0, pre[k] - 1]], dtype, f"{k} batched prompt")
        live = list(batch)
        t = 0
        while live:
            ending = [k for k in live if t + 1 == dec[k]]
            got = rp.step([{"id": k, "tokens": [reqs[k][pre[k] + t]], "want": [0]} for k in live], end=ending)
            for j, k in enumerate(live):
                assert_logits_close(got[j], refs[k][pre[k] + t], dtype, f"{k} batched decode {t}")
            live = [k for k in live if k not in ending]
            t += 1
    rp.close()


def test_steps_without_wanted_logits_and_a_full_cache(tmp_path):
    rp = Replay("A", "float32", tmp_path, max_tokens=128)
    toks = random_tokens(512, 100, 300)
    assert rp.step([{"id": "x", "tokens": toks[:90], "want": []}]) is None
    got = rp.step([{"id": "x", "tokens": toks[90:], "want": [9]}], end=["x"])
    assert_logits_close(got, plain_logits("A", toks)[-1:], "float32", "after a step that wanted nothing")
    # a second request fits only because the first one was given back
    got = rp.step([{"id": "y", "tokens": toks, "want": [99]}], end=["y"])
    assert_logits_close(got, plain_logits("A", toks)[-1:], "float32", "reused pages")
    rp.close()
