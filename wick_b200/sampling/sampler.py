"""Turning logits into the next token, the way wick does.

Options, defaults and the order of operations follow ``src/sampler.rs``:
repetition penalty over the distinct tokens of the context (``:76-85``), greedy
when ``temperature <= 0`` (first maximum, ``:86-88,129-137``), otherwise top-k
candidates sorted by logit (``:89-94``), probabilities ``exp((l - max) / T)``
normalised (``:95-98``), min-p (``:100-104``), top-p (``:105-115``) and one draw
``r = next_f32() * total`` walked down the sorted candidates (``:116-125``).
The generator is xoshiro256** seeded through splitmix64 (``:29-61``); every
sequence gets a generator of its own from the seed, so a sequence samples the
same tokens alone or in a batch.

Device side: the argmax, the top-k selection (up to 1024 candidates per row),
the cuts and the draw are CUDA kernels; only each sequence's uniform number comes
from the host, from that sequence's generator.  :func:`pick_from_sorted` is the
plain form of the cuts and the draw (float32 on the host, one operation at a
time) that the tests hold the kernel against.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import numpy as np
import torch

_M64 = (1 << 64) - 1


@dataclasses.dataclass
class SamplerConfig:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = 0x5EED

    @classmethod
    def greedy(cls) -> "SamplerConfig":
        return cls(temperature=0.0)


class Rng:
    """xoshiro256** seeded through splitmix64 (sampler.rs:29-61)."""

    def __init__(self, seed: int):
        z = seed & _M64
        s = []
        for _ in range(4):
            z = (z + 0x9E3779B97F4A7C15) & _M64
            x = z
            x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
            x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
            s.append(x ^ (x >> 31))
        self.s = s

    @staticmethod
    def _rotl(x: int, k: int) -> int:
        return ((x << k) | (x >> (64 - k))) & _M64

    def next_u64(self) -> int:
        s = self.s
        out = (self._rotl((s[1] * 5) & _M64, 7) * 9) & _M64
        t = (s[1] << 17) & _M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return out

    def next_f32(self) -> float:
        """Uniform in [0, 1) with 24 bits."""
        return float(np.float32(self.next_u64() >> 40) / np.float32(1 << 24))


def pick_from_sorted(vals: np.ndarray, idx: np.ndarray, cfg: SamplerConfig, rng: Rng) -> int:
    """vals: float32 candidates sorted descending, idx their token ids.  Steps
    sampler.rs:95-125 in float32."""
    f = np.float32
    t = f(cfg.temperature)
    probs = np.exp(((vals.astype(f) - vals[0]) / t).astype(f)).astype(f)
    total = f(0)
    for p in probs:                      # sequential float32 sum, as the reference's iterator sum
        total = f(total + p)
    probs = (probs / total).astype(f)
    keep = len(probs)
    if cfg.min_p > 0.0:
        floor = f(probs[0] * f(cfg.min_p))
        below = np.nonzero(probs < floor)[0]
        keep = max(int(below[0]) if len(below) else keep, 1)
    if cfg.top_p < 1.0:
        acc = f(0)
        for i in range(keep):
            acc = f(acc + probs[i])
            if acc >= f(cfg.top_p):
                keep = i + 1
                break
    tot = f(0)
    for p in probs[:keep]:
        tot = f(tot + p)
    r = f(f(rng.next_f32()) * tot)
    for i in range(keep):
        r = f(r - probs[i])
        if r <= 0:
            return int(idx[i])
    return int(idx[keep - 1])


def rng_state(seed: int) -> List[int]:
    """The four 64-bit words of a freshly seeded generator, as signed integers (the form an
    int64 tensor holds them in for the device's generator kernel)."""
    return [w - (1 << 64) if w >= (1 << 63) else w for w in Rng(seed).s]


def sample_on_device(cfg: SamplerConfig, logits: torch.Tensor, uniforms, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 ``logits`` [rows, vocab] on the device, as int32 [rows] on
    the device; nothing is copied to the host.  ``uniforms`` is a function that returns this
    step's uniform numbers (float32 [rows] on the device); it is called only if a draw is made.
    A repetition penalty is applied by the caller beforehand.  ``out``: where to write (int32 [rows]).

    Where every token is a candidate (``top_k`` 0, no min-p, no top-p) and the vocabulary is
    larger than the selection kernel's 1,024 candidates, the draw walks the candidates in the
    order of their ids, not sorted by logit as sampler.rs:116-125 does: the same distribution,
    but for one uniform number another token than the reference picks."""
    from .. import ops
    rows, vocab = logits.shape
    if cfg.temperature <= 0.0:
        return ops.argmax(logits, out)
    k = vocab if cfg.top_k == 0 else min(cfg.top_k, vocab)
    if k == vocab and cfg.top_p >= 1.0 and cfg.min_p <= 0.0 and vocab > Sampler.DEVICE_TOP_K:
        return ops.sample_temperature(logits, cfg.temperature, uniforms(), out)
    if k <= Sampler.DEVICE_TOP_K:
        vals, idx = ops.top_k(logits, k)
    else:
        # More candidates than the selection kernel takes (rare): a library sort, ties by index.
        vals, order = torch.sort(logits, dim=1, descending=True, stable=True)
        vals, idx = vals[:, :k].contiguous(), order[:, :k].to(torch.int32).contiguous()
    return ops.pick_sorted(vals, idx, uniforms(), cfg.temperature, cfg.min_p, cfg.top_p, out)


class Sampler:
    """Samples one token per row of a batch of logits; one :class:`Rng` per sequence.  (The
    form for callers that hold the logits of a step in their hands; a batch that decodes
    without the host in between keeps its generators on the device instead.)"""

    DEVICE_TOP_K = 1024

    def __init__(self, cfg: SamplerConfig, n_seqs: int):
        self.cfg = cfg
        self.rngs = [Rng(cfg.seed) for _ in range(n_seqs)]

    def sample(self, logits: torch.Tensor, seq_ids: Sequence[int],
               histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """logits: float32 [rows, vocab] on the device, row i belonging to sequence
        ``seq_ids[i]`` (its index in this sampler); histories[i]: that sequence's
        tokens so far (needed only with a repetition penalty)."""
        from .. import ops
        cfg = self.cfg
        rows, vocab = logits.shape
        if rows == 0:
            return []
        if cfg.repetition_penalty != 1.0:
            if histories is None:
                raise ValueError("a repetition penalty needs the sequences' tokens")
            logits = logits.clone()
            ops.repetition_penalty(logits, histories, cfg.repetition_penalty)

        def uniforms():
            u = torch.tensor([self.rngs[s].next_f32() for s in seq_ids], dtype=torch.float32)
            return u.to(logits.device)

        return sample_on_device(cfg, logits, uniforms).tolist()
