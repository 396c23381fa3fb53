"""A batch of sequences that start together, stepped for the generation loop.

The loop (``engine/generate.py``) drives an object with three calls:

``start(slots, prompts, limits)``
    run all prompts in one step and sample each sequence's first token;
``launch(slots)``
    run one more step for these sequences, each fed the token sampled for it last,
    and sample again;
``collect() -> list of token ids``
    the tokens of the oldest step not collected yet, in that step's order of slots.

``depth`` says how many steps may be launched beyond the one being collected.

:class:`DeviceRun` (depth 1) keeps everything between two steps on the device: the
sampled token goes into the sequence's state record, the next step's token,
position and cached length come out of it (``csrc/state.cu``), the generators of
the draws and the tokens seen (for the repetition penalty) live on the device
too.  The host uploads a step's description (slots and page tables) only when the
batch's composition changes, launches step k + 1 before it has read the tokens of
step k, and reads those through a pinned buffer behind an event.  A sequence that
sampled a stop token or reached its limit is frozen by the device at once; the
host learns of it one step later and leaves it out from then on.

:class:`StepRun` (depth 0) is the same interface over anything with a ``step``
function and a sampler that returns host integers: one step at a time.
"""
from __future__ import annotations

import collections
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache import PAGE
from ..sampling.sampler import SamplerConfig, rng_state, sample_on_device


class StepRun:
    depth = 0

    def __init__(self, engine, sampler, needs_history: bool):
        self.engine, self.sampler, self.needs_history = engine, sampler, needs_history
        self.row: Dict[int, int] = {}
        self.last: Dict[int, int] = {}
        self.hist: Dict[int, List[int]] = {}
        self.result: Deque[List[int]] = collections.deque()

    def start(self, slots: Sequence[int], prompts: Sequence[Sequence[int]], limits: Sequence[int]) -> None:
        for i, (s, p) in enumerate(zip(slots, prompts)):
            self.row[s] = i
            self.hist[s] = list(p)
        self._step(slots, [list(p) for p in prompts])

    def launch(self, slots: Sequence[int]) -> None:
        self._step(slots, [[self.last[s]] for s in slots])

    def _step(self, slots, feed) -> None:
        logits = self.engine.step(list(slots), feed, [[len(f) - 1] for f in feed])
        hist = [self.hist[s] for s in slots] if self.needs_history else None
        toks = [int(t) for t in self.sampler.sample(logits, [self.row[s] for s in slots], hist)]
        for s, t in zip(slots, toks):
            self.last[s] = t
            if self.needs_history:
                self.hist[s].append(t)
        self.result.append(toks)

    def collect(self) -> List[int]:
        return self.result.popleft()


class DeviceRun:
    depth = 1

    def __init__(self, engine, cfg: SamplerConfig, stop_token_ids: Sequence[int] = ()):
        self.engine, self.cfg = engine, cfg
        dev = engine.device
        stops = sorted(set(int(t) for t in stop_token_ids))
        self.stops = torch.tensor(stops, dtype=torch.int32, device=dev) if stops else None
        self.vocab = engine.spec.vocab
        self.rng: Optional[torch.Tensor] = None
        self.seen: Optional[torch.Tensor] = None
        self.ids: Optional[torch.Tensor] = None
        self.uniforms: Optional[torch.Tensor] = None
        self._pinned: List[torch.Tensor] = []
        self._events: List[torch.cuda.Event] = []
        self._turn = 0
        self.pending: Deque[Tuple[int, int]] = collections.deque()
        self.uploads = 0                     # descriptions copied to the device (a test reads it)
        self.h2d_bytes = 0
        self.left: Dict[int, int] = {}       # tokens each sequence may still be given, as far as the host knows
        self.last_logits: Optional[torch.Tensor] = None   # the last step's rows (a view: the next step overwrites them)

    # ---- the first step: all prompts ----
    def start(self, slots: Sequence[int], prompts: Sequence[Sequence[int]], limits: Sequence[int]) -> None:
        e = self.engine
        B = len(slots)
        dev = e.device
        self.ids = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        self.uniforms = torch.zeros(B, dtype=torch.float32, device=dev)
        for _ in range(self.depth + 2):
            self._pinned.append(torch.zeros(B + 1, dtype=torch.int32, pin_memory=True))
            self._events.append(torch.cuda.Event())
        if self.cfg.temperature > 0.0:
            self.rng = torch.tensor([rng_state(self.cfg.seed)] * B, dtype=torch.int64).to(dev)
        if self.cfg.repetition_penalty != 1.0:
            self.seen = torch.zeros((B, self.vocab), dtype=torch.uint8, device=dev)
        # the sequences' records: nothing cached, nothing generated, their limits and rows
        rec = np.zeros((B, ops.SEQ_STATE_WORDS + 1), dtype=np.int32)
        rec[:, ops.SEQ_LIMIT] = limits
        rec[:, ops.SEQ_ROW] = np.arange(B)
        rec[:, ops.SEQ_STATE_WORDS] = slots
        up = torch.from_numpy(rec).pin_memory().to(dev, non_blocking=True)
        self.h2d_bytes += rec.nbytes
        ops.seq_state_set(e.seq_state, up[:, ops.SEQ_STATE_WORDS].contiguous(), up[:, :ops.SEQ_STATE_WORDS].contiguous())
        starts = [e.cache.length(s) for s in slots]
        for s, st, p in zip(slots, starts, prompts):
            e.cache.reserve(s, st + len(p))
        q_lens = [len(p) for p in prompts]
        logits, batch = e._forward_prompt(list(slots), [list(p) for p in prompts], [[q - 1] for q in q_lens], starts, q_lens)
        self.h2d_bytes += batch.layout.size * 4
        with ops.stream_scope():
            if self.seen is not None:                    # (a captured step's padding tokens belong to slot 0: not marked)
                ops.seen_prompt(self.seen, e.seq_state, batch.slots, batch.tokens, batch.seq_of_token)
            self._sample_and_advance(logits[:B], batch.slots[:B], batch.kv_len[:B], B)
        self.last_logits = logits[:B]
        for s, q, lim in zip(slots, q_lens, limits):
            e.cache.advance(s, q)
            self.left[s] = lim - 1

    # ---- one more token each ----
    def launch(self, slots: Sequence[int]) -> None:
        e = self.engine
        cache = e.cache
        B = len(slots)
        longest = 0
        for s in slots:
            n = cache.length(s) + 1
            cache.reserve(s, n)
            longest = max(longest, n)
        # (A batch that has shrunk and will end within 64 steps keeps the captured step it has.)
        ending = max(self.left.get(s, 0) for s in slots) < 64
        g = e._decode_graph(B, (longest + PAGE - 1) // PAGE, capture=e.use_graphs, prefer_captured=ending)
        composition = (tuple(slots), tuple(len(cache.pages_of(s)) for s in slots))
        if g.composition != composition:
            # (token, position and lengths of the description are written by step_prepare)
            e._fill_graph_batch(g, slots, [[0]] * B, [0] * B)
            g.composition = composition
            self.uploads += 1
            self.h2d_bytes += g.layout.size * 4
        b = g.batch
        with ops.stream_scope():
            ops.step_prepare(e.seq_state, b.slots, b.tokens, b.positions, b.start, b.kv_len)
            if e.use_graphs:
                g.graph.replay()
                ops.launches[0] += g.kernels
                logits = g.logits
            else:                                        # (graphs switched off: the same step as separate launches)
                b.memo.clear()
                logits = e.model.forward(b, cache)
            self._sample_and_advance(logits[:B], b.slots[:B], b.kv_len[:B], B)
        self.last_logits = logits[:B]
        for s in slots:
            cache.advance(s, 1)
            self.left[s] = self.left.get(s, 1) - 1

    def _sample_and_advance(self, logits: torch.Tensor, slots_dev: torch.Tensor, kv_len_dev: torch.Tensor, B: int) -> None:
        e = self.engine
        if self.seen is not None:
            ops.penalty_seen(logits, self.seen, e.seq_state, slots_dev, self.cfg.repetition_penalty)
        ids = self.ids[:B + 1]                       # the sampled tokens, then the kernels' status word
        sample_on_device(self.cfg, logits, lambda: ops.rng_uniforms(self.rng, e.seq_state, slots_dev, self.uniforms[:B]),
                         out=ids[:B])
        ops.step_advance(e.seq_state, slots_dev, ids, kv_len_dev, self.stops, self.seen, self.vocab)
        i = self._turn
        self._turn = (i + 1) % len(self._pinned)
        self._pinned[i][:B + 1].copy_(ids, non_blocking=True)
        self._events[i].record()
        self.pending.append((i, B))

    def collect(self) -> List[int]:
        i, B = self.pending.popleft()
        self._events[i].synchronize()
        out = self._pinned[i][:B + 1].tolist()
        if out[B] != 0:
            ops.check_status()               # raises with the kernel's message
        return out[:B]
