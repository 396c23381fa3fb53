"""The engine: a model, its cache, and ONE step function.

``Engine.step(slots, tokens, want)`` runs a batch of sequences that start
together: in their first step each brings its whole prompt (unequal lengths, all
tokens flat in one batch), afterwards one token each.  Only the tokens given are
run; everything earlier comes from the cache.  The logits of the wanted places
come back as one float32 tensor.  A step of one token per sequence is replayed
from a captured CUDA graph (one graph per padded batch size); padded entries
read and write the reserved page 0 and change no real sequence's result.

Reference: wick ``src/model.rs:420-516`` (``Model::forward``: tokens at positions
``cache.len..``, cache append before attention, length advanced once after all
layers, logits of the last or of all tokens) generalised from one sequence to a
batch.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache import PAGE, Cache
from ..config.base import ModelConfig, get_architecture, load_config
from ..models.model import Model
from ..weights.loader import load_weights
from ..weights.random_init import random_fetch
from .batch import BatchLayout, StepBatch, fill_host

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "f32": torch.float32, "float32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(d) -> torch.dtype:
    try:
        return _DTYPES[d]
    except KeyError:
        raise ValueError(f"unknown dtype {d} (bfloat16 or float32)") from None


class Workspace:
    """Named scratch buffers that grow on demand and are reused across steps."""

    def __init__(self, device):
        self.device = device
        self.buffers: Dict[str, torch.Tensor] = {}
        self.frozen = False

    def get(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """zero: the buffer is zero when it is made (its users leave it zero)."""
        b = self.buffers.get(name)
        if b is None or b.numel() < numel or b.dtype != dtype:
            if self.frozen:
                raise RuntimeError(f"scratch buffer {name} would have to grow to {numel} elements while a CUDA "
                                   f"graph is being captured")
            make = torch.zeros if zero else torch.empty
            b = self.buffers[name] = make(max(numel, 1), dtype=dtype, device=self.device)
        return b


class _Staging:
    """Pinned host buffers for the packed batch description, used in turn."""

    def __init__(self, n: int = 4):
        self.bufs: List[Optional[torch.Tensor]] = [None] * n
        self.events: List[Optional[torch.cuda.Event]] = [None] * n
        self.i = 0

    def take(self, size: int) -> Tuple[torch.Tensor, int]:
        i = self.i
        self.i = (i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        b = self.bufs[i]
        if b is None or b.numel() < size:
            b = self.bufs[i] = torch.empty(max(size, 1024), dtype=torch.int32, pin_memory=True)
        return b, i

    def mark(self, i: int) -> None:
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class _DecodeGraph:
    def __init__(self, n_pad: int, table_width: int):
        self.n_pad, self.table_width = n_pad, table_width
        self.layout = BatchLayout(n_pad, n_pad, table_width, n_pad)
        self.buffer: Optional[torch.Tensor] = None
        self.batch: Optional[StepBatch] = None
        # What a batch that decodes on the device last wrote into the buffer (its slots and
        # how many pages each held); None after anyone else filled it.
        self.composition: Optional[tuple] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None


PROMPT_GRAPH_TOKENS = 512     # prompt steps of up to this many tokens are captured, padded to a multiple of 64
PROMPT_GRAPH_SEQS = 64        # ... and of up to this many sequences (padded to a power of two or three quarters of one)
PROMPT_GRAPH_COUNT = 24       # captured prompt steps an engine keeps (each holds its output rows); further shapes are launched


class _PromptGraph:
    """A captured prompt step of ``n_tokens`` tokens in ``n_seqs`` sequences, the last of
    which is padding: it lives in slot 0 and on the reserved page 0 and takes the tokens
    that fill the step up.  Sequences between the real ones and the padding bring no token."""

    def __init__(self, n_tokens: int, n_seqs: int, n_want: int):
        self.n_tokens, self.n_seqs, self.n_want = n_tokens, n_seqs, n_want
        self.table_width = PROMPT_GRAPH_TOKENS // PAGE
        self.layout = BatchLayout(n_seqs, n_tokens, self.table_width, n_want)
        self.buffer: Optional[torch.Tensor] = None
        self.batch: Optional[StepBatch] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None


class Engine:
    def __init__(self, model: Model, *, max_tokens: int, max_seqs: Optional[int] = None,
                 use_graphs: Optional[bool] = None):
        if model.ctx.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only (there is no CPU path)")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available")
        self.model = model
        self.spec = model.spec
        self.device = model.ctx.device
        self.dtype = model.ctx.dtype
        self.cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=self.dtype, device=self.device,
                           max_seqs=max_seqs, max_position=self.spec.max_position)
        self.workspace = Workspace(self.device)
        self._staging = _Staging()
        if use_graphs is None:
            use_graphs = os.environ.get("WICK_B200_NO_GRAPHS", "") == ""
        self.use_graphs = use_graphs
        self._graphs: Dict[Tuple[int, int], _DecodeGraph] = {}
        # Short prompt steps are bound by the host's time per launch: they are captured too,
        # where every part of the model allows it (WICK_B200_NO_PROMPT_GRAPHS=1: never).
        self.prompt_graphs = (os.environ.get("WICK_B200_NO_PROMPT_GRAPHS", "") == "") and model.prompt_capturable()
        self._prompt_graphs: Dict[Tuple[int, int, int], _PromptGraph] = {}
        self._prompt_pool = None
        self._steps_since_check = 0
        # One record per cache slot on the device (length, next token, finished, ...): what a
        # batch that decodes without the host in between is advanced by.  Slot 0 (padding) is
        # finished for ever.
        self.seq_state = torch.zeros((self.cache.max_seqs + 1, ops.SEQ_STATE_WORDS), dtype=torch.int32,
                                     device=self.device)
        self.seq_state[0, ops.SEQ_FINISHED] = 1

    # ---- construction ----------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, *, dtype="bfloat16", max_tokens: int = 4096, device="cuda:0", **kw) -> "Engine":
        cfg = load_config(model_dir)
        arch = get_architecture(cfg.architecture)
        model = Model(arch.build_spec(cfg), parse_dtype(dtype), device)
        load_weights(model, model_dir)
        eng = cls(model, max_tokens=max_tokens, **kw)
        eng.config = cfg
        return eng

    @classmethod
    def from_config(cls, cfg: ModelConfig, seed: int, *, dtype="bfloat16", max_tokens: int = 4096, device="cuda:0",
                    **kw) -> "Engine":
        """Random weights drawn on the device (no files)."""
        arch = get_architecture(cfg.architecture)
        model = Model(arch.build_spec(cfg), parse_dtype(dtype), device)
        model.load(random_fetch(model, seed))
        eng = cls(model, max_tokens=max_tokens, **kw)
        eng.config = cfg
        return eng

    def check_kernels(self) -> None:
        """Raise if a kernel reported that it gave up a bounded wait (this
        synchronises the device, so it runs only now and then)."""
        self._steps_since_check = 0
        ops.check_status()

    def warm_up(self, max_batch: int = 1, context: Optional[int] = None, prompt_tokens: int = 0) -> int:
        """Capture now what generation would capture on first use: the decode steps of every
        padded batch size up to ``max_batch`` and every page-table width up to ``context``
        positions (default: what the cache can hold per sequence), and the prompt steps of one
        to ``max_batch`` sequences of up to ``prompt_tokens`` tokens together (at most 512: longer
        steps are not captured).  Touches only the reserved page and slot.  Returns how many
        steps were captured; with graphs switched off it captures nothing."""
        if not self.use_graphs:
            return 0
        before = sum(g.graph is not None for g in self._graphs.values()) + len(self._prompt_graphs)
        context = min(context or self.spec.max_position, self.spec.max_position, self.cache.max_tokens)
        batches = sorted({self._bucket(b) for b in range(1, max(1, max_batch) + 1)})
        pages, widths = (context + PAGE - 1) // PAGE, []
        w = 8
        while True:
            widths.append(w)
            if w >= pages:
                break
            w *= 2
        for b in batches:
            for w in widths:
                self._decode_graph(b, w)
        for t in range(PAGE, min(prompt_tokens, PROMPT_GRAPH_TOKENS) + PAGE, PAGE):
            for b in batches:
                if b <= min(t, PROMPT_GRAPH_SEQS):
                    self._prompt_graph([t - b + 1] + [1] * (b - 1), [t - b + 1] + [1] * (b - 1), b)
        return sum(g.graph is not None for g in self._graphs.values()) + len(self._prompt_graphs) - before

    # ---- sequences ---------------------------------------------------------
    def open_seq(self) -> int:
        return self.cache.open_seq()

    def close_seq(self, slot: int) -> None:
        self.cache.close_seq(slot)

    def seq_len(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate_seq(self, slot: int, length: int) -> None:
        """Forget what the sequence holds from position ``length`` on, so that its next step
        continues from there: a new prompt that shares its first ``length`` tokens with the
        last one runs only the rest (wick src/engine.rs:127-132 keeps the common prefix of
        consecutive prompts in the same way).  Pages beyond the new length are given back."""
        self.cache.truncate(slot, length)

    def begin_run(self, sampler, stop_token_ids=()):
        """A batch of sequences that start together and then decode on the device: see
        :class:`~wick_b200.engine.run.DeviceRun`."""
        from .run import DeviceRun
        return DeviceRun(self, sampler, stop_token_ids)

    # ---- the step ------------------------------------------------------------
    def _check(self, slots, tokens, want) -> None:
        if not (len(slots) == len(tokens) == len(want)):
            raise ValueError("slots, tokens and want must have one entry per sequence")
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        vocab = self.spec.vocab
        for b, (s, t, w) in enumerate(zip(slots, tokens, want)):
            if len(t) == 0:
                raise ValueError(f"sequence {b} (slot {s}) brings no token")
            lo, hi = min(t), max(t)
            if lo < 0 or hi >= vocab:
                raise ValueError(f"token id {lo if lo < 0 else hi} of sequence {b} is outside the vocabulary "
                                 f"of {vocab}")
            for i in w:
                if not 0 <= i < len(t):
                    raise ValueError(f"wanted place {i} of sequence {b} is outside its {len(t)} tokens")

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Run ``tokens[b]`` after what slot ``slots[b]`` already holds.

        want[b]: indices into tokens[b] whose logits are returned (default: the
        last one).  Returns float32 [sum(len(want[b])), vocab], rows in the order
        of the sequences and of ``want``.

        The result of a captured decode step (one token per sequence, graphs on) is a
        view of that captured step's output buffer: it is valid until the next step of
        the same batch size runs, so copy it (``.clone()``) to keep it longer.  (Prompt
        steps of up to 512 tokens are replayed from captured steps too, padded to a
        multiple of 64 tokens; their result is copied out before it is returned.)"""
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        self._check(slots, tokens, want)
        cache = self.cache
        starts = [cache.length(s) for s in slots]
        for s, st, t in zip(slots, starts, tokens):
            cache.reserve(s, st + len(t))
        q_lens = [len(t) for t in tokens]
        decode = all(q == 1 for q in q_lens)
        if decode and self.use_graphs:
            logits = self._step_graph(slots, tokens, want, starts)
        else:
            logits, batch = self._forward_prompt(slots, tokens, want, starts, q_lens)
            if batch.q_tiles is not None:
                logits = logits.clone()              # (a captured step's output buffer: the next one overwrites it)
        for s, q in zip(slots, q_lens):
            cache.advance(s, q)
        return logits

    def _upload(self, layout: BatchLayout, dev: Optional[torch.Tensor], **fields) -> Tuple[torch.Tensor, np.ndarray]:
        host, idx = self._staging.take(layout.size)
        arr = host.numpy()[:layout.size]
        fill_host(layout, arr, **fields)
        if dev is None:
            dev = torch.empty(layout.size, dtype=torch.int32, device=self.device)
        dev.copy_(host[:layout.size], non_blocking=True)
        self._staging.mark(idx)
        return dev, arr

    def _forward_prompt(self, slots, tokens, want, starts, q_lens) -> Tuple[torch.Tensor, StepBatch]:
        """A step of any shape: replayed from a captured step of its padded size where there
        can be one, else launched kernel by kernel.  Returns the logits of the wanted places
        and the batch description that ran (a captured step's has padding behind the
        ``len(slots)`` real sequences)."""
        g = self._prompt_graph(q_lens, [s + q for s, q in zip(starts, q_lens)], sum(len(w) for w in want))
        if g is None:
            return self._forward_eager(slots, tokens, want, starts, q_lens)
        B, cache = len(slots), self.cache
        idle = g.n_seqs - 1 - B
        fill = g.n_tokens - sum(q_lens)
        pages = [cache.pages_of(s)[:(st + q + PAGE - 1) // PAGE] for s, st, q in zip(slots, starts, q_lens)]
        self._upload(g.layout, g.buffer, tokens=[list(t) for t in tokens] + [[]] * idle + [[0] * fill],
                     starts=list(starts) + [0] * (idle + 1), slots=list(slots) + [0] * (idle + 1),
                     pages=pages + [[0]] * (idle + 1), want=[list(w) for w in want] + [[]] * (idle + 1), pad_want=True)
        g.graph.replay()
        ops.launches[0] += g.kernels
        self._count_step()
        return g.logits[:sum(len(w) for w in want)], g.batch

    def _prompt_graph(self, q_lens, kv_lens, n_want: int) -> Optional[_PromptGraph]:
        """The captured step that serves a prompt step of these lengths (captured on first
        use), or None: graphs are off, a part of the model does not allow it, or the step is
        larger than what is captured."""
        if not (self.use_graphs and self.prompt_graphs):
            return None
        n_tokens, B = sum(q_lens), len(q_lens)
        if n_tokens > PROMPT_GRAPH_TOKENS or B > PROMPT_GRAPH_SEQS or max(kv_lens) > PROMPT_GRAPH_TOKENS:
            return None
        t_pad = (n_tokens + PAGE - 1) // PAGE * PAGE
        n_seqs = self._bucket(B) + 1
        if n_want > t_pad:
            return None
        w_pad = n_seqs if n_want <= n_seqs else t_pad
        key = (t_pad, n_seqs, w_pad)
        g = self._prompt_graphs.get(key)
        if g is None and len(self._prompt_graphs) >= PROMPT_GRAPH_COUNT:
            return None
        if g is None:
            g = _PromptGraph(t_pad, n_seqs, w_pad)
            g.buffer = torch.zeros(g.layout.size, dtype=torch.int32, device=self.device)
            # (host lists: all tokens in one sequence, which is what the capture below runs)
            g.batch = StepBatch(g.layout, g.buffer, q_lens=[0] * (n_seqs - 1) + [t_pad], starts=[0] * n_seqs,
                                workspace=self.workspace, q_tiles=t_pad // ops.Q_TILE + n_seqs)
            # Captured on padding only: every token in the padding sequence, whose page table
            # names the reserved page 0 throughout, so that no live sequence is touched.
            self._upload(g.layout, g.buffer, tokens=[[]] * (n_seqs - 1) + [[0] * t_pad], starts=[0] * n_seqs,
                         slots=[0] * n_seqs, pages=[[0]] * n_seqs, want=[[]] * n_seqs, pad_want=True)
            if self._prompt_pool is None:
                self._prompt_pool = torch.cuda.graph_pool_handle()
            self._capture(g, pool=self._prompt_pool)
            self._prompt_graphs[key] = g
        return g

    def _forward_eager(self, slots, tokens, want, starts, q_lens) -> Tuple[torch.Tensor, StepBatch]:
        cache = self.cache
        B = len(slots)
        kv_lens = [s + q for s, q in zip(starts, q_lens)]
        width = max(1, max((k + PAGE - 1) // PAGE for k in kv_lens))
        layout = BatchLayout(B, sum(q_lens), width, sum(len(w) for w in want))
        pages = [cache.pages_of(s)[:(k + PAGE - 1) // PAGE] for s, k in zip(slots, kv_lens)]
        dev, _ = self._upload(layout, None, tokens=tokens, starts=starts, slots=slots, pages=pages, want=want)
        batch = StepBatch(layout, dev, q_lens=q_lens, starts=starts, workspace=self.workspace)
        with ops.stream_scope():
            logits = self.model.forward(batch, cache)
        self._count_step()
        return logits, batch

    def _count_step(self) -> None:
        """Every 64 steps (replayed ones too) the kernels' status word is read."""
        self._steps_since_check += 1
        if self._steps_since_check >= 64:
            self.check_kernels()

    # ---- captured decode -------------------------------------------------------
    @staticmethod
    def _bucket(n: int) -> int:
        """The padded size of a batch of ``n``: a power of two, or (from 24 on) three quarters of
        one: 1, 2, 4, 8, 16, 24, 32, 48, 64, 96, ...  (A batch of 40 pays for 48 rows in the matrix
        products and for 48 sequences' pairs in the attention, not for 64.)"""
        b = 1
        while b < n:
            b *= 2
        return b // 4 * 3 if b >= 32 and n <= b // 4 * 3 else b

    def _decode_graph(self, n_seqs: int, max_pages: int, capture: bool = True, prefer_captured: bool = False) -> _DecodeGraph:
        """The captured step for ``n_seqs`` sequences (padded, see :meth:`_bucket`) whose page
        tables hold up to ``max_pages`` pages (padded to 8, 16, 32 ...); captured on first use
        (``capture`` False: only its buffer and batch description are made)."""
        n_pad = self._bucket(n_seqs)
        width = 8
        while width < max_pages:
            width *= 2
        key = (n_pad, width)
        g = self._graphs.get(key)
        if prefer_captured and capture and (g is None or g.graph is None):
            # A larger captured step of the same page-table width serves as well (more padded
            # rows) and saves a capture in the middle of a generation that is about to end.
            have = [k for k, c in self._graphs.items() if k[1] == width and k[0] > n_pad and c.graph is not None]
            if have:
                return self._graphs[min(have)]
        if g is None:
            g = self._graphs[key] = _DecodeGraph(n_pad, width)
            g.buffer = torch.zeros(g.layout.size, dtype=torch.int32, device=self.device)
            g.batch = StepBatch(g.layout, g.buffer, q_lens=[1] * n_pad, starts=[0] * n_pad, workspace=self.workspace,
                                kv_bound=width * PAGE)
        if g.graph is None and capture:
            # Capture (and its warm-up run) on a batch of padding entries only, so
            # that no live sequence's cache or state is touched twice.
            self._upload(g.layout, g.buffer, tokens=[[0]] * n_pad, starts=[0] * n_pad, slots=[0] * n_pad,
                         pages=[[0]] * n_pad, want=[[0]] * n_pad)
            self._capture(g)
        return g

    def _fill_graph_batch(self, g: _DecodeGraph, slots, tokens, starts) -> None:
        """The description of a decode step of ``slots`` into the captured step's buffer;
        padded entries are one token (id 0) at position 0 of the reserved page 0 / slot 0."""
        cache = self.cache
        pad = g.n_pad - len(slots)
        f_pages = [cache.pages_of(s)[:g.table_width] for s in slots] + [[0]] * pad
        self._upload(g.layout, g.buffer, tokens=[list(t) for t in tokens] + [[0]] * pad, starts=list(starts) + [0] * pad,
                     slots=list(slots) + [0] * pad, pages=f_pages, want=[[0]] * g.n_pad)
        g.composition = None

    def _step_graph(self, slots, tokens, want, starts) -> torch.Tensor:
        B = len(slots)
        g = self._decode_graph(B, max((s + 1 + PAGE - 1) // PAGE for s in starts))
        self._fill_graph_batch(g, slots, tokens, starts)
        g.graph.replay()
        ops.launches[0] += g.kernels
        self._count_step()
        rows = [b for b in range(B) for _ in want[b]]
        if rows == list(range(B)):
            return g.logits[:B]
        if not rows:
            return g.logits[:0]
        return g.logits[torch.tensor(rows, device=self.device)]

    def _capture(self, g, pool=None) -> None:
        def run():
            g.batch.memo.clear()
            with ops.stream_scope():                # (entered on the stream that runs or captures the step)
                return self.model.forward(g.batch, self.cache)

        # Warm-up outside capture (compiles/loads kernels, grows scratch buffers).
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            run()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        self.workspace.frozen = True
        before = ops.launches[0]
        try:
            with torch.cuda.graph(graph, pool=pool):     # (prompt steps share one pool: they never run at the same time)
                g.logits = run()
        finally:
            self.workspace.frozen = False
        g.kernels = ops.launches[0] - before
        ops.launches[0] = before
        # The graph holds raw pointers into the scratch buffers: keep those alive
        # even if the workspace later replaces them by larger ones.
        g.keepalive = dict(self.workspace.buffers)
        g.graph = graph
        self.check_kernels()
