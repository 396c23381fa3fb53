"""The description of one step's work, as the kernels read it.

A step runs, for each of ``n_seqs`` sequences, ``q_len[b]`` new tokens that
follow the ``start[b]`` tokens the cache already holds.  All tokens of the step
lie flat in one array; ``cu_seqlens`` gives each sequence's range in it.

Everything the device needs is packed into ONE int32 buffer that is filled in
pinned host memory and copied with one transfer; the fields below are views of
the device copy.  A captured decode step reads the same device buffer at every
replay, so the buffer's layout depends only on (``n_seqs``, ``n_tokens``,
``table_width``, number of wanted rows).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..layout import PAGE


class BatchLayout:
    """Offsets (in int32 elements) of each field inside the packed buffer."""

    def __init__(self, n_seqs: int, n_tokens: int, table_width: int, n_want: int):
        self.n_seqs, self.n_tokens, self.table_width = n_seqs, n_tokens, table_width
        self.n_want = n_want
        off = 0

        def take(n: int) -> int:
            nonlocal off
            o = off
            off += (n + 3) // 4 * 4          # keep every field 16-byte aligned
            return o

        self.tokens = take(n_tokens)
        self.positions = take(n_tokens)
        self.seq_of_token = take(n_tokens)
        self.cu_seqlens = take(n_seqs + 1)
        self.start = take(n_seqs)
        self.kv_len = take(n_seqs)
        self.slots = take(n_seqs)
        self.page_table = take(n_seqs * table_width)
        self.want = take(n_want)
        self.size = off


class StepBatch:
    """Host-side values plus device views of one step.

    tokens        int32 [n_tokens]   token ids
    positions     int32 [n_tokens]   absolute position of each token in its sequence
    seq_of_token  int32 [n_tokens]   index (0..n_seqs) of the sequence a token belongs to
    cu_seqlens    int32 [n_seqs+1]
    start         int32 [n_seqs]     tokens cached before this step
    kv_len        int32 [n_seqs]     start + q_len: tokens cached after this step
    slots         int32 [n_seqs]     the cache slot (sequence record) of each sequence
    page_table    int32 [n_seqs, table_width]  page ids, in position order
    want          int32 [n_want]     flat token indices whose logits are returned

    ``memo`` holds what parts compute once a step and share between layers (position
    tables, a mixer's own work lists), under keys of their choosing.
    """

    def __init__(self, layout: BatchLayout, dev: torch.Tensor, *, q_lens: Sequence[int],
                 starts: Sequence[int], host: Optional[np.ndarray] = None, workspace=None,
                 kv_bound: Optional[int] = None, q_tiles: Optional[int] = None):
        L = layout
        self.layout = L
        self.buffer = dev
        self.n_seqs, self.n_tokens, self.table_width = L.n_seqs, L.n_tokens, L.table_width
        self.n_want = L.n_want
        self.q_lens = list(q_lens)
        self.starts = list(starts)
        self.max_q_len = max(self.q_lens) if self.q_lens else 0
        self.max_kv_len = max((s + q for s, q in zip(self.starts, self.q_lens)), default=0)
        self.is_decode = self.max_q_len == 1 and self.n_tokens == self.n_seqs
        self.host = host
        # Scratch buffers that outlive the step (an object with ``get(name, numel, dtype)``),
        # and the number of cached positions that kernels size their work by: the longest
        # sequence of this step, or more (a captured step is sized for its page table).
        self.workspace = workspace
        self.kv_bound = self.max_kv_len if kv_bound is None else kv_bound
        # A captured prompt step: the most 64-row work items its sequences can make (the host
        # lists above then describe no real prompt, see Part.PROMPT_CAPTURABLE); None otherwise.
        self.q_tiles = q_tiles
        v = lambda off, n: dev[off:off + n]
        self.tokens = v(L.tokens, L.n_tokens)
        self.positions = v(L.positions, L.n_tokens)
        self.seq_of_token = v(L.seq_of_token, L.n_tokens)
        self.cu_seqlens = v(L.cu_seqlens, L.n_seqs + 1)
        self.start = v(L.start, L.n_seqs)
        self.kv_len = v(L.kv_len, L.n_seqs)
        self.slots = v(L.slots, L.n_seqs)
        self.page_table = v(L.page_table, L.n_seqs * L.table_width).view(L.n_seqs, L.table_width)
        self.want = v(L.want, L.n_want)
        # Values that several layers share within the step (position tables and
        # the like), keyed by whoever computes them.
        self.memo: Dict[object, object] = {}


def fill_host(layout: BatchLayout, out: np.ndarray, *, tokens: Sequence[Sequence[int]],
              starts: Sequence[int], slots: Sequence[int], pages: Sequence[Sequence[int]],
              want: Sequence[Sequence[int]], pad_page: int = 0, pad_want: bool = False) -> None:
    """Write every field of the packed buffer ``out`` (int32 [layout.size]).  A sequence
    may bring no token.  pad_want: fewer places may be wanted than the layout holds; the
    rest name the step's first token."""
    L = layout
    B = L.n_seqs
    out[:] = 0
    t = 0
    w = 0
    pt = out[L.page_table:L.page_table + B * L.table_width].reshape(B, L.table_width)
    pt[:] = pad_page
    for b in range(B):
        toks = tokens[b]
        n = len(toks)
        out[L.cu_seqlens + b] = t
        out[L.tokens + t:L.tokens + t + n] = toks
        out[L.positions + t:L.positions + t + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
        out[L.seq_of_token + t:L.seq_of_token + t + n] = b
        out[L.start + b] = starts[b]
        out[L.kv_len + b] = starts[b] + n
        out[L.slots + b] = slots[b]
        pg = pages[b]
        pt[b, :len(pg)] = pg
        for i in want[b]:
            out[L.want + w] = t + i
            w += 1
        t += n
    out[L.cu_seqlens + B] = t
    assert t == L.n_tokens and (w == L.n_want or (pad_want and w < L.n_want))
