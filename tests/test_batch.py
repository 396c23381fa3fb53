"""The packed description of a step (host side): field layout, sequences that bring no token,
wanted places padded for a captured step, and the padded batch sizes of captured steps."""
import numpy as np
import pytest

from wick_b200.engine.batch import BatchLayout, fill_host
from wick_b200.engine.engine import Engine


def test_fields_are_16_byte_aligned_and_do_not_overlap():
    L = BatchLayout(n_seqs=5, n_tokens=131, table_width=3, n_want=7)
    fields = [("tokens", 131), ("positions", 131), ("seq_of_token", 131), ("cu_seqlens", 6), ("start", 5), ("kv_len", 5),
              ("slots", 5), ("page_table", 15), ("want", 7)]
    end = 0
    for name, n in fields:
        off = getattr(L, name)
        assert off % 4 == 0 and off >= end, name
        end = off + n
    assert L.size >= end


def test_fill_of_a_ragged_prompt_step():
    L = BatchLayout(n_seqs=3, n_tokens=6, table_width=2, n_want=4)
    out = np.full(L.size, -7, dtype=np.int32)
    fill_host(L, out, tokens=[[5, 6, 7], [8], [9, 10]], starts=[0, 70, 3], slots=[2, 1, 4], pages=[[3], [5, 6], [7]],
              want=[[0, 2], [0], [1]])
    f = lambda name, n: out[getattr(L, name):getattr(L, name) + n].tolist()
    assert f("tokens", 6) == [5, 6, 7, 8, 9, 10]
    assert f("positions", 6) == [0, 1, 2, 70, 3, 4]
    assert f("seq_of_token", 6) == [0, 0, 0, 1, 2, 2]
    assert f("cu_seqlens", 4) == [0, 3, 4, 6]
    assert f("start", 3) == [0, 70, 3] and f("kv_len", 3) == [3, 71, 5] and f("slots", 3) == [2, 1, 4]
    assert f("page_table", 6) == [3, 0, 5, 6, 7, 0]
    assert f("want", 4) == [0, 2, 3, 5]


def test_fill_of_a_padded_prompt_step_with_idle_and_padding_sequences():
    """A captured prompt step: two real sequences, one entry without tokens, and the padding
    sequence (slot 0, page 0) that takes the tokens filling the step up; unused wanted places
    name the step's first token."""
    L = BatchLayout(n_seqs=4, n_tokens=8, table_width=2, n_want=4)
    out = np.full(L.size, -7, dtype=np.int32)
    fill_host(L, out, tokens=[[5, 6, 7], [8, 9], [], [0, 0, 0]], starts=[0, 64, 0, 0], slots=[2, 3, 0, 0],
              pages=[[4], [5, 6], [0], [0]], want=[[2], [1], [], []], pad_want=True)
    f = lambda name, n: out[getattr(L, name):getattr(L, name) + n].tolist()
    assert f("cu_seqlens", 5) == [0, 3, 5, 5, 8]
    assert f("seq_of_token", 8) == [0, 0, 0, 1, 1, 3, 3, 3]
    assert f("positions", 8) == [0, 1, 2, 64, 65, 0, 1, 2]
    assert f("kv_len", 4) == [3, 66, 0, 3] and f("slots", 4) == [2, 3, 0, 0]
    assert f("page_table", 8) == [4, 0, 5, 6, 0, 0, 0, 0]
    assert f("want", 4) == [2, 4, 0, 0]
    with pytest.raises(AssertionError):
        fill_host(L, out, tokens=[[5, 6, 7], [8, 9], [], [0, 0, 0]], starts=[0, 64, 0, 0], slots=[2, 3, 0, 0],
                  pages=[[4], [5, 6], [0], [0]], want=[[2], [1], [], []])      # fewer wanted places than the layout holds


def test_padded_batch_sizes():
    sizes = [Engine._bucket(n) for n in range(1, 100)]
    assert sizes[:8] == [1, 2, 4, 4, 8, 8, 8, 8]
    assert all(b >= n for n, b in zip(range(1, 100), sizes))
    assert sorted(set(sizes)) == [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128]
    assert Engine._bucket(17) == 24 and Engine._bucket(24) == 24 and Engine._bucket(25) == 32
    assert Engine._bucket(33) == 48 and Engine._bucket(49) == 64 and Engine._bucket(65) == 96
