"""The engine against the plain implementation, in float32 and bfloat16: each
request alone and whole; the last 32 tokens one by one; batches of unequal
lengths whose shorter requests end earlier, one batch after another so that
slots and pages are used again; long decoding; the first tokens of a sequence;
uneven chunks; captured and eager decode steps."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from helpers import (CONFIGS, assert_logits_close, make_engine, plain_logits, poison_all,  # noqa: E402
                     poison_free_pages, random_tokens)

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B"]


def vocab_of(name):
    return CONFIGS[name]["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES + ["C"])
def test_each_request_alone_and_whole(name, dtype):
    eng = make_engine(name, dtype)
    poison_all(eng)
    for n, seed in ((1, 1), (5, 2), (64, 3), (65, 4), (200, 5)):
        toks = random_tokens(vocab_of(name), n, seed)
        s = eng.open_seq()
        got = eng.step([s], [toks], [list(range(n))])
        eng.close_seq(s)
        assert_logits_close(got, plain_logits(name, toks), dtype, f"{name} whole n={n}")
    eng.cache.check()


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(name, dtype, graphs):
    eng = make_engine(name, dtype, use_graphs=graphs)
    poison_all(eng)
    toks = random_tokens(vocab_of(name), 150, 11)
    ref = plain_logits(name, toks)
    s = eng.open_seq()
    head = len(toks) - 32
    got = [eng.step([s], [toks[:head]], [list(range(head))]).clone()]
    for i in range(head, len(toks)):
        got.append(eng.step([s], [[toks[i]]]).clone())
    eng.close_seq(s)
    assert_logits_close(torch.cat(got), ref, dtype, f"{name} decode of the last 32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_uneven_chunks_match_one_pass(name, dtype):
    # wick tests/tiny_models.rs:73-95
    eng = make_engine(name, dtype)
    poison_all(eng)
    toks = random_tokens(vocab_of(name), 48, 12)
    ref = plain_logits(name, toks)
    s = eng.open_seq()
    pos, got = 0, []
    for size in [1, 5, 2, 7, 1, 1, 13, 3, 15]:
        got.append(eng.step([s], [toks[pos:pos + size]], [list(range(size))]).clone())
        pos += size
    eng.close_seq(s)
    assert pos == len(toks)
    assert_logits_close(torch.cat(got), ref, dtype, f"{name} uneven chunks")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another_reuse_slots(name, dtype, graphs):
    """Three batches through a cache that holds only one of them at a time.
    Every request runs prompt-then-decode; shorter requests end earlier and the
    batch shrinks; freed pages are filled with NaN before the next batch starts."""
    lens_per_batch = [(5, 11, 17, 70), (1, 7, 30, 64), (33, 2, 129)]
    dec = {0: 3, 1: 9, 2: 5, 3: 12}
    eng = make_engine(name, dtype, max_tokens=64 * 8, use_graphs=graphs)
    poison_all(eng)
    seed = 100
    for lens in lens_per_batch:
        seqs = []
        for i, n in enumerate(lens):
            seed += 1
            seqs.append(random_tokens(vocab_of(name), n + dec[i], seed))
        refs = [plain_logits(name, s) for s in seqs]
        slots = [eng.open_seq() for _ in seqs]
        live = list(range(len(seqs)))
        got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], [list(range(n)) for n in lens]).clone()
        off = 0
        for i, n in enumerate(lens):
            assert_logits_close(got[off:off + n], refs[i][:n], dtype, f"{name} batch prompt {i}")
            off += n
        step = 0
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][lens[i] + step]] for i in live]).clone()
            for r, i in enumerate(live):
                assert_logits_close(got[r], refs[i][lens[i] + step], dtype, f"{name} seq {i} decode step {step}")
            step += 1
            for i in list(live):
                if step >= dec[i]:
                    eng.close_seq(slots[i])
                    live.remove(i)
            poison_free_pages(eng)
        eng.cache.check()
        assert eng.cache.pages.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_crosses_pages_and_splits(dtype):
    """A 3-token prompt, then 300 tokens one by one: crosses page boundaries
    (64) and the decode kernel's split size (256)."""
    name = "A"
    eng = make_engine(name, dtype)
    poison_all(eng)
    toks = random_tokens(vocab_of(name), 256 - 3 + 50, 21)[:256]   # max_position_embeddings of A is 256
    ref = plain_logits(name, toks)
    s = eng.open_seq()
    got = [eng.step([s], [toks[:3]], [[0, 1, 2]]).clone()]
    for t in toks[3:]:
        got.append(eng.step([s], [[t]]).clone())
    assert_logits_close(torch.cat(got), ref, dtype, "long decode")
    with pytest.raises(ValueError, match="context length exceeded"):
        eng.step([s], [[1]])
    eng.close_seq(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_several_splits(dtype):
    name = "B"
    eng = make_engine(name, dtype)
    toks = random_tokens(vocab_of(name), 512, 22)
    ref = plain_logits(name, toks)
    s = eng.open_seq()
    eng.step([s], [toks[:200]], [[]])
    got = [eng.step([s], [[t]]).clone() for t in toks[200:]]
    eng.close_seq(s)
    assert_logits_close(torch.cat(got), ref[200:], dtype, "decode from 200 to 512")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_head_dim_64_prompt_then_long_decode_in_a_batch(dtype, graphs):
    """Config D (head_dim 64, group of 4): in bfloat16 both attention kernels run
    on the tensor cores.  Three sequences, prompts of unequal length, then 150
    decoded tokens each (several decode splits, partial last pages)."""
    name = "D"
    eng = make_engine(name, dtype, use_graphs=graphs)
    poison_all(eng)
    lens = (3, 100, 260)
    seqs = [random_tokens(vocab_of(name), n + 150, 60 + n) for n in lens]
    refs = [plain_logits(name, s) for s in seqs]
    slots = [eng.open_seq() for _ in seqs]
    got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], [[n - 1] for n in lens]).clone()
    for i, n in enumerate(lens):
        assert_logits_close(got[i], refs[i][n - 1], dtype, f"D prompt {i}")
    for k in range(150):
        got = eng.step(slots, [[s[n + k]] for s, n in zip(seqs, lens)]).clone()
        if k % 7 == 0 or k > 140:
            for i, n in enumerate(lens):
                assert_logits_close(got[i], refs[i][n + k], dtype, f"D seq {i} decode {k}")
    for s in slots:
        eng.close_seq(s)


@pytest.mark.parametrize("graphs", [False, True])
def test_short_kernels_overlap_in_a_captured_step(graphs):
    """Config E in bfloat16: kernels of a few microseconds each, launched back to
    back from a captured step, each allowed to start before the one before it has
    ended.  A kernel that read its input before waiting for its producer gave
    logits that were off by half their range here (and nowhere else)."""
    name = "E"
    eng = make_engine(name, "bfloat16", use_graphs=graphs)
    poison_all(eng)
    lens = (290, 130)
    seqs = [random_tokens(vocab_of(name), n + 40, 70 + n) for n in lens]
    refs = [plain_logits(name, s) for s in seqs]
    slots = [eng.open_seq() for _ in seqs]
    got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], [[n - 1] for n in lens]).clone()
    for i, n in enumerate(lens):
        assert_logits_close(got[i], refs[i][n - 1], "bfloat16", f"E prompt {i}")
    for k in range(40):
        got = eng.step(slots, [[s[n + k]] for s, n in zip(seqs, lens)]).clone()
        for i, n in enumerate(lens):
            assert_logits_close(got[i], refs[i][n + k], "bfloat16", f"E seq {i} decode {k}")
    for s in slots:
        eng.close_seq(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(name, dtype):
    """Position 0 sees only itself; a one-token prompt, then its first decoded tokens."""
    eng = make_engine(name, dtype)
    poison_all(eng)
    toks = random_tokens(vocab_of(name), 4, 31)
    ref = plain_logits(name, toks)
    s = eng.open_seq()
    got = [eng.step([s], [[t]]).clone() for t in toks]
    eng.close_seq(s)
    assert_logits_close(torch.cat(got), ref, dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_and_batch_composition_change_nothing(dtype):
    """The same request decoded alone, in a batch of 3 (padded to 4 in the
    captured step) and in a batch of 5 (padded to 8) gives the same logits."""
    name = "B"
    eng = make_engine(name, dtype, use_graphs=True)
    seqs = [random_tokens(vocab_of(name), n, 40 + n) for n in (20, 6, 77, 41, 9)]
    outs = {}
    for group in ([0], [0, 1, 2], [0, 1, 2, 3, 4]):
        slots = [eng.open_seq() for _ in group]
        eng.step(slots, [seqs[i][:-4] for i in group], [[] for _ in group])
        rows = []
        for k in range(4, 0, -1):
            rows.append(eng.step(slots, [[seqs[i][-k]] for i in group])[0].clone())
        for s in slots:
            eng.close_seq(s)
        outs[len(group)] = torch.stack(rows)
    assert torch.equal(outs[1], outs[3]) and torch.equal(outs[1], outs[5])
    assert_logits_close(outs[5], plain_logits(name, seqs[0])[-4:], dtype, "batched decode")


def test_step_checks_its_arguments():
    eng = make_engine("A", "float32")
    s = eng.open_seq()
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.step([s], [[512]])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.step([s], [[-1]])
    with pytest.raises(ValueError, match="brings no token"):
        eng.step([s], [[]])
    with pytest.raises(ValueError, match="wanted place"):
        eng.step([s], [[1, 2]], [[2]])
    with pytest.raises(ValueError, match="twice"):
        eng.step([s, s], [[1], [2]])
    from wick_b200.cache import PoolError
    with pytest.raises(PoolError, match="not open"):
        eng.step([s + 1], [[1]])
    assert eng.seq_len(s) == 0, "a refused step changes nothing"
    out = eng.step([s], [[1, 2, 3]], [[]])
    assert out.shape == (0, 512) and eng.seq_len(s) == 3
    eng.close_seq(s)


def test_wanted_rows_come_in_order_of_entries_and_want():
    name, dtype = "A", "float32"
    eng = make_engine(name, dtype)
    a, b = random_tokens(512, 9, 50), random_tokens(512, 4, 51)
    sa, sb = eng.open_seq(), eng.open_seq()
    got = eng.step([sa, sb], [a, b], [[8, 0, 8], [2, 2]])       # a place may be asked for more than once
    ra, rb = plain_logits(name, a), plain_logits(name, b)
    assert_logits_close(got, torch.stack([ra[8], ra[0], ra[8], rb[2], rb[2]]), dtype, "want order")
    assert torch.equal(got[0], got[2]) and torch.equal(got[3], got[4])
    eng.close_seq(sa)
    eng.close_seq(sb)


def test_model_with_random_weights_drawn_on_the_device():
    cfg = wick.config_from_json(CONFIGS["B"])
    eng = wick.Engine.from_config(cfg, seed=3, dtype="bfloat16", max_tokens=256)
    s = eng.open_seq()
    out = eng.step([s], [[1, 2, 3]])
    assert out.shape == (1, 1000) and torch.isfinite(out).all() and out.abs().max() > 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lens", [(150, 37), (300, 25)])
def test_real_layer_widths_of_qwen3_8b(dtype, lens):
    """One layer at the real widths (config R): a prompt whole, a second prompt in
    the same batch, then decoded tokens — so that the kernels run with their real
    tile counts, splits and strides.  float32 must match the plain implementation
    to 1e-4 here too.  (313 tokens in a step: the matrix products on pairs of thread
    blocks, the narrow ones with their inner dimension cut into runs.)"""
    name = "R"
    eng = make_engine(name, dtype, max_tokens=1024)
    poison_all(eng)
    seqs = [random_tokens(vocab_of(name), n, 900 + n) for n in lens]
    refs = [plain_logits(name, s) for s in seqs]
    slots = [eng.open_seq() for _ in seqs]
    heads = [len(s) - 6 for s in seqs]
    got = eng.step(slots, [s[:h] for s, h in zip(seqs, heads)], [[0, h // 2, h - 1] for h in heads]).clone()
    for i, h in enumerate(heads):
        assert_logits_close(got[3 * i:3 * i + 3], refs[i][[0, h // 2, h - 1]], dtype, f"R prompt {i}")
    for k in range(6):
        got = eng.step(slots, [[s[h + k]] for s, h in zip(seqs, heads)]).clone()
        for i, h in enumerate(heads):
            assert_logits_close(got[i], refs[i][h + k], dtype, f"R seq {i} decode {k}")
    for s in slots:
        eng.close_seq(s)


def _run_batch_against_plain(name, dtype, eng, lens, n_decode, seed0, every=1):
    """Prompts of ``lens`` tokens in one step, then ``n_decode[i]`` tokens one by one for
    sequence i (shorter ones leave earlier); every logit row against the plain implementation."""
    seqs = [random_tokens(vocab_of(name), n + d, seed0 + i) for i, (n, d) in enumerate(zip(lens, n_decode))]
    refs = [plain_logits(name, s) for s in seqs]
    slots = [eng.open_seq() for _ in seqs]
    got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], [[n - 1] for n in lens]).clone()
    for i, n in enumerate(lens):
        assert_logits_close(got[i], refs[i][n - 1], dtype, f"{name} prompt {i} of {n} tokens")
    live = [i for i in range(len(seqs)) if n_decode[i] > 0]
    for i in range(len(seqs)):
        if n_decode[i] == 0:
            eng.close_seq(slots[i])
    step = 0
    while live:
        got = eng.step([slots[i] for i in live], [[seqs[i][lens[i] + step]] for i in live]).clone()
        if step % every == 0 or step + 1 >= max(n_decode):
            for r, i in enumerate(live):
                assert_logits_close(got[r], refs[i][lens[i] + step], dtype, f"{name} seq {i} ({lens[i]} tokens) decode step {step}")
        step += 1
        for i in list(live):
            if step >= n_decode[i]:
                eng.close_seq(slots[i])
                live.remove(i)
        poison_free_pages(eng)
    eng.cache.check()
    assert eng.cache.pages.n_held == 0


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_batch_beyond_148_pairs_at_real_widths(dtype, graphs):
    """22 sequences of 1 to 700 tokens at the real widths (config R: 8 kv heads, so 176
    (sequence, kv head) pairs): the prompts in one step, then up to 9 decoded tokens each,
    the shorter requests leaving earlier, so that the batch runs at 22, 19, 17 ... sequences
    (captured steps of 24 and 16 rows) and the decode attention for many pairs runs inside the engine."""
    name = "R"
    lens = (1, 700, 3, 64, 65, 127, 128, 129, 130, 2, 255, 256, 257, 31, 300, 20, 5, 385, 77, 200, 192, 193)
    n_decode = tuple(9 - (i % 4) * 2 if i % 5 else 9 for i in range(len(lens)))
    eng = make_engine(name, dtype, max_tokens=sum((n + 9 + 63) // 64 * 64 for n in lens), use_graphs=graphs)
    poison_all(eng)
    _run_batch_against_plain(name, dtype, eng, lens, n_decode, 3000)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_batch_of_80_sequences(dtype, graphs):
    """Config D (2 kv heads of 64) with 80 sequences: 160 pairs, the batch bucket of 128,
    then 64 as requests leave."""
    name = "D"
    g = torch.Generator().manual_seed(5)
    lens = tuple(int(x) for x in torch.randint(1, 330, (80,), generator=g))
    n_decode = tuple(3 + (i * 7) % 10 for i in range(80))
    eng = make_engine(name, dtype, max_tokens=sum((n + 12 + 63) // 64 * 64 for n in lens), use_graphs=graphs)
    poison_all(eng)
    _run_batch_against_plain(name, dtype, eng, lens, n_decode, 4000)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E"])
def test_decoding_across_512_and_1024_cached_tokens(name, dtype, graphs):
    """Sequences decode across 512 and across 1,024 cached positions: a captured step is made
    for page tables of 8, 16 and 32 pages, and a live sequence changes from one captured step
    to the next in mid-flight."""
    eng = make_engine(name, dtype, max_tokens=4096, use_graphs=graphs)
    poison_all(eng)
    _run_batch_against_plain(name, dtype, eng, (500, 40), (30, 12), 5000 + len(name))
    _run_batch_against_plain(name, dtype, eng, (1015, 300, 7), (30, 30, 5), 5100 + len(name))
    if graphs:
        widths = sorted(set(w for (_, w) in eng._graphs))
        assert widths == [8, 16, 32], widths


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E"])
def test_batch_composition_changes_no_bit_with_tensor_core_attention(name, dtype, graphs):
    """Head sizes 64 and 128 (in bfloat16 the one-launch decode attention): a request of 1,100
    cached tokens (nine runs of 128 positions) decoded alone, among 3 and among 24 gives the
    same bits, eagerly and from captured steps: how a sequence's positions are cut into runs,
    and the order in which the runs' results are merged, depend on its own length only."""
    eng = make_engine(name, dtype, max_tokens=8192, use_graphs=graphs)
    lens = [1100, 6, 77, 500, 9] + [20 + 11 * i for i in range(19)]
    seqs = [random_tokens(vocab_of(name), n + 4, 40 + n) for n in lens]
    outs = {}
    for count in (1, 3, 24):
        group = list(range(count))
        slots = [eng.open_seq() for _ in group]
        eng.step(slots, [seqs[i][:-4] for i in group], [[] for _ in group])
        rows = []
        for k in range(4, 0, -1):
            rows.append(eng.step(slots, [[seqs[i][-k]] for i in group])[0].clone())
        for s in slots:
            eng.close_seq(s)
        outs[count] = torch.stack(rows)
    assert_logits_close(outs[24], plain_logits(name, seqs[0])[-4:], dtype, "batched decode")
    assert torch.equal(outs[1], outs[3]), "alone and among 3"
    assert torch.equal(outs[1], outs[24]), "alone and among 24"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_a_shared_prefix_is_kept_and_only_the_rest_runs(name, dtype):
    """Prefix reuse (wick src/engine.rs:127-132): a sequence is cut back to the 70 tokens its
    next prompt shares with the last one (inside its second page), the pages beyond are given
    back and poisoned, and only the new prompt's remaining tokens run."""
    eng = make_engine(name, dtype, max_tokens=1024)
    poison_all(eng)
    first = random_tokens(vocab_of(name), 200, 61)
    second = first[:70] + random_tokens(vocab_of(name), 90, 62)
    s = eng.open_seq()
    eng.step([s], [first], [[]])
    for t in random_tokens(vocab_of(name), 3, 63):
        eng.step([s], [[t]])
    held = eng.cache.pages.n_held
    eng.truncate_seq(s, 70)
    assert eng.seq_len(s) == 70 and eng.cache.pages.n_held == 2 < held
    poison_free_pages(eng)
    got = eng.step([s], [second[70:]], [list(range(90))]).clone()
    ref = plain_logits(name, second)
    assert_logits_close(got, ref[70:], dtype, f"{name} after a cut to 70 tokens")
    got = eng.step([s], [[5]]).clone()
    assert_logits_close(got, plain_logits(name, second + [5])[-1:], dtype, f"{name} decode after the cut")
    with pytest.raises(ValueError, match="cannot truncate"):
        eng.truncate_seq(s, 500)
    eng.close_seq(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_tensors_by_name_come_back_as_the_checkpoint_stores_them(dtype):
    """Fused and tiled matrices are split and put back row by row: every tensor of the folder
    is found under its name with its values (bfloat16 values are exact in float32)."""
    from helpers import model_dir
    from plain import qwen3_plain as P
    for name in ("B", "D"):
        eng = make_engine(name, dtype)
        _, stored = P.read_model_dir(model_dir(name))
        held = eng.model.tensors()
        assert set(held) == set(stored)
        for k, t in stored.items():
            assert torch.equal(held[k].float().cpu(), t), k
        assert torch.equal(eng.model.tensor("model.layers.1.self_attn.k_proj.weight").float().cpu(),
                           stored["model.layers.1.self_attn.k_proj.weight"])
        with pytest.raises(KeyError):
            eng.model.tensor("model.layers.1.self_attn.nothing")


def test_four_layers_at_the_real_sizes_of_qwen3_8b_in_float32():
    """Four layers with the widths of Qwen3-8B and its full vocabulary of 151,936, random
    float32 weights drawn on the device and handed to the plain implementation by tensor name:
    a 300-token prompt and 8 decoded tokens, every wanted row within 1e-4."""
    from plain import qwen3_plain as P
    j = dict(CONFIGS["R"], num_hidden_layers=4, vocab_size=151936)
    cfg = wick.config_from_json(j)
    eng = wick.Engine.from_config(cfg, seed=5, dtype="float32", max_tokens=512)
    w = {k: t.cpu() for k, t in eng.model.tensors().items()}
    toks = random_tokens(151936, 308, 77)
    ref = P.forward(P.plain_config(j), w, toks)
    del w
    s = eng.open_seq()
    got = [eng.step([s], [toks[:300]], [[0, 150, 299]]).clone()]
    for t in toks[300:]:
        got.append(eng.step([s], [[t]]).clone())
    eng.close_seq(s)
    want = torch.cat([ref[[0, 150, 299]], ref[300:]])
    assert_logits_close(torch.cat(got), want, "float32", "four real layers")
    eng.check_kernels()


@pytest.mark.parametrize("graphs", [False, True])
def test_the_kernels_status_word_is_read_now_and_then(graphs, monkeypatch):
    """Replayed steps count like launched ones: every 64 steps the status word is read, so a
    kernel that gave up a wait cannot go unnoticed for long."""
    from wick_b200 import ops
    eng = make_engine("A", "float32", use_graphs=graphs)
    s = eng.open_seq()
    eng.step([s], [[1, 2, 3]])
    calls = []
    real = ops.check_status
    monkeypatch.setattr(ops, "check_status", lambda: (calls.append(1), real())[1])
    for t in range(130):
        eng.step([s], [[t % 500]])
    assert len(calls) >= 2
    eng.close_seq(s)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_group_of_five_query_heads_per_kv_head(dtype, graphs):
    """Config F: 10 heads over 2 kv heads of 128 (the grouping of Qwen3-14B): unequal prompts,
    then decoding, the shorter requests leaving earlier."""
    name = "F"
    eng = make_engine(name, dtype, max_tokens=4096, use_graphs=graphs)
    poison_all(eng)
    _run_batch_against_plain(name, dtype, eng, (130, 1, 700, 64, 300), (12, 5, 12, 3, 9), 6000)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_beyond_64_pages(dtype, graphs):
    """A 4,150-token prompt (33 blocks of 128 keys in the prompt attention) and a 70-token one,
    then 10 decoded tokens each: beyond 64 pages the decode attention's parts grow from two
    pages to four, and the captured step is made for a page table of 128 pages."""
    name = "E"
    eng = make_engine(name, dtype, max_tokens=8192, use_graphs=graphs)
    poison_all(eng)
    _run_batch_against_plain(name, dtype, eng, (4150, 70), (10, 10), 7000, every=3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_steps_replayed_from_captured_steps_of_padded_sizes(dtype):
    """Prompt steps of up to 512 tokens are replayed from captured steps, padded to a multiple of
    64 tokens and to a power of two of sequences plus a padding sequence on the reserved page.
    Steps of different compositions share one captured step; idle sequence entries, the padding
    tokens and what page 0 holds (NaN here) change no row; a step that is longer, or that
    continues a sequence beyond 512 positions, is launched kernel by kernel."""
    name = "D"
    eng = make_engine(name, dtype, max_tokens=4096, use_graphs=True)
    assert eng.model.prompt_capturable()
    eng.prompt_graphs = True                                   # (whatever the environment's switches say)
    poison_all(eng)
    V = vocab_of(name)

    def run(lens, seed, whole):
        seqs = [random_tokens(V, n, seed + i) for i, n in enumerate(lens)]
        slots = [eng.open_seq() for _ in seqs]
        want = [list(range(n)) for n in lens] if whole else None
        got = eng.step(slots, seqs, want)
        off = 0
        for i, s in enumerate(seqs):
            ref = plain_logits(name, s)
            if whole:
                assert_logits_close(got[off:off + len(s)], ref, dtype, f"lens {lens} seq {i}")
                off += len(s)
            else:
                assert_logits_close(got[i], ref[-1], dtype, f"lens {lens} seq {i} (last)")
        return slots, seqs

    def close(slots):
        for s in slots:
            eng.close_seq(s)
        poison_free_pages(eng)

    close(run((30, 41), 300, whole=False)[0])
    assert set(eng._prompt_graphs) == {(128, 3, 3)}
    close(run((64, 7), 310, whole=False)[0])                  # the same padded size: the same captured step
    close(run((1, 127), 320, whole=False)[0])                 # no padding token at all
    assert set(eng._prompt_graphs) == {(128, 3, 3)}
    close(run((70,), 330, whole=True)[0])                     # every position wanted: as many rows as tokens
    assert set(eng._prompt_graphs) == {(128, 3, 3), (128, 2, 128)}
    close(run((1, 2, 64, 9, 3), 340, whole=True)[0])          # five sequences in eight entries
    assert (128, 9, 128) in eng._prompt_graphs
    n_captured = len(eng._prompt_graphs)
    # a sequence continued beyond 512 positions, and a step of more than 512 tokens: not captured
    slots, seqs = run((500,), 350, whole=False)
    more = random_tokens(V, 30, 351)
    got = eng.step(slots, [more], [list(range(30))])
    assert_logits_close(got, plain_logits(name, seqs[0] + more)[500:], dtype, "continued beyond 512 positions")
    close(slots)
    close(run((300, 290), 360, whole=False)[0])
    assert len(eng._prompt_graphs) == n_captured + 1          # (the 500-token step)
    eng.cache.check()
    assert eng.cache.pages.n_held == 0
    eng.check_kernels()


def test_a_captured_prompt_step_and_the_same_step_launched_give_the_same_logits():
    """Bits are not promised (the padded size may choose other kernels), closeness is: the
    same prompts through a captured step and through separate launches."""
    name = "F"
    V = vocab_of(name)
    seqs = [random_tokens(V, n, 400 + n) for n in (90, 3, 33)]
    out = []
    for captured in (True, False):
        eng = make_engine(name, "bfloat16", use_graphs=True)
        eng.prompt_graphs = captured
        slots = [eng.open_seq() for _ in seqs]
        out.append(eng.step(slots, seqs).float().cpu())
        assert (len(eng._prompt_graphs) > 0) == captured
    for i, s in enumerate(seqs):
        assert_logits_close(out[0][i], plain_logits(name, s)[-1], "bfloat16", f"captured, seq {i}")
        assert_logits_close(out[1][i], plain_logits(name, s)[-1], "bfloat16", f"launched, seq {i}")


def test_the_plain_kernels_switch_runs_the_bfloat16_model_without_tensor_cores(monkeypatch):
    """WICK_B200_PLAIN=1: every matrix product and attention of the bfloat16 model through the
    plain CUDA-core twins; no tensor-core kernel is called, and the logits hold against the
    plain implementation like the fast kernels' do."""
    from wick_b200 import ops
    from wick_b200.ops import gemm_tc

    def never(*a, **k):
        raise AssertionError("a tensor-core kernel ran under the plain-kernels switch")

    monkeypatch.setattr(ops, "PLAIN_KERNELS", True)
    monkeypatch.setattr(gemm_tc, "gemm_tc", never)
    monkeypatch.setattr(gemm_tc, "gemm_tc_pair", never)
    monkeypatch.setattr(ops, "attention_decode_parts_fused", never)
    monkeypatch.setattr(ops, "attention_decode_parts", never)
    name = "D"
    eng = make_engine(name, "bfloat16")
    poison_all(eng)
    assert ops.attention_prompt_kind(64, torch.bfloat16) == "plain" and ops.attention_decode_kind(64, torch.bfloat16) == "plain"
    _run_batch_against_plain(name, "bfloat16", eng, (70, 5, 130), (6, 3, 6), 9000)


@pytest.mark.parametrize("seed", [21, 22])
def test_random_configurations_prompt_decode_and_chunked_prompt(seed):
    """Configurations drawn at random (head sizes, groups, widths and vocabularies that are no
    power of two, tied and untied heads): unequal prompts in one step, decoding, then the same
    prompts in two chunks on reused slots, in float32 and bfloat16 against the plain implementation."""
    import random

    import helpers as H
    rnd = random.Random(seed)
    for ci in range(3):
        hd = rnd.choice([16, 32, 64, 128])
        kv = rnd.choice([1, 2, 3])
        heads = kv * rnd.choice([1, 2, 3, 5, 8])
        vocab = rnd.choice([257, 1003, 5003])
        cfgj = dict(architectures=["Qwen3ForCausalLM"], hidden_size=rnd.choice([72, 200, 320, 520]), num_attention_heads=heads,
                    num_key_value_heads=kv, head_dim=hd, intermediate_size=rnd.choice([88, 160, 1000]),
                    num_hidden_layers=rnd.choice([1, 2, 3]), vocab_size=vocab, max_position_embeddings=1024,
                    rope_theta=rnd.choice([10000.0, 1000000.0]), rms_norm_eps=rnd.choice([1e-6, 1e-5]),
                    tie_word_embeddings=rnd.random() < 0.5)
        name = f"random-{seed}-{ci}"
        H.CONFIGS[name] = cfgj
        lens = [rnd.choice([1, 2, 5, 63, 64, 65, 129, 200, 257]) for _ in range(rnd.choice([1, 3, 5]))]
        n_dec = rnd.choice([3, 20])
        seqs = [random_tokens(vocab, n + n_dec, 100 * ci + i) for i, n in enumerate(lens)]
        refs = [plain_logits(name, s) for s in seqs]
        for dtype in DTYPES:
            what = f"{cfgj} lens {lens} {dtype}"
            eng = make_engine(name, dtype, max_tokens=4096)
            poison_all(eng)
            slots = [eng.open_seq() for _ in seqs]
            got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], [list(range(n)) for n in lens]).clone()
            off = 0
            for i, n in enumerate(lens):
                assert_logits_close(got[off:off + n], refs[i][:n], dtype, f"prompt {i} of {what}")
                off += n
            for k in range(n_dec):
                got = eng.step(slots, [[s[n + k]] for s, n in zip(seqs, lens)]).clone()
                for i, n in enumerate(lens):
                    assert_logits_close(got[i], refs[i][n + k], dtype, f"seq {i} decode {k} of {what}")
            for s in slots:
                eng.close_seq(s)
            poison_free_pages(eng)
            slots = [eng.open_seq() for _ in seqs]
            cut = [max(1, n // 2) for n in lens]
            eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], [[] for _ in lens])
            live = [i for i, n in enumerate(lens) if n > cut[i]]
            if live:
                got = eng.step([slots[i] for i in live], [seqs[i][cut[i]:lens[i]] for i in live],
                               [[lens[i] - cut[i] - 1] for i in live]).clone()
                for j, i in enumerate(live):
                    assert_logits_close(got[j], refs[i][lens[i] - 1], dtype, f"chunked prompt {i} of {what}")
            for s in slots:
                eng.close_seq(s)
            eng.cache.check()
            eng.check_kernels()
            del eng
