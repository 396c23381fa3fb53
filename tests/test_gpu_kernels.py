"""Each kernel alone against a plain PyTorch float32 reference of the same
operation, at sizes other than the tiny models' (odd widths, vocabularies that
are no power of two, head sizes 16..128, groups of 1, 2, 5 and 8)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from plain import qwen3_plain as P  # noqa: E402

DTYPES = [torch.float32, torch.bfloat16]


def dev(t):
    return t.to("cuda")


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.2e-2) * scale


@pytest.fixture(scope="module")
def ops():
    from wick_b200 import ops
    return ops


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(ops, dtype):
    table = torch.randn(333, 72).to(dtype)
    tok = torch.tensor([0, 332, 5, 5, 17], dtype=torch.int32)
    out = ops.embed(dev(table), dev(tok))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table.float()[tok.long()])


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 1000, 4096 + 8])
def test_rmsnorm_plain_with_delta_and_with_rows(ops, out_dtype, width):
    torch.manual_seed(width)
    x, w = torch.randn(9, width) * 3, 1 + 0.1 * torch.randn(width)
    ref = P.rms_norm(x, w, 1e-5)
    got = ops.rmsnorm(dev(x), dev(w), 1e-5, out_dtype)
    assert got.dtype == out_dtype and (got.float().cpu() - ref).abs().max() < tol(out_dtype, ref.abs().max())
    # fused residual addition of three partial sums, on selected rows
    delta = torch.randn(3, 9, width)
    rows = torch.tensor([7, 2, 2, 0], dtype=torch.int32)
    xd = dev(x.clone())
    got = ops.rmsnorm(xd, dev(w), 1e-5, out_dtype, delta=dev(delta), rows=dev(rows))
    xs = x + ((delta[0] + delta[1]) + delta[2])
    ref = P.rms_norm(xs[rows.long()], w, 1e-5)
    assert (got.float().cpu() - ref).abs().max() < tol(out_dtype, ref.abs().max())
    assert torch.equal(xd.cpu(), x), "with selected rows (one of them named twice here) x stays as it was"
    xd = dev(x.clone())
    got = ops.rmsnorm(xd, dev(w), 1e-5, out_dtype, delta=dev(delta))
    assert torch.allclose(xd.cpu(), xs, atol=1e-6), "without selected rows the residual is updated in place"
    assert (got.float().cpu() - P.rms_norm(xs, w, 1e-5)).abs().max() < tol(out_dtype, ref.abs().max())


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 1000, 4096])
def test_rmsnorm_of_many_rows_gives_the_bits_of_few_rows(ops, out_dtype, width):
    """600 rows take the kernel with a warp per row, 9 rows the one with a block
    per row: a token's norm must not depend on how many others share its step."""
    torch.manual_seed(width + 1)
    n = 600
    x, w, delta = torch.randn(n, width) * 3, 1 + 0.1 * torch.randn(width), torch.randn(2, n, width)
    xs = x + (delta[0] + delta[1])
    ref = P.rms_norm(xs, w, 1e-5)
    xd = dev(x.clone())
    got = ops.rmsnorm(xd, dev(w), 1e-5, out_dtype, delta=dev(delta))
    assert (got.float().cpu() - ref).abs().max() < tol(out_dtype, ref.abs().max())
    assert torch.allclose(xd.cpu(), xs, atol=1e-6)
    pick = [0, 1, 77, 300, 598, 599, 5, 6, 7]
    few = ops.rmsnorm(dev(x[pick].clone()), dev(w), 1e-5, out_dtype, delta=dev(delta[:, pick].contiguous()))
    assert torch.equal(few.cpu(), got.cpu()[pick])


def test_add_delta(ops):
    x, d = torch.randn(5, 33), torch.randn(2, 5, 33)
    got = ops.add_delta(dev(x.clone()), dev(d))
    assert torch.allclose(got.cpu(), x + (d[0] + d[1]), atol=1e-6)


def test_rope_table_uses_float32_angles(ops):
    inv = P.rope_inv_freq(1e6, 48)
    pos = torch.tensor([0, 1, 77, 40000], dtype=torch.int32)
    cos, sin = ops.rope_table(dev(pos), dev(inv))
    ang = pos.float()[:, None] * inv[None, :]
    assert (cos.cpu() - torch.cos(ang)).abs().max() < 2e-6 and (sin.cpu() - torch.sin(ang)).abs().max() < 2e-6


def _paged(n_pages, n_kv, hd, dtype, fill=float("nan")):
    return torch.full((n_pages, 2, n_kv, 64, hd), fill, dtype=dtype, device="cuda")


class FakeBatch:
    """The fields of a step batch that the attention kernels read."""

    def __init__(self, q_lens, starts, pages, width=None):
        from wick_b200.engine.batch import BatchLayout, StepBatch, fill_host
        B = len(q_lens)
        width = width or max(len(p) for p in pages)
        lay = BatchLayout(B, sum(q_lens), width, 0)
        host = np.zeros(lay.size, dtype=np.int32)
        fill_host(lay, host, tokens=[[0] * q for q in q_lens], starts=starts, slots=list(range(1, B + 1)),
                  pages=pages, want=[[] for _ in q_lens])
        self.sb = StepBatch(lay, torch.from_numpy(host).cuda(), q_lens=q_lens, starts=starts)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, hd", [(4, 2, 16), (5, 1, 48), (8, 8, 64), (16, 2, 128)])
def test_qk_norm_rope_append_and_attention(ops, dtype, heads, kv_heads, hd):
    """Two sequences with a cached prefix each, pages in scrambled order, cache
    full of NaN where nothing was written: the fused norm/rotation/append kernel,
    then the prompt kernel and the decode kernel, against the plain parts."""
    torch.manual_seed(hd + heads)
    q_lens, starts = [70, 3], [130, 0]
    totals = [s + q for s, q in zip(starts, q_lens)]
    pages = [[9, 2, 5, 7], [4]]
    kv = _paged(12, kv_heads, hd, dtype)
    qw, kw = 1 + 0.1 * torch.randn(hd), 1 + 0.1 * torch.randn(hd)
    inv = P.rope_inv_freq(10000.0, hd)
    eps = 1e-6
    full = [torch.randn(t, (heads + 2 * kv_heads) * hd).to(dtype) for t in totals]

    def plain_qkv(x):
        t = x.shape[0]
        x = x.float()
        q = x[:, :heads * hd].view(t, heads, hd)
        k = x[:, heads * hd:(heads + kv_heads) * hd].view(t, kv_heads, hd)
        v = x[:, (heads + kv_heads) * hd:].view(t, kv_heads, hd)
        pos = torch.arange(t)
        return (P.rope(P.rms_norm(q, qw, eps), pos, inv), P.rope(P.rms_norm(k, kw, eps), pos, inv), v)

    # step 1: the prefixes (sequence 0 only), step 2: the new tokens of both
    fb0 = FakeBatch([starts[0]], [0], [pages[0]], width=4).sb
    cos, sin = ops.rope_table(fb0.positions, dev(inv))
    ops.qk_norm_rope_append(dev(full[0][:starts[0]]), heads, kv_heads, hd, q_weight=dev(qw), k_weight=dev(kw),
                            eps=eps, cos=cos, sin=sin, kv=kv, page_table=fb0.page_table,
                            seq_of_token=fb0.seq_of_token, positions=fb0.positions)
    fb = FakeBatch(q_lens, starts, pages).sb
    new = torch.cat([full[0][starts[0]:], full[1]])
    cos, sin = ops.rope_table(fb.positions, dev(inv))
    q = ops.qk_norm_rope_append(dev(new), heads, kv_heads, hd, q_weight=dev(qw), k_weight=dev(kw), eps=eps,
                                cos=cos, sin=sin, kv=kv, page_table=fb.page_table, seq_of_token=fb.seq_of_token,
                                positions=fb.positions)
    refs = [plain_qkv(x) for x in full]
    ref_q = torch.cat([refs[0][0][starts[0]:], refs[1][0]])
    assert (q.float().cpu() - ref_q).abs().max() < tol(dtype, 4)
    # the cache holds k (normed, rotated) and v (raw) at every position, in the right page
    for b in range(2):
        for p in (0, totals[b] - 1, min(64, totals[b] - 1)):
            page = pages[b][p // 64]
            assert (kv[page, 0, :, p % 64].float().cpu() - refs[b][1][p]).abs().max() < tol(dtype, 4)
            assert torch.equal(kv[page, 1, :, p % 64].float().cpu(), refs[b][2][p].to(dtype).float())
    # prompt attention over prefix + new tokens
    out = ops.attention_prompt(q, kv, fb, 1 / math.sqrt(hd))
    out_plain = ops.attention_prompt(q, kv, fb, 1 / math.sqrt(hd), plain=True)
    ref_o = []
    for b in range(2):
        qq, kk, vv = refs[b]
        if dtype == torch.bfloat16:           # the kernel reads the rounded cache
            qq, kk, vv = (t.to(dtype).float() for t in (qq, kk, vv))
        ref_o.append(P.causal_attention(qq, kk, vv)[starts[b]:])
    ref_o = torch.cat(ref_o)
    assert torch.isfinite(out.float()).all(), "a NaN from an unwritten cache position leaked"
    assert (out.float().cpu() - ref_o).abs().max() < tol(dtype, 2)
    assert (out_plain.float().cpu() - ref_o).abs().max() < tol(dtype, 2), "the CUDA-core twin"
    if dtype == torch.bfloat16 and hd <= 128:
        out_mma = ops.attention_prompt(q, kv, fb, 1 / math.sqrt(hd), kind="mma")
        assert (out_mma.float().cpu() - ref_o).abs().max() < tol(dtype, 2), "the mma.sync form"
    # decode attention: the last token of each sequence alone
    fd = FakeBatch([1, 1], [t - 1 for t in totals], pages).sb
    last = torch.tensor([q_lens[0] - 1, sum(q_lens) - 1], device="cuda")
    for plain in (False, True):
        scratch = torch.full((ops.attention_decode_scratch_floats(2, heads, hd, fd.max_kv_len, dtype, plain),),
                             float("nan"), device="cuda")
        outd = ops.attention_decode(q[last].contiguous(), kv, fd, 1 / math.sqrt(hd), scratch, plain=plain)
        assert torch.isfinite(outd.float()).all()
        assert (outd.float().cpu() - ref_o[last.cpu()]).abs().max() < tol(dtype, 2)
    ops.check_status()
    # the projection output as float32 partial sums gives the same q and cache
    parts = torch.stack([new.float() * 0.25, new.float() * 0.5, new.float() * 0.25])
    kv2 = _paged(12, kv_heads, hd, dtype)
    q2 = ops.qk_norm_rope_append(dev(parts), heads, kv_heads, hd, q_weight=dev(qw), k_weight=dev(kw), eps=eps,
                                 cos=cos, sin=sin, kv=kv2, page_table=fb.page_table, seq_of_token=fb.seq_of_token,
                                 positions=fb.positions, dtype=dtype)
    assert (q2.float() - q.float()).abs().max() < tol(dtype, 4)
    page = pages[1][0]
    assert (kv2[page, :, :, :3].float() - kv[page, :, :, :3].float()).abs().max() < tol(dtype, 4)


@pytest.mark.parametrize("hd", [32, 64])
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(ops, dtype, hd):
    """One key far back gets a score that dominates: the output must be its
    value.  Random keys would hide a kernel that skips a page or a split.
    (head_dim 64 in bfloat16 runs the tensor-core kernels.)"""
    heads, kv_heads = 4, 2
    n = 700
    for far in (3, 64 * 4 + 1, 511, 640):
        torch.manual_seed(far)
        k = torch.randn(n, kv_heads, hd) * 0.1
        v = torch.randn(n, kv_heads, hd)
        q = torch.randn(1, heads, hd) * 0.1
        k[far] = 0
        k[far, :, 0] = 8.0
        q[0, :, 0] = 40.0                                   # score 40*8/sqrt(hd) >= 40 above all others
        kv = _paged(13, kv_heads, hd, dtype)
        pages = [list(range(12, 12 - 11, -1))]              # 11 pages in descending order
        for p in range(n):
            kv[pages[0][p // 64], 0, :, p % 64] = k[p].to(dtype).cuda()
            kv[pages[0][p // 64], 1, :, p % 64] = v[p].to(dtype).cuda()
        fd = FakeBatch([1], [n - 1], pages).sb
        want = v[far].to(dtype).float().repeat_interleave(heads // kv_heads, 0)
        for plain in (False, True):
            scratch = torch.empty(ops.attention_decode_scratch_floats(1, heads, hd, n, dtype, plain), device="cuda")
            out = ops.attention_decode(dev(q.to(dtype)), kv, fd, 1 / math.sqrt(hd), scratch, plain=plain).float().cpu()
            assert (out[0] - want).abs().max() < 1e-2, f"decode kernel (plain={plain}) missed key {far}"
        # the same through the prompt kernel: 5 new tokens whose last one carries the query
        qs = torch.zeros(5, heads, hd)
        qs[4] = q[0]
        fp = FakeBatch([5], [n - 5], pages).sb
        outp = ops.attention_prompt(dev(qs.to(dtype)), kv, fp, 1 / math.sqrt(hd)).float().cpu()
        assert (outp[4] - want).abs().max() < 1e-2, f"prompt kernel missed key {far}"


def _many_lengths(n, seed):
    g = torch.Generator().manual_seed(seed)
    edge = [1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257, 700]
    return tuple(edge[i % len(edge)] if i % 3 == 0 else int(torch.randint(1, 600, (1,), generator=g)) for i in range(n))


@pytest.mark.parametrize("heads, kv_heads, hd", [(4, 2, 128), (6, 3, 64), (3, 1, 128)])
def test_prompt_attention_on_tcgen05(ops, heads, kv_heads, hd):
    """The tcgen05 prompt kernel against the plain parts and its two twins: several
    sequences with and without a cached prefix, blocks of 128 rows that end inside a
    sequence, lengths around the 128-key step, scrambled pages, NaN wherever the cache
    holds no token, and scores whose maximum jumps far up late in a row (so that the
    accumulator in tensor memory is rescaled) and early in a row (so that it is not)."""
    if ops.plain_kernels():
        pytest.skip("WICK_B200_PLAIN is set: this test is about a fast kernel, which the switch takes out")
    assert ops.attention_prompt_kind(hd, torch.bfloat16) == "tc"
    torch.manual_seed(hd + heads)
    q_lens, starts = [300, 128, 1, 129, 257], [77, 0, 500, 127, 0]
    totals = [s + q for s, q in zip(starts, q_lens)]
    n_pages = sum((t + 63) // 64 for t in totals) + 1
    perm = (torch.randperm(n_pages - 1) + 1).tolist()
    pages, o = [], 0
    for t in totals:
        n = (t + 63) // 64
        pages.append(perm[o:o + n])
        o += n
    kv = _paged(n_pages, kv_heads, hd, torch.bfloat16)          # NaN everywhere
    ks, vs, qs = [], [], []
    for b, t in enumerate(totals):
        k = torch.randn(t, kv_heads, hd)
        v = torch.randn(t, kv_heads, hd)
        q = torch.randn(q_lens[b], heads, hd)
        if t > 200:                                              # one key that dominates from position 190 on
            k[190] *= 0.0
            k[190, :, 1] = 30.0
            q[:, :, 1] = q[:, :, 1].abs() * 0 + 12.0
        if b == 4:                                               # and one at position 2
            k[2] *= 0.0
            k[2, :, 3] = 30.0
            q[:, :, 3] = 9.0
        k, v, q = k.bfloat16(), v.bfloat16(), q.bfloat16()
        for p in range(t):
            kv[pages[b][p // 64], 0, :, p % 64] = k[p].cuda()
            kv[pages[b][p // 64], 1, :, p % 64] = v[p].cuda()
        ks.append(k.float()), vs.append(v.float()), qs.append(q)
    fb = FakeBatch(q_lens, starts, pages).sb
    q_all = dev(torch.cat(qs))
    ref = []
    for b in range(len(q_lens)):
        qq = torch.zeros(totals[b], heads, hd)
        qq[starts[b]:] = qs[b].float()
        ref.append(P.causal_attention(qq, ks[b], vs[b])[starts[b]:])
    ref = torch.cat(ref)
    got = {kind: ops.attention_prompt(q_all, kv, fb, 1 / math.sqrt(hd), kind=kind).float().cpu() for kind in ("tc", "mma", "plain")}
    ops.check_status()
    for kind, out in got.items():
        assert torch.isfinite(out).all(), kind
        assert (out - ref).abs().max() < tol(torch.bfloat16, 2), kind
    assert (got["tc"] - got["mma"]).abs().max() < tol(torch.bfloat16, 2)


@pytest.mark.parametrize("m, n, k", [(1, 72, 64), (7, 333, 100), (130, 192, 96), (64, 1000, 72)])
@pytest.mark.parametrize("combo", ["f32", "bf16", "bf16_f32", "f32_gated", "bf16_gated"])
def test_gemm_simt(ops, m, n, k, combo):
    torch.manual_seed(m * n + k)
    dt = torch.float32 if combo.startswith("f32") else torch.bfloat16
    out_dt = torch.float32 if combo in ("f32", "bf16_f32", "f32_gated") else torch.bfloat16
    gated = combo.endswith("gated")
    x = torch.randn(m, k).to(dt)
    w = (torch.randn(2 * n if gated else n, k) / math.sqrt(k)).to(dt)
    got = ops.gemm_simt(dev(x), dev(w), out_dt, gated=gated).float().cpu()
    y = x.double() @ w.double().T
    ref = (y[:, :n] / (1 + torch.exp(-y[:, :n])) * y[:, n:]) if gated else y
    assert got.shape == (m, n)
    assert (got - ref.float()).abs().max() < (2e-5 if out_dt == torch.float32 else 2e-2)


def test_gemm_rows_do_not_depend_on_the_batch(ops):
    x = torch.randn(65, 96)
    w = torch.randn(160, 96)
    full = ops.gemm_simt(dev(x), dev(w), torch.float32)
    one = ops.gemm_simt(dev(x[13:14].contiguous()), dev(w), torch.float32)
    assert torch.equal(full[13:14], one)


def test_argmax_first_maximum(ops):
    x = torch.randn(6, 151936 // 8 + 3)
    x[1, 77] = x[1, 5000] = 50.0                    # a tie: the first index wins
    x[2, 0] = float("nan")                          # nothing compares greater than a leading NaN
    x[3, 10] = float("nan")
    x[4] = float("-inf")
    got = ops.argmax(dev(x)).tolist()
    assert got == [P.argmax_first(r) for r in x]
    assert got[1] == 77 and got[2] == 0 and got[4] == 0


def test_sample_temperature_follows_the_cumulative_distribution(ops):
    torch.manual_seed(0)
    vocab = 5003
    logits = torch.randn(64, vocab) * 2
    u = torch.rand(64)
    u[0], u[1] = 0.0, 0.9999999
    for temp in (0.7, 1.5):
        got = ops.sample_temperature(dev(logits), temp, dev(u)).tolist()
        p = torch.softmax(logits.double() / temp, -1)
        c = p.cumsum(-1)
        for i, t in enumerate(got):
            lo = c[i, t - 1].item() if t > 0 else 0.0
            assert lo - 1e-5 <= u[i].item() <= c[i, t].item() + 1e-5, (i, t)
    # empirical frequencies (sampler.rs:164-172): 1/4 and 3/4
    l2 = torch.tensor([[0.0, math.log(3.0)]]).repeat(4000, 1)
    got = ops.sample_temperature(dev(l2), 1.0, dev(torch.rand(4000)))
    assert abs(got.float().mean().item() - 0.75) < 0.03


@pytest.mark.parametrize("vocab, k", [(333, 1), (1000, 40), (5003, 333), (151936, 40), (2048, 1024)])
def test_top_k_sorted_with_index_tie_break(ops, vocab, k):
    torch.manual_seed(vocab + k)
    x = torch.randn(5, vocab)
    x[1, :] = x[1, :].round()                       # many ties
    x[2, 7] = x[2, 900 % vocab] = 99.0
    x[3, :] = 1.0                                   # all equal: the lowest indices
    vals, idx = ops.top_k(dev(x), k)
    vals, idx = vals.cpu(), idx.cpu()
    for r in range(5):
        # descending in the total order of floats (-0.0 below +0.0, as f32::total_cmp), ties by index
        bits = x[r].numpy().view(np.uint32).astype(np.int64)
        keys = np.where(bits & 0x80000000, ~bits & 0xFFFFFFFF, bits | 0x80000000)
        order = sorted(range(vocab), key=lambda i: (-int(keys[i]), i))[:k]
        assert idx[r].tolist() == order
        assert torch.equal(vals[r], x[r][order])


@pytest.mark.parametrize("k, temperature, min_p, top_p", [(40, 0.7, 0.0, 0.9), (20, 1.1, 0.05, 0.8), (1, 0.5, 0.0, 0.9),
                                                            (333, 1.0, 0.0, 1.0), (1024, 0.3, 0.2, 0.5), (7, 2.0, 0.9, 1.0)])
def test_pick_from_sorted_candidates(ops, k, temperature, min_p, top_p):
    """The cuts and the draw on the device against their plain form on the host, from
    the same sorted candidates and the same uniform numbers.  (The two exponentials may
    differ in the last bit: a draw that falls on a boundary may then take the neighbour.)"""
    from wick_b200.sampling.sampler import SamplerConfig, pick_from_sorted

    class Fixed:
        def __init__(self, u):
            self.u = u

        def next_f32(self):
            return self.u

    torch.manual_seed(k)
    rows = 300
    logits = torch.randn(rows, 5003) * 3
    logits[5, :] = 0.25                                           # all candidates equal
    vals, idx = ops.top_k(dev(logits), k)
    u = torch.rand(rows)
    u[0], u[1] = 0.0, 1.0 - 2.0 ** -24                            # the ends of the generator's range
    got = ops.pick_sorted(vals, idx, dev(u), temperature, min_p, top_p).tolist()
    cfg = SamplerConfig(temperature=temperature, top_k=k, top_p=top_p, min_p=min_p)
    v, ix = vals.cpu().numpy(), idx.cpu().numpy()
    off = 0
    for r in range(rows):
        want = pick_from_sorted(v[r], ix[r], cfg, Fixed(float(u[r])))
        if got[r] != want:
            off += 1
            place = {int(t): i for i, t in enumerate(ix[r])}
            assert abs(place[got[r]] - place[want]) == 1, (r, got[r], want)
    assert off <= 1


def test_repetition_penalty(ops):
    x = torch.tensor([[2.0, -2.0, 4.0, 1.0], [1.0, 1.0, -1.0, 0.0]])
    got = ops.repetition_penalty(dev(x.clone()), [[0, 1, 1, 0], [2, 9]], 2.0).cpu()
    assert torch.equal(got, torch.tensor([[1.0, -4.0, 4.0, 1.0], [1.0, 1.0, -2.0, 0.0]]))


def test_kernels_refuse_what_they_cannot_do(ops):
    from wick_b200.ops import KernelError
    with pytest.raises(KernelError, match="CUDA tensor"):
        ops.embed(torch.zeros(3, 4), torch.zeros(2, dtype=torch.int32))
    with pytest.raises(KernelError, match="float16"):
        ops.embed(torch.zeros(3, 4, dtype=torch.float16, device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"))
    with pytest.raises(KernelError, match="multiple of 16"):
        ops.attention_prompt(torch.zeros(1, 2, 24, device="cuda"), torch.zeros(1, 2, 1, 64, 24, device="cuda"),
                             FakeBatch([1], [0], [[0]]).sb, 1.0)
    with pytest.raises(KernelError, match="top_k"):
        ops.top_k(torch.zeros(1, 5000, device="cuda"), 2000)
    with pytest.raises(KernelError, match="contiguous"):
        ops.argmax(torch.zeros(4, 8, device="cuda").t())


# ---- the tensor-core matrix product ------------------------------------------
def _tc_ref(x, w, gated):
    y = x.double() @ w.double().T
    if gated:
        n = w.shape[0] // 2
        y = y[:, :n] / (1 + torch.exp(-y[:, :n])) * y[:, n:]
    return y.float()


@pytest.mark.parametrize("t, n, k, gated", [
    (1, 128, 64, False), (5, 333, 72, False), (8, 256, 128, False), (64, 1000, 96, False), (3, 200, 104, True),
    (16, 384, 1024, False), (65, 333, 72, False), (128, 16, 64, False), (300, 520, 200, False), (300, 520, 200, True),
    (1000, 1024, 512, True), (33, 4096, 4096, False), (8, 1000, 256, True), (40, 333, 2048, True),
    (100, 520, 2056, False), (255, 4096, 1024, False), (100, 333, 328, True), (255, 520, 200, True), (130, 1000, 4096, True)])
def test_gemm_tensor_core_both_ways_round(t, n, k, gated):
    """Few tokens (weights as the 128-row operand, transposed output, split inner
    dimension) and many tokens (tokens as the 128-row operand), plain and gated,
    with ragged edges in every dimension, against a float64 product."""
    from wick_b200.ops import gemm_tc as G
    torch.manual_seed(t + n + k)
    x = torch.randn(t, k).bfloat16()
    w = (torch.randn(2 * n if gated else n, k) / math.sqrt(k)).bfloat16()
    plan = G.plan_for(dev(w), gated)
    assert plan is not None
    ref = _tc_ref(x, w, gated)
    got32 = plan.forward(dev(x), torch.float32)
    got16 = plan.forward(dev(x), torch.bfloat16)
    assert got32.shape == (t, n)
    assert (got32.cpu() - ref).abs().max() < 2e-4 * max(1.0, ref.abs().max())
    assert (got16.float().cpu() - ref).abs().max() < 1e-2 * max(1.0, ref.abs().max())
    if not gated:
        parts = plan.forward_delta(dev(x))
        assert parts.dtype == torch.float32 and parts.shape[1:] == (t, n)
        assert (parts.sum(0).cpu() - ref).abs().max() < 2e-4 * max(1.0, ref.abs().max())
        if t < G.PAIR_MIN and k >= 1024:
            assert parts.shape[0] > 1, "a product with few tiles splits its inner dimension"
    G.check_status()
    # the CUDA-core kernel is the plain twin of this one
    twin = ops_gemm_simt(dev(x), dev(w), gated)
    assert (got32 - twin).abs().max() < (1e-2 if gated else 2e-4) * max(1.0, ref.abs().max())   # gated twin: bf16 out


@pytest.mark.parametrize("t, n, k, gated", [(256, 256, 64, False), (257, 100, 72, True), (700, 520, 200, False),
                                            (1000, 333, 328, True), (2100, 1536, 1024, False),
                                            (512, 1024, 4096, False), (300, 300, 8264, False)])
def test_gemm_tensor_core_single_blocks_and_pairs(monkeypatch, t, n, k, gated):
    """From 256 tokens on two thread blocks share a 256 x 256 tile; the kernel for
    single blocks takes the same sizes.  Both against a float64 product.  (The last two
    sizes make few tiles with a long inner dimension: it is cut into 2 and 4 runs.)"""
    from wick_b200.ops import gemm_tc as G
    torch.manual_seed(t + n + k)
    x = torch.randn(t, k).bfloat16()
    w = (torch.randn(2 * n if gated else n, k) / math.sqrt(k)).bfloat16()
    ref = _tc_ref(x, w, gated)
    plan = G.plan_for(dev(w), gated)
    assert t >= G.PAIR_MIN
    for pair_min in (G.PAIR_MIN, 1 << 30):
        monkeypatch.setattr(G, "PAIR_MIN", pair_min)
        got32 = plan.forward(dev(x), torch.float32)
        got16 = plan.forward(dev(x), torch.bfloat16)
        G.check_status()
        assert (got32.cpu() - ref).abs().max() < 2e-4 * max(1.0, ref.abs().max()), pair_min
        assert (got16.float().cpu() - ref).abs().max() < 1e-2 * max(1.0, ref.abs().max()), pair_min
    if not gated:
        # the epilogue that adds into a float32 residual: same numbers as product + addition
        monkeypatch.setattr(G, "PAIR_MIN", 256)
        res = torch.randn(t, n)
        acc = dev(res.clone())
        runs = plan.prompt_splits(t)
        assert runs == {(512, 1024, 4096): 2, (300, 300, 8264): 4}.get((t, n, k), 1)
        if runs == 1:
            assert plan.forward_add(dev(x), acc)
            G.check_status()
            assert torch.equal(acc, dev(res) + plan.forward(dev(x), torch.float32))
        else:
            assert not plan.forward_add(dev(x), acc), "few tiles: partial sums over runs of the inner dimension"
            parts = plan.forward_delta(dev(x))
            G.check_status()
            assert parts.shape == (runs, t, n)
            assert (parts.sum(0).cpu() - ref).abs().max() < 2e-4 * max(1.0, ref.abs().max())
            assert torch.equal(parts, plan.forward_delta(dev(x))), "the same bits in every run"
        assert not plan.forward_add(dev(x[:100]), dev(res[:100].clone())), "few tokens: the caller adds"


def ops_gemm_simt(x, w, gated):
    from wick_b200 import ops
    return ops.gemm_simt(x, w, torch.bfloat16 if gated else torch.float32, gated=gated).float()


def test_gemm_tensor_core_rows_do_not_depend_on_the_batch():
    from wick_b200.ops import gemm_tc as G
    torch.manual_seed(5)
    w = dev((torch.randn(512, 2048) / 45).bfloat16())
    x = dev(torch.randn(40, 2048).bfloat16())
    plan = G.plan_for(w)
    full = plan.forward_delta(x)
    for rows in (1, 7, 16, 17):
        part = plan.forward_delta(x[:rows].contiguous())
        assert torch.equal(part, full[:, :rows]), rows
    assert G.plan_for(dev(torch.zeros(64, 100, dtype=torch.bfloat16))) is None, "rows of 200 bytes cannot be fetched by TMA"
    assert G.plan_for(dev(torch.zeros(64, 96))) is None, "float32 weights take the CUDA-core kernel"


def test_a_wait_that_nothing_satisfies_gives_up_and_is_reported(ops):
    """Every ring kernel waits through the same bounded wait.  A kernel made for this test
    (one block, one barrier that nobody arrives on, no copy in flight, a limit of one
    millisecond) runs it out: the wait returns, the status word names it, the error is raised
    once, and the device goes on working."""
    ops.check_status()
    assert ops.wait_gives_up(1.0) is True
    with pytest.raises(ops.KernelError, match="gave up waiting for nothing"):
        ops.check_status()
    ops.check_status()                                       # the word was cleared
    x = torch.randn(5, 72, device="cuda")
    got = ops.rmsnorm(x, torch.ones(72, device="cuda"), 1e-6, torch.float32)
    assert (got.cpu() - P.rms_norm(x.cpu(), torch.ones(72), 1e-6)).abs().max() < 1e-5


def _decode_case(ops, heads, kv_heads, hd, lens, seed):
    """Random cache contents for sequences of `lens` positions (the last one is the new
    token, written by the norm/rotation/append kernel), scrambled pages, NaN wherever the
    cache holds nothing.  Returns what the decode kernels and the plain attention need."""
    torch.manual_seed(seed)
    B = len(lens)
    n_pages = sum((t + 63) // 64 for t in lens) + 1
    perm = (torch.randperm(n_pages - 1) + 1).tolist()
    pages, o = [], 0
    for t in lens:
        n = (t + 63) // 64
        pages.append(perm[o:o + n])
        o += n
    kv = _paged(n_pages, kv_heads, hd, torch.bfloat16)
    for b, t in enumerate(lens):
        for i, pg in enumerate(pages[b]):
            n = min(64, t - 1 - 64 * i)
            if n > 0:
                kv[pg, :, :, :n] = torch.randn(2, kv_heads, n, hd, device="cuda").bfloat16()
    fd = FakeBatch([1] * B, [t - 1 for t in lens], pages).sb
    width = (heads + 2 * kv_heads) * hd
    parts = dev(torch.randn(3, B, width) * 0.6)
    qw, kw = dev(1 + 0.1 * torch.randn(hd)), dev(1 + 0.1 * torch.randn(hd))
    cos, sin = ops.rope_table(fd.positions, dev(P.rope_inv_freq(10000.0, hd)))
    q = ops.qk_norm_rope_append(parts, heads, kv_heads, hd, q_weight=qw, k_weight=kw, eps=1e-6, cos=cos, sin=sin, kv=kv,
                                page_table=fd.page_table, seq_of_token=fd.seq_of_token, positions=fd.positions,
                                dtype=torch.bfloat16)
    return q, kv, fd, pages


def _plain_last_row(q_row, kv, pages_b, t, heads, kv_heads, scale):
    kk = torch.cat([kv[pg, 0].float() for pg in pages_b], dim=1)[:, :t].transpose(0, 1).cpu()
    vv = torch.cat([kv[pg, 1].float() for pg in pages_b], dim=1)[:, :t].transpose(0, 1).cpu()
    qq = q_row.float().cpu()
    g = heads // kv_heads
    return torch.stack([P.softmax_rows(((qq[h] @ kk[:, h // g].T) * scale)[None])[0] @ vv[:, h // g] for h in range(heads)])


def _run_parts(ops, q, kv, fd, heads, kv_heads, hd, max_kv_len=None):
    mk = max_kv_len or fd.max_kv_len
    scratch = torch.full((max(1, ops.attention_decode_parts_scratch(fd.n_seqs, heads, kv_heads, hd, mk)),), float("nan"),
                         device="cuda")
    out = ops.attention_decode_parts(q, kv, fd, 1 / math.sqrt(hd), scratch, max_kv_len=mk)
    ops.check_status()
    return out


@pytest.mark.parametrize("heads, kv_heads, hd, lens", [
    (8, 2, 128, (1, 130, 700, 64)), (4, 4, 64, (129, 5)), (16, 2, 128, (300,)), (6, 2, 64, (2000, 65, 128, 127, 1, 1025)),
    (5, 1, 128, (4097, 4096, 4160, 3)), (8, 1, 64, (9000, 200)),
    (8, 2, 128, _many_lengths(74, 1)), (6, 3, 64, _many_lengths(49, 2)), (8, 8, 128, _many_lengths(19, 3)),
    (4, 1, 128, _many_lengths(300, 4)), (32, 8, 128, (1537,) * 24 + (1, 700, 1300, 128)),
    (40, 8, 128, _many_lengths(16, 5)), (64, 8, 128, (1025,) * 8)])
def test_decode_attention_by_parts(ops, heads, kv_heads, hd, lens):
    """The tensor-core decode attention against the plain attention over the cache as it
    stands: lengths around the 64-position page and the 128-position part, one part and many,
    more than 64 pages (parts of more than two pages), groups of 1 to 8 query heads per kv
    head (5 and 8: the shapes of Qwen3-14B and 32B), from one pair to 300, scrambled pages,
    NaN wherever the cache holds no token and in the scratch."""
    assert ops.attention_decode_parts_supported(len(lens), heads, kv_heads, hd, torch.bfloat16)
    assert not ops.attention_decode_parts_supported(4, 18, 2, hd, torch.bfloat16), "9 query heads per kv head"
    q, kv, fd, pages = _decode_case(ops, heads, kv_heads, hd, lens, hd + heads + len(lens))
    before = torch.nan_to_num(kv.float(), nan=-7.0)
    got = _run_parts(ops, q, kv, fd, heads, kv_heads, hd).float().cpu()
    assert torch.isfinite(got).all()
    scale = 1 / math.sqrt(hd)
    check = range(len(lens)) if len(lens) <= 30 else list(range(0, len(lens), 7)) + [len(lens) - 1]
    for b in check:
        ref = _plain_last_row(q[b], kv, pages[b], lens[b], heads, kv_heads, scale)
        assert (got[b] - ref).abs().max() < tol(torch.bfloat16, 1), f"sequence {b} of {lens[b]} positions"
    assert torch.equal(torch.nan_to_num(kv.float(), nan=-7.0), before), "the cache is only read"
    # a captured step sizes its work by the page table, not by the longest sequence: same bits
    again = _run_parts(ops, q, kv, fd, heads, kv_heads, hd, max_kv_len=fd.table_width * 64).float().cpu()
    assert torch.equal(again, got)


@pytest.mark.parametrize("heads, kv_heads, hd, lens", [
    (8, 2, 128, (1, 130, 700, 64)), (4, 4, 64, (129, 5)), (6, 2, 64, (2000, 65, 128, 127, 1, 1025)),
    (5, 1, 128, (4097, 3)), (8, 8, 128, _many_lengths(19, 3)), (4, 1, 128, _many_lengths(300, 4)),
    (32, 8, 128, (1537,) * 24 + (1, 700, 1300, 128)), (40, 8, 128, _many_lengths(16, 5)), (64, 8, 128, (1025,) * 8)])
def test_decode_attention_by_parts_from_the_projections_sums(ops, heads, kv_heads, hd, lens):
    """The form that starts from the q/k/v projection's float32 partial sums (sum, per-head norm,
    rotation, the new key and value into the cache, attention) against the two kernels that do
    the same in two steps: same output within the rounding of q, the same value row and (to
    the last bfloat16 bit) key row in the cache and nothing else written; and with write_kv
    off nothing is written and the cache's own row is used."""
    torch.manual_seed(hd + heads + len(lens))
    B = len(lens)
    n_pages = sum((t + 63) // 64 for t in lens) + 1
    perm = (torch.randperm(n_pages - 1) + 1).tolist()
    pages, o = [], 0
    for t in lens:
        n = (t + 63) // 64
        pages.append(perm[o:o + n])
        o += n
    kv_a = _paged(n_pages, kv_heads, hd, torch.bfloat16)
    for b, t in enumerate(lens):
        for i, pg in enumerate(pages[b]):
            n = min(64, t - 1 - 64 * i)
            if n > 0:
                kv_a[pg, :, :, :n] = torch.randn(2, kv_heads, n, hd, device="cuda").bfloat16()
    kv_b = kv_a.clone()
    fd = FakeBatch([1] * B, [t - 1 for t in lens], pages).sb
    sums = dev(torch.randn(3, B, (heads + 2 * kv_heads) * hd) * 0.6)
    qw, kw = dev(1 + 0.1 * torch.randn(hd)), dev(1 + 0.1 * torch.randn(hd))
    cos, sin = ops.rope_table(fd.positions, dev(P.rope_inv_freq(10000.0, hd)))
    scale = 1 / math.sqrt(hd)
    q = ops.qk_norm_rope_append(sums, heads, kv_heads, hd, q_weight=qw, k_weight=kw, eps=1e-6, cos=cos, sin=sin, kv=kv_a,
                                page_table=fd.page_table, seq_of_token=fd.seq_of_token, positions=fd.positions,
                                dtype=torch.bfloat16)
    want = _run_parts(ops, q, kv_a, fd, heads, kv_heads, hd).float()
    scratch = torch.full((max(1, ops.attention_decode_parts_scratch(B, heads, kv_heads, hd, fd.max_kv_len)),), float("nan"), device="cuda")
    got = ops.attention_decode_parts_fused(sums, heads, kv_heads, hd, q_weight=qw, k_weight=kw, eps=1e-6, cos=cos, sin=sin,
                                           kv=kv_b, batch=fd, scale=scale, scratch=scratch).float()
    ops.check_status()
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < tol(torch.bfloat16, 1)
    check = range(B) if B <= 30 else list(range(0, B, 11)) + [B - 1]
    for b in check:
        ref = _plain_last_row(q[b], kv_a, pages[b], lens[b], heads, kv_heads, scale)
        assert (got[b].cpu() - ref).abs().max() < tol(torch.bfloat16, 1), f"sequence {b} of {lens[b]} positions"
    for b, t in enumerate(lens):
        page, row = pages[b][(t - 1) // 64], (t - 1) % 64
        a, bb = kv_a[page, :, :, row].float(), kv_b[page, :, :, row].float()
        assert torch.equal(a[1], bb[1]), "the value is the projection's sum, rounded once"
        assert ((a[0] - bb[0]).abs() <= 2.0 ** -7 * a[0].abs() + 1e-30).all()
        kv_b[page, 0, :, row] = kv_a[page, 0, :, row]
    assert torch.equal(torch.nan_to_num(kv_b.float(), nan=-7.0), torch.nan_to_num(kv_a.float(), nan=-7.0))
    kv_c = kv_a.clone()
    again = ops.attention_decode_parts_fused(sums, heads, kv_heads, hd, q_weight=qw, k_weight=kw, eps=1e-6, cos=cos, sin=sin,
                                             kv=kv_c, batch=fd, scale=scale, scratch=scratch, write_kv=False).float()
    assert torch.equal(torch.nan_to_num(kv_c.float(), nan=-7.0), torch.nan_to_num(kv_a.float(), nan=-7.0))
    assert (again - want).abs().max() < tol(torch.bfloat16, 1)


@pytest.mark.parametrize("heads, kv_heads, hd", [(32, 8, 128), (8, 2, 64), (5, 1, 128)])
def test_decode_attention_bits_do_not_depend_on_the_batch(ops, heads, kv_heads, hd):
    """A sequence's output rows are the same bits whether it is alone, among 8 or among 70
    sequences: alone and among few, a cluster of one-warp blocks computes its parts and merges
    them through shared memory; among many, its parts are dealt to the warps of persistent
    blocks and merged by a second kernel; and a captured step sizes everything by its page
    table (more blocks per cluster than the sequence has parts)."""
    lens = (1100, 3, 640, 77, 129, 2049, 64, 500) + _many_lengths(62, 9)
    q, kv, fd, pages = _decode_case(ops, heads, kv_heads, hd, lens, 5)
    full = _run_parts(ops, q, kv, fd, heads, kv_heads, hd)
    for pick in ([0], [5], list(range(8)), [7, 0, 5], [2], [3, 4]):
        sub = FakeBatch([1] * len(pick), [lens[i] - 1 for i in pick], [pages[i] for i in pick]).sb
        got = _run_parts(ops, q[pick].contiguous(), kv, sub, heads, kv_heads, hd)
        assert torch.equal(got, full[pick]), pick
        wide = FakeBatch([1] * len(pick), [lens[i] - 1 for i in pick], [pages[i] for i in pick], width=64).sb
        got = _run_parts(ops, q[pick].contiguous(), kv, wide, heads, kv_heads, hd, max_kv_len=64 * 64)
        assert torch.equal(got, full[pick]), (pick, "sized by a page table of 64 pages")


def test_decode_attention_refuses_a_length_beyond_its_page_table(ops):
    """A length that its page table cannot hold is left out and reported (status 10); nothing
    outside the table or the cache is touched."""
    heads, kv_heads, hd = 8, 2, 128
    q, kv, fd, pages = _decode_case(ops, heads, kv_heads, hd, (200, 70), 3)
    fd.kv_len[0] = fd.table_width * 64 + 1
    scratch = torch.zeros(ops.attention_decode_parts_scratch(2, heads, kv_heads, hd, 4096), device="cuda")
    out = ops.attention_decode_parts(q, kv, fd, 1 / math.sqrt(hd), scratch, max_kv_len=4096)
    with pytest.raises(ops.KernelError, match="a length or a page outside its page table"):
        ops.check_status()
    ref = _plain_last_row(q[1], kv, pages[1], 70, heads, kv_heads, 1 / math.sqrt(hd))
    assert (out[1].float().cpu() - ref).abs().max() < tol(torch.bfloat16, 1), "the other sequence is served"


@pytest.mark.parametrize("dtype", DTYPES)
def test_cuda_core_decode_attention_cuts_a_length_back_to_its_table(ops, dtype):
    """A length one split beyond what the call was sized for: the kernel reports it and works
    on what the page table and the scratch hold (the cache and the table given here are large
    enough that even an unguarded kernel would have stayed inside them)."""
    if ops.plain_kernels():
        pytest.skip("WICK_B200_PLAIN is set: this test is about a fast kernel, which the switch takes out")
    heads, kv_heads, hd = 4, 2, 32
    split = ops.attention_decode_split(hd, dtype)
    n = 2 * split
    torch.manual_seed(1)
    kv = torch.randn(2 * n // 64 + 2, 2, kv_heads, 64, hd, device="cuda").to(dtype)
    q = torch.randn(1, heads, hd, device="cuda").to(dtype)
    pages = [list(range(1, 2 * n // 64 + 1))]
    fd = FakeBatch([1], [n + split - 1], pages, width=2 * n // 64).sb        # kv_len = n + split
    scratch = torch.zeros(4 * ops.attention_decode_scratch_floats(1, heads, hd, n + split, dtype), device="cuda")
    out = ops.attention_decode(q, kv, fd, 1 / math.sqrt(hd), scratch, max_kv_len=n)
    with pytest.raises(ops.KernelError, match="outside its page table"):
        ops.check_status()
    fd_ok = FakeBatch([1], [n - 1], pages, width=2 * n // 64).sb
    want = ops.attention_decode(q, kv, fd_ok, 1 / math.sqrt(hd), scratch, max_kv_len=n)
    ops.check_status()
    assert torch.equal(out, want), "the first max_kv_len positions were attended to"
