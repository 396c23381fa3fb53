"""The tiled form in which the tensor-core kernels hold a weight matrix."""
import torch

from wick_b200.ops.gemm_tc import pack


def test_pack_is_tiles_of_128_rows_by_64_columns_with_zero_padding():
    torch.manual_seed(0)
    w = torch.randn(300, 200).bfloat16()
    p = pack(w)
    assert p.shape == (3, 4, 128, 64) and p.is_contiguous()
    for tile, kb, r, c in [(0, 0, 0, 0), (1, 2, 5, 63), (2, 3, 43, 7), (0, 3, 127, 0)]:
        assert p[tile, kb, r, c] == w[tile * 128 + r, kb * 64 + c]
    assert (p[2, :, 44:, :] == 0).all(), "rows beyond the matrix"
    assert (p[:, 3, :, 8:] == 0).all(), "columns beyond the matrix"
    back = p.permute(0, 2, 1, 3).reshape(384, 256)[:300, :200]
    assert torch.equal(back, w)


def test_pack_pads_the_halves_of_a_gated_pair_separately():
    torch.manual_seed(1)
    w = torch.randn(2 * 130, 64).bfloat16()           # gate rows 0..129, up rows 130..259
    p = pack(w, gated=True)
    assert p.shape == (4, 1, 128, 64)
    assert torch.equal(p[0, 0], w[:128]) and torch.equal(p[1, 0, :2], w[128:130]) and (p[1, 0, 2:] == 0).all()
    assert torch.equal(p[2, 0], w[130:258]) and torch.equal(p[3, 0, :2], w[258:260]) and (p[3, 0, 2:] == 0).all()


def test_how_a_plan_cuts_the_inner_dimension_at_the_sizes_of_qwen3_8b():
    """The rules that decide how many blocks stream a matrix, at the shapes the bench
    runs (hidden 4096, q 4096 + kv 2 x 1024, intermediate 12288).  Pure host logic."""
    from wick_b200.ops.gemm_tc import Plan
    qkv = Plan(torch.zeros(6144, 4096, dtype=torch.bfloat16), False)
    o = Plan(torch.zeros(4096, 4096, dtype=torch.bfloat16), False)
    down = Plan(torch.zeros(4096, 12288, dtype=torch.bfloat16), False)
    gate_up = Plan(torch.zeros(2 * 1024, 4096, dtype=torch.bfloat16), True)
    # decode steps (up to 64 tokens): about two blocks per SM, the same for every batch
    assert (qkv.decode_splits, o.decode_splits, down.decode_splits) == (6, 8, 8)
    # short prompts (65 to 255 tokens): at most one block per SM
    assert (qkv.short_prompt_splits(), o.short_prompt_splits(), down.short_prompt_splits()) == (3, 4, 4)
    # prompts on pairs of thread blocks: runs only where 256 x 256 tiles are few
    assert [o.prompt_splits(t) for t in (256, 512, 1024, 2048)] == [2, 2, 1, 1]
    assert [down.prompt_splits(t) for t in (256, 512, 1024, 2048)] == [4, 2, 1, 1]
    assert [qkv.prompt_splits(t) for t in (256, 512, 2048)] == [2, 1, 1]
    assert gate_up.prompt_splits(256) == 1 and gate_up.mid_splits(100) == 1, "a gated pair has no partial sums"
    assert gate_up.pair_offset == 1024 and gate_up.n_out == 1024


def test_unpack_gives_the_matrix_back():
    from wick_b200.ops.gemm_tc import unpack
    torch.manual_seed(2)
    for rows, k, gated in [(300, 200, False), (2 * 130, 72, True), (128, 64, False), (2 * 128, 4096, True)]:
        w = torch.randn(rows, k).bfloat16()
        assert torch.equal(unpack(pack(w, gated), rows, k, gated), w)
