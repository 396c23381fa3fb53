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
