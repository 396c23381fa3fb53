"""The decode-attention entry point that allocates nothing
(``wick_attn_decode_noalloc_bf16``), called the way a host without an allocator
would call it: through the shared object's exported C symbol, with raw pointers.
Its output must equal the ordinary entry point's, on two calls in a row that
share the built-in scratch array.  This file is collected last on purpose."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library(head_dim):
    from wick_b200.ops import ATTN_SOURCES
    from wick_b200.ops.build import compile_library
    path = compile_library(f"wick_attn_hd{head_dim}", ATTN_SOURCES, [f"WICK_HD={head_dim}"])
    lib = ctypes.CDLL(path)
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.wick_last_error.restype = ctypes.c_char_p
    lib.wick_attn_decode_noalloc_capacity.restype = ctypes.c_longlong
    lib.wick_attn_decode_noalloc_bf16.restype = I
    lib.wick_attn_decode_noalloc_bf16.argtypes = [P, P, P, P, I, I, P, I, I, I, F, P, P]
    lib.wick_attn_decode_bf16.restype = I
    lib.wick_attn_decode_bf16.argtypes = [P, P, P, P, ctypes.c_int64, P, I, I, P, I, I, I, F, P, P]
    lib.wick_attn_decode_split_bf16.restype = I
    return lib


def _case(seed, n_seqs, heads, kv_heads, hd, lens, n_pages):
    g = torch.Generator().manual_seed(seed)
    kv = torch.randn(n_pages, 2, kv_heads, 64, hd, generator=g).bfloat16().cuda()
    q = torch.randn(n_seqs, heads, hd, generator=g).bfloat16().cuda()
    width = max(-(-l // 64) for l in lens)
    table = torch.zeros(n_seqs, width, dtype=torch.int32)
    perm = torch.randperm(n_pages - 1, generator=g) + 1
    k = 0
    for b, l in enumerate(lens):
        for p in range(-(-l // 64)):
            table[b, p] = perm[k]
            k += 1
    return q, kv, torch.tensor(lens, dtype=torch.int32).cuda(), table.cuda(), width


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    hd, heads, kv_heads = 64, 8, 2
    lib = _library(hd)
    split = lib.wick_attn_decode_split_bf16()
    assert lib.wick_attn_decode_noalloc_capacity() == 2 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    # the second call is smaller than the first, so it finds the first call's leftovers in the array
    for seed, lens in ((1, [700, 3, 257, 64]), (2, [5, 130])):
        n = len(lens)
        q, kv, kv_len, table, width = _case(seed, n, heads, kv_heads, hd, lens, 24)
        want, got = torch.empty_like(q), torch.full_like(q, float("nan"))
        floats = n * heads * (-(-max(lens) // split)) * (hd + 2)
        scratch = torch.empty(floats, dtype=torch.float32, device="cuda")
        rc = lib.wick_attn_decode_bf16(q.data_ptr(), kv.data_ptr(), want.data_ptr(), scratch.data_ptr(), floats,
                                       kv_len.data_ptr(), n, max(lens), table.data_ptr(), width, heads, kv_heads,
                                       scale, status.data_ptr(), stream)
        assert rc == 0, lib.wick_last_error()
        rc = lib.wick_attn_decode_noalloc_bf16(q.data_ptr(), kv.data_ptr(), got.data_ptr(), kv_len.data_ptr(), n,
                                               max(lens), table.data_ptr(), width, heads, kv_heads, scale,
                                               status.data_ptr(), stream)
        assert rc == 0, lib.wick_last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.isfinite(got.float()).all()
        # same kernels, same order of sums: the tests' bfloat16 tolerance is met with room to spare
        assert (got.float() - want.float()).abs().max().item() <= 1.2e-2
        assert torch.equal(got, want)
        # and both agree with a plain float32 computation of the same attention
        for b, l in enumerate(lens):
            pages = table[b, :-(-l // 64)].long()
            k = kv[pages, 0].permute(1, 0, 2, 3).reshape(kv_heads, -1, hd)[:, :l].float()
            v = kv[pages, 1].permute(1, 0, 2, 3).reshape(kv_heads, -1, hd)[:, :l].float()
            for h in range(heads):
                w = torch.softmax((k[h // (heads // kv_heads)] @ q[b, h].float()) * scale, 0)
                ref = w @ v[h // (heads // kv_heads)]
                assert (got[b, h].float() - ref).abs().max().item() < 1.2e-2 * 2


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    hd = 64
    lib = _library(hd)
    q = torch.zeros(1, dtype=torch.bfloat16, device="cuda")
    rc = lib.wick_attn_decode_noalloc_bf16(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 4096, 4096,
                                           q.data_ptr(), 64, 64, 8, 1.0, None, None)
    assert rc != 0
    msg = lib.wick_last_error().decode()
    assert "need" in msg and "the built-in array holds 2097152" in msg
