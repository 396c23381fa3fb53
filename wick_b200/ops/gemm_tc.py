"""Plans for the tensor-core (tcgen05) matrix product of ``csrc/gemm_tc.cu``.

A plan belongs to one bfloat16 weight matrix [out, in] and decides, per call,
which way round the kernel runs:

* fewer than 256 tokens: the weights are the 128-row operand, the tokens the
  narrow one (tile width = tokens rounded up to 16), the result is written
  transposed.  Matrices with few 128-row slabs split their inner dimension over
  several blocks, so that enough of them stream weights at once; the float32
  partial sums are added by the consumer in index order.  Up to 64 tokens (a
  decode step) the number of splits depends on the matrix alone, never on the
  batch, and two blocks of 100 KB share an SM; short prompts of 65 to 255 tokens
  take fewer splits (and one 200 KB block per SM beyond 128 tokens).
* 256 tokens and more: the kernel of ``csrc/gemm_tc2.cu``, in which two thread
  blocks on neighbouring SMs share one 256 x 256 tile (few tiles: the inner
  dimension in 2 to 4 runs).
* the tokens as the 128-row operand of single blocks (weight tiles 256 rows wide,
  128 + 128 for a gated pair) is the form the tests hold the pair kernel against.

Inner sizes that are no multiple of 8 (rows that are no multiple of 16 bytes
cannot be fetched by TMA) have no plan; the caller then uses the CUDA-core kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import KernelError, _Lib, _libs, _p, _stream, check_status, status_tensor  # noqa: F401

SMALL = 64                  # up to this many tokens: weights as the 128-row operand, two 100 KB blocks per SM
SWAP_MAX = 255              # up to this many tokens: weights as the 128-row operand (measured: 5-14 % faster than
                            # tokens on the 128-row side for 100-200 tokens, whose one or two slabs leave SMs idle)
PAIR_MIN = 256              # from this many tokens on, pairs of thread blocks share 256 x 256 tiles
_sms = {}


def sm_count(device) -> int:
    """Multiprocessors of the device a weight lives on (148 on a B200; the same number for a
    matrix that is not on a CUDA device, e.g. when only the plan's rules are looked at)."""
    dev = torch.device(device)
    if dev.type != "cuda":
        return 148
    n = _sms.get(dev)
    if n is None:
        n = _sms[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


SOURCES = ["gemm_tc.cu", "gemm_tc2.cu"]


def _lib() -> _Lib:
    lib = _libs.get("gemm_tc")
    if lib is None:
        lib = _libs["gemm_tc"] = _Lib("wick_gemm_tc", SOURCES)
    return lib


_SIG = "plipliiiiiiiiiiiplilipp"


def gemm_tc(a: torch.Tensor, a_rows: int, b: torch.Tensor, b_rows: int, *, bn: int, out: torch.Tensor, ldo: int,
            gated: int = 0, pair_offset: int = 0, transposed: bool = False, splits: int = 1, split_stride: int = 0,
            max_smem: int = 0, a_static: bool = False, b_static: bool = False, a_packed: bool = False,
            b_packed: bool = False, k: Optional[int] = None) -> None:
    """The raw kernel call (see ``wick_gemm_tc`` in gemm_tc.cu).  A packed operand is a
    :func:`pack` result [tiles, k blocks, 128, 64]; ``k`` then names the inner size."""
    def rows_and_k(nm, t, packed):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
            raise KernelError(f"gemm_tc: {nm} must be a contiguous bfloat16 CUDA tensor")
        if packed:
            if t.dim() != 4 or tuple(t.shape[2:]) != (128, 64):
                raise KernelError(f"gemm_tc: packed {nm} must be [tiles, k blocks, 128, 64]")
            return t.shape[0] * 128, None
        if t.dim() != 2:
            raise KernelError(f"gemm_tc: {nm} must be 2-D")
        return t.shape[0], t.shape[1]
    ra, ka = rows_and_k("a", a, a_packed)
    rb, kb = rows_and_k("b", b, b_packed)
    k = k if k is not None else (ka if ka is not None else kb)
    for kk in (ka, kb):
        if kk is not None and kk != k:
            raise KernelError(f"gemm_tc: inner sizes differ: {ka} and {kb} (k = {k})")
    if out.dtype not in (torch.float32, torch.bfloat16) or not out.is_contiguous():
        raise KernelError("gemm_tc: out must be contiguous float32 or bfloat16")
    st = status_tensor(a.device)
    _lib().call("wick_gemm_tc", _SIG, _p(a), ra, a_rows, _p(b), rb, b_rows, k, bn, gated,
                pair_offset, 1 if transposed else 0, 1 if out.dtype == torch.float32 else 0, 1 if a_static else 0,
                1 if b_static else 0, 1 if a_packed else 0, 1 if b_packed else 0, _p(out), ldo, splits,
                split_stride, max_smem, _p(st), _stream())


def pack(w: torch.Tensor, gated: bool = False) -> torch.Tensor:
    """A [rows, k] matrix as [tiles, ceil(k / 64), 128, 64]: tiles of 128 rows x 64
    columns, each contiguous, rows and columns padded with zeros; the two halves of a
    gated pair are padded each on its own.  A kernel then fetches a weight tile as one
    contiguous 16 KB piece of DRAM instead of 128 pieces of 128 bytes."""
    rows, k = w.shape
    halves = [w[:rows // 2], w[rows // 2:]] if gated else [w]
    kp = (k + 63) // 64 * 64
    out = []
    for h in halves:
        r = h.shape[0]
        rp = (r + 127) // 128 * 128
        if rp != r or kp != k:
            t = torch.zeros((rp, kp), dtype=w.dtype, device=w.device)
            t[:r, :k] = h
        else:
            t = h
        out.append(t.view(rp // 128, 128, kp // 64, 64).permute(0, 2, 1, 3))
    return torch.cat(out, 0).contiguous() if len(out) > 1 else out[0].contiguous()


def unpack(packed: torch.Tensor, rows: int, k: int, gated: bool = False) -> torch.Tensor:
    """The [rows, k] matrix that :func:`pack` made ``packed`` from."""
    tiles, k_blocks = packed.shape[:2]
    full = packed.permute(0, 2, 1, 3).reshape(tiles * 128, k_blocks * 64)
    if gated:
        half = rows // 2
        return torch.cat([full[:half, :k], full[(tiles // 2) * 128:(tiles // 2) * 128 + half, :k]], 0).contiguous()
    return full[:rows, :k].contiguous()


def gemm_tc_pair(a: torch.Tensor, b: torch.Tensor, b_rows: int, *, out: torch.Tensor, ldo: int, gated: bool = False,
                 pair_offset: int = 0, accumulate: bool = False, b_packed: bool = False, splits: int = 1,
                 split_stride: int = 0) -> None:
    """The kernel for pairs of thread blocks (see ``wick_gemm_tc2`` in gemm_tc2.cu): out[m, n] = a[m] . b[n],
    or out[m, n] += ... with ``accumulate`` (float32 output), or ``splits`` partial sums over runs of the inner
    dimension, ``split_stride`` elements apart (float32 output)."""
    for nm, t in (("a", a), ("b", b)):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
            raise KernelError(f"gemm_tc_pair: {nm} must be a contiguous bfloat16 CUDA tensor")
    if a.dim() != 2 or (b.dim() != 2 if not b_packed else (b.dim() != 4 or tuple(b.shape[2:]) != (128, 64))):
        raise KernelError("gemm_tc_pair: a must be 2-D, b 2-D or a packed [tiles, k blocks, 128, 64]")
    if not b_packed and a.shape[1] != b.shape[1]:
        raise KernelError(f"gemm_tc_pair: inner sizes differ: {a.shape[1]} and {b.shape[1]}")
    if b_packed and b.shape[1] != (a.shape[1] + 63) // 64:
        raise KernelError(f"gemm_tc_pair: packed b has {b.shape[1]} k blocks, a an inner size of {a.shape[1]}")
    if out.dtype not in (torch.float32, torch.bfloat16) or not out.is_contiguous():
        raise KernelError("gemm_tc_pair: out must be contiguous float32 or bfloat16")
    st = status_tensor(a.device)
    _lib().call("wick_gemm_tc2", "pipliiiiiiiplilpp", _p(a), a.shape[0], _p(b), b.shape[0] * 128 if b_packed else b.shape[0],
                b_rows, a.shape[1], 1 if gated else 0, pair_offset, 1 if out.dtype == torch.float32 else 0,
                1 if accumulate else 0, 1 if b_packed else 0, _p(out), ldo, splits, split_stride, _p(st), _stream())


def _ceil16(n: int) -> int:
    return (n + 15) // 16 * 16


class Plan:
    """Holds the matrix in the packed form (:func:`pack`); the row-major original is
    not kept."""

    def __init__(self, weight: torch.Tensor, gated: bool):
        self.gated = gated
        self.rows, self.k = weight.shape
        self.n_out = self.rows // 2 if gated else self.rows
        self.w = pack(weight, gated)
        self.sms = sm_count(weight.device)
        self.pair_offset = (self.n_out + 127) // 128 * 128            # in padded rows
        k_blocks = (self.k + 63) // 64
        tiles = (self.n_out + 127) // 128
        # Decode: about two blocks per SM (just under two per SM) stream best; every
        # split keeps at least eight 64-wide steps of the inner dimension.
        self.decode_splits = max(1, min(2 * self.sms // tiles, 8, k_blocks // 8))
        self.k_blocks = k_blocks

    def matrix(self) -> torch.Tensor:
        """The weight as it was given: [rows, k], row-major (a copy)."""
        return unpack(self.w, self.rows, self.k, self.gated)

    def prompt_splits(self, t: int) -> int:
        """Runs of the inner dimension for ``t`` >= PAIR_MIN tokens: a few hundred tokens times
        a narrow matrix make fewer 256 x 256 tiles than there are pairs of SMs (512 tokens
        x 4096 outputs: 32 tiles for 74 pairs); two to four runs of at least 32 steps each
        fill the part."""
        if self.gated:
            return 1
        tiles = ((t + 255) // 256) * ((self.n_out + 255) // 256)
        return max(1, min(4, (self.sms // 2) // tiles, self.k_blocks // 32))

    def short_prompt_splits(self) -> int:
        """Runs of the inner dimension for SMALL < tokens <= SWAP_MAX (weights as the 128-row
        operand, at most one block per SM)."""
        return max(1, min(self.sms // ((self.n_out + 127) // 128), 8, self.k_blocks // 8))

    def mid_splits(self, t: int) -> int:
        """Runs of the inner dimension when SWAP_MAX < ``t`` < PAIR_MIN tokens take the form with
        the tokens as the 128-row operand of single blocks: one or two slabs of tokens times
        256-wide slabs of the matrix are a handful of tiles; up to eight runs of at least eight
        steps each give every SM a block."""
        if self.gated:
            return 1
        tiles = ((t + 127) // 128) * ((self.n_out + 255) // 256)
        return max(1, min(8, self.sms // tiles, self.k_blocks // 8))

    # ---- [n, in] -> [n, out] ----
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        t = x.shape[0]
        out = torch.empty((t, self.n_out), dtype=out_dtype, device=x.device)
        if t == 0:
            return out
        self._run(x, out, splits=1)
        return out

    def forward_delta(self, x: torch.Tensor) -> torch.Tensor:
        t = x.shape[0]
        if self.gated:
            raise KernelError("gemm_tc: a gated pair has no partial sums")
        if t <= SMALL:
            splits = self.decode_splits
        elif t <= SWAP_MAX:
            splits = self.short_prompt_splits()
        else:
            splits = self.prompt_splits(t) if t >= PAIR_MIN else self.mid_splits(t)
        out = torch.empty((splits, t, self.n_out), dtype=torch.float32, device=x.device)
        if t:
            self._run(x, out, splits=splits)
        return out

    def forward_add(self, x: torch.Tensor, residual: torch.Tensor) -> bool:
        """residual [n, out] (float32) += x W^T, every element by one thread, where the
        kernel for many tokens runs; False (and nothing done) otherwise."""
        t = x.shape[0]
        if self.gated or t < PAIR_MIN or residual.dtype != torch.float32 or not residual.is_contiguous() \
                or tuple(residual.shape) != (t, self.n_out) or self.prompt_splits(t) > 1:
            return False                                   # (few tiles: partial sums over runs of the inner dimension instead)
        gemm_tc_pair(x, self.w, self.n_out, out=residual, ldo=self.n_out, accumulate=True, b_packed=True)
        return True

    def _run(self, x: torch.Tensor, out: torch.Tensor, splits: int) -> None:
        t = x.shape[0]
        if t <= max(SMALL, SWAP_MAX):
            # Two blocks of 100 KB per SM: one block's start and end overlap the
            # other's streaming.  A gated pair shares one 128-row tile (64 gate rows,
            # 64 up rows), which doubles the number of blocks.  (More than 128 tokens make
            # stages of 48 KB: one block of 200 KB per SM then.)
            gemm_tc(self.w, self.n_out, x, t, bn=_ceil16(t), out=out, ldo=self.n_out,
                    gated=3 if self.gated else 0, pair_offset=self.pair_offset, transposed=True, splits=splits,
                    split_stride=t * self.n_out, max_smem=(100 if t <= 128 else 200) * 1024, a_static=True,
                    a_packed=True, k=self.k)
        elif t >= PAIR_MIN:
            gemm_tc_pair(x, self.w, self.n_out, out=out, ldo=self.n_out, gated=self.gated, pair_offset=self.pair_offset,
                         b_packed=True, splits=splits, split_stride=t * self.n_out)
        else:
            bn = min(128 if self.gated else 256, _ceil16(self.n_out))
            if bn > 128:
                bn = 256                               # two packed tiles of 128 rows
            gemm_tc(x, t, self.w, self.n_out, bn=bn, out=out, ldo=self.n_out, gated=2 if self.gated else 0,
                    pair_offset=self.pair_offset, transposed=False, splits=splits, split_stride=t * self.n_out,
                    max_smem=200 * 1024, b_static=True, b_packed=True, k=self.k)


def plan_for(weight: torch.Tensor, gated: bool = False) -> Optional[Plan]:
    """A plan for this weight, or None where the kernel does not take its sizes."""
    if weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.dim() != 2:
        return None
    if weight.shape[1] % 8 != 0 or weight.data_ptr() % 16 != 0:
        return None
    if gated and weight.shape[0] % 2 != 0:
        return None
    return Plan(weight, gated)
