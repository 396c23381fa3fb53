"""The kernels, as Python functions over CUDA tensors.

Every function checks its arguments (device, dtype, shape, contiguity), passes
raw pointers and the current CUDA stream to an exported C function of one of
the libraries built from ``wick_b200/csrc``, and raises :class:`KernelError`
with the library's message if the call is refused.  There is no fallback of
any kind: without a CUDA device or without ``nvcc`` these functions raise.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
import os
from typing import Dict, List, Optional, Tuple

import torch

from .build import BuildError, load_library

from ..layout import PAGE


class KernelError(RuntimeError):
    pass


_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_int64, "f": ctypes.c_float}

# Argument kinds of an exported function: p pointer, i int32, l int64, f float; the
# last pointer is always the stream.


def _dt(t: torch.Tensor) -> str:
    if t.dtype == torch.bfloat16:
        return "bf16"
    if t.dtype == torch.float32:
        return "f32"
    raise KernelError(f"unsupported element type {t.dtype} (bfloat16 and float32 are built)")


class _Lib:
    """A loaded library with lazily configured functions."""

    def __init__(self, name, sources, defines=()):
        self._lib = load_library(name, sources, defines)
        self._fns: Dict[str, object] = {}
        self._lib.wick_page_size.restype = ctypes.c_int
        built_for = int(self._lib.wick_page_size())
        if built_for != PAGE:
            raise KernelError(f"{name} was built for cache pages of {built_for} positions, the package uses {PAGE}")

    def fn(self, name: str, sig: str):
        f = self._fns.get(name)
        if f is None:
            try:
                f = getattr(self._lib, name)
            except AttributeError:
                raise KernelError(f"{name} is not exported by {self._lib._name}") from None
            f.argtypes = [_CT[c] for c in sig]
            f.restype = ctypes.c_int
            self._fns[name] = f
        return f

    def call(self, name: str, sig: str, *args, kernels: int = 1):
        rc = self.fn(name, sig)(*args)
        if rc != 0:
            raise KernelError(self._lib.wick_last_error().decode("utf-8", "replace"))
        launches[0] += kernels


_libs: Dict[str, _Lib] = {}

# Kernels launched through this module so far (a captured step counts them once,
# at capture; the engine adds them again at every replay).
launches = [0]

# WICK_B200_PLAIN=1 (or PLAIN_KERNELS = True): every matrix product and every attention runs
# through its plain CUDA-core twin (float32 accumulation, no tensor cores, no bulk copies),
# whatever the compute dtype: the slow form that the fast kernels are held against, for
# telling a kernel's fault from a model's.
PLAIN_KERNELS = os.environ.get("WICK_B200_PLAIN", "") not in ("", "0")


def plain_kernels() -> bool:
    return PLAIN_KERNELS


CORE_SOURCES = ["core.cu", "sample.cu", "state.cu"]


def _core() -> _Lib:
    lib = _libs.get("core")
    if lib is None:
        lib = _libs["core"] = _Lib("wick_core", CORE_SOURCES)
    return lib


def _simt() -> _Lib:
    lib = _libs.get("simt")
    if lib is None:
        lib = _libs["simt"] = _Lib("wick_gemm_simt", ["gemm_simt.cu"])
    return lib


ATTN_SOURCES = ["attn.cu", "attn_decode.cu", "attn_decode_parts.cu", "attn_prompt_mma.cu", "attn_prompt_tc.cu"]


def _attn(head_dim: int) -> _Lib:
    key = f"attn{head_dim}"
    lib = _libs.get(key)
    if lib is None:
        if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
            raise KernelError(f"attention kernels take a head_dim that is a multiple of 16 between 16 and 256, "
                              f"not {head_dim}")
        # WICK_B200_ATTN_DEFINES: further -D definitions for experiments (e.g. "WICK_DECODE_WARPS=4,WICK_DECODE_TILES=3")
        more = [d for d in os.environ.get("WICK_B200_ATTN_DEFINES", "").split(",") if d]
        lib = _libs[key] = _Lib(f"wick_attn_hd{head_dim}", ATTN_SOURCES, [f"WICK_HD={head_dim}"] + more)
    return lib


# One device word that kernels write a code to when a bounded wait gives up or an index they
# were given lies outside its table.
_status: Optional[torch.Tensor] = None
_STATUS_TEXT = {1: "gemm_tc gave up waiting for a free shared-memory stage", 2: "gemm_tc gave up waiting for a TMA copy",
                3: "gemm_tc gave up waiting for the accumulator", 4: "attention decode gave up waiting for its bulk copies",
                5: "gemm_tc gave up waiting for a free accumulator",
                7: "attention (tcgen05) gave up waiting for a copy or an accumulator",
                8: "attention decode (tensor cores) gave up waiting for its TMA copies",
                10: "attention decode was given a length or a page outside its page table or its cache",
                99: "the test kernel gave up waiting for nothing (nobody arrives on its barrier)"}


def status_tensor(device) -> torch.Tensor:
    global _status
    if _status is None or _status.device != torch.device(device):
        _status = torch.zeros(1, dtype=torch.int32, device=device)
    return _status


def check_status() -> None:
    """Raise if a kernel gave up a bounded wait (this synchronises the device)."""
    if _status is not None:
        code = int(_status.item())
        if code != 0:
            _status.zero_()
            raise KernelError(f"a kernel reported a fault: {_STATUS_TEXT.get(code, 'code %d' % code)}; its output is invalid")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_scope_stream: List[Optional[int]] = [None]


@contextlib.contextmanager
def stream_scope():
    """Inside the scope every kernel of this module goes to the stream that is
    current at entry.  (Asked once: torch's lookup of the current stream costs as
    much host time as a launch, and a short prompt's step is bound by the host.)"""
    before = _scope_stream[0]
    _scope_stream[0] = torch.cuda.current_stream().cuda_stream
    try:
        yield
    finally:
        _scope_stream[0] = before


def _stream() -> int:
    s = _scope_stream[0]
    return torch.cuda.current_stream().cuda_stream if s is None else s


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(name: str, t: torch.Tensor, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the kernels have no CPU form)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, has {tuple(t.shape)}")


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [n, width] rows of ``table`` [vocab, width] at int32 ``tokens`` [n]."""
    _cuda("table", table)
    _cuda("tokens", tokens, torch.int32)
    n, (vocab, width) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, width), dtype=torch.float32, device=table.device)
    _cuda("out", out, torch.float32, (n, width))
    _core().call(f"wick_embed_{_dt(table)}", "pppiilp", _p(table), _p(tokens), _p(out), n, width, vocab, _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype, *,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norm of float32 ``x`` [n, width] into ``out_dtype``.

    delta: float32 [splits, n, width]; added to ``x`` (in index order) before the norm,
    and, when every row is normalised, in place.  rows: int32 indices (a row may be named
    more than once); only those rows are normalised, the result has len(rows) rows, and
    ``x`` itself is left as it was."""
    _cuda("x", x, torch.float32)
    n, width = x.shape
    _cuda("weight", weight, torch.float32, (width,))
    splits = 0
    if delta is not None:
        _cuda("delta", delta, torch.float32)
        _need(delta.dim() == 3 and tuple(delta.shape[1:]) == (n, width),
              f"delta must be [splits, {n}, {width}], is {tuple(delta.shape)}")
        splits = delta.shape[0]
    if rows is not None:
        _cuda("rows", rows, torch.int32)
    n_out = n if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n_out, width), dtype=out_dtype, device=x.device)
    _cuda("out", out, out_dtype, (n_out, width))
    _core().call(f"wick_rmsnorm_{_dt(out)}", "ppilpfppiip", _p(x), _p(delta), splits, n, _p(weight), float(eps),
                 _p(rows), _p(out), n_out, width, _stream())
    return out


def add_delta(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta[0] + delta[1] + ... in place (float32)."""
    _cuda("x", x, torch.float32)
    _cuda("delta", delta, torch.float32)
    _need(delta.dim() == 3 and tuple(delta.shape[1:]) == tuple(x.shape), "delta must be [splits, *x.shape]")
    _core().call("wick_add_delta", "ppilp", _p(x), _p(delta), delta.shape[0], x.numel(), _stream())
    return x


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of ``positions[t] * inv_freq[i]`` (float32 product), each [n, half]."""
    _cuda("positions", positions, torch.int32)
    _cuda("inv_freq", inv_freq, torch.float32)
    n, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _core().call("wick_rope_table", "ppppiip", _p(positions), _p(inv_freq), _p(cos), _p(sin), n, half, _stream())
    return cos, sin


def qk_norm_rope_append(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, *,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kv: Optional[torch.Tensor],
                        page_table: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                        write_kv: bool = True, q_out: Optional[torch.Tensor] = None,
                        dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Per-head RMS norm of q and k (if weights are given), half-split rotation
    (if tables are given), then q -> ``q_out`` [n, n_heads, head_dim] and k, v ->
    the cache ``kv`` [pages, 2, n_kv, 64, head_dim] at each token's position.

    qkv: [n, (n_heads + 2 n_kv) head_dim] in the activation dtype, or float32
    partial sums [splits, n, ...] (then ``dtype`` names the activation dtype)."""
    _cuda("qkv", qkv)
    width = (n_heads + 2 * n_kv) * head_dim
    parts = qkv.dim() == 3
    if parts:
        _need(qkv.dtype == torch.float32 and qkv.shape[2] == width and dtype is not None,
              f"partial sums must be float32 [splits, n, {width}] and come with the activation dtype")
        n, splits, act = qkv.shape[1], qkv.shape[0], dtype
    else:
        _need(qkv.dim() == 2 and qkv.shape[1] == width, f"qkv must be [n, {width}], is {tuple(qkv.shape)}")
        n, splits, act = qkv.shape[0], 0, qkv.dtype
    for nm, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _cuda(nm, w, torch.float32, (head_dim,))
    _need((q_weight is None) == (k_weight is None), "q and k norm weights come together")
    if cos is not None:
        _cuda("cos", cos, torch.float32, (n, head_dim // 2))
        _cuda("sin", sin, torch.float32, (n, head_dim // 2))
    if write_kv:
        _cuda("kv", kv, act)
        _need(kv.dim() == 5 and tuple(kv.shape[1:]) == (2, n_kv, PAGE, head_dim),
              f"kv must be [pages, 2, {n_kv}, {PAGE}, {head_dim}], is {tuple(kv.shape)}")
    _cuda("page_table", page_table, torch.int32)
    _cuda("seq_of_token", seq_of_token, torch.int32, (n,))
    _cuda("positions", positions, torch.int32, (n,))
    if q_out is None:
        q_out = torch.empty((n, n_heads, head_dim), dtype=act, device=qkv.device)
    _cuda("q_out", q_out, act, (n, n_heads, head_dim))
    _core().call(f"wick_qk_norm_rope_append_{_dt(q_out)}", "ppiiiiippfpppppippip",
                 None if parts else _p(qkv), _p(qkv) if parts else None, splits, n, n_heads, n_kv, head_dim,
                 _p(q_weight), _p(k_weight), float(eps), _p(cos), _p(sin), _p(q_out), _p(kv) if write_kv else None,
                 _p(page_table), page_table.shape[-1], _p(seq_of_token), _p(positions), 1 if write_kv else 0,
                 _stream())
    return q_out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    _cuda("gate", gate)
    _cuda("up", up, gate.dtype, gate.shape)
    out = torch.empty_like(gate)
    _core().call(f"wick_silu_mul_{_dt(gate)}", "ppplp", _p(gate), _p(up), _p(out), gate.numel(), _stream())
    return out


# ---------------------------------------------------------------------------
def gemm_simt(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, *, gated: bool = False,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [m, k] times w [n, k] transposed on the CUDA cores, float32 accumulation.
    gated: w is [2n, k] (gate rows, then up rows); returns silu(x gate^T) * (x up^T)."""
    _cuda("x", x)
    _cuda("w", w, x.dtype)
    m, k = x.shape
    _need(w.dim() == 2 and w.shape[1] == k, f"w must be [n, {k}], is {tuple(w.shape)}")
    n = w.shape[0] // 2 if gated else w.shape[0]
    if gated:
        _need(w.shape[0] % 2 == 0, "gated weight needs an even number of rows")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _cuda("out", out, out_dtype, (m, n))
    name = f"wick_gemm_simt_{_dt(x)}_{_dt(out)}" + ("_gated" if gated else "")
    if name not in ("wick_gemm_simt_bf16_bf16", "wick_gemm_simt_bf16_f32", "wick_gemm_simt_f32_f32",
                    "wick_gemm_simt_bf16_bf16_gated", "wick_gemm_simt_f32_f32_gated"):
        raise KernelError(f"no matrix product from {x.dtype} to {out_dtype}" + (" (gated)" if gated else ""))
    _simt().call(name, "pppiiip", _p(x), _p(w), _p(out), m, n, k, _stream())
    return out


# ---------------------------------------------------------------------------
Q_TILE = 64         # query rows per work item of the prompt attention kernels


def attention_tiles(batch) -> int:
    """How many work items the prompt attention kernels cut this step into: one per 64 new
    tokens of a sequence, numbered sequence by sequence (a kernel finds its item's sequence
    and first row from the step's ``cu_seqlens``)."""
    if getattr(batch, "q_tiles", None) is not None:
        return batch.q_tiles                 # (a captured step: the most there can be; a kernel skips items beyond the last)
    return sum((q + Q_TILE - 1) // Q_TILE for q in batch.q_lens)


def attention_prompt_kind(head_dim: int, dtype: torch.dtype, plain: bool = False) -> str:
    """Which prompt kernel runs: ``tc`` (tcgen05: bfloat16, head sizes 64 and 128),
    ``mma`` (mma.sync: bfloat16, other head sizes up to 128) or ``plain`` (CUDA
    cores: float32, larger heads, and the twin the others are checked against)."""
    if plain or PLAIN_KERNELS or dtype != torch.bfloat16 or head_dim > 128:
        return "plain"
    return "tc" if head_dim in (64, 128) else "mma"


def attention_prompt(q: torch.Tensor, kv: torch.Tensor, batch, scale: float,
                     out: Optional[torch.Tensor] = None, plain: bool = False, kind: Optional[str] = None) -> torch.Tensor:
    """Causal attention of the step's new tokens over the cache (which already
    holds their keys and values).  q: [n, heads, d]; kv: [pages, 2, kv_heads, 64, d].
    ``kind`` (see :func:`attention_prompt_kind`) picks a kernel by hand."""
    _cuda("q", q)
    n, n_heads, hd = q.shape
    _cuda("kv", kv, q.dtype)
    _need(kv.dim() == 5 and kv.shape[1] == 2 and kv.shape[3] == PAGE and kv.shape[4] == hd,
          f"kv must be [pages, 2, kv_heads, {PAGE}, {hd}], is {tuple(kv.shape)}")
    n_kv = kv.shape[2]
    _need(n == batch.n_tokens, f"q has {n} rows, the batch {batch.n_tokens} tokens")
    if out is None:
        out = torch.empty_like(q)
    _cuda("out", out, q.dtype, q.shape)
    kind = kind or attention_prompt_kind(hd, q.dtype, plain)
    _need(kind == "plain" or q.dtype == torch.bfloat16, "the tensor-core attention kernels take bfloat16")
    n_tiles = attention_tiles(batch)
    if kind == "tc":
        _attn(hd).call("wick_attn_prompt_tc_bf16", "plplpipippiiifpp", _p(q), n, _p(kv), kv.shape[0], _p(out),
                       n_tiles, _p(batch.cu_seqlens), batch.n_seqs, _p(batch.start),
                       _p(batch.page_table), batch.table_width, n_heads, n_kv, float(scale),
                       _p(status_tensor(q.device)), _stream())
        return out
    _attn(hd).call("wick_attn_prompt_mma_bf16" if kind == "mma" else f"wick_attn_prompt_{_dt(q)}", "pppipippiiifp",
                   _p(q), _p(kv), _p(out), n_tiles, _p(batch.cu_seqlens), batch.n_seqs, _p(batch.start), _p(batch.page_table),
                   batch.table_width, n_heads, n_kv, float(scale), _stream())
    return out


_decode_split: Dict[tuple, int] = {}


def attention_decode_kind(head_dim: int, dtype: torch.dtype, plain: bool = False) -> str:
    """Which of the CUDA-core decode kernels :func:`attention_decode` runs: ``fast`` (from
    bulk-copied page tiles) or ``plain``.  (The tensor-core decode attention, bfloat16 at head
    sizes 64 and 128, is :func:`attention_decode_parts`.)"""
    return "plain" if plain or PLAIN_KERNELS else "fast"


def attention_decode_split(head_dim: int, dtype: torch.dtype, plain: bool = False) -> int:
    """Cached positions handled by one block of the decode kernel."""
    kind = attention_decode_kind(head_dim, dtype, plain)
    key = (head_dim, dtype, kind)
    v = _decode_split.get(key)
    if v is None:
        lib = _attn(head_dim)._lib
        name = {"plain": "wick_attn_decode_plain_split",
                "fast": f"wick_attn_decode_split_{'bf16' if dtype == torch.bfloat16 else 'f32'}"}[kind]
        f = getattr(lib, name)
        f.restype = ctypes.c_int
        f.argtypes = []
        v = _decode_split[key] = int(f())
    return v


def attention_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, max_kv_len: int,
                                    dtype: torch.dtype = torch.bfloat16, plain: bool = False) -> int:
    split = attention_decode_split(head_dim, dtype, plain)
    return n_seqs * n_heads * max(1, -(-max_kv_len // split)) * (head_dim + 2)


def attention_decode(q: torch.Tensor, kv: torch.Tensor, batch, scale: float, scratch: torch.Tensor,
                     out: Optional[torch.Tensor] = None, max_kv_len: Optional[int] = None,
                     plain: bool = False) -> torch.Tensor:
    """One new token per sequence, on the CUDA cores (float32, and bfloat16 at head sizes the
    tensor-core kernel does not take).  scratch: float32, at least
    :func:`attention_decode_scratch_floats` elements; it holds the per-split partial results
    between the two kernels.  plain: the form without shared-memory staging."""
    _cuda("q", q)
    n, n_heads, hd = q.shape
    _cuda("kv", kv, q.dtype)
    _need(kv.dim() == 5 and kv.shape[1] == 2 and kv.shape[3] == PAGE and kv.shape[4] == hd,
          f"kv must be [pages, 2, kv_heads, {PAGE}, {hd}], is {tuple(kv.shape)}")
    n_kv = kv.shape[2]
    _need(n == batch.n_seqs, f"decode attention takes one token per sequence: {n} rows, {batch.n_seqs} sequences")
    _cuda("scratch", scratch, torch.float32)
    if out is None:
        out = torch.empty_like(q)
    _cuda("out", out, q.dtype, q.shape)
    mk = batch.max_kv_len if max_kv_len is None else max_kv_len
    kind = attention_decode_kind(hd, q.dtype, plain)
    if kind == "plain":
        _attn(hd).call(f"wick_attn_decode_plain_{_dt(q)}", "pppplpiipiiifp", _p(q), _p(kv), _p(out),
                       _p(scratch), scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table),
                       batch.table_width, n_heads, n_kv, float(scale), _stream(), kernels=2)
    else:
        _attn(hd).call(f"wick_attn_decode_{_dt(q)}", "pppplpiipiiifpp", _p(q), _p(kv), _p(out),
                       _p(scratch), scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table),
                       batch.table_width, n_heads, n_kv, float(scale), _p(status_tensor(q.device)), _stream(),
                       kernels=2)
    return out


def attention_decode_parts_supported(n_seqs: int, n_heads: int, n_kv: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core decode attention whose work is cut by each sequence's own
    length takes this problem: bfloat16, head size 64 or 128, at most 8 query heads per kv head."""
    if dtype != torch.bfloat16 or head_dim not in (64, 128) or n_kv <= 0 or n_heads % n_kv != 0 or n_heads // n_kv > 8:
        return False
    return n_seqs <= 2048


def attention_decode_parts_scratch(n_seqs: int, n_heads: int, n_kv: int, head_dim: int, max_kv_len: int) -> int:
    """float32 words of scratch that :func:`attention_decode_parts` needs."""
    f = _attn(head_dim)._lib.wick_attn_decode_parts_scratch
    f.restype = ctypes.c_longlong
    f.argtypes = [ctypes.c_int] * 4
    return int(f(n_seqs, n_heads, n_kv, max_kv_len))


def attention_decode_parts(q: torch.Tensor, kv: torch.Tensor, batch, scale: float, scratch: torch.Tensor,
                           out: Optional[torch.Tensor] = None, max_kv_len: Optional[int] = None) -> torch.Tensor:
    """One new token per sequence over the cache (which already holds its key and value).
    q: bfloat16 [n, heads, d].  scratch: float32, at least
    :func:`attention_decode_parts_scratch` words.  How a sequence's positions are cut into
    parts, and the order in which the parts are merged, depend on its own length only."""
    _cuda("q", q, torch.bfloat16)
    n, n_heads, hd = q.shape
    _cuda("kv", kv, torch.bfloat16)
    _need(kv.dim() == 5 and kv.shape[1] == 2 and kv.shape[3] == PAGE and kv.shape[4] == hd,
          f"kv must be [pages, 2, kv_heads, {PAGE}, {hd}], is {tuple(kv.shape)}")
    n_kv = kv.shape[2]
    _need(n == batch.n_seqs, f"decode attention takes one token per sequence: {n} rows, {batch.n_seqs} sequences")
    _cuda("scratch", scratch, torch.float32)
    if out is None:
        out = torch.empty_like(q)
    _cuda("out", out, torch.bfloat16, q.shape)
    mk = batch.max_kv_len if max_kv_len is None else max_kv_len
    _attn(hd).call("wick_attn_decode_parts_bf16", "pplpplpiipiiifpp", _p(q), _p(kv), kv.shape[0], _p(out), _p(scratch),
                   scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table), batch.table_width,
                   n_heads, n_kv, float(scale), _p(status_tensor(q.device)), _stream(), kernels=2 if mk > 128 else 1)
    return out


def attention_decode_parts_fused(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, *,
                                 q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kv: torch.Tensor, batch,
                                 scale: float, scratch: torch.Tensor, write_kv: bool = True,
                                 max_kv_len: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`attention_decode_parts` from the projection's float32 partial sums ``qkv``
    [splits, n, (n_heads + 2 n_kv) head_dim]: per-head norm of q and k, rotation, the new key
    and value into the cache (unless ``write_kv`` is False), attention, merge — two launches."""
    _cuda("qkv", qkv, torch.float32)
    width = (n_heads + 2 * n_kv) * head_dim
    n = batch.n_seqs
    _need(qkv.dim() == 3 and tuple(qkv.shape[1:]) == (n, width), f"qkv must be [splits, {n}, {width}], is {tuple(qkv.shape)}")
    for nm, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _cuda(nm, w, torch.float32, (head_dim,))
    _need((q_weight is None) == (k_weight is None), "q and k norm weights come together")
    if cos is not None:
        _cuda("cos", cos, torch.float32, (n, head_dim // 2))
        _cuda("sin", sin, torch.float32, (n, head_dim // 2))
    _cuda("kv", kv, torch.bfloat16)
    _need(kv.dim() == 5 and tuple(kv.shape[1:]) == (2, n_kv, PAGE, head_dim),
          f"kv must be [pages, 2, {n_kv}, {PAGE}, {head_dim}], is {tuple(kv.shape)}")
    _cuda("scratch", scratch, torch.float32)
    if out is None:
        out = torch.empty((n, n_heads, head_dim), dtype=torch.bfloat16, device=qkv.device)
    _cuda("out", out, torch.bfloat16, (n, n_heads, head_dim))
    mk = batch.max_kv_len if max_kv_len is None else max_kv_len
    _attn(head_dim).call("wick_attn_decode_parts_fused_bf16", "pippfppiplpplpiipiiifpp", _p(qkv), qkv.shape[0], _p(q_weight),
                         _p(k_weight), float(eps), _p(cos), _p(sin), 1 if write_kv else 0, _p(kv), kv.shape[0], _p(out),
                         _p(scratch), scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table), batch.table_width,
                         n_heads, n_kv, float(scale), _p(status_tensor(qkv.device)), _stream(), kernels=2 if mk > 128 else 1)
    return out


# ---------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of each row's maximum (int32 [rows])."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _cuda("out", out, torch.int32, (rows,))
    _core().call("wick_argmax", "ppiip", _p(logits), _p(out), rows, vocab, _stream())
    return out


def sample_temperature(logits: torch.Tensor, temperature: float, uniforms: torch.Tensor,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row from softmax(logits / temperature): the first index whose
    cumulative probability (in index order) reaches uniforms[row] times the total."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _cuda("uniforms", uniforms, torch.float32, (rows,))
    _need(temperature > 0, "temperature must be positive (0 means greedy: use argmax)")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _cuda("out", out, torch.int32, (rows,))
    _core().call("wick_sample_temperature", "pppiifp", _p(logits), _p(uniforms), _p(out), rows, vocab,
                 float(1.0 / temperature), _stream())
    return out


def top_k(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The k largest entries of each row, sorted by value (descending), ties by
    index (ascending): (float32 [rows, k], int32 [rows, k])."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _need(1 <= k <= min(vocab, 1024), f"top_k on the device takes 1 <= k <= min(vocab, 1024), not {k}")
    vals = torch.empty((rows, k), dtype=torch.float32, device=logits.device)
    idx = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
    _core().call("wick_top_k", "pppiiip", _p(logits), _p(vals), _p(idx), rows, vocab, k, _stream())
    return vals, idx


def pick_sorted(vals: torch.Tensor, idx: torch.Tensor, uniforms: torch.Tensor, temperature: float, min_p: float,
                top_p: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row from candidates sorted by logit (descending): the
    probabilities at ``temperature``, the min-p and top-p cuts and the draw with
    the row's uniform number, as ``sampling.sampler.pick_from_sorted`` does them
    on the host (int32 [rows])."""
    _cuda("vals", vals, torch.float32)
    rows, k = vals.shape
    _cuda("idx", idx, torch.int32, (rows, k))
    _cuda("uniforms", uniforms, torch.float32, (rows,))
    _need(temperature > 0.0, "pick_sorted needs a temperature above 0")
    probs = torch.empty_like(vals)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=vals.device)
    _cuda("out", out, torch.int32, (rows,))
    _core().call("wick_pick_sorted", "pppppiifffp", _p(vals), _p(idx), _p(uniforms), _p(probs), _p(out), rows, k,
                 float(temperature), float(min_p), float(top_p), _stream())
    return out


def repetition_penalty(logits: torch.Tensor, histories, penalty: float) -> torch.Tensor:
    """In place: every distinct token of histories[row] has its logit divided by
    ``penalty`` if positive, multiplied otherwise."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _need(len(histories) == rows, "one history per row")
    r, t = [], []
    for i, h in enumerate(histories):
        d = sorted(set(int(x) for x in h))
        r += [i] * len(d)
        t += d
    if not t:
        return logits
    dev = torch.tensor([r, t], dtype=torch.int32).to(logits.device)
    _core().call("wick_repetition_penalty", "pppiifp", _p(logits), _p(dev[0]), _p(dev[1]), len(t), vocab,
                 float(penalty), _stream())
    return logits


# ---------------------------------------------------------------------------
# The per-sequence state record on the device (csrc/state.cu) and the kernels that
# move a batch from one decode step to the next without the host.
SEQ_STATE_WORDS = 8
SEQ_LENGTH, SEQ_NEXT, SEQ_FINISHED, SEQ_GENERATED, SEQ_LIMIT, SEQ_ROW = range(6)


def seq_state_set(state: torch.Tensor, slots: torch.Tensor, values: torch.Tensor) -> None:
    """state[slots[i]] = values[i] (int32 records of SEQ_STATE_WORDS words)."""
    _cuda("state", state, torch.int32)
    n = slots.numel()
    _cuda("slots", slots, torch.int32, (n,))
    _cuda("values", values, torch.int32, (n, SEQ_STATE_WORDS))
    _need(state.dim() == 2 and state.shape[1] == SEQ_STATE_WORDS, "state must be [slots, 8]")
    _core().call("wick_seq_state_set", "pppip", _p(state), _p(slots), _p(values), n, _stream())


def step_prepare(state: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor,
                 start: torch.Tensor, kv_len: torch.Tensor) -> None:
    """The fields of a decode step from the sequences' records: the token sampled last, its
    position, and the cached length before and after the step."""
    n = slots.numel()
    _cuda("state", state, torch.int32)
    for nm, t in (("slots", slots), ("tokens", tokens), ("positions", positions), ("start", start), ("kv_len", kv_len)):
        _cuda(nm, t, torch.int32, (n,))
    _core().call("wick_step_prepare", "ppppppip", _p(state), _p(slots), _p(tokens), _p(positions), _p(start), _p(kv_len),
                 n, _stream())


def step_advance(state: torch.Tensor, slots: torch.Tensor, ids: torch.Tensor, kv_len: torch.Tensor,
                 stops: Optional[torch.Tensor], seen: Optional[torch.Tensor], vocab: int) -> None:
    """After sampling: every running sequence of the step takes its sampled token (ids[i]) as
    its next one and its new length, or is marked finished (a stop token, or its limit).
    ids has one element more than there are rows; it receives the kernels' status word."""
    n = slots.numel()
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32, (n,))
    _cuda("ids", ids, torch.int32, (n + 1,))
    _cuda("kv_len", kv_len, torch.int32, (n,))
    n_stops = 0
    if stops is not None and stops.numel():
        _cuda("stops", stops, torch.int32)
        n_stops = stops.numel()
    if seen is not None:
        _cuda("seen", seen, torch.uint8)
        _need(seen.dim() == 2 and seen.shape[1] == vocab, f"seen must be [rows, {vocab}]")
    _core().call("wick_step_advance", "pppppipipip", _p(state), _p(slots), _p(ids), _p(kv_len),
                 _p(stops) if n_stops else None, n_stops, _p(seen), vocab, _p(status_tensor(state.device)), n, _stream())


def rng_uniforms(rng: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One uniform number in [0, 1) per row from the generator (xoshiro256**, int64 [rows of the
    batch, 4]) of the row's sequence; the generators of running sequences move on."""
    n = slots.numel()
    _cuda("rng", rng, torch.int64)
    _need(rng.dim() == 2 and rng.shape[1] == 4, "rng must be [rows, 4]")
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32, (n,))
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=state.device)
    _cuda("out", out, torch.float32, (n,))
    _core().call("wick_rng_uniforms", "ppppip", _p(rng), _p(state), _p(slots), _p(out), n, _stream())
    return out


def seen_prompt(seen: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor,
                seq_of_token: torch.Tensor) -> None:
    """Mark a prompt step's tokens as seen in their sequences' rows of ``seen`` (uint8 [rows, vocab])."""
    _cuda("seen", seen, torch.uint8)
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32)
    n = tokens.numel()
    _cuda("tokens", tokens, torch.int32, (n,))
    _cuda("seq_of_token", seq_of_token, torch.int32, (n,))
    _core().call("wick_seen_prompt", "pippppip", _p(seen), seen.shape[1], _p(state), _p(slots), _p(tokens),
                 _p(seq_of_token), n, _stream())


def penalty_seen(logits: torch.Tensor, seen: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, penalty: float) -> None:
    """In place: the logit of every token seen in the row's sequence is divided by ``penalty``
    if positive, multiplied otherwise."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _cuda("seen", seen, torch.uint8)
    _need(seen.dim() == 2 and seen.shape[1] == vocab, f"seen must be [rows, {vocab}]")
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32, (rows,))
    _core().call("wick_penalty_seen", "ppippfip", _p(logits), _p(seen), vocab, _p(state), _p(slots), float(penalty), rows,
                 _stream())


def wait_gives_up(limit_ms: float = 1.0) -> bool:
    """Run the kernel whose wait nothing can satisfy (one block, one barrier, no copies): its
    bounded wait gives up after ``limit_ms`` and leaves code 99 in the status word, which
    :func:`check_status` then reports.  Returns whether the wait gave up."""
    st = status_tensor("cuda")
    flag = torch.zeros(1, dtype=torch.int32, device=st.device)
    _core().call("wick_wait_gives_up", "pilpp", _p(st), 99, int(limit_ms * 1e6), _p(flag), _stream())
    return bool(flag.item())
