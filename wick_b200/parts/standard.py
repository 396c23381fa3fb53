"""The parts the Qwen3 dense decoder is put together from.

Each class takes its sizes and constants from ``params`` and nothing else:

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
norm           ``rms``                 width, eps
position       ``rotary_half_split``   head_dim, theta
position       ``none``                —
mixer          ``gqa_attention``       width, heads, kv_heads, head_dim,
                                       qk_norm (PartSpec or None),
                                       position (PartSpec), scale (or None)
ffn            ``gated_mlp``           width, intermediate, activation ("silu")
block          ``prenorm_residual``    —
embedding      ``table``               vocab, width
head           ``linear``              vocab, width, tied
=============  ======================  ==========================================

Formulas and their place in wick: RMS norm ``src/kernels.rs:343-357``; rotation
``src/model.rs:404-414`` with ``inv_freq`` from ``src/config.rs:162-167``;
attention ``src/model.rs:452-487,520-553``; SwiGLU MLP ``src/model.rs:490-503``;
output head ``src/model.rs:508-515`` with the tie rule of ``src/model.rs:190``.
"""
from __future__ import annotations

import math
from typing import Any, List, Mapping, Optional

import torch

from .. import ops
from ..models.spec import PartSpec
from .base import (Block, BuildContext, CacheNeed, Embedding, FeedForward, Fetch, Head, Hidden, Mixer,
                   Norm, Part, Position, TensorSpec, as_splits, build_part, register_part)
from .linear import Linear


# ---------------------------------------------------------------------------
class RMSNorm(Norm):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self):
        return [TensorSpec("weight", (self.width,), "vector")]

    def load(self, fetch):
        self.weight = self.ctx.hold(fetch("weight"), "vector")

    def tensor(self, name):
        return self.weight if name == "weight" else None

    def forward(self, x, out_dtype, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, rows=rows)

    def add_forward(self, x, delta, out_dtype, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, delta=delta, rows=rows)

    def weight_bytes(self):
        return self.width * 4


# ---------------------------------------------------------------------------
class RotaryHalfSplit(Position):
    """Whole-head rotation of the pairs (i, i + head_dim/2) by the angle
    ``position * inv_freq[i]`` with ``inv_freq[i] = theta ** (-2i / head_dim)``,
    evaluated in float64 and rounded to float32 once."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        d = self.head_dim
        inv = [1.0 / (self.theta ** (2.0 * i / d)) for i in range(d // 2)]
        self.inv_freq = torch.tensor(inv, dtype=torch.float64).to(torch.float32).to(ctx.device)

    def rotary_inv_freq(self):
        return self.inv_freq

    def tables(self, batch):
        """cos/sin [tokens, head_dim/2] of this step, computed once and shared by
        every layer that uses an equal encoding."""
        key = ("rotary_half_split", self.head_dim, self.theta)
        t = batch.memo.get(key)
        if t is None:
            t = batch.memo[key] = ops.rope_table(batch.positions, self.inv_freq)
        return t


class NoPosition(Position):
    PROMPT_CAPTURABLE = True

    def rotary_inv_freq(self):
        return None

    def apply(self, q, k, positions):
        return None


# ---------------------------------------------------------------------------
class GQAttention(Mixer):
    """Causal attention with grouped key/value heads over a paged cache.

    q, k, v = x Wq^T, x Wk^T, x Wv^T (no bias); optional per-head norm of q and k
    (one weight vector shared by all heads) before the position encoding; k and v
    are appended to the cache; every new token attends to positions 0..its own;
    the result goes through Wo.  The three projections are held as one matrix.
    """

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.heads, self.kv_heads, self.head_dim = (int(p["width"]), int(p["heads"]),
                                                                int(p["kv_heads"]), int(p["head_dim"]))
        if self.heads % self.kv_heads != 0:
            raise ValueError("heads must be a multiple of kv_heads")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"the attention kernels take a head_dim that is a multiple of 16 between 16 and 256, "
                             f"not {self.head_dim}")
        self.q_dim, self.kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = p.get("window")
        if self.window is not None:
            raise ValueError("windowed attention is not built")
        qk = p.get("qk_norm")
        self.q_norm = build_part("norm", qk, ctx) if qk is not None else None
        self.k_norm = build_part("norm", qk, ctx) if qk is not None else None
        if qk is not None and not isinstance(self.q_norm, RMSNorm):
            raise ValueError("the fused q/k norm kernel is an RMS norm; another norm needs its own kernel")
        self.position = build_part("position", p.get("position") or PartSpec("none"), ctx)
        self.PROMPT_CAPTURABLE = bool(self.position.PROMPT_CAPTURABLE)   # (its own kernels read the step from the device)
        self.qkv = Linear(self.q_dim + 2 * self.kv_dim, self.width, ctx)
        self.o = Linear(self.width, self.q_dim, ctx)

    def tensor_specs(self):
        specs = [TensorSpec("q_proj.weight", (self.q_dim, self.width)),
                 TensorSpec("k_proj.weight", (self.kv_dim, self.width)),
                 TensorSpec("v_proj.weight", (self.kv_dim, self.width)),
                 TensorSpec("o_proj.weight", (self.width, self.q_dim))]
        if self.q_norm is not None:
            specs += [TensorSpec("q_norm." + s.name, s.shape, s.role) for s in self.q_norm.tensor_specs()]
            specs += [TensorSpec("k_norm." + s.name, s.shape, s.role) for s in self.k_norm.tensor_specs()]
        return specs

    def load(self, fetch):
        self.qkv.load_rows([fetch("q_proj.weight"), fetch("k_proj.weight"), fetch("v_proj.weight")])
        self.o.load_rows([fetch("o_proj.weight")])
        if self.q_norm is not None:
            self.q_norm.load(lambda n: fetch("q_norm." + n))
            self.k_norm.load(lambda n: fetch("k_norm." + n))

    def tensor(self, name):
        q, kv = self.q_dim, self.kv_dim
        if name in ("q_proj.weight", "k_proj.weight", "v_proj.weight"):
            lo, hi = {"q": (0, q), "k": (q, q + kv), "v": (q + kv, q + 2 * kv)}[name[0]]
            return self.qkv.rows(lo, hi)
        if name == "o_proj.weight":
            return self.o.rows(0, self.width)
        for prefix, norm in (("q_norm.", self.q_norm), ("k_norm.", self.k_norm)):
            if name.startswith(prefix) and norm is not None:
                return norm.tensor(name[len(prefix):])
        return None

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.o.weight_bytes() + (2 * self.head_dim * 4 if self.q_norm else 0)

    ADDS_TO_RESIDUAL = True

    def forward(self, x, batch, cache, write_cache, residual=None):
        inv_freq = self.position.rotary_inv_freq()
        if inv_freq is None and not isinstance(self.position, NoPosition):
            q = self._encode_unfused(x, batch, cache, write_cache)
        else:
            qkv = self.qkv.forward_delta(x)              # float32 partial sums [splits, n, q_dim + 2 kv_dim]
            cos = sin = None
            if inv_freq is not None:
                cos, sin = self.position.tables(batch)
            if batch.is_decode and qkv.shape[0] <= 8 and not ops.plain_kernels() and ops.attention_decode_parts_supported(
                    batch.n_seqs, self.heads, self.kv_heads, self.head_dim, self.ctx.dtype):
                # the tensor-core decode attention: the projection's sums, the q/k norm, the rotation,
                # the cache append, the attention and the merge in one or two launches
                need = ops.attention_decode_parts_scratch(batch.n_seqs, self.heads, self.kv_heads, self.head_dim, batch.kv_bound)
                att = ops.attention_decode_parts_fused(
                    qkv, self.heads, self.kv_heads, self.head_dim, q_weight=self.q_norm.weight if self.q_norm else None,
                    k_weight=self.k_norm.weight if self.k_norm else None, eps=self.q_norm.eps if self.q_norm else 0.0,
                    cos=cos, sin=sin, kv=cache.kv, batch=batch, scale=self.scale,
                    scratch=batch.workspace.get("attention_decode_parts", need, torch.float32), write_kv=write_cache,
                    max_kv_len=batch.kv_bound)
                return self.o.forward_delta(att.view(batch.n_tokens, self.q_dim), residual)
            q = ops.qk_norm_rope_append(
                qkv, self.heads, self.kv_heads, self.head_dim,
                q_weight=self.q_norm.weight if self.q_norm else None,
                k_weight=self.k_norm.weight if self.k_norm else None,
                eps=self.q_norm.eps if self.q_norm else 0.0,
                cos=cos, sin=sin, kv=cache.kv, page_table=batch.page_table,
                seq_of_token=batch.seq_of_token, positions=batch.positions, write_kv=write_cache,
                dtype=self.ctx.dtype)
        if batch.is_decode:
            need = ops.attention_decode_scratch_floats(batch.n_seqs, self.heads, self.head_dim, batch.kv_bound,
                                                       self.ctx.dtype)
            att = ops.attention_decode(q, cache.kv, batch, self.scale,
                                       batch.workspace.get("attention_decode", need, torch.float32),
                                       max_kv_len=batch.kv_bound)
        else:
            att = ops.attention_prompt(q, cache.kv, batch, self.scale)
        return self.o.forward_delta(att.view(batch.n_tokens, self.q_dim), residual)


    def _encode_unfused(self, x, batch, cache, write_cache):
        """The way for a position encoding that the fused kernel does not know:
        project, norm q and k per head, let the encoding's own ``apply`` work on
        float32 q [n, heads, d] and k [n, kv_heads, d], then append k and v to the
        cache.  Slower than the fused kernel by a few copies."""
        n = x.shape[0]
        qkv = self.qkv.forward(x, torch.float32)
        q = qkv[:, :self.q_dim].reshape(n * self.heads, self.head_dim)
        k = qkv[:, self.q_dim:self.q_dim + self.kv_dim].reshape(n * self.kv_heads, self.head_dim)
        v = qkv[:, self.q_dim + self.kv_dim:]
        if self.q_norm is not None:
            q = self.q_norm.forward(q, torch.float32)
            k = self.k_norm.forward(k, torch.float32)
        q, k = q.view(n, self.heads, self.head_dim), k.view(n, self.kv_heads, self.head_dim)
        self.position.apply(q, k, batch.positions)
        encoded = torch.cat([q.view(n, -1), k.view(n, -1), v], dim=1).to(self.ctx.dtype)
        return ops.qk_norm_rope_append(
            encoded, self.heads, self.kv_heads, self.head_dim, q_weight=None, k_weight=None, eps=0.0, cos=None,
            sin=None, kv=cache.kv, page_table=batch.page_table, seq_of_token=batch.seq_of_token,
            positions=batch.positions, write_kv=write_cache)


# ---------------------------------------------------------------------------
class GatedMLP(FeedForward):
    """down( act(x gate^T) * (x up^T) ), no biases; gate and up are one matrix."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.intermediate = int(params["width"]), int(params["intermediate"])
        act = params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"unsupported activation {act}")
        self.gate_up = Linear(2 * self.intermediate, self.width, ctx, gated=True)
        self.down = Linear(self.width, self.intermediate, ctx)

    def tensor_specs(self):
        return [TensorSpec("gate_proj.weight", (self.intermediate, self.width)),
                TensorSpec("up_proj.weight", (self.intermediate, self.width)),
                TensorSpec("down_proj.weight", (self.width, self.intermediate))]

    def load(self, fetch):
        self.gate_up.load_rows([fetch("gate_proj.weight"), fetch("up_proj.weight")])
        self.down.load_rows([fetch("down_proj.weight")])

    def tensor(self, name):
        i = self.intermediate
        if name == "gate_proj.weight":
            return self.gate_up.rows(0, i)
        if name == "up_proj.weight":
            return self.gate_up.rows(i, 2 * i)
        return self.down.rows(0, self.width) if name == "down_proj.weight" else None

    def weight_bytes(self):
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    ADDS_TO_RESIDUAL = True

    def forward(self, x, batch, residual=None):
        act = self.gate_up.forward(x, self.ctx.dtype)                   # [n, intermediate]
        return self.down.forward_delta(act, residual)


# ---------------------------------------------------------------------------
class PreNormResidual(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x)).  An addition is either left pending,
    so that the following norm's kernel performs it, or done by the part itself: a
    part whose class says ``ADDS_TO_RESIDUAL`` is handed the residual stream and
    returns None when it has added its result to it (its last kernel did)."""

    PROMPT_CAPTURABLE = True

    def forward(self, h, batch, cache, write_cache):
        dt = self.ctx.dtype
        if h.pending is not None:
            xn = self.mixer_norm.add_forward(h.x, h.pending, dt)
        else:
            xn = self.mixer_norm.forward(h.x, dt)
        if getattr(self.mixer, "ADDS_TO_RESIDUAL", False):
            d = self.mixer.forward(xn, batch, cache, write_cache, residual=h.x)
        else:
            d = self.mixer.forward(xn, batch, cache, write_cache)
        xn = self.ffn_norm.forward(h.x, dt) if d is None else self.ffn_norm.add_forward(h.x, as_splits(d), dt)
        if getattr(self.ffn, "ADDS_TO_RESIDUAL", False):
            d = self.ffn.forward(xn, batch, residual=h.x)
        else:
            d = self.ffn.forward(xn, batch)
        h.pending = None if d is None else as_splits(d)
        return h


# ---------------------------------------------------------------------------
class TableEmbedding(Embedding):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self):
        return [TensorSpec("weight", (self.vocab, self.width))]

    def load(self, fetch):
        self.weight = self.ctx.hold(fetch("weight"), "matrix")

    def tensor(self, name):
        return self.weight if name == "weight" else None

    def forward(self, tokens):
        return ops.embed(self.weight, tokens)

    def weight_bytes(self):
        return 0            # a step reads one row per token, not the table


class LinearHead(Head):
    """logits = x W^T in float32.  ``tied``: W is the embedding table.  As in wick
    (model.rs:190) the head is also tied when its own tensor is absent."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])
        self.tied = bool(params.get("tied", False))
        self.linear = Linear(self.vocab, self.width, ctx)
        self.is_tied = self.tied
        self.embedding: Optional[Embedding] = None

    PEERS = ("embedding",)

    def attach(self, peers):
        self.embedding = peers.get("embedding")

    def tensor_specs(self):
        return [TensorSpec("weight", (self.vocab, self.width), optional=True)]

    def load(self, fetch):
        w = None if self.tied else fetch("weight")
        if w is None:
            table = self.embedding.tensor("weight") if self.embedding is not None else None
            if table is None:
                raise ValueError("a tied head needs the embedding table (loaded before it)")
            self.linear.use(table)
            self.is_tied = True
        else:
            self.linear.load_rows([w])
            self.is_tied = False

    def tensor(self, name):
        return self.linear.rows(0, self.vocab) if name == "weight" and not self.is_tied else None

    def forward(self, x):
        return self.linear.forward(x, torch.float32)

    def weight_bytes(self):
        return self.linear.weight_bytes()


register_part("norm", "rms", RMSNorm)
register_part("position", "rotary_half_split", RotaryHalfSplit)
register_part("position", "none", NoPosition)
register_part("mixer", "gqa_attention", GQAttention)
register_part("ffn", "gated_mlp", GatedMLP)
register_part("block", "prenorm_residual", PreNormResidual)
register_part("embedding", "table", TableEmbedding)
register_part("head", "linear", LinearHead)
