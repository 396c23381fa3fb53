"""The interfaces of the parts a layer is put together from, and their registry.

Categories: ``mixer`` (token mixing over the sequence: attention here),
``ffn`` (feed-forward), ``norm``, ``position`` (position encoding), ``block``
(the arrangement of the former in one layer), ``embedding`` and ``head``.

A part is built from a :class:`~wick_b200.models.spec.PartSpec` — its registered
kind plus its sizes and constants — and a :class:`BuildContext` (compute dtype
and device).  It declares the tensors it needs by local name, receives them
through :meth:`Part.load`, and computes with the kernels of ``wick_b200.ops``.
No part knows which model it is in, which layer it is, or what its neighbours
are: everything it needs is in its parameters and in the arguments of
``forward``.

Adding a part: subclass the category's base class, implement its methods,
and call :func:`register_part` with a new kind name; a model spec can then
name that kind.  Nothing else in the package has to change.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..models.spec import PartSpec

CATEGORIES = ("mixer", "ffn", "norm", "position", "block", "embedding", "head")


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs.  ``role`` decides how it is held:
    ``matrix``: in the compute dtype (bfloat16 or float32);
    ``vector``: always float32 (norm weights and the like: tensors that a
    checkpoint stores in 32-bit stay 32-bit, and 16-bit vectors are widened
    exactly, as wick does for every 1-D tensor, model.rs:136-142);
    ``table``: integers, as int32."""

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclasses.dataclass(frozen=True)
class BuildContext:
    dtype: torch.dtype            # torch.bfloat16 or torch.float32
    device: torch.device

    def hold(self, t: torch.Tensor, role: str) -> torch.Tensor:
        """Move a loaded tensor to the device in the dtype its role asks for."""
        if role == "matrix":
            dt = self.dtype
        elif role == "vector":
            dt = torch.float32
        elif role == "table":
            dt = torch.int32
        else:
            raise ValueError(f"unknown tensor role {role}")
        if t.dtype == torch.float16 and dt == torch.bfloat16:
            t = t.to(torch.float32)          # f16 -> f32 -> bf16, round to nearest even (model.rs:67-71)
        return t.to(device=self.device, dtype=dt).contiguous()


Fetch = Callable[[str], Optional[torch.Tensor]]


@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the cache for one schedule entry.

    kind ``paged_kv``: keys and values of every position, ``kv_heads`` x
    ``head_dim`` each, in pages; ``window`` (tokens) if only the last ones are
    ever read.  kind ``state``: one record of fixed ``shape`` and ``dtype`` per
    sequence, zeroed when the sequence starts."""

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    shape: Tuple[int, ...] = ()
    dtype: Optional[torch.dtype] = None   # None: the compute dtype


class Part:
    category = ""
    # Other places of the model whose part this one needs to see ("embedding", "final_norm",
    # "head"): the model hands them over through :meth:`attach` before any weight is loaded.
    # (An output head that shares the embedding table names "embedding".)
    PEERS: Tuple[str, ...] = ()
    # True if a prompt step of this part reads the step's shape (which token belongs to which
    # sequence, lengths, positions, pages) from the batch's DEVICE arrays only and sizes its
    # launches by ``batch.n_tokens``, ``batch.n_seqs`` and ``batch.q_tiles`` alone.  The engine
    # captures prompt steps of padded sizes and replays them for other prompts only if every
    # part of the model says so; the host lists of such a captured batch (``q_lens``,
    # ``starts``) describe no real prompt.
    PROMPT_CAPTURABLE = False

    def __init__(self, params: Mapping[str, Any], ctx: BuildContext):
        self.params = dict(params)
        self.ctx = ctx

    def attach(self, peers: Mapping[str, "Part"]) -> None:
        """Receive the parts named in ``PEERS`` (place -> part)."""

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, fetch: Fetch) -> None:
        """Take the tensors named by :meth:`tensor_specs` (``fetch(local_name)``
        returns a tensor of the declared shape, or None for an absent optional
        one) and keep them on the device."""

    def tensor(self, name: str) -> Optional[torch.Tensor]:
        """The tensor held under the local ``name``, in the shape and layout a checkpoint
        stores it in (on the device, in the dtype it is held in), however the part keeps
        it for its kernels; None if the part holds none of that name.  For handing a
        model's weights to another implementation."""
        return None

    def weight_bytes(self) -> int:
        """Bytes of weights one forward pass of this part reads."""
        return 0


class Norm(Part):
    category = "norm"

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normalise the float32 rows of ``x`` [n, width] (only ``rows`` of
        them, if given) into a new [n or len(rows), width] tensor."""
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x += sum(delta)`` in float32 and in place (``delta`` is
        [splits, n, width], summed in index order), then normalise.  With
        ``rows`` only those rows are normalised and ``x`` need not be brought up
        to date (nobody reads it afterwards)."""
        x.add_(delta.sum(0) if delta.shape[0] > 1 else delta[0])
        return self.forward(x, out_dtype, rows)


class Position(Part):
    category = "position"

    def rotary_inv_freq(self) -> Optional[torch.Tensor]:
        """If this encoding is a half-split rotation of whole heads by
        ``position * inv_freq[i]``, the float32 table [head_dim/2] (kernels then
        fuse it); otherwise None and :meth:`apply` is called."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode positions into q [n, heads, d] and k [n, kv_heads, d] in place."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, x: torch.Tensor, batch: "Any", cache: "Any", write_cache: bool) -> torch.Tensor:
        """x: [tokens, width] in the compute dtype (already normalised).
        batch: the step's :class:`~wick_b200.engine.batch.StepBatch`.
        cache: the view of this schedule entry's cache storage for this batch
        (None if :meth:`cache_need` is None).  write_cache is False when the
        entry reads an earlier entry's cache.
        Returns float32 [splits, tokens, width], to be summed into the residual.

        A mixer (or feed-forward) whose class sets ``ADDS_TO_RESIDUAL = True`` is
        also given ``residual=`` (the float32 residual stream [tokens, width]); it
        may add its result to it itself (each element once, in a fixed order) and
        return None."""
        raise NotImplementedError


class FeedForward(Part):
    category = "ffn"

    def forward(self, x: torch.Tensor, batch: "Any") -> torch.Tensor:
        """x: [tokens, width], compute dtype.  Returns float32 [splits, tokens, width]."""
        raise NotImplementedError


class Hidden:
    """The residual stream between blocks: float32 ``x`` [tokens, width] and a
    float32 ``pending`` [splits, tokens, width] that has still to be added to it
    (kept apart so that the next norm's kernel can do the addition)."""

    __slots__ = ("x", "pending")

    def __init__(self, x: torch.Tensor, pending: Optional[torch.Tensor] = None):
        self.x, self.pending = x, pending

    def resolved(self) -> torch.Tensor:
        if self.pending is not None:
            p = self.pending
            self.x.add_(p.sum(0) if p.shape[0] > 1 else p[0])
            self.pending = None
        return self.x


class Block(Part):
    category = "block"

    def __init__(self, params, ctx, mixer: Mixer, mixer_norm: Norm, ffn: FeedForward, ffn_norm: Norm):
        super().__init__(params, ctx)
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = mixer, mixer_norm, ffn, ffn_norm

    def forward(self, h: Hidden, batch: "Any", cache: "Any", write_cache: bool) -> Hidden:
        raise NotImplementedError


class Embedding(Part):
    category = "embedding"

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """int32 [n] -> float32 [n, width]."""
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[n, width] in the compute dtype -> float32 logits [n, vocab]."""
        raise NotImplementedError


_PARTS: Dict[str, Dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type) -> type:
    if category not in _PARTS:
        raise ValueError(f"unknown part category {category}")
    _PARTS[category][kind] = cls
    return cls


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[category][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(category, {})))
        raise KeyError(f"no {category} part of kind {kind!r} is registered (known: {known})") from None


def build_part(category: str, spec: PartSpec, ctx: BuildContext, *args) -> Part:
    return part_class(category, spec.kind)(spec.params, ctx, *args)


def as_splits(delta: torch.Tensor) -> torch.Tensor:
    """A part may return [tokens, width]; the residual path wants [splits, tokens, width]."""
    return delta if delta.dim() == 3 else delta.unsqueeze(0)
