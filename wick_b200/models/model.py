"""A model built from a :class:`ModelSpec`: parts, their tensors, one forward pass.

The class is the same for every architecture: it builds each layer's parts from
the spec through the part registry, knows every tensor's full name (the part's
local name behind the prefixes the spec gives), and runs the layers in the
order of the spec's schedule over one :class:`StepBatch`.
"""
from __future__ import annotations

import fnmatch
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..parts.base import Block, BuildContext, CacheNeed, Hidden, Part, TensorSpec, build_part
from ..parts import standard as _standard_parts   # registers the standard kinds  # noqa: F401
from .spec import ModelSpec


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype {dtype} is not built (bfloat16 or float32)")
        spec.validate()
        self.spec = spec
        self.ctx = BuildContext(dtype=dtype, device=torch.device(device))
        ctx = self.ctx
        self.embedding = build_part("embedding", spec.embedding, ctx)
        self.blocks: List[Block] = []
        for ls in spec.layers:
            mixer = build_part("mixer", ls.mixer, ctx)
            mixer_norm = build_part("norm", ls.mixer_norm, ctx)
            ffn = build_part("ffn", ls.ffn, ctx)
            ffn_norm = build_part("norm", ls.ffn_norm, ctx)
            self.blocks.append(build_part("block", ls.block, ctx, mixer, mixer_norm, ffn, ffn_norm))
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        self.head = build_part("head", spec.head, ctx)
        named = {"embedding": self.embedding, "final_norm": self.final_norm, "head": self.head}
        for _, part in self._places():
            if part.PEERS:
                part.attach({k: named[k] for k in part.PEERS})
        self.loaded = False

    # ---- tensors ---------------------------------------------------------
    def _places(self) -> List[Tuple[str, Part]]:
        s = self.spec
        out: List[Tuple[str, Part]] = [(s.embedding_prefix, self.embedding)]
        for ls, blk in zip(s.layers, self.blocks):
            out += [(ls.prefix + ls.names["mixer_norm"], blk.mixer_norm),
                    (ls.prefix + ls.names["mixer"], blk.mixer),
                    (ls.prefix + ls.names["ffn_norm"], blk.ffn_norm),
                    (ls.prefix + ls.names["ffn"], blk.ffn)]
        out += [(s.final_norm_prefix, self.final_norm), (s.head_prefix, self.head)]
        return out

    def tensor_table(self) -> Dict[str, TensorSpec]:
        """Full tensor name -> what is expected under it."""
        table: Dict[str, TensorSpec] = {}
        for prefix, part in self._places():
            for ts in part.tensor_specs():
                table[prefix + ts.name] = ts
        return table

    def tensor(self, name: str) -> torch.Tensor:
        """The loaded tensor of this full name, in the layout a checkpoint stores it in
        (fused matrices split again, tiled ones put back row by row)."""
        for prefix, part in self._places():
            if name.startswith(prefix):
                t = part.tensor(name[len(prefix):])
                if t is not None:
                    return t
        raise KeyError(f"the model holds no tensor {name!r}")

    def tensors(self) -> Dict[str, torch.Tensor]:
        """Every loaded tensor by its full name (see :meth:`tensor`); absent optional ones
        (a tied head) are left out."""
        out: Dict[str, torch.Tensor] = {}
        for prefix, part in self._places():
            for ts in part.tensor_specs():
                t = part.tensor(ts.name)
                if t is not None:
                    out[prefix + ts.name] = t
        return out

    def is_ignored(self, name: str) -> bool:
        return any(fnmatch.fnmatchcase(name, pat) for pat in self.spec.ignore_tensors)

    def load(self, get: Callable[[str], Optional[torch.Tensor]]) -> None:
        """``get(full_name)`` returns a tensor (any device) or None.  Parts load in the order
        embedding, layers, final norm, head."""
        for prefix, part in self._places():
            part.load((lambda p: (lambda local: get(p + local)))(prefix))
        self.loaded = True

    # ---- sizes -------------------------------------------------------------
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """For each schedule entry, the cache storage it owns (None if it reads
        another entry's or its mixer keeps nothing)."""
        needs: List[Optional[CacheNeed]] = []
        for e in self.spec.schedule:
            needs.append(None if e.read_cache_of is not None else self.blocks[e.layer].mixer.cache_need())
        return needs

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads (each schedule entry reads its layer's)."""
        n = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for e in self.spec.schedule:
            b = self.blocks[e.layer]
            n += b.mixer.weight_bytes() + b.ffn.weight_bytes() + b.mixer_norm.weight_bytes() + b.ffn_norm.weight_bytes()
        return n

    def prompt_capturable(self) -> bool:
        """Whether every part reads a prompt step's shape from the device only, so that a
        captured prompt step can be replayed for other prompts of the same padded size."""
        parts: List[Part] = [self.embedding, self.final_norm, self.head]
        for b in self.blocks:
            parts += [b, b.mixer, b.mixer_norm, b.ffn, b.ffn_norm]
        return all(p.PROMPT_CAPTURABLE for p in parts)

    # ---- forward -------------------------------------------------------------
    def forward(self, batch, cache) -> torch.Tensor:
        """Run the batch's tokens through every scheduled layer, appending to the
        cache, and return float32 logits [len(batch.want), vocab]."""
        if not self.loaded:
            raise RuntimeError("the model has no weights yet")
        h = Hidden(self.embedding.forward(batch.tokens))
        for i, e in enumerate(self.spec.schedule):
            src = i if e.read_cache_of is None else e.read_cache_of
            h = self.blocks[e.layer].forward(h, batch, cache.view(src, batch), e.read_cache_of is None)
        if batch.n_want == 0:
            return torch.empty((0, self.spec.vocab), dtype=torch.float32, device=self.ctx.device)
        if h.pending is not None:
            xn = self.final_norm.add_forward(h.x, h.pending, self.ctx.dtype, batch.want)
        else:
            xn = self.final_norm.forward(h.x, self.ctx.dtype, batch.want)
        return self.head.forward(xn)
