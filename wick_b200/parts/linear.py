"""A weight matrix [out, in] and its product with activations, y = x W^T.

This is the one place that chooses a matrix-product kernel: the tensor-core
kernels for bfloat16 when they take the sizes at hand, the CUDA-core float32
kernel for the 32-bit path (and as the plain form of the former).  Several
tensors that share an input (q/k/v, gate/up) are held as one matrix, rows
concatenated in the order given.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch

from .. import ops
from .base import BuildContext


class Linear:
    def __init__(self, out_features: int, in_features: int, ctx: BuildContext, gated: bool = False):
        self.out_features, self.in_features, self.ctx, self.gated = out_features, in_features, ctx, gated
        self.weight: Optional[torch.Tensor] = None
        self._tc = None

    # ---- weights ----
    def load_rows(self, parts: Sequence[torch.Tensor]) -> None:
        held = [self.ctx.hold(p, "matrix") for p in parts]
        w = held[0] if len(held) == 1 else torch.cat(held, dim=0)
        del held
        self.use(w)

    def use(self, w: torch.Tensor) -> None:
        if tuple(w.shape) != (self.out_features, self.in_features):
            raise ValueError(f"weight of shape {tuple(w.shape)} given, "
                             f"[{self.out_features}, {self.in_features}] expected")
        self.weight = w.contiguous()
        self._tc = None
        if self.ctx.dtype == torch.bfloat16 and self._tensor_core() is not None:
            self.weight = None                 # the plan holds the matrix in its packed form

    def rows(self, start: int, stop: int) -> torch.Tensor:
        """Rows ``start..stop`` of the matrix as it was loaded, [stop - start, in] row-major,
        whatever form it is held in."""
        w = self.weight if self.weight is not None else self._tc.matrix()
        return w[start:stop].contiguous()

    def weight_bytes(self) -> int:
        return self.out_features * self.in_features * (2 if self.ctx.dtype == torch.bfloat16 else 4)

    # ---- products ----
    def _tensor_core(self):
        """The tensor-core plan of this matrix, or None where it does not apply."""
        if self._tc is None:
            from ..ops import gemm_tc
            self._tc = (not ops.plain_kernels() and gemm_tc.plan_for(self.weight, gated=self.gated)) or False
        return self._tc or None

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """[n, in] -> [n, out] (or [n, out/2] for a gated pair) in ``out_dtype``."""
        if self.ctx.dtype == torch.bfloat16:
            tc = self._tensor_core()
            if tc is not None:
                return tc.forward(x, out_dtype)
        return ops.gemm_simt(x, self.weight, out_dtype, gated=self.gated)

    def forward_delta(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """[n, in] -> float32 [splits, n, out]: partial sums over slices of the
        inner dimension, to be added up (in index order) by whoever consumes them.
        With ``residual`` (float32 [n, out]) the product may instead be added to it
        by the kernel itself (each element by one thread); then None is returned."""
        if self.ctx.dtype == torch.bfloat16:
            tc = self._tensor_core()
            if tc is not None:
                if residual is not None and tc.forward_add(x, residual):
                    return None
                return tc.forward_delta(x)
        return ops.gemm_simt(x, self.weight, torch.float32).unsqueeze(0)
