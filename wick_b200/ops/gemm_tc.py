"""Tensor-core (tcgen05) matrix products for bfloat16 weights."""
from __future__ import annotations

from typing import Optional

import torch


def plan_for(weight: torch.Tensor, gated: bool = False):
    """A plan object with ``forward`` / ``forward_delta`` for this weight, or
    None where the tensor-core kernels do not take its sizes."""
    return None
