"""Random weights for a configuration.

``write_random_model`` writes a model folder (``config.json`` and
``model.safetensors``) from a configuration and a seed; the folder loads like
any checkpoint.  ``random_fetch`` produces the same kind of tensors directly
on a device, for sizes that are not worth a round trip through a file.

Matrices are N(0, std) and vectors (norm weights) 1 + N(0, vector_std), each
tensor from a generator seeded by (seed, tensor name) so that a tensor's values
do not depend on which other tensors exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict, Optional

import torch

from ..config.base import ModelConfig, get_architecture
from ..models.model import Model
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _make(name: str, ts, seed: int, device, dtype: torch.dtype, std: float, vector_std: float) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    if ts.role == "table":
        raise ValueError(f"{name}: no random rule for an integer table")
    t = torch.randn(ts.shape, generator=g, device=device, dtype=torch.float32)
    if ts.role == "vector":
        t = 1.0 + vector_std * t
    else:
        t = std * t
    return t.to(dtype)


def random_fetch(model: Model, seed: int, *, std: float = 0.02, vector_std: float = 0.1,
                 tied: Optional[bool] = None) -> Callable[[str], Optional[torch.Tensor]]:
    """A ``get(name)`` for :meth:`Model.load` that draws each tensor on the
    model's device.  Optional tensors (an untied head) are drawn unless the
    model's spec ties them."""
    table = model.tensor_table()
    dev = model.ctx.device
    store_dtype = model.ctx.dtype

    def get(name: str):
        ts = table.get(name)
        if ts is None:
            return None
        if ts.optional and getattr(model.head, "tied", False):
            return None
        return _make(name, ts, seed, dev, torch.float32 if ts.role == "vector" else store_dtype, std, vector_std)

    return get


def write_random_model(config: ModelConfig, seed: int, out_dir: str, *, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02, vector_std: float = 0.1) -> str:
    """Write ``config.json`` and ``model.safetensors`` under ``out_dir``."""
    arch = get_architecture(config.architecture)
    model = Model(arch.build_spec(config), torch.float32, "cpu")
    tensors: Dict[str, torch.Tensor] = {}
    for name, ts in model.tensor_table().items():
        if ts.optional and getattr(model.head, "tied", False):
            continue
        tensors[name] = _make(name, ts, seed, "cpu", dtype, std, vector_std)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_json(), f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    return out_dir
