"""Binding a checkpoint's tensors to a model by name.

Every problem of a checkpoint is collected and reported in ONE error: tensors
the model needs and the files lack, tensors the files carry and the model does
not know, and tensors of the wrong shape (wording after wick
``src/model.rs:137-140,180-183``: "missing tensor NAME", "NAME: expected shape
[r, c], found [...]").  bf16 stays bf16, f16 goes through f32 to bf16, f32 is
rounded to bf16 for matrices of the bfloat16 path and kept for everything the
parts declare as 32-bit (``src/model.rs:64-85,136-142``).
"""
from __future__ import annotations

from typing import List

import torch

from ..models.model import Model
from .safetensors_io import SafeTensorsDir, SafeTensorsError


class WeightError(ValueError):
    """The checkpoint does not fit the model; ``missing``, ``unexpected`` and
    ``wrong_shape`` list the tensor names concerned."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)


_FLOAT_FILE_DTYPES = ("F32", "F16", "BF16")


def check_tensors(model: Model, st: SafeTensorsDir) -> None:
    table = model.tensor_table()
    missing: List[str] = []
    wrong: List[str] = []
    lines: List[str] = []
    for name, ts in table.items():
        info = st.get(name)
        if info is None:
            if not ts.optional:
                missing.append(name)
                lines.append(f"missing tensor {name}")
            continue
        if tuple(info.shape) != tuple(ts.shape):
            wrong.append(name)
            lines.append(f"{name}: expected shape {list(ts.shape)}, found {list(info.shape)}")
        elif ts.role in ("matrix", "vector") and info.dtype_name not in _FLOAT_FILE_DTYPES:
            wrong.append(name)
            lines.append(f"{name}: unsupported dtype {info.dtype_name}")
    unexpected = sorted(n for n in st.names() if n not in table and not model.is_ignored(n))
    lines += [f"unexpected tensor {n}" for n in unexpected]
    if lines:
        head = (f"checkpoint does not fit {model.spec.architecture}: {len(missing)} missing, "
                f"{len(unexpected)} unexpected, {len(wrong)} of the wrong shape or type")
        raise WeightError(head + "\n  " + "\n  ".join(lines), missing, unexpected, wrong)


def load_weights(model: Model, model_dir: str) -> SafeTensorsDir:
    """Check every tensor name and shape, then hand the tensors to the parts."""
    try:
        st = SafeTensorsDir(model_dir)
    except SafeTensorsError as e:
        raise WeightError(str(e)) from None
    check_tensors(model, st)

    def get(name: str):
        info = st.get(name)
        return None if info is None else info.tensor()

    model.load(get)
    return st
