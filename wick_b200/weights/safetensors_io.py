"""Reading and writing safetensors files.

The format (wick ``src/safetensors.rs:81-119``): an 8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw
tensor bytes.  ``__metadata__`` is skipped (``:94``); a header longer than the
file or than 100 MiB is refused (``:86``); every byte range must equal
``numel * itemsize`` (``:112-114``).  A directory holds either one
``model.safetensors`` or the shards named by ``model.safetensors.index.json``'s
``weight_map`` (``:56-74``).

Files are memory-mapped; a tensor is handed out as a torch view of the mapping
(no copy) and is copied once, by the caller, to where it is used.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Sequence, Tuple

import numpy as np
import torch


class SafeTensorsError(ValueError):
    pass


# dtype name -> (torch dtype, numpy carrier dtype, item size)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I64": (torch.int64, np.dtype("<i8"), 8),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.int32: "I32", torch.int64: "I64"}

_MAX_HEADER = 100 << 20


class TensorInfo:
    __slots__ = ("name", "dtype_name", "shape", "_buf", "_begin", "_end")

    def __init__(self, name: str, dtype_name: str, shape: Tuple[int, ...], buf, begin: int, end: int):
        self.name, self.dtype_name, self.shape = name, dtype_name, shape
        self._buf, self._begin, self._end = buf, begin, end

    @property
    def dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype_name][0]

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def tensor(self) -> torch.Tensor:
        """A read-only view of the file's bytes as a torch tensor."""
        tdt, ndt, _ = _DTYPES[self.dtype_name]
        arr = np.frombuffer(self._buf, dtype=ndt, count=self.numel, offset=self._begin)
        # torch warns about non-writable arrays; the view is never written to.
        arr = arr.reshape(self.shape)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.from_numpy(arr)
        if self.dtype_name == "BF16":
            t = t.view(torch.bfloat16)
        return t


class SafeTensorsFile:
    """One memory-mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        try:
            with open(path, "rb") as f:
                size = os.fstat(f.fileno()).st_size
                if size < 8:
                    raise SafeTensorsError(f"{path}: file too short")
                self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        except OSError as e:
            raise SafeTensorsError(f"{path}: {e.strerror or e}") from None
        try:
            self.tensors = self._parse(size)
        except SafeTensorsError as e:
            raise SafeTensorsError(f"{path}: {e}") from None

    def _parse(self, size: int) -> Dict[str, TensorInfo]:
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > size - 8 or hlen > _MAX_HEADER:
            raise SafeTensorsError("bad header length")
        try:
            header = json.loads(bytes(self._map[8:8 + hlen]).decode("utf-8"))
        except UnicodeDecodeError:
            raise SafeTensorsError("header is not UTF-8") from None
        except json.JSONDecodeError as e:
            raise SafeTensorsError(str(e)) from None
        if not isinstance(header, dict):
            raise SafeTensorsError("header is not an object")
        base = 8 + hlen
        out: Dict[str, TensorInfo] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(info, dict):
                raise SafeTensorsError(f"{name}: bad entry")
            dt = info.get("dtype")
            if not isinstance(dt, str):
                raise SafeTensorsError("missing dtype")
            if dt not in _DTYPES:
                raise SafeTensorsError(f"{name}: unsupported dtype {dt}")
            shape = info.get("shape")
            if not isinstance(shape, list) or not all(isinstance(d, int) and d >= 0 for d in shape):
                raise SafeTensorsError("missing shape")
            offs = info.get("data_offsets")
            if (not isinstance(offs, list) or len(offs) != 2
                    or not all(isinstance(o, int) and o >= 0 for o in offs)):
                raise SafeTensorsError("bad data_offsets")
            begin, end = offs
            numel = 1
            for d in shape:
                numel *= d
            if end < begin or base + end > size or end - begin != numel * _DTYPES[dt][2]:
                raise SafeTensorsError(f"{name}: data range does not match its shape")
            out[name] = TensorInfo(name, dt, tuple(shape), self._map, base + begin, base + end)
        return out


class SafeTensorsDir:
    """All tensors of a model directory, single file or sharded, by name."""

    def __init__(self, model_dir: str):
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    j = json.load(f)
            except (OSError, json.JSONDecodeError) as e:
                raise SafeTensorsError(f"{index}: {e}") from None
            wm = j.get("weight_map") if isinstance(j, dict) else None
            if not isinstance(wm, dict):
                raise SafeTensorsError("index has no weight_map")
            shards = sorted({v for v in wm.values() if isinstance(v, str)})
            paths = [os.path.join(model_dir, s) for s in shards]
        else:
            paths = [os.path.join(model_dir, "model.safetensors")]
        self.files: List[SafeTensorsFile] = [SafeTensorsFile(p) for p in paths]
        self.tensors: Dict[str, TensorInfo] = {}
        for f in self.files:
            self.tensors.update(f.tensors)

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def get(self, name: str):
        return self.tensors.get(name)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def __len__(self) -> int:
        return len(self.tensors)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor] | Sequence[Tuple[str, torch.Tensor]]) -> None:
    """Write CPU tensors in the order given (layout as safetensors.rs:139-169:
    header padded with spaces so that the data starts on an 8-byte boundary)."""
    items = list(tensors.items()) if isinstance(tensors, Mapping) else list(tensors)
    header: Dict[str, dict] = {}
    offset = 0
    blobs: List[bytes | memoryview] = []
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafeTensorsError(f"{name}: unsupported dtype {t.dtype}")
        t = t.detach().contiguous().cpu()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        carrier = t.view(torch.uint8) if t.dim() > 0 else t.reshape(1).view(torch.uint8)
        blobs.append(memoryview(carrier.numpy()).cast("B") if nbytes else b"")
        offset += nbytes
    text = json.dumps(header, separators=(",", ":"))
    while (8 + len(text)) % 8 != 0:
        text += " "
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text.encode("utf-8"))
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)
