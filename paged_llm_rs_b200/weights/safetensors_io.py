"""Reading and writing the safetensors container, without a library.

The format: an 8-byte little-endian header length N, N bytes of JSON mapping
each tensor name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets
relative to the end of the header), then the raw little-endian data.  The
reference reads the same files through candle
(crates/pagedllm/src/weights.rs:24-32).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch

from ..errors import WeightError

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One open file: header parsed, data memory-mapped, tensors made on demand."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightError(f"{path}: {e}") from e
        size = os.fstat(self._f.fileno()).st_size
        head = self._f.read(8)
        if len(head) != 8:
            raise WeightError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n > size - 8:
            raise WeightError(f"{path}: header length {n} exceeds the file")
        try:
            self.header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{path}: header is not JSON: {e}") from e
        self.header.pop("__metadata__", None)
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None
        for name, info in self.header.items():
            if info.get("dtype") not in _DTYPES:
                raise WeightError(f"{path}: {name} has dtype {info.get('dtype')!r}, which is not handled")
            b, e = info["data_offsets"]
            count = int(np.prod(info["shape"], dtype=np.int64)) if info["shape"] else 1
            if e - b != count * _DTYPES[info["dtype"]][1] or self._base + e > size:
                raise WeightError(f"{path}: {name} has data offsets that do not fit its shape")

    def names(self) -> List[str]:
        return list(self.header)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.header[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.header[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor viewing the mapped file (copy-on-write pages)."""
        info = self.header[name]
        dt, _ = _DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        if e == b:
            return torch.empty(tuple(info["shape"]), dtype=dt)
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._base + b)
        return torch.from_numpy(raw).view(dt).reshape(tuple(info["shape"]))

    def close(self):
        # Tensors handed out may still view the map; let the garbage collector unmap it.
        self._f.close()


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The weight files of a model folder: model.safetensors, or the shards
    that model.safetensors.index.json lists."""
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(single):
        return [SafetensorsFile(single)]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise WeightError(f"{model_dir}: no model.safetensors and no model.safetensors.index.json")


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write tensors (host, contiguous) under their names, in the given order."""
    header = {}
    offset = 0
    items = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightError(f"{name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        items.append(t)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for t in items:
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
