"""Weights by tensor name, checked against what the model's parts ask for.

The reference fetches tensors one at a time and stops at the first that is
missing or misshapen (crates/pagedllm/src/weights.rs:51-66).  Here every part
states its tensors up front (``TensorSpec``), so one pass over the file finds
all that is missing, unexpected or of the wrong shape and reports it in one
``WeightError``.

What dtype a tensor is kept in follows its role (see ``TensorSpec``): matrices in
the compute dtype, gains in float32, integer tables as int32, and "keep" as
stored, so a tensor stored in 32-bit stays 32-bit.
"""

from __future__ import annotations

from typing import Dict, Iterable, List

import torch

from ..errors import WeightError
from ..parts.spec import TensorSpec
from .safetensors_io import SafetensorsFile, open_model_files


def check_tensors(specs: Iterable[TensorSpec], available: Dict[str, tuple]) -> None:
    """Raise one WeightError listing every missing, unexpected and misshapen tensor.
    ``available`` maps each name in the file to its shape."""
    specs = list(specs)
    wanted = {}
    for s in specs:
        if s.name in wanted and wanted[s.name].shape != tuple(s.shape):
            raise WeightError(f"two parts ask for {s.name} at different shapes")
        # a tensor is optional only if every part asking for it says so
        if s.name in wanted:
            s = TensorSpec(s.name, tuple(s.shape), s.role, s.optional and wanted[s.name].optional)
        wanted[s.name] = s
    missing = [n for n, s in wanted.items() if n not in available and not s.optional]
    unexpected = [n for n in available if n not in wanted]
    wrong = [
        f"{n} has shape {list(available[n])}, expected {list(s.shape)}"
        for n, s in wanted.items()
        if n in available and tuple(available[n]) != tuple(s.shape)
    ]
    if missing or unexpected or wrong:
        lines = ["the weight file does not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightError("\n".join(lines))


def _kept_dtype(role: str, stored: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return compute_dtype
    if role == "gain":
        return torch.float32
    if role == "index":
        return torch.int32
    if role == "keep":
        return stored
    raise ValueError(f"unknown tensor role {role!r}")


def load_weights(model_dir: str, specs: Iterable[TensorSpec], compute_dtype: torch.dtype,
                 device) -> Dict[str, torch.Tensor]:
    """Read the tensors the specs name from ``model_dir`` onto ``device``."""
    specs = list(specs)
    files: List[SafetensorsFile] = open_model_files(model_dir)
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for n in f.names():
            where[n] = f
    check_tensors(specs, {n: f.shape(n) for n, f in where.items()})
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name in out or s.name not in where:
            continue
        f = where[s.name]
        host = f.tensor(s.name)
        dt = _kept_dtype(s.role, host.dtype, compute_dtype)
        # One copy to the device, then the cast there (exact for bfloat16 -> float32).
        out[s.name] = host.to(device=device).to(dtype=dt).contiguous()
    for f in files:
        f.close()
    return out
