"""Random weights: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode in its engine; its fixture script draws a tiny
model once (scripts/dump_reference.py:229-241).  Here matrices are N(0, 0.02)
and norm gains 1 + N(0, 0.1).  Every value is a function of (seed, tensor name,
index in the tensor) alone, computed in integers: the same bytes whatever the
order in which tensors are drawn and on whatever device they are drawn (a folder
written on the GPU for the bench holds what one written on the CPU holds).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..config.registry import resolve_architecture
from ..parts.decoder import tensor_specs_of
from .safetensors_io import write_safetensors


_M64 = (1 << 64) - 1


def _mix(z: torch.Tensor) -> torch.Tensor:
    """splitmix64's finaliser on int64 tensors (products wrap; shifts are made logical by masks)."""
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * -4658895280553007687           # 0xBF58476D1CE4E5B9 as int64
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * -7723592293110705685           # 0x94D049BB133111EB as int64
    return z ^ ((z >> 31) & ((1 << 33) - 1))


def _standard_normal(seed: int, name: str, shape, device) -> torch.Tensor:
    """float32 values of unit variance: the sum of twelve 16-bit uniform numbers per value (its variance is
    exactly one, its tails end at six standard deviations), formed in integers so that every device gives the
    same bits; then ONE float32 multiplication."""
    n = 1
    for d in shape:
        n *= int(d)
    key = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")
    key = key - (1 << 64) if key >= (1 << 63) else key
    total = torch.zeros(n, dtype=torch.int64, device=device)
    index = torch.arange(n, dtype=torch.int64, device=device)
    for r in range(3):
        # (0x9E3779B97F4A7C15 as int64 is -7046029254386353131: splitmix64's increment)
        z = _mix((index * 3 + r + 1) * -7046029254386353131 + key)
        for k in range(4):
            total += (z >> (16 * k)) & 0xFFFF
    # sum of 12 uniforms on 0..65535: mean 6 * 65535, standard deviation 65536 (to 1e-10)
    return ((total * 2 - 12 * 65535).to(torch.float32) * (1.0 / 131072.0)).reshape(tuple(shape))


def random_tensors(model_spec, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                   matrix_std: float = 0.02, gain_std: float = 0.1,
                   write_optional: bool = True) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for s in tensor_specs_of(model_spec):
        if s.name in out or (s.optional and not write_optional):
            continue
        if s.role == "gain":
            t = 1.0 + gain_std * _standard_normal(seed, s.name, s.shape, device)
        elif s.role == "index":
            t = torch.zeros(s.shape, dtype=torch.int32, device=device)
        else:
            t = matrix_std * _standard_normal(seed, s.name, s.shape, device)
        out[s.name] = t if s.role == "index" else t.to(dtype)
    return out


def write_random_model(model_dir: str, config_dict: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       device="cpu", write_optional: bool = False, matrix_std: float = 0.02,
                       gain_std: float = 0.1) -> str:
    """Make ``model_dir`` with config.json and model.safetensors.  Optional
    tensors (a tied head's own copy) are left out unless asked for."""
    arch = resolve_architecture(config_dict)
    cfg = arch.parse(config_dict)
    spec = arch.describe(cfg)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=1)
    tensors = random_tensors(spec, seed, dtype=dtype, device=device, matrix_std=matrix_std, gain_std=gain_std,
                             write_optional=write_optional)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
    return model_dir
