"""Random weights: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode in its engine; its fixture script draws a tiny
model once (scripts/dump_reference.py:229-241).  Here matrices are N(0, 0.02)
and norm gains 1 + N(0, 0.1), each tensor from its own generator keyed by the
seed and the tensor's name, so that the bytes do not depend on the order in
which tensors are drawn.
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


def _generator(seed: int, name: str, device) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(model_spec, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                   matrix_std: float = 0.02, gain_std: float = 0.1,
                   write_optional: bool = True) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for s in tensor_specs_of(model_spec):
        if s.name in out or (s.optional and not write_optional):
            continue
        g = _generator(seed, s.name, device)
        if s.role == "gain":
            t = 1.0 + gain_std * torch.randn(s.shape, generator=g, device=device, dtype=torch.float32)
        elif s.role == "index":
            t = torch.zeros(s.shape, dtype=torch.int32, device=device)
        else:
            t = matrix_std * torch.randn(s.shape, generator=g, device=device, dtype=torch.float32)
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
