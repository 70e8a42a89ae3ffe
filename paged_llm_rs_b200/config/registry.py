"""One registry from an architecture's name to its configuration class and its
description as parts.

The reference has a single ``model_type == "qwen3"`` check
(crates/pagedllm/src/config.rs:89-94) and no registry; this one is keyed on
``config.json["architectures"][0]`` and falls back to ``model_type``.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from ..errors import ConfigError, UnsupportedModelError
from .schema import read_json


@dataclass(frozen=True)
class Architecture:
    name: str
    # parse(dict) -> typed config; raises ConfigError / UnsupportedModelError
    parse: Callable[[Mapping[str, Any]], Any]
    # describe(config) -> parts.spec.ModelSpec
    describe: Callable[[Any], Any]
    # names under which config.json may call it (architectures[0] or model_type)
    aliases: tuple = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    for key in (arch.name,) + tuple(arch.aliases):
        if key in _ARCHITECTURES and not replace and _ARCHITECTURES[key] is not arch:
            raise ValueError(f"architecture {key!r} is already registered")
        _ARCHITECTURES[key] = arch


def architecture_names():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_dict: Mapping[str, Any]) -> Architecture:
    archs = config_dict.get("architectures")
    tried = []
    if isinstance(archs, (list, tuple)):
        for a in archs:
            tried.append(a)
            if a in _ARCHITECTURES:
                return _ARCHITECTURES[a]
    mt = config_dict.get("model_type")
    if mt is not None:
        tried.append(mt)
        if mt in _ARCHITECTURES:
            return _ARCHITECTURES[mt]
    if not tried:
        raise ConfigError("config.json names no architecture: neither `architectures` nor `model_type`")
    raise UnsupportedModelError(
        f"architecture {tried!r} is not registered; known: {architecture_names()}"
    )


def load_config(model_dir: str):
    """Read ``model_dir/config.json``; return (architecture, typed config)."""
    d = read_json(os.path.join(model_dir, "config.json"))
    arch = resolve_architecture(d)
    return arch, arch.parse(d)
