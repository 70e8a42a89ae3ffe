"""Typed configurations read from a model folder's JSON files.

``Qwen3Config`` holds exactly the keys the Qwen3 dense decoder's config.json
gives (reference: crates/pagedllm/src/config.rs:17-66) and refuses what the
engine would otherwise silently ignore (config.rs:87-131).  Every size and
constant the model code uses comes from here; none stands in code.

One thing goes beyond the reference: it refuses any ``sliding_window``
(config.rs:104-106).  This engine implements the window (``use_sliding_window``
with ``layer_types`` / ``max_window_layers``, the architecture's own keys), so it
is accepted when the config switches it on, and refused as in the reference when
a window is given but not switched on.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError, UnsupportedModelError

_MISSING = object()


def _take(d: Mapping[str, Any], key: str, kind, default=_MISSING):
    """Read ``d[key]`` as ``kind`` (int, float, bool, str) or raise ConfigError."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"missing field `{key}`")
        return default
    v = d[key]
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"`{key}` must be true or false, got {v!r}")
        return v
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"`{key}` must be an integer, got {v!r}")
        if v < 0:
            raise ConfigError(f"`{key}` must not be negative, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"`{key}` must be a number, got {v!r}")
        if not math.isfinite(float(v)):
            raise ConfigError(f"`{key}` must be finite, got {v!r}")
        return float(v)
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"`{key}` must be a string, got {v!r}")
        return v
    raise TypeError(kind)


FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config:
    """Shape and constants of one Qwen3 dense decoder (config.rs:17-66)."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int  # its own key, not hidden_size / heads (config.rs:30-35)
    rms_norm_eps: float
    vocab_size: int
    max_position_embeddings: int
    tie_word_embeddings: bool
    rope_theta: float
    # One entry per layer: "full_attention" or "sliding_attention".
    layer_types: Tuple[str, ...] = ()
    # Keys a sliding layer may see, itself included; None when no layer slides.
    sliding_window: Optional[int] = None
    model_type: str = "qwen3"
    hidden_act: str = "silu"
    architecture: str = "Qwen3ForCausalLM"

    # --- derived widths (config.rs:147-160) ---------------------------------
    @property
    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def query_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def window_of_layer(self, layer: int) -> Optional[int]:
        return self.sliding_window if self.layer_types[layer] == SLIDING_ATTENTION else None

    # --- reading -------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        model_type = _take(d, "model_type", str)
        if model_type != "qwen3":
            raise UnsupportedModelError(f"model_type {model_type!r}, only qwen3 is implemented")
        hidden_act = _take(d, "hidden_act", str)
        if hidden_act != "silu":
            raise UnsupportedModelError(f"hidden_act {hidden_act!r}, only silu is implemented")
        if _take(d, "attention_bias", bool, False):
            raise UnsupportedModelError("attention_bias, the projections here carry no bias")
        if d.get("rope_scaling") is not None:
            raise UnsupportedModelError("rope_scaling, the rotary table here is unscaled")

        # rope_theta: flat (older writers) or nested under rope_parameters
        # (config.rs:139-145); the nested rope_type must be absent or "default".
        theta = None
        if d.get("rope_theta") is not None:
            theta = _take(d, "rope_theta", float)
        nested = d.get("rope_parameters")
        if nested is not None:
            if not isinstance(nested, Mapping):
                raise ConfigError("`rope_parameters` must be an object")
            kind = nested.get("rope_type")
            if kind is not None and kind != "default":
                raise UnsupportedModelError(f"rope_type {kind!r}, the rotary table here is unscaled")
            if theta is None and nested.get("rope_theta") is not None:
                theta = _take(nested, "rope_theta", float)
        if theta is None:
            raise ConfigError("no rope_theta, in either the flat or the nested layout")
        if theta <= 0:
            raise ConfigError(f"rope_theta must be positive, got {theta}")

        n_layers = _take(d, "num_hidden_layers", int)
        heads = _take(d, "num_attention_heads", int)
        kv_heads = _take(d, "num_key_value_heads", int)
        if heads == 0 or kv_heads == 0 or heads % kv_heads != 0:
            raise UnsupportedModelError(
                f"{heads} query heads over {kv_heads} key heads, which do not group evenly"
            )
        head_dim = _take(d, "head_dim", int)
        if head_dim == 0 or head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be a positive even number, got {head_dim}")

        # The window.  The reference refuses every sliding_window; here it runs
        # when use_sliding_window switches it on.
        window = _take(d, "sliding_window", int, None)
        use_window = _take(d, "use_sliding_window", bool, False)
        layer_types = d.get("layer_types")
        if window is not None and not use_window:
            raise UnsupportedModelError(
                f"sliding_window {window} without use_sliding_window: the config gives a window "
                "and switches it off; remove it or set use_sliding_window"
            )
        if use_window:
            if window is None or window < 1:
                raise ConfigError("use_sliding_window needs a positive sliding_window")
            if layer_types is None:
                first_sliding = _take(d, "max_window_layers", int, n_layers)
                layer_types = [
                    SLIDING_ATTENTION if i >= first_sliding else FULL_ATTENTION for i in range(n_layers)
                ]
        if layer_types is None:
            layer_types = [FULL_ATTENTION] * n_layers
        if not isinstance(layer_types, (list, tuple)) or len(layer_types) != n_layers:
            raise ConfigError(f"layer_types must list {n_layers} layers")
        for t in layer_types:
            if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise UnsupportedModelError(f"layer type {t!r} is not implemented")
        if SLIDING_ATTENTION in layer_types and not use_window:
            raise UnsupportedModelError("layer_types names a sliding layer but use_sliding_window is off")
        if SLIDING_ATTENTION not in layer_types:
            window = None

        archs = d.get("architectures")
        arch = archs[0] if isinstance(archs, (list, tuple)) and archs else "Qwen3ForCausalLM"

        eps = _take(d, "rms_norm_eps", float)
        if eps <= 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {eps}")
        cfg = cls(
            hidden_size=_take(d, "hidden_size", int),
            intermediate_size=_take(d, "intermediate_size", int),
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=eps,
            vocab_size=_take(d, "vocab_size", int),
            max_position_embeddings=_take(d, "max_position_embeddings", int),
            tie_word_embeddings=_take(d, "tie_word_embeddings", bool),
            rope_theta=theta,
            layer_types=tuple(layer_types),
            sliding_window=window,
            model_type=model_type,
            hidden_act=hidden_act,
            architecture=arch,
        )
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size",
                    "max_position_embeddings"):
            if getattr(cfg, key) < 1:
                raise ConfigError(f"`{key}` must be at least 1")
        return cfg

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "rope_theta": self.rope_theta,
            "layer_types": list(self.layer_types),
            "use_sliding_window": self.sliding_window is not None,
            "sliding_window": self.sliding_window,
        }
        return d


def read_json(path: str) -> dict:
    try:
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
    except OSError as e:
        raise ConfigError(f"reading {path}: {e}") from e
    try:
        d = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return d


@dataclass(frozen=True)
class GenerationDefaults:
    """What generation_config.json says about how to run the model
    (config.rs:170-211): stop ids (falling back to config.json's eos_token_id)
    and the sampling defaults.  All optional."""

    eos_token_ids: Tuple[int, ...] = ()
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None

    @staticmethod
    def _token_ids(v) -> Optional[Tuple[int, ...]]:
        if isinstance(v, bool):
            return None
        if isinstance(v, int) and v >= 0:
            return (v,)
        if isinstance(v, list):
            ids = tuple(x for x in v if isinstance(x, int) and not isinstance(x, bool) and x >= 0)
            return ids or None
        return None

    @classmethod
    def from_dir(cls, model_dir: str) -> "GenerationDefaults":
        gen = None
        p = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(p):
            try:
                gen = read_json(p)
            except ConfigError:
                gen = None
        eos = cls._token_ids(gen.get("eos_token_id")) if gen else None
        if eos is None:
            try:
                eos = cls._token_ids(read_json(os.path.join(model_dir, "config.json")).get("eos_token_id"))
            except ConfigError:
                eos = None

        def number(key):
            if not gen:
                return None
            v = gen.get(key)
            return float(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else None

        top_k = number("top_k")
        return cls(
            eos_token_ids=eos or (),
            temperature=number("temperature"),
            top_p=number("top_p"),
            top_k=int(top_k) if top_k is not None and int(top_k) > 0 else None,
        )
