from .schema import Qwen3Config, GenerationDefaults, read_json, FULL_ATTENTION, SLIDING_ATTENTION
from .registry import (Architecture, register_architecture, resolve_architecture, load_config,
                       architecture_names)
