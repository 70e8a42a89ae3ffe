"""A paged-KV inference engine for one B200: Qwen3 dense decoder, token ids in,
token ids out.

    from paged_llm_rs_b200 import Engine
    engine = Engine("model_dir", dtype="bfloat16")
    print(engine.generate([[1, 2, 3]], max_tokens=8))

The CUDA kernels are compiled for sm_100a at the first call that needs them.
"""

from . import models  # registers the architectures
from .config import (Architecture, GenerationDefaults, Qwen3Config, load_config, register_architecture,
                     resolve_architecture)
from .errors import (CacheError, ConfigError, EngineError, KernelError, UnsupportedModelError, WeightError)
from .sampling import Rng, SamplingParams


def __getattr__(name):
    # heavier pieces load on first use
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "ModelRunner":
        from .engine.runner import ModelRunner
        return ModelRunner
    if name == "StepEntry":
        from .engine.step import StepEntry
        return StepEntry
    if name == "write_random_model":
        from .weights.random_init import write_random_model
        return write_random_model
    raise AttributeError(name)


def generate(model: str, prompts, max_tokens: int = 512, dtype="bfloat16", **options):
    """One-call generation: build an engine for ``model`` and run the prompts.
    ``options`` are Engine's (block_size, cache_mib, blocks, max_batch, chunk,
    prefix_cache) and generate's (temperature, top_k, top_p, seed, stop_tokens)."""
    from .engine.engine import Engine

    gen_keys = ("temperature", "top_k", "top_p", "seed", "stop_tokens")
    gen = {k: options.pop(k) for k in gen_keys if k in options}
    return Engine(model, dtype=dtype, **options).generate(prompts, max_tokens=max_tokens, **gen)
