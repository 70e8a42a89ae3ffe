"""Error classes of the engine.

They mirror the classes of the reference's error enum
(crates/pagedllm/src/error.rs:9-22): a config that is not valid, a model that
this engine would have to misread in order to run, and a weight file that does
not fit the model.  Cache and kernel errors are this engine's own.
"""


class EngineError(Exception):
    """Base of every error the engine raises on purpose."""


class ConfigError(EngineError):
    """config.json is not valid JSON, misses a key, or holds a value out of range."""


class UnsupportedModelError(EngineError):
    """The config names something this engine does not implement and will not ignore."""


class WeightError(EngineError):
    """The weight file misses tensors, holds unexpected ones, or holds wrong shapes."""


class CacheError(EngineError):
    """The cache manager was asked for something it cannot give (no pages, bad request id)."""


class KernelError(EngineError):
    """A kernel refused its arguments (size not supported, wrong dtype, extension missing)."""
