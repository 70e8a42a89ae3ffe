"""A model as data: which parts each layer is made of and in which order layers run.

An architecture's ``describe(config)`` returns a ``ModelSpec``.  The generic
decoder (``parts/decoder.py``) builds it from the part registries; no part and
no builder code knows which architecture it serves.

The reference assembles one fixed block type in code
(crates/pagedllm/src/model/mod.rs:84-136, 174-257); here the same assembly is a
list, so that a later architecture can give different layers different mixers
and feed-forwards, run a layer twice, or let a layer read another layer's cache.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs from the weight file.

    role decides the dtype it is kept in:
      "matrix"  compute dtype (bfloat16 when serving, float32 on the 32-bit path)
      "gain"    float32 always (norm gains; an exact upcast from bfloat16)
      "index"   int32 (integer tables)
      "keep"    as stored (a tensor stored in 32-bit stays so)
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclass
class PartSpec:
    """kind picks the class from a registry; params are its sizes and constants;
    prefix is where its tensors live in the weight file."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass
class LayerSpec:
    block: str  # arrangement, e.g. "prenorm_residual"
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]  # the norms the arrangement names, e.g. "mixer", "feed_forward"
    prefix: str = ""


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ModelSpec.layers and may appear
    several times in a schedule.  ``reads_cache_of`` names an earlier schedule
    entry whose cache this run attends over instead of writing its own."""

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    position_encodings: Dict[str, PartSpec] = field(default_factory=dict)

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.reads_cache_of is not None:
                j = e.reads_cache_of
                if not 0 <= j < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {j}, which does not run before it")
                if self.schedule[j].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {j}, which owns none")
