"""Interfaces of the parts a model is put together from, and their registries.

A part is built from its sizes and constants (``PartSpec.params``) and the
prefix of its tensors; it states the tensors it needs (``tensors()``), receives
them (``bind``) and then runs (``forward``).  No part knows which model it is in.

  Norm               forward(x) and add_norm(residual, delta)
  PositionEncoding   what a mixer needs to place tokens (rotary tables here)
  Mixer              forward(x, step, cache): mixes tokens of a request; says what
                     cache it needs (paged keys/values, or a slot of fixed-size state)
  FeedForward        forward(x, step): acts on each token alone
  Block              arrangement of one mixer, one feed-forward and their norms

Another kind of part is added by subclassing and ``register_*``; an architecture
names it in its ``ModelSpec`` by the registered kind.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from .spec import PartSpec, TensorSpec


@dataclass
class Runtime:
    """Where and in which dtype a model runs."""

    device: torch.device
    dtype: torch.dtype
    # one int32 the kernels raise bits in when an index is out of range
    status: torch.Tensor = None
    # While a step runs with a dict here, parts store copies of what they leave at their
    # boundaries under "<tensor prefix>.<what>" ("model.layers.0.self_attn.o_proj.in"): the
    # reference's Trace (crates/pagedllm/src/model/mod.rs:33-80).  Only what a kernel stores
    # can be named: a fused kernel's intermediate values are not.
    trace: Optional[Dict[str, torch.Tensor]] = None

    def __post_init__(self):
        if self.status is None:
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def record(self, name: str, tensor: torch.Tensor) -> None:
        if self.trace is not None:
            self.trace[name] = tensor.detach().clone()


# --- what a mixer needs of the cache manager ------------------------------------

@dataclass(frozen=True)
class KVNeed:
    """Paged keys and values.  kind "full": every key stays; "window": only the
    last ``window`` keys of a request are ever read, so older pages are given back."""

    kind: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    # rows stored with their 16-byte chunks XOR-ed by the offset in the page (what the
    # tensor-core attention kernels read); the mixer that reads the pool decides
    swizzled: bool = False

    def group_key(self) -> tuple:
        return (self.kind, self.window, self.num_kv_heads, self.head_dim, self.swizzled)


@dataclass(frozen=True)
class StateNeed:
    """A slot of fixed size per request: ``shape`` elements of ``dtype``, zeroed
    when a request takes the slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# --- the step as parts see it ---------------------------------------------------

@dataclass
class GroupStep:
    """One cache group's share of a step: where tokens are written and what the
    attention kernels read (see engine/step.py for how it is made)."""

    block_tables: torch.Tensor  # int32 [segments, table_width]; -1 where a page was given back
    slots: torch.Tensor         # int32 [tokens]: page * page_size + offset for each token
    work: torch.Tensor          # int32 [max_work, 8] attention work items
    n_work: torch.Tensor        # int32 [1]
    max_work: int
    red: torch.Tensor           # int32 [max_red, 4] reductions of split items
    n_red: torch.Tensor         # int32 [1]
    max_red: int
    part_o: torch.Tensor        # float32 scratch for split items
    part_ml: torch.Tensor
    kinds: int = 3              # what the work items are: 1 single tokens only, 2 portions only, 3 both
    counters: Optional[torch.Tensor] = None   # int32 zeros [max_work * CTAs an item]: a kernel that combines
                                              # the splits itself counts them off here and leaves zeros
    cluster: int = 0            # > 1: the list holds that many items for every (single) token, which the
                                # attention kernel combines inside a thread-block cluster; red is empty


@dataclass
class StepState:
    """One batch on the device.  Tokens of a request are contiguous (a segment)."""

    n_tokens: int
    tokens: torch.Tensor          # int32 [tokens]
    positions: torch.Tensor       # int32 [tokens] absolute positions
    groups: List[GroupStep]
    logit_rows: torch.Tensor      # int32 [wanted]
    n_wanted: int
    # segments, for mixers with state of their own: per segment
    # (first token, token count, tokens in the cache before this step, state slot)
    segments: torch.Tensor = None  # int32 [segments, 4]
    host_segments: List[Tuple[int, int, int, int]] = field(default_factory=list)
    # per wanted row, for the sampling kernel: temperature (<= 0: greedy) and the request's uniform number
    temperature: torch.Tensor = None
    uniform: torch.Tensor = None


# --- parts ------------------------------------------------------------------------

class Part:
    kind = ""

    def __init__(self, spec: PartSpec, rt: Runtime):
        self.spec = spec
        self.prefix = spec.prefix
        self.rt = rt

    def tensors(self) -> List[TensorSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the tensors named in tensors() (present unless optional)."""

    def _name(self, leaf: str) -> str:
        return f"{self.prefix}.{leaf}" if self.prefix else leaf


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual += delta (in place, when delta is given), then the norm of it.
        With ``rows`` only those rows are normed and residual is left as it is."""
        if delta is not None:
            if rows is None:
                residual.add_(delta)
            else:
                return self.forward(residual.index_select(0, rows.long()) + delta.index_select(0, rows.long()))
        return self.forward(residual, rows)

    def add_norm_deferred(self, residual: torch.Tensor, delta: Optional[torch.Tensor]):
        """The same as ``add_norm`` but not yet run: an object that the kernels'
        products take in place of a tensor (ops.NormedInput), whose ``residual_out``
        is the new residual stream; or None when this norm has no such form for
        these rows.  Only handed to parts with ``takes_normed_input``."""
        return None


class PositionEncoding(Part):
    """Built once per model and handed to the mixers that name it."""

    def rotary(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        """(cos, sin, rotary_dim) with float32 tables [max_positions, rotary_dim/2],
        or None when this encoding does not rotate."""
        return None


class Mixer(Part):
    # True when forward() hands x straight to a product (ops.linear / ops.linear_glu), so
    # that the block may pass a norm that is not yet formed (ops.NormedInput) instead of a tensor.
    takes_normed_input = False
    # True when forward() only launches kernels whose arguments do not depend on the
    # step's contents, so that a decode step can be captured once and replayed.
    graph_safe = False

    def cache_need(self):
        """KVNeed, StateNeed or None."""
        return None

    def cluster_limit(self, page_size: int) -> int:
        """For a mixer that reads its group's attention work items: the most items of one single
        token it can take as a cluster (GroupStep.cluster), 0 when it wants split items with
        partial rows and reductions.  The packer plans a group for the least of its mixers."""
        return 0

    def forward(self, x: torch.Tensor, step: StepState, cache, writes_cache: bool = True) -> torch.Tensor:
        """x [tokens, hidden] -> [tokens, hidden].  ``cache`` is what the cache
        manager made for this run of the layer: (k_pool, v_pool, group index) for a
        KVNeed, the state tensor [slots, *shape] for a StateNeed, None otherwise."""
        raise NotImplementedError


class FeedForward(Part):
    takes_normed_input = False   # as for Mixer

    def forward(self, x: torch.Tensor, step: StepState) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of built parts.  ``forward`` takes the residual stream and a
    pending addition to it (the previous block's last output, not yet added) and
    returns the same pair, so that the add can be fused into the next norm."""

    kind = ""
    prefix = ""   # the layer's tensor prefix ("model.layers.3"), set by the decoder that builds it

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm]):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def forward(self, residual, delta, step: StepState, cache, writes_cache: bool):
        raise NotImplementedError


# --- registries -------------------------------------------------------------------

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}


def _register(table: Dict[str, type], kind: str, cls: type, replace: bool) -> type:
    if kind in table and table[kind] is not cls and not replace:
        raise ValueError(f"{kind!r} is already registered")
    table[kind] = cls
    cls.kind = kind
    return cls


def register_mixer(kind, cls, replace=False): return _register(MIXERS, kind, cls, replace)
def register_feed_forward(kind, cls, replace=False): return _register(FEED_FORWARDS, kind, cls, replace)
def register_norm(kind, cls, replace=False): return _register(NORMS, kind, cls, replace)
def register_position_encoding(kind, cls, replace=False): return _register(POSITION_ENCODINGS, kind, cls, replace)
def register_block(kind, cls, replace=False): return _register(BLOCKS, kind, cls, replace)
def register_embedding(kind, cls, replace=False): return _register(EMBEDDINGS, kind, cls, replace)
def register_head(kind, cls, replace=False): return _register(HEADS, kind, cls, replace)


def make(table: Dict[str, type], what: str, spec: PartSpec, rt: Runtime, **extra):
    if spec.kind not in table:
        raise KeyError(f"no {what} of kind {spec.kind!r} is registered; known: {sorted(table)}")
    return table[spec.kind](spec, rt, **extra)
