"""Interfaces of the parts a model is put together from, and their registries.

A part is built from its sizes and constants (``PartSpec.params``) and the
prefix of its tensors; it states the tensors it needs (``tensors()``), receives
them (``bind``) and then runs (``forward``).  No part knows which model it is in.

  Norm               forward(x) and add_norm(residual, delta)
  PositionEncoding   what a mixer needs to place tokens (rotary tables here), and what it adds
                     to the residual stream behind the embedding (nothing here)
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

class PagedNeed:
    """Something kept for every token of a request, in pages that the cache manager hands out and
    takes back.  kind "full": everything stays until the request ends; "window": only the last
    ``window`` tokens are ever read, so older pages are given back.  A need says how its pages lie
    in memory; needs with equal ``group_key()`` share pages, an allocator and block tables.
    Every need has the fields ``kind``, ``window`` and ``dtype`` (None: the model's dtype)."""

    def group_key(self) -> tuple:
        raise NotImplementedError

    def pool_shape(self, entries: int, pages: int, page_size: int) -> Tuple[int, ...]:
        """The shape of the one tensor that holds the pages of ``entries`` runs of layers."""
        raise NotImplementedError

    def layer_view(self, pool: torch.Tensor, index: int) -> tuple:
        """What run ``index`` of the group's layers is handed of the pool (the cache manager adds the group's number)."""
        raise NotImplementedError

    def bytes_per_token(self, element_size: int) -> int:
        raise NotImplementedError


@dataclass(frozen=True)
class KVNeed(PagedNeed):
    """Paged keys and values, a layer's keys (and likewise values) as [pages, kv_heads, page_size, head_dim]."""

    kind: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    # rows stored with their 16-byte chunks XOR-ed by the offset in the page (what the
    # tensor-core attention kernels read); the mixer that reads the pool decides
    swizzled: bool = False
    group_size: int = 1          # query heads to a kv head
    dtype: Optional[torch.dtype] = None

    def group_key(self) -> tuple:
        return ("kv", self.kind, self.window, self.num_kv_heads, self.head_dim, self.swizzled, self.group_size, self.dtype)

    def pool_shape(self, entries, pages, page_size):
        return (entries, 2, pages, self.num_kv_heads, page_size, self.head_dim)

    def layer_view(self, pool, index):
        return (pool[index, 0], pool[index, 1])

    def bytes_per_token(self, element_size):
        return 2 * self.num_kv_heads * self.head_dim * element_size


@dataclass(frozen=True)
class RowNeed(PagedNeed):
    """One row of ``width`` values for every token (a latent vector, say), a layer's rows as
    [pages, page_size, width]: the page of a mixer that does not keep keys and values per head."""

    width: int
    kind: str = "full"
    window: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    def group_key(self) -> tuple:
        return ("rows", self.kind, self.window, self.width, self.dtype)

    def pool_shape(self, entries, pages, page_size):
        return (entries, pages, page_size, self.width)

    def layer_view(self, pool, index):
        return (pool[index],)

    def bytes_per_token(self, element_size):
        return self.width * element_size


@dataclass(frozen=True)
class StateNeed:
    """A slot of fixed size per request: ``shape`` elements of ``dtype``, zeroed
    when a request takes the slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class PlanWish:
    """What a mixer whose kernels read attention work items asks of the step packer: items of at
    most ``tile_tokens`` query tokens, for a kernel that launches ``ctas_per_item`` CTAs an item
    and leaves partial results of ``heads`` x ``head_dim`` a token where a key range was split."""

    tile_tokens: int
    ctas_per_item: int
    heads: int
    head_dim: int


# --- the step as parts see it ---------------------------------------------------

@dataclass
class AttentionWork:
    """A step's attention cut into work items for a cache group (kernels/attention_plan.py), with
    the scratch for split items: made only for groups whose mixers wish for it (Mixer.plan_wish)."""

    work: torch.Tensor          # int32 [max_work, 8] attention work items
    n_work: torch.Tensor        # int32 [1]
    max_work: int
    red: torch.Tensor           # int32 [max_red, 4] reductions of split items
    n_red: torch.Tensor         # int32 [1]
    max_red: int
    part_o: torch.Tensor        # float32 scratch for split items
    part_ml: torch.Tensor
    kinds: int = 3              # what the work items are: 1 single tokens only, 2 portions only, 3 both
    many_splits: bool = False   # the step is cut into eight splits a tile or more (the reduction then shares them out)


@dataclass
class GroupStep:
    """One cache group's share of a step: where each token is written and where its request's
    pages lie (see engine/step.py for how it is made)."""

    block_tables: torch.Tensor  # int32 [segments, table_width]; -1 where a page was given back
    slots: torch.Tensor         # int32 [tokens]: page * page_size + offset for each token
    plan: Optional[AttentionWork] = None


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


class PositionEncoding(Part):
    """Built once per model and handed to the mixers that name it."""

    def rotary(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        """(cos, sin, rotary_dim) with float32 tables [max_positions, rotary_dim/2],
        or None when this encoding does not rotate."""
        return None

    def at_embedding(self, hidden: torch.Tensor, step: "StepState") -> torch.Tensor:
        """What the encoding does to the residual stream right behind the embedding (learned
        absolute positions add a row for ``step.positions`` here); the default leaves it as it is.
        It runs inside a captured step, so it may launch kernels over the step's device tensors only."""
        return hidden


class Mixer(Part):
    # True when forward() only launches kernels whose arguments do not depend on the
    # step's contents, so that a decode step can be captured once and replayed.
    graph_safe = False

    def cache_need(self):
        """KVNeed, StateNeed or None."""
        return None

    def plan_wish(self, page_size: int) -> Optional[PlanWish]:
        """For a mixer that reads attention work items (``GroupStep.plan``): how it wants the step's
        attention cut for pages of ``page_size`` tokens.  None (the default): its group gets block
        tables and slots only.  The mixers that share a cache group must wish alike."""
        return None

    def forward(self, x: torch.Tensor, step: StepState, cache, writes_cache: bool = True) -> torch.Tensor:
        """x [tokens, hidden] -> [tokens, hidden].  ``cache`` is what the cache manager made for
        this run of the layer: for a paged need its ``layer_view`` and the group's number
        ((k_pool, v_pool, group) for a KVNeed, (rows, group) for a RowNeed; the group's
        tables and slots are ``step.groups[group]``), the state tensor [slots, *shape] for a
        StateNeed, None otherwise."""
        raise NotImplementedError


class FeedForward(Part):
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

    # An arrangement may also give its forward in two halves around the mixer:
    #   h = pre_mixer(residual, delta);  a = mixer.forward(h, step, cache, writes_cache);
    #   residual, delta = post_mixer(residual, a, step)
    # Then a step is still captured and replayed when the mixer is not ``graph_safe``: the
    # capture ends before the mixer and begins again behind it, and the mixer alone is launched
    # kernel by kernel at every replay.  Without them such a mixer keeps the whole model on
    # plain launches.
    pre_mixer = None
    post_mixer = None


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
