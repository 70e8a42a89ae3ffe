"""The cache manager: pages for keys and values, grouped by what layers need, a
block table per request and group, and slots for per-request state.

The reference has one group (every layer keeps every key), one table per
sequence and no state slots (crates/pagedllm/src/batch.rs:279-315,
crates/pagedllm/src/blocks.rs:296-430).  Here layers whose mixers ask for the
same kind of cache (all keys, or a window of them; the same kv heads and head
size) form a group with pages, an allocator and tables of its own; a window
group gives pages back as soon as the window has passed them.  Mixers that ask
for a ``StateNeed`` get a slot of fixed size per request instead.

One page holds ``page_size`` tokens of every layer of its group.  How a page
lies in memory is the need's business (``PagedNeed.pool_shape``): keys and
values per kv head for a ``KVNeed`` (a layer's keys, and likewise values, as
[pages, kv_heads, page_size, head_dim]), one row per token for a ``RowNeed``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import CacheError
from ..parts.base import PagedNeed, StateNeed
from .allocator import BlockAllocator, block_hash

FREED = -1  # a table entry whose page was given back (window groups only)


class BlockTable:
    """Where one request's tokens live in one group: logical page -> physical page
    (blocks.rs:296-430)."""

    def __init__(self, page_size: int):
        self.page_size = page_size
        self.blocks: List[int] = []
        self.tokens = 0            # tokens written and committed
        self.hashes: List[int] = []  # names of the full pages, chained
        self.first_live = 0        # logical pages before this one were given back

    def capacity(self) -> int:
        return len(self.blocks) * self.page_size

    def blocks_needed(self, count: int) -> int:
        wanted = self.tokens + count
        return max(0, -(-(wanted - self.capacity()) // self.page_size)) if wanted > self.capacity() else 0

    def slot_of(self, position: int) -> int:
        """page * page_size + offset of a position (blocks.rs:411-414)."""
        b = position // self.page_size
        if b >= len(self.blocks) or self.blocks[b] < 0:
            raise CacheError(f"position {position} has no page")
        return self.blocks[b] * self.page_size + position % self.page_size

    def live_blocks(self) -> List[int]:
        return [b for b in self.blocks if b >= 0]

    def array(self):
        """The table as an int32 numpy array, rebuilt only when pages were added or
        given back since the last call (a page is added every page_size tokens, and
        the step packer asks every step)."""
        sig = (len(self.blocks), self.first_live)
        if getattr(self, "_arr_sig", None) != sig:
            import numpy as np
            self._arr = np.asarray(self.blocks, dtype=np.int32)
            self._arr_ptr = self._arr.ctypes.data
            self._arr_sig = sig
        return self._arr

    def pointer(self):
        """(address, entries) of ``array()``: what the native step packer reads."""
        arr = self.array()
        return self._arr_ptr, len(arr)


@dataclass
class CacheGroup:
    need: PagedNeed
    entries: List[int]                 # schedule entries whose caches live here
    allocator: BlockAllocator
    page_size: int
    pool: Optional[torch.Tensor] = None  # need.pool_shape(entries, pages, page_size)

    @property
    def window(self) -> Optional[int]:
        return self.need.window if self.need.kind == "window" else None


@dataclass
class RequestCache:
    request_id: object
    tables: List[BlockTable]
    state_slot: int = -1

    _tokens: int = 0  # count kept here when the model has no paged group at all

    @property
    def tokens(self) -> int:
        """Tokens written and committed."""
        return self.tables[0].tokens if self.tables else self._tokens


class CacheManager:
    def __init__(self, needs: Sequence[Optional[object]], page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype, device, prefix_cache: bool = True, allocate_device: bool = True):
        """``needs[i]`` is what schedule entry i asks for (a PagedNeed, a StateNeed or None).
        Every group gets ``num_pages`` pages of ``page_size`` tokens."""
        if page_size < 1:
            raise CacheError("page_size must be at least 1")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.dtype, self.device = dtype, device
        self.groups: List[CacheGroup] = []
        self._entry_group: Dict[int, Tuple[int, int]] = {}  # entry -> (group, index in group)
        self._state_entries: Dict[int, StateNeed] = {}
        by_key: Dict[tuple, int] = {}
        for i, need in enumerate(needs):
            if isinstance(need, PagedNeed):
                key = need.group_key()
                if key not in by_key:
                    by_key[key] = len(self.groups)
                    self.groups.append(CacheGroup(need, [], BlockAllocator(num_pages), page_size))
                g = self.groups[by_key[key]]
                self._entry_group[i] = (by_key[key], len(g.entries))
                g.entries.append(i)
            elif isinstance(need, StateNeed):
                self._state_entries[i] = need
            elif need is not None:
                raise CacheError(f"schedule entry {i} asks for {need!r}, which the cache manager does not know")
        self._n_entries = len(needs)
        # state slots: one index per live request, shared by every entry that keeps state
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._state: Dict[int, torch.Tensor] = {}
        self._requests: Dict[object, RequestCache] = {}
        # Sharing rests on pages that never change and are never dropped while held:
        # true for groups that keep every key, not for windows or state.
        self.prefix_cache = bool(prefix_cache) and bool(self.groups) and not self._state_entries \
            and all(g.window is None for g in self.groups)
        if allocate_device:
            for g in self.groups:
                g.pool = torch.zeros(g.need.pool_shape(len(g.entries), num_pages, page_size),
                                     dtype=g.need.dtype or dtype, device=device)
            for i, need in self._state_entries.items():
                self._state[i] = torch.zeros((max_requests,) + tuple(need.shape), dtype=need.dtype, device=device)

    # -- what layers get -------------------------------------------------------------
    def layer_caches(self) -> List[object]:
        """Per schedule entry what its mixer is handed: its view of the group's pool and the
        group's number ((k_pool, v_pool, group) for a KVNeed), a state tensor
        [max_requests, *shape], or None."""
        out: List[object] = [None] * self._n_entries
        for i, (gi, li) in self._entry_group.items():
            g = self.groups[gi]
            out[i] = g.need.layer_view(g.pool, li) + (gi,) if g.pool is not None else (None, gi)
        for i, t in self._state.items():
            out[i] = t
        return out

    def bytes_per_token(self) -> int:
        return sum(len(g.entries) * g.need.bytes_per_token(torch.empty((), dtype=g.need.dtype or self.dtype).element_size())
                   for g in self.groups)

    # -- requests ----------------------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already open")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        for t in self._state.values():
            t[slot].zero_()
        rc = RequestCache(request_id, [BlockTable(self.page_size) for _ in self.groups], slot)
        self._requests[request_id] = rc
        return rc

    def get(self, request_id) -> RequestCache:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not open") from None

    def has(self, request_id) -> bool:
        return request_id in self._requests

    def slots_free(self) -> int:
        return len(self._free_slots)

    def tokens_of(self, request_id) -> int:
        return self.get(request_id).tokens

    def close(self, request_id) -> None:
        """Give back everything the request holds."""
        rc = self._requests.pop(request_id, None)
        if rc is None:
            raise CacheError(f"request {request_id!r} is not open (closed twice?)")
        for g, t in zip(self.groups, rc.tables):
            for b in t.blocks:
                if b >= 0:
                    g.allocator.release(b)
            t.blocks, t.hashes, t.tokens = [], [], 0
        self._free_slots.append(rc.state_slot)

    # -- pages ---------------------------------------------------------------------------
    def available(self) -> int:
        """Free pages of the tightest group."""
        return min((g.allocator.available() for g in self.groups), default=self.num_pages)

    def pages_for(self, tokens: int, step_tokens: Optional[int] = None) -> int:
        """Pages a request of ``tokens`` tokens holds at its largest, in the group
        that needs most.  A window group holds the window plus what one step adds."""
        most = 0
        for g in self.groups:
            if g.window is None:
                n = -(-tokens // self.page_size)
            else:
                span = min(tokens, g.window + (step_tokens or tokens))
                n = min(-(-tokens // self.page_size), -(-span // self.page_size) + 1)
            most = max(most, n)
        return most

    def blocks_needed(self, request_id, count: int) -> int:
        """Pages (in the group that needs most) still to be taken for ``count`` more tokens."""
        rc = self.get(request_id)
        return max((t.blocks_needed(count) for t in rc.tables), default=0)

    def reserve(self, request_id, count: int) -> bool:
        """Take the pages ``count`` more tokens need, in every group, or none at all."""
        rc = self.get(request_id)
        taken: List[Tuple[int, int]] = []
        for gi, (g, t) in enumerate(zip(self.groups, rc.tables)):
            for _ in range(t.blocks_needed(count)):
                b = g.allocator.allocate()
                if b is None:
                    for gj, bb in reversed(taken):
                        self.groups[gj].allocator.release(bb)
                        rc.tables[gj].blocks.pop()
                    return False
                t.blocks.append(b)
                taken.append((gi, b))
        return True

    def reserve_up_to(self, request_id, count: int) -> int:
        """Take pages for as many of ``count`` more tokens as the pools allow; return
        how many tokens fit (crates/pagedllm/src/scheduler.rs:452-460)."""
        rc = self.get(request_id)
        if not rc.tables or self.reserve(request_id, count):
            return count
        while True:  # page by page, every group in step
            room = min(t.capacity() - t.tokens for t in rc.tables)
            if room >= count:
                return count
            if not self.reserve(request_id, room + 1):
                return room

    def claim_prefix(self, request_id, tokens: Sequence[int]) -> int:
        """Take the pages that already hold the leading full pages of ``tokens``, never
        the last page (scheduler.rs:596-621).  Returns how many tokens are thereby
        already in the cache."""
        rc = self.get(request_id)
        if not self.prefix_cache or any(t.blocks for t in rc.tables):
            return 0
        ps = self.page_size
        candidates = max(0, -(-len(tokens) // ps) - 1)
        parent, shared = None, 0
        for index in range(candidates):
            name = block_hash(parent, tokens[index * ps:(index + 1) * ps])
            got = []
            for g in self.groups:
                b = g.allocator.acquire_cached(name)
                if b is None:
                    g.allocator.record_miss()
                    break
                got.append(b)
            if len(got) < len(self.groups):
                for g, b in zip(self.groups, got):
                    g.allocator.release(b)
                break
            for t, b in zip(rc.tables, got):
                t.blocks.append(b)
                t.hashes.append(name)
                t.tokens += ps
            shared += ps
            parent = name
        return shared

    def commit(self, request_id, count: int, history: Optional[Sequence[int]] = None) -> None:
        """Record that ``count`` tokens were written.  Names the pages that became
        full (``history`` = every token of the request so far) and gives back the
        pages a window has passed."""
        rc = self.get(request_id)
        if not rc.tables:
            rc._tokens += count
        for g, t in zip(self.groups, rc.tables):
            if t.tokens + count > t.capacity():
                raise CacheError(f"{t.tokens + count} tokens written into {t.capacity()} of capacity")
            t.tokens += count
            if self.prefix_cache and history is not None:
                full = min(t.tokens // self.page_size, len(t.blocks))
                while len(t.hashes) < full:
                    i = len(t.hashes)
                    chunk = history[i * self.page_size:(i + 1) * self.page_size]
                    if len(chunk) < self.page_size:
                        break
                    name = block_hash(t.hashes[-1] if t.hashes else None, chunk)
                    t.hashes.append(name)
                    g.allocator.publish(t.blocks[i], name)
            if g.window is not None:
                # The next query sits at position t.tokens or later and sees keys
                # from t.tokens - window + 1 on: pages wholly before that are done.
                first_needed = max(0, t.tokens - g.window + 1)
                while (t.first_live + 1) * self.page_size <= first_needed:
                    b = t.blocks[t.first_live]
                    if b >= 0:
                        g.allocator.release(b)
                        t.blocks[t.first_live] = FREED
                    t.first_live += 1

    def set_prefix_cache(self, enabled: bool) -> None:
        enabled = bool(enabled) and bool(self.groups) and not self._state_entries and all(g.window is None for g in self.groups)
        self.prefix_cache = enabled
        if not enabled:
            for g in self.groups:
                g.allocator.clear_cache()

    # -- checking ------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, none held by a table without the allocator knowing."""
        for gi, g in enumerate(self.groups):
            g.allocator.check()
            held: Dict[int, int] = {}
            for rc in self._requests.values():
                for b in rc.tables[gi].blocks:
                    if b >= 0:
                        held[b] = held.get(b, 0) + 1
            for b in range(g.allocator.total):
                if g.allocator.holders(b) != held.get(b, 0):
                    raise CacheError(f"group {gi} page {b}: allocator counts {g.allocator.holders(b)} holders, "
                                     f"tables hold it {held.get(b, 0)} times")
        slots = [rc.state_slot for rc in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a state slot was lost")
