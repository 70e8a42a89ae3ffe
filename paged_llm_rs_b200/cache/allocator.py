"""Pages of the cache as numbers: a free list, holder counts, and names for full
pages so that requests that begin alike can share them.

Behaviour follows the reference's allocator
(crates/pagedllm/src/blocks.rs:75-293): a page with no name is handed out
first; only when every free page has a name does one lose it, the one released
longest ago (blocks.rs:138-162); a released page keeps its name and contents
until the space is needed (blocks.rs:207-219); the first page to carry a name
keeps it (blocks.rs:191-203).  Nothing here touches a device.
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional

from ..errors import CacheError

_MASK = (1 << 64) - 1


def block_hash(parent: Optional[int], tokens: Iterable[int]) -> int:
    """Name of a full page: FNV-1a over the little-endian bytes of the parent's
    name (0 for none), the token count and each token as 64-bit values, finished
    by splitmix64 (blocks.rs:53-72).  Chained, so it stands for the whole prefix."""
    h = 0xCBF29CE484222325
    tokens = list(tokens)

    def mix(h: int, value: int) -> int:
        for i in range(8):
            h ^= (value >> (8 * i)) & 0xFF
            h = (h * 0x100000001B3) & _MASK
        return h

    h = mix(h, parent or 0)
    h = mix(h, len(tokens))
    for t in tokens:
        h = mix(h, int(t))
    z = (h + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


class BlockAllocator:
    def __init__(self, total: int):
        if total < 1:
            raise CacheError("a page pool needs at least one page")
        self.total = total
        self._holders = [0] * total
        self._hash: List[Optional[int]] = [None] * total
        self._released_at = [0] * total
        # popped from the end, so an untouched pool hands out page 0 first
        self._free: List[int] = list(range(total - 1, -1, -1))
        self._cached: Dict[int, int] = {}
        self._clock = 0
        self.handed_out = self.hits = self.misses = self.evictions = 0

    # -- taking ------------------------------------------------------------------
    def allocate(self) -> Optional[int]:
        """A page for a request's own use, or None when none is free."""
        if not self._free:
            return None
        index = None
        for i in range(len(self._free) - 1, -1, -1):
            if self._hash[self._free[i]] is None:
                index = i
                break
        if index is None:
            index = min(range(len(self._free)), key=lambda i: self._released_at[self._free[i]])
            self.evictions += 1
        block = self._free[index]
        self._free[index] = self._free[-1]
        self._free.pop()
        self._forget(block)
        self._holders[block] = 1
        self.handed_out += 1
        return block

    def acquire_cached(self, name: int) -> Optional[int]:
        """The page that already holds this prefix, with one more holder."""
        block = self._cached.get(name)
        if block is None:
            return None
        self._holders[block] += 1
        if self._holders[block] == 1:
            self._free.remove(block)  # resident but unheld: no longer a candidate for eviction
        self.hits += 1
        return block

    def record_miss(self) -> None:
        self.misses += 1

    def publish(self, block: int, name: int) -> None:
        """Name a page that has just been filled.  Only full pages get names."""
        if self._holders[block] == 0:
            raise CacheError(f"page {block} is named while nobody holds it")
        existing = self._cached.get(name)
        if existing is not None and existing != block:
            return  # another request filled the same prefix first; its page keeps the name
        if self._hash[block] is not None and self._hash[block] != name:
            self._forget(block)
        self._hash[block] = name
        self._cached[name] = block

    # -- giving back ---------------------------------------------------------------
    def release(self, block: int) -> None:
        if not 0 <= block < self.total:
            raise CacheError(f"page {block} is not in a pool of {self.total}")
        if self._holders[block] == 0:
            raise CacheError(f"page {block} released more often than it was taken")
        self._holders[block] -= 1
        if self._holders[block] == 0:
            self._clock += 1
            self._released_at[block] = self._clock
            self._free.append(block)

    def clear_cache(self) -> None:
        """Forget every name: sharing off, nothing else changed (blocks.rs:276-281)."""
        self._hash = [None] * self.total
        self._cached.clear()

    def _forget(self, block: int) -> None:
        name = self._hash[block]
        if name is not None:
            self._hash[block] = None
            if self._cached.get(name) == block:
                del self._cached[name]

    # -- looking -------------------------------------------------------------------
    def available(self) -> int:
        return len(self._free)

    def in_use(self) -> int:
        return self.total - len(self._free)

    def cached_blocks(self) -> int:
        return len(self._cached)

    def holders(self, block: int) -> int:
        return self._holders[block]

    def check(self) -> None:
        """Every page is either free (no holder) or held, never both or neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for b in range(self.total):
            if (self._holders[b] == 0) != (b in free):
                raise CacheError(f"page {b} has {self._holders[b]} holders and is {'on' if b in free else 'off'} the free list")
        for name, b in self._cached.items():
            if self._hash[b] != name:
                raise CacheError(f"name {name:#x} points at page {b}, which does not carry it")
