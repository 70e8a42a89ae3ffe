from .allocator import BlockAllocator, block_hash
from .manager import BlockTable, CacheGroup, CacheManager, RequestCache, FREED
