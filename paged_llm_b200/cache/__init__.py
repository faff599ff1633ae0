from .manager import CacheManager, GroupSpec, Page, PageCopy, PagePool, chain_hash
from .storage import CacheStorage, LayerCache

BlockManager = CacheManager      # the reference's name for it

__all__ = ["BlockManager", "CacheManager", "CacheStorage", "GroupSpec", "LayerCache", "Page", "PageCopy",
           "PagePool", "chain_hash"]
