from .manager import (CacheError, CacheManager, GroupSpec, Opened, OutOfPages, PagePool,
                      chain_hashes, hash_page)
from .storage import CacheStorage

__all__ = ["CacheError", "CacheManager", "CacheStorage", "GroupSpec", "Opened", "OutOfPages",
           "PagePool", "chain_hashes", "hash_page"]
