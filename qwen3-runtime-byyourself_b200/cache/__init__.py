"""The cache: slots per sequence, paged keys and values per layer group, fixed-size state."""
from .book import PAGE_TOKENS, CacheBook, CacheError, CacheFull, CacheNeed, PageGroup

__all__ = ["PAGE_TOKENS", "CacheBook", "CacheError", "CacheFull", "CacheNeed", "PageGroup", "KVCache", "LayerCache"]


def __getattr__(name):  # the storage needs torch; the bookkeeping does not
    if name in ("KVCache", "LayerCache"):
        from . import storage
        return getattr(storage, name)
    raise AttributeError(name)
