from .pages import (CacheInvariantError, CacheLayout, GroupLayout, OutOfPages, PagePool,
                    RequestPages)

__all__ = ["CacheInvariantError", "CacheLayout", "GroupLayout", "OutOfPages", "PagePool",
           "RequestPages", "KVCacheManager", "bytes_per_page", "cache_groups_of"]


def __getattr__(name):
    # the tensor side imports torch and the kernels; the bookkeeping does not need them
    if name in ("KVCacheManager", "bytes_per_page", "cache_groups_of"):
        from . import manager
        return getattr(manager, name)
    raise AttributeError(name)
