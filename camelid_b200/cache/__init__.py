from .book import PAGE, CacheBook, FreeList, KVSpec, StateSpec, flatten_specs

__all__ = ["PAGE", "CacheBook", "FreeList", "KVSpec", "StateSpec", "SequenceCache", "flatten_specs"]


def __getattr__(name):
    if name == "SequenceCache":            # needs torch; the bookkeeping above does not
        from .sequence_cache import SequenceCache
        return SequenceCache
    raise AttributeError(name)
