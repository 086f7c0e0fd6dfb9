"""Embedding caches: GPU set-associative LRU cache, HBM hash-table shard, cached-embedding front ends."""
from .gpu_cache import GpuCache, GpuHashTable, CacheQueryResult, merge_op, uva_cache_query_op, unique_keys  # noqa: F401
