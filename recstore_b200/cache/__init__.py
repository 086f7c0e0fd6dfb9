"""Embedding caches: GPU set-associative LRU cache, HBM hash-table shard, cached-embedding front ends."""
from .gpu_cache import GpuCache, GpuHashTable, CacheQueryResult, merge_op, uva_cache_query_op, unique_keys  # noqa: F401
from .embeddings import (CacheShardingPolicy, AbsEmb, TorchNativeStdEmb, TorchNativeStdEmbDDP, KnownLocalCachedEmbedding,  # noqa: F401,E402
                         KnownLocalCachedEmbeddingSoftware, KnownShardedCachedEmbedding, KGExternelEmbedding, NVGPUCache, ShmTensorStore,
                         CacheEmbFactory)
from .lookahead_table import LookaheadCachedTable  # noqa: F401,E402
