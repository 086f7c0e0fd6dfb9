"""Parameter server: shard object, loopback server, clients (sync, async, sharded)."""
from .client import (ParameterServer, ParameterClient, PythonParameterClient, AllShardsParameterClient,  # noqa: F401
                     ShardManager, pack_records, unpack_records)
