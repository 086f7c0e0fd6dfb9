"""Who is who in a parameter-server job: roles, ids and the servers' addresses, met through a small key-value store.

``Postoffice(role, num_servers, num_clients, global_id, store_host, store_port)``: servers are the first
``num_servers`` global ids, clients follow; server *i* publishes ``server/<i> = host:port`` once it listens, every
member can ``server_address(i)`` (blocking with a timeout) and ``barrier(name)``.  The store is a
``torch.distributed.TCPStore`` hosted by global id 0 -- the reference meets through memcached with the same
role / id scheme (src/ps_common/Postoffice.{h,cc}; flags ``global_id``, ``num_server_processes``,
``num_client_processes``); ``ShardManager.KeyPartition`` (``ps/client.py``) maps keys to server ids.
"""
from __future__ import annotations

import datetime
from typing import List, Tuple

from torch.distributed import TCPStore


class Postoffice:
    def __init__(self, num_servers: int, num_clients: int, global_id: int, store_host: str = "127.0.0.1", store_port: int = 29400,
                 timeout_s: float = 60.0):
        assert 0 <= global_id < num_servers + num_clients
        self.num_servers, self.num_clients, self.global_id = num_servers, num_clients, global_id
        self.store = TCPStore(store_host, store_port, world_size=None, is_master=(global_id == 0),
                              timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)

    # ---- roles
    @property
    def is_server(self) -> bool:
        return self.global_id < self.num_servers

    @property
    def is_client(self) -> bool:
        return not self.is_server

    @property
    def server_id(self) -> int:
        assert self.is_server
        return self.global_id

    @property
    def client_id(self) -> int:
        assert self.is_client
        return self.global_id - self.num_servers

    @property
    def num_members(self) -> int:
        return self.num_servers + self.num_clients

    # ---- rendezvous
    def publish_server(self, host: str, port: int) -> None:
        self.store.set(f"server/{self.server_id}", f"{host}:{port}")

    def server_address(self, i: int) -> Tuple[str, int]:
        host, port = self.store.get(f"server/{i}").decode().rsplit(":", 1)     # blocks until published (store timeout)
        return host, int(port)

    def all_servers(self) -> List[Tuple[str, int]]:
        return [self.server_address(i) for i in range(self.num_servers)]

    def barrier(self, name: str = "default") -> None:
        """All members arrive; reusable (a generation counter per name)."""
        key = f"barrier/{name}"
        n = self.store.add(key, 1)
        gen = (n - 1) // self.num_members
        self.store.wait([f"{key}/done/{gen}"]) if n % self.num_members else self.store.set(f"{key}/done/{gen}", "1")
