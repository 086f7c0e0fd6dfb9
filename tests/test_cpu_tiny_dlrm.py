"""Tiny DLRM on the CPU with 2 gloo ranks: 8 tables x 10,000 rows x dim 16 on a 2-way sharded KV parameter server,
Zipf(1.05) ids, 13 dense features, bottom 13-64-16, dot interaction, top 52-64-1, batch 256, SGD lr 0.1."""
import os
import socket

import torch


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, q):
    import numpy as np
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from recstore_b200.ps import ParameterServer, ParameterClient, AllShardsParameterClient
        from recstore_b200.models.ps_dlrm import PSDLRM, PSEmbeddingBag
        from recstore_b200.utils.data import zipf_ids
        T, N, D, B = 8, 10_000, 16, 256
        srv = ParameterServer("KVEngineMap", {"dim": D, "capacity": T * N, "optimizer": "sgd", "lr": 0.1})
        ports = [None] * world
        dist.all_gather_object(ports, srv.serve(0))
        client = AllShardsParameterClient([ParameterClient("127.0.0.1", p, i, D) for i, p in enumerate(ports)])
        bags = [PSEmbeddingBag(client, t, N, D) for t in range(T)]
        for b in bags:
            b.init_uniform(rank, world, seed=1)
        dist.barrier()
        assert len(srv) > 0.4 * T * N                      # both shards hold about half of the keys
        torch.manual_seed(0)
        model = PSDLRM(bags, 13, (64, 16), (64, 1))
        ddp = DDP(model)
        opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
        rng = np.random.default_rng(100 + rank)
        # a fixed labelling rule so that there is something to learn: label depends on table 0's id parity
        losses = []
        for step in range(60):
            ids = [torch.from_numpy(zipf_ids(B // world, N, 1.05, rng)) for _ in range(T)]
            dense = torch.from_numpy(np.log1p(rng.exponential(1.0, size=(B // world, 13))).astype(np.float32))
            labels = ((ids[0] % 2 == 0) & (rng.random(B // world) < 0.5)).float()
            emb = model.lookup(ids)
            logit = ddp(dense, emb)
            loss = torch.nn.functional.binary_cross_entropy_with_logits(logit, labels)
            opt.zero_grad()
            loss.backward()
            opt.step()
            assert model.sparse_step() == T * (B // world)
            losses.append(loss.item())
        dist.barrier()
        q.put((rank, losses[0], sum(losses[-10:]) / 10))
        for c in client.clients:
            c.close()
        dist.barrier()
        srv.close()
    finally:
        dist.destroy_process_group()


def test_tiny_dlrm_trains_on_two_cpu_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    res = [q.get(timeout=300) for _ in range(2)]
    [p.join(60) for p in ps]
    assert all(p.exitcode == 0 for p in ps)
    for rank, first, last in res:
        assert last < first, (rank, first, last)          # it learns
        assert last < 0.66
