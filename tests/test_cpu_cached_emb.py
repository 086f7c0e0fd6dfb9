"""Differential test of the cached-embedding placements against a golden replicated nn.Embedding (2 gloo ranks on
the CPU), step by step: identical ids, loss = emb.sum()-like, forward values must agree at every step."""
import json
import os
import socket

import pytest
import torch


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, ns, cache_type, mode, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import recstore_b200 as rs
        from recstore_b200 import ipc
        from recstore_b200.cache import CacheEmbFactory
        from recstore_b200.controller import KGCacheControllerWrapperBase, BasePerfSampler
        ipc.set_namespace(ns)
        if rank == 0:
            KGCacheControllerWrapperBase.BeforeDDPInit()
        dist.barrier()
        rs.kvinit()
        N, D, L, steps, per, clr = 400, 8, 4, 25, 48, 0.5

        def init(t, shape, dtype):
            t.copy_(torch.arange(shape[0], dtype=dtype).unsqueeze(1).expand(shape) * 0.01)   # row i == 0.01 * i
        emb = rs.DistEmbedding(N, D, name="full_emb", init_func=init) if rank == 0 else None
        dist.barrier()
        if rank != 0:
            emb = rs.DistEmbedding(N, D, name="full_emb", init_func=init)
        assert torch.allclose(emb.weight[7], torch.full((D,), 0.07))
        cfg = json.dumps({"num_gpus": world, "L": L, "clr": clr, "dim": D, "backwardMode": mode, "full_emb_capacity": N,
                          "cache_ratio": 0.1})
        ctrl = KGCacheControllerWrapperBase.FactoryNew("RecStore", cfg, rank, world)
        ctrl.init(emb.get_shm_tensor() if rank == 0 else None)
        golden = CacheEmbFactory.New("TorchNativeStdEmbDDP", emb)
        gopt = torch.optim.SGD(golden.std_emb.parameters(), lr=clr)
        cached = CacheEmbFactory.New(cache_type, emb, {"cache_ratio": 0.1, "backwardMode": mode, "clr": clr, "controller": ctrl})
        sampler = BasePerfSampler(rank, L, per, N, mode, None, seed=11)
        # every rank publishes its future reads to rank 0's controller through a gather (control plane)
        from recstore_b200.utils import comm

        def publish(step, ids):
            allids = comm.gather_variable_shape_tensor(ids, 0)
            if rank == 0 and ctrl.controller is not None:
                for r, t in enumerate(allids):
                    ctrl.controller.PublishReads(r, step, t)
        future = [sampler.gen_next_sample() for _ in range(L)]
        for s, ids in enumerate(future):
            publish(s, ids)
        worst = 0.0
        for step in range(steps):
            nxt = sampler.gen_next_sample()
            publish(step + L, nxt)
            future.append(nxt)
            ids = future.pop(0)
            a = cached.forward(ids)
            b = golden.forward(ids)
            worst = max(worst, (a - b).abs().max().item())
            w = torch.arange(1, per + 1, dtype=torch.float32).unsqueeze(1) * (rank + 1)
            (a * w).sum().backward()
            gopt.zero_grad()
            (b * w).sum().backward()
            gopt.step()
            cached.after_backward()
        ctrl.GraceFullyStopThreads()
        dist.barrier()
        q.put((rank, worst))
        dist.barrier()
        if rank == 0:
            ipc.IPCTensorFactory.ClearIPCMemory()          # leave nothing in shared memory
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cache_type,mode", [("KnownLocalCachedEmbedding", "CppSync"), ("KnownLocalCachedEmbedding", "CppAsyncV2"),
                                             ("KnownShardedCachedEmbedding", "CppAsyncV2"), ("KGExternelEmbedding", "CppSync"),
                                             ("LocalCachedEmbedding", "CppAsyncV2"), ("ShardedCachedEmbedding", "CppSync"),
                                             ("ShardedCachedEmbedding", "CppAsync")])
def test_cached_embedding_matches_golden(cache_type, mode):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, ns = _free_port(), f"pytest_ce_{os.getpid()}"
    ps = [ctx.Process(target=_worker, args=(r, 2, port, ns, cache_type, mode, q)) for r in range(2)]
    [p.start() for p in ps]
    res = [q.get(timeout=180) for _ in range(2)]
    [p.join(60) for p in ps]
    assert all(p.exitcode == 0 for p in ps)
    for rank, worst in res:
        assert worst < 1e-4, (cache_type, mode, rank, worst)
