"""Multi-GPU tests (one process per GPU, NCCL bootstrap, NVLink peer windows).  Skipped with < 2 GPUs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _init(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    import torch.distributed as dist
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"),
                            timeout=datetime.timedelta(seconds=90))
    return dist


def _spawn(fn, args, nprocs):
    """mp.spawn that leaves the verdict to the workers' own reports (a failed rank has written its traceback)."""
    import torch.multiprocessing as mp
    try:
        mp.spawn(fn, args=args, nprocs=nprocs, join=True)
    except Exception as e:              # noqa: BLE001
        print("spawn:", type(e).__name__, str(e)[:300])


def _leave(dist, rank, out, err):
    """End of a worker.  After a failure the rank records it and exits at once: tearing the process group down would
    wait for peers that sit in a collective this rank never joins, and the parent ends the other ranks when one fails."""
    if err is None:
        dist.destroy_process_group()
        return
    import traceback
    out[rank] = "".join(traceback.format_exception(type(err), err, err.__traceback__))[-1500:]
    os._exit(1)


def _dlrm_worker(rank, world, port, graph, out, kind="dot"):
    dist = _init(rank, world, port)
    try:
        from recstore_b200.models.dlrm import DLRM, DLRMConfig
        from recstore_b200.parallel.peer import PeerContext
        from recstore_b200.utils.data import DLRMBatchSource
        rows = [1000, 37, 5000, 12, 300, 20000, 64]
        hot = [1, 2, 1, 3, 1, 1, 1]
        B = 512
        cfg = DLRMConfig(table_rows=rows, batch=B, hotness=hot, emb_lr=0.05, mlp_lr=0.05 if kind == "dot" else 0.002, seed=5,
                         use_cuda_graph=graph, interaction=kind, dcn_layers=2, dcn_rank=64, projection_sizes=(3, 4))
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{rank}"))
        eng = DLRM(cfg, ctx)
        solo = DLRM(cfg) if rank == 0 else None          # same seeds -> identical initial state
        src = DLRMBatchSource(rows, hot, B, alpha=1.2, seed=9)
        # The first step is bit-exact between the sharded and the single-GPU run; afterwards fp32 summation order
        # differs and row-wise Adagrad (a normalised step while a row's state is still tiny) amplifies the difference
        # step over step - faster for the interactions with more stacked GEMMs, which are compared over fewer steps.
        for step in range({"dot": 4, "projection": 2, "dcn": 1}[kind]):
            b = src.next()
            l = eng.train_step(eng.make_pinned_batch(b.dense, b.ids, b.labels))
            lt = torch.tensor([l], device="cuda", dtype=torch.float64)
            dist.all_reduce(lt)
            if rank == 0:
                ls = solo.train_step(solo.make_pinned_batch(b.dense, b.ids, b.labels))
                assert abs(lt.item() - ls) < 2e-3 * max(1.0, abs(ls)), (step, lt.item(), ls)
        eng.check()
        # tables: every rank sends its tables to rank 0 for comparison with the single-GPU run
        for t in range(len(rows)):
            if eng.owner[t] == rank and rank != 0:
                dist.send(eng.table_weight(t).contiguous(), dst=0)
            if rank == 0:
                if eng.owner[t] == 0:
                    w = eng.table_weight(t)
                else:
                    w = torch.empty(rows[t], cfg.emb_dim, device="cuda")
                    dist.recv(w, src=eng.owner[t])
                ref = solo.table_weight(t)
                err = ((w - ref).norm() / ref.norm()).item()
                assert err < 5e-2, (t, err)
        if rank == 0:
            sd, sr = eng.dense_state(), solo.dense_state()
            for k in sd:
                err = ((sd[k] - sr[k]).norm() / (sr[k].norm() + 1e-12)).item()
                assert err < 1e-3, (k, err)
        # inference path agrees between the sharded and the single-GPU engine
        b = src.next()
        p = eng.predict(eng.make_pinned_batch(b.dense, b.ids, b.labels))
        if rank == 0:
            ps = solo.predict(solo.make_pinned_batch(b.dense, b.ids, b.labels))
            assert (p - ps[:p.numel()]).abs().max().item() < 5e-2
        dist.barrier()
        out[rank] = "ok"
    except BaseException as e:          # noqa: BLE001 - reported to the parent, then the process exits
        _leave(dist, rank, out, e)
    _leave(dist, rank, out, None)


@pytest.mark.parametrize("graph", [False, True])
def test_dlrm_two_ranks_match_single(graph):
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = min(_ngpus(), 4) if _ngpus() in (2, 4) else 2
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_dlrm_worker, (world, _free_port(), graph, out), world)
    assert all(out.get(r) == "ok" for r in range(world)), dict(out)


@pytest.mark.parametrize("kind", ["dcn", "projection"])
def test_dlrm_two_ranks_match_single_other_interactions(kind):
    """The cross-network and projection interactions: sharded run == single-GPU run (losses, tables, dense weights)."""
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_dlrm_worker, (2, _free_port(), True, out, kind), 2)
    assert all(out.get(r) == "ok" for r in range(2)), dict(out)


def _timeout_worker(rank, world, port, out):
    """A wait whose signal never comes must return an error status, not hang, and leave the context usable."""
    dist = _init(rank, world, port)
    try:
        from recstore_b200.parallel.peer import PeerContext
        from recstore_b200 import _lib
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{rank}"), wait_timeout_s=0.2)
        ctx.barrier()                       # a normal round works
        torch.cuda.synchronize()
        ctx.check_status()
        if rank == 0:
            ctx.wait(5)                     # nobody signals channel 5
            torch.cuda.synchronize()
            try:
                ctx.check_status()
                out[rank] = "no error raised"
            except _lib.DeviceStatusError as e:
                assert "wait_timeout" in str(e)
                x = torch.ones(4, device="cuda") * 2   # context still usable
                assert x.sum().item() == 8
                out[rank] = "ok"
        else:
            out[rank] = "ok"
        dist.barrier()
    except BaseException as e:          # noqa: BLE001
        _leave(dist, rank, out, e)
    _leave(dist, rank, out, None)


def test_bounded_wait_reports_timeout():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_timeout_worker, (2, _free_port(), out), 2)
    assert all(out.get(r) == "ok" for r in range(2)), dict(out)


def _sharded_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    try:
        from recstore_b200.parallel.peer import PeerContext
        from recstore_b200.parallel.sharded_table import ShardedEmbeddingTable
        from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{rank}"))
        N, D, n = 5000, 32, 3000
        for dedup, ratio in ((True, 1.0), (False, 1.0), (True, 0.2), (False, 0.2)):   # ratio < 1: host tier behind the HBM rows
            tab = ShardedEmbeddingTable(ctx, f"t{int(dedup)}{int(ratio * 10)}", N, D, max_keys=n, lr=0.1, eps=1e-8, dedup=dedup,
                                        init="row_index", hbm_ratio=ratio)
            # oracle: full table replicated on every rank
            W = torch.arange(N, device="cuda", dtype=torch.float32).unsqueeze(1).repeat(1, D)
            S = torch.zeros(N, device="cuda")
            g = torch.Generator(device="cuda").manual_seed(7 + rank)
            for step in range(3):
                ids = torch.randint(0, N, (n,), device="cuda", generator=g)
                ids[::5] = 3                                            # hot key, owned by rank 3 % world
                rows = tab.lookup(ids)
                assert torch.allclose(rows, W[ids], atol=1e-4), (rank, dedup, step)
                grads = torch.randn(n, D, device="cuda", generator=g)
                tab.update(grads)
                # every rank's (ids, grads) reach the oracle on every rank
                all_ids = [torch.empty_like(ids) for _ in range(world)]
                all_g = [torch.empty_like(grads) for _ in range(world)]
                dist.all_gather(all_ids, ids); dist.all_gather(all_g, grads)
                rowwise_adagrad_update(W, S, torch.cat(all_ids), torch.cat(all_g), 0.1, 1e-8)
            torch.cuda.synchronize()
            ctx.check_status()
            mine = tab.local_global_ids()
            mine = mine[mine < N]
            w_all = torch.cat([tab.weight.cpu(), tab.cold]) if tab.tiered else tab.weight.cpu()
            s_all = torch.cat([tab.state.cpu(), tab.cold_state]) if tab.tiered else tab.state.cpu()
            assert torch.allclose(w_all[: mine.numel()], W[mine].cpu(), atol=2e-3, rtol=2e-3), (rank, dedup, ratio)
            assert torch.allclose(s_all[: mine.numel()], S[mine].cpu(), atol=1e-2, rtol=2e-3), (rank, dedup, ratio)
        dist.barrier()
        out[rank] = "ok"
    except BaseException as e:          # noqa: BLE001 - reported to the parent, then the process exits
        _leave(dist, rank, out, e)
    _leave(dist, rank, out, None)


def test_sharded_table_lookup_update_matches_replicated_oracle():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = 4 if _ngpus() >= 4 else 2
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_sharded_worker, (world, _free_port(), out), world)
    assert all(out.get(r) == "ok" for r in range(world)), dict(out)


def test_kge_driver_two_gpus_native_path():
    """TransE-L2 on entity / relation tables sharded over two GPUs, through the training driver."""
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    from recstore_b200.cli import kge_main
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    out, info = kge_main.main(["--device", "cuda", "--num_proc", "2", "--model_name", "TransE_l2", "--max_step", "120",
                               "--n_entities", "20000", "--n_triples", "200000", "--hidden_dim", "128", "--gamma", "10",
                               "--batch_size", "512", "--neg_sample_size", "128", "--rel_part", "--test", "--log_interval", "1000"])
    assert len(out) == 2
    for r in (0, 1):
        assert out[r]["last_loss"] < 0.6 * out[r]["first_loss"], out[r]
        assert out[r]["test"]["MRR"] > 0.2, out[r]
