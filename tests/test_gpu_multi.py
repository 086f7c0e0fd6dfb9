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


def _world(cap=8):
    """Largest of 8 / 4 / 2 ranks that the box (and the test's cap) allows."""
    n = min(_ngpus(), cap)
    return 8 if n >= 8 else 4 if n >= 4 else 2


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


def _dlrm_worker(rank, world, port, graph, out, kind="dot", split=None):
    dist = _init(rank, world, port)
    try:
        from recstore_b200.models.dlrm import DLRM, DLRMConfig
        from recstore_b200.parallel.peer import PeerContext
        from recstore_b200.utils.data import DLRMBatchSource
        rows = [1000, 37, 5000, 12, 300, 20000, 64, 900]
        hot = [1, 2, 1, 3, 1, 1, 1, 1] if split is None else [1, 2, 40, 3, 1, 1, 1, 1]
        B = 512 if world <= 4 else 1024
        # The dot model is compared under row-wise Adagrad.  The interactions with more stacked GEMMs are compared under
        # plain SGD on the embeddings: Adagrad's normalised step (while a row's state is still tiny) would amplify the
        # fp32 summation-order noise of the all-reduce step over step, which says nothing about the exchange itself.
        opt = "rowwise_adagrad" if kind == "dot" else "sgd"
        # What is compared, and how tightly.  From identical parameters the sharded and the single-GPU run do the same
        # arithmetic per sample; only fp32 summation order differs (split reductions, the all-reduce), so the FIRST step's
        # parameter updates must agree almost to rounding: that is the check that catches a wrong exchange, a dropped id or
        # a misrouted gradient.  Later steps compound those last-bit differences through bf16 re-rounding of the weights
        # and the multiplicative cross layers, so they only have to stay close.  Row-sharded tables send their pooled
        # partial sums as bf16, one rounding more than the single-GPU run has (the model's backward turns that 0.3 % into
        # several per cent of gradient difference, measured); so that the first step can still be compared tightly, that
        # test starts from table values on a coarse grid (multiples of 1/32, |v| <= 1/16) whose partial sums of up to 40
        # rows are exact in bf16, which makes its forward pass bit-identical to the single-GPU one.
        lr_e, lr_m = (0.05, 0.05 if kind == "dot" else 0.002) if split is None else (0.01, 0.01 if kind == "dot" else 0.002)
        tol_pred, tol_upd, tol_loss = (2e-3, 2e-3, 5e-3) if split is None else (2e-3, 2e-3, 5e-2)
        cfg = DLRMConfig(table_rows=rows, batch=B, hotness=hot, emb_lr=lr_e, mlp_lr=lr_m, seed=5,
                         use_cuda_graph=graph, interaction=kind, dcn_layers=2, dcn_rank=64, projection_sizes=(3, 4),
                         emb_optimizer=opt, row_split=split)
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{rank}"))
        eng = DLRM(cfg, ctx)
        solo = DLRM(cfg) if rank == 0 else None          # same seeds -> identical initial state
        if split is not None:
            assert eng.split_tables == sorted(split) and eng.K == len(split)
        src = DLRMBatchSource(rows, hot, B, alpha=1.2, seed=9)
        if split is not None:
            for t in range(len(rows)):
                full = torch.randint(-2, 3, (rows[t], cfg.emb_dim), generator=torch.Generator().manual_seed(100 + t)).float() / 32
                if rank == 0:
                    solo.table_weight(t).copy_(full)
                if t in eng.local_tables:
                    eng.table_weight(t).copy_(full[rank::world] if t in split else full)

        def rel(a, b):
            return ((a - b).norm() / (b.norm() + 1e-20)).item()

        # forward only, before any update
        b = src.next()
        p = eng.predict(eng.make_pinned_batch(b.dense, b.ids, b.labels))
        if rank == 0:
            ps = solo.predict(solo.make_pinned_batch(b.dense, b.ids, b.labels))
            assert (p - ps[:p.numel()]).abs().max().item() < tol_pred
        dense0 = {k: v.clone() for k, v in eng.dense_state().items()}
        tab0 = [eng.gather_table(t) for t in range(len(rows))]
        for step in range(4):
            b = src.next()
            l = eng.train_step(eng.make_pinned_batch(b.dense, b.ids, b.labels))
            lt = torch.tensor([l], device="cuda", dtype=torch.float64)
            dist.all_reduce(lt)
            if rank == 0:
                ls = solo.train_step(solo.make_pinned_batch(b.dense, b.ids, b.labels))
                assert abs(lt.item() - ls) < (2e-3 if step == 0 else tol_loss) * max(1.0, abs(ls)), (step, lt.item(), ls)
            if step == 0:
                # first-step UPDATES (parameter minus its initial value), dense and every table
                errs = {}
                tabs = [eng.gather_table(t) for t in range(len(rows))]
                if rank == 0:
                    sd, sr = eng.dense_state(), solo.dense_state()
                    for k in sd:
                        if (sr[k] - dense0[k]).abs().sum() > 0:
                            errs[k] = rel(sd[k] - dense0[k], sr[k] - dense0[k])
                    for t in range(len(rows)):
                        errs[f"table{t}"] = rel(tabs[t] - tab0[t], solo.table_weight(t) - tab0[t])
                    # (a table update is the difference of two fp32 numbers of the size of the weights: with weights on the
                    # coarse grid, ~1000 x larger than the update, the subtraction alone costs a few 1e-3)
                    bad = {k: round(v, 5) for k, v in errs.items()
                           if v >= (1e-2 if split is not None and k.startswith("table") else tol_upd)}
                    assert not bad, (bad, {k: round(v, 5) for k, v in errs.items()})
        eng.check()
        # after four steps: parameters still close
        for t in range(len(rows)):
            w = eng.gather_table(t)
            if rank == 0:
                assert rel(w, solo.table_weight(t)) < (5e-2 if split is None else 1e-1), (t, rel(w, solo.table_weight(t)))
        if rank == 0:
            sd, sr = eng.dense_state(), solo.dense_state()
            for k in sd:
                assert rel(sd[k], sr[k]) < 5e-2, (k, rel(sd[k], sr[k]))
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
    world = _world() if graph else _world(4)
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_dlrm_worker, (world, _free_port(), graph, out), world)
    assert all(out.get(r) == "ok" for r in range(world)), dict(out)


@pytest.mark.parametrize("kind", ["dcn", "projection"])
def test_dlrm_two_ranks_match_single_other_interactions(kind):
    """The cross-network and projection interactions: sharded run == single-GPU run (losses, tables, dense weights) over
    four steps."""
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_dlrm_worker, (2, _free_port(), True, out, kind), 2)
    assert all(out.get(r) == "ok" for r in range(2)), dict(out)


@pytest.mark.parametrize("kind", ["dot", "dcn"])
def test_dlrm_row_sharded_tables_match_single(kind):
    """Tables spread row-wise over the ranks (owner = id % world; a 40-hot, a 3-hot and a 1-hot one): keys travel to the
    owners, pooled partial sums come back, gradients fan out to every owner.  Result == single-GPU run."""
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = _world() if kind == "dot" else _world(4)
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_dlrm_worker, (world, _free_port(), True, out, kind, [2, 3, 5]), world)
    assert all(out.get(r) == "ok" for r in range(world)), dict(out)


def _pipe_worker(rank, world, port, out):
    """Pipelined lookup on several GPUs against the single-GPU engine: a chain of submits whose results are read one step
    late (every step's graph ends with the next batch's lookup and forward all-to-all)."""
    dist = _init(rank, world, port)
    try:
        from recstore_b200.models.dlrm import DLRM, DLRMConfig
        from recstore_b200.parallel.peer import PeerContext
        from recstore_b200.utils.data import DLRMBatchSource
        rows = [1000, 37, 5000, 12, 300, 20000, 64, 900]
        hot = [1, 2, 1, 3, 1, 1, 1, 1]
        B = 512 if world <= 4 else 1024
        kw = dict(table_rows=rows, batch=B, hotness=hot, emb_lr=0.05, mlp_lr=0.05, seed=5)
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{rank}"))
        eng = DLRM(DLRMConfig(pipeline_lookup=True, **kw), ctx)
        assert eng._pipe
        solo = DLRM(DLRMConfig(**kw)) if rank == 0 else None
        src = DLRMBatchSource(rows, hot, B, alpha=1.2, seed=9)
        batches = [src.next() for _ in range(4)]
        got, prev = [], None
        for b in batches:
            h = eng.submit(eng.make_pinned_batch(b.dense, b.ids, b.labels))
            if prev is not None:
                got.append(prev.result())
            prev = h
        got.append(prev.result())
        eng.check()
        lt = torch.tensor(got, device="cuda", dtype=torch.float64)
        dist.all_reduce(lt)
        tabs = [eng.gather_table(t) for t in range(len(rows))]
        if rank == 0:
            ref = [solo.train_step(solo.make_pinned_batch(b.dense, b.ids, b.labels)) for b in batches]
            for i, (a, r) in enumerate(zip(lt.tolist(), ref)):
                assert abs(a - r) < (2e-3 if i == 0 else 5e-3) * max(1.0, abs(r)), (i, lt.tolist(), ref)
            rel = lambda a, b: ((a - b).norm() / (b.norm() + 1e-20)).item()
            for t in range(len(rows)):
                assert rel(tabs[t], solo.table_weight(t)) < 5e-2, (t, rel(tabs[t], solo.table_weight(t)))
            sd, sr = eng.dense_state(), solo.dense_state()
            for k in sd:
                assert rel(sd[k], sr[k]) < 5e-2, (k, rel(sd[k], sr[k]))
        else:
            eng.dense_state()
        ms = eng.time_steps_on_device(4)          # look-ahead graphs back to back, then a normal step
        assert ms > 0
        b = src.next()
        eng.train_step(eng.make_pinned_batch(b.dense, b.ids, b.labels))
        eng.check()
        dist.barrier()
        out[rank] = "ok"
    except BaseException as e:          # noqa: BLE001
        _leave(dist, rank, out, e)
    _leave(dist, rank, out, None)


def test_dlrm_pipelined_lookup_matches_single():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = _world()
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_pipe_worker, (world, _free_port(), out), world)
    assert all(out.get(r) == "ok" for r in range(world)), dict(out)


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
        # ratio < 1: host tier behind the HBM rows; fused = False: the exchange as separate count / signal / wait launches
        for dedup, ratio, fused in ((True, 1.0, True), (False, 1.0, True), (True, 0.2, True), (False, 0.2, True), (True, 1.0, False)):
            tab = ShardedEmbeddingTable(ctx, f"t{int(dedup)}{int(ratio * 10)}{int(fused)}", N, D, max_keys=n, lr=0.1, eps=1e-8,
                                        dedup=dedup, init="row_index", hbm_ratio=ratio, fused=fused)
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
    world = _world()
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_sharded_worker, (world, _free_port(), out), world)
    assert all(out.get(r) == "ok" for r in range(world)), dict(out)


@pytest.mark.parametrize("choice", ["KnownShardedCachedEmbedding", "KnownLocalCachedEmbedding", "LocalCachedEmbedding",
                                    "ShardedCachedEmbedding"])
def test_cached_embeddings_on_the_native_plane_match_replicated_embedding(choice):
    """The reference-named cached embeddings on two GPUs (hot ranges as range-owned shards on the peer-window
    transport, rows of other ranges from the device-mapped host table, gradients delivered by ``push_update``): every
    step's forward output equals a replicated ``nn.Embedding`` trained with the same gradients (the driver's --diff_test).
    The two hash-cache placements run their ``GpuCache`` (query, fill on miss, update of cached copies in backward) with
    NCCL all-to-alls around it."""
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    from recstore_b200.cli import perf_emb
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    out = perf_emb.main(["--num_workers", "2", "--device", "cuda", "--run_steps", "25", "--diff_test", "--emb_choice", choice,
                         "--backwardMode", "CppAsyncV2", "--batch_size", "3000", "--num_embs", "50000", "--log_interval", "1000"])
    assert len(out) == 2 and all(v[0] == 25 and v[1] < 1e-3 for v in out.values()), out


def _ps_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    try:
        from recstore_b200.parallel.peer import PeerContext
        from recstore_b200.ps.gpu_client import NvlinkParameterClient
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{rank}"))
        D = 16
        ps = NvlinkParameterClient(ctx, emb_dim=D, capacity=40000, max_batch=4096, lr=0.5, name="ps_multi")
        g = torch.Generator().manual_seed(5)
        keys = torch.randperm(1 << 20, generator=g)[:4000] + (1 << 35)        # the same key set on every rank
        vals = torch.randn(4000, D, generator=g)
        mine = slice(rank, 4000, world)                                       # every rank puts ITS part; owners are key % world
        ps.PutParameter(keys[mine], vals[mine])
        ctx.barrier()
        rows, found = ps.GetParameterWithMask(keys[:1500])                    # most of them put by, and stored on, other ranks
        assert found.all() and torch.equal(rows.cpu(), vals[:1500]), rank
        gg = torch.Generator().manual_seed(9 + rank)
        idx = torch.randint(0, 300, (800,), generator=gg)
        grads = torch.randn(800, D, generator=gg)
        ps.UpdateParameter(keys[idx], grads)                                  # every rank updates overlapping keys
        all_idx = [torch.empty_like(idx).cuda() for _ in range(world)]
        all_g = [torch.empty_like(grads).cuda() for _ in range(world)]
        dist.all_gather(all_idx, idx.cuda()); dist.all_gather(all_g, grads.cuda())
        ref = vals.clone().cuda()
        ref.index_add_(0, torch.cat(all_idx), -0.5 * torch.cat(all_g))
        ctx.barrier()
        got = ps.GetParameter(keys[:300])
        assert torch.allclose(got, ref[:300], atol=1e-4), (rank, (got - ref[:300]).abs().max().item())
        assert ps.Stats()["keys_stored"] == 4000
        ctx.check_status()
        dist.barrier()
        out[rank] = "ok"
    except BaseException as e:          # noqa: BLE001 - reported to the parent, then the process exits
        _leave(dist, rank, out, e)
    _leave(dist, rank, out, None)


def test_nvlink_parameter_client_across_ranks():
    """PS verbs served by HBM hash-table shards on two GPUs: keys put by one rank are read and updated by the other over
    the peer windows; concurrent updates of the same keys from both ranks add up on the owner."""
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_ps_worker, (2, _free_port(), out), 2)
    assert all(out.get(r) == "ok" for r in range(2)), dict(out)


def _hbm_emb_worker(rank, world, port, ns, out):
    """The reference-named training API (DistEmbedding + SparseRowWiseAdaGrad) on the HBM plane against the same loop on
    the host shared-memory table: identical ids and gradients, ranks touching disjoint rows (so the host path, where every
    rank applies its own update, is order-free), duplicates inside a rank."""
    dist = _init(rank, world, port)
    try:
        import recstore_b200 as rs
        from recstore_b200 import ipc
        from recstore_b200.dist_opt import SparseRowWiseAdaGrad
        from recstore_b200.parallel.peer import PeerContext
        ipc.set_namespace(ns)
        rs.kvinit()
        N, D, lr = 5000, 32, 0.1

        def init(t, shape, dtype):
            t.copy_((torch.arange(shape[0], dtype=dtype) % 97).unsqueeze(1).expand(shape) * 0.01 + 0.05)
        host = rs.DistEmbedding(N, D, name="hbm_ref", init_func=init) if rank == 0 else None
        dist.barrier()
        if rank != 0:
            host = rs.DistEmbedding(N, D, name="hbm_ref", init_func=init)
        ctx = PeerContext(rank, world, device=torch.device(f"cuda:{rank}"))
        hbm = rs.HbmDistEmbedding(ctx, N, D, "hbm_emb", init_func=init, max_keys=4096)
        o_host, o_hbm = SparseRowWiseAdaGrad([host], lr), SparseRowWiseAdaGrad([hbm], lr)
        g = torch.Generator().manual_seed(100 + rank)
        for step in range(3):
            ids = torch.randint(0, N // world, (600,), generator=g) * world + rank        # rows of this rank's own residue class
            ids[::7] = ids[0]                                                              # duplicates
            w = torch.randn(600, D, generator=g)
            a = host(ids, torch.device("cuda"))
            b = hbm(ids, torch.device("cuda"))
            assert torch.allclose(a, b, atol=1e-6), (step, (a - b).abs().max().item())
            (a * w.cuda()).sum().backward()
            (b * w.cuda()).sum().backward()
            o_host.step(); o_hbm.step()
            o_host.zero_grad(); o_hbm.zero_grad()
            torch.cuda.synchronize()
            dist.barrier()
        ctx.check_status()
        full = hbm.to_dense_tensor()
        if rank == 0:
            assert torch.allclose(full, host.weight, atol=1e-5, rtol=1e-5), (full - host.weight).abs().max().item()
        sd = o_hbm.local_state_dict()
        assert len(sd["emb_states"]["hbm_emb"]["ids"]) == hbm.table.local_global_ids()[hbm.table.local_global_ids() < N].numel()
        dist.barrier()
        out[rank] = "ok"
    except BaseException as e:          # noqa: BLE001
        _leave(dist, rank, out, e)
    _leave(dist, rank, out, None)


def test_dist_embedding_api_on_the_hbm_plane_matches_the_host_table():
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    _spawn(_hbm_emb_worker, (2, _free_port(), f"pytest_hbm_{os.getpid()}", out), 2)
    assert all(out.get(r) == "ok" for r in range(2)), dict(out)


@pytest.mark.parametrize("model", ["RESCAL", "TransR"])
def test_kge_matrix_models_two_gpus(model):
    """The models with a matrix per relation on two GPUs: the D rows of a relation's matrix are spread over both ranks
    (cyclic ownership of the row-blocked table) and still share one Adagrad accumulator value; training reduces the loss."""
    if _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    from recstore_b200.cli import kge_main
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    out, info = kge_main.main(["--device", "cuda", "--num_proc", "2", "--model_name", model, "--max_step", "150",
                               "--n_entities", "3000", "--n_triples", "30000", "--hidden_dim", "16", "--gamma", "8",
                               "--batch_size", "128", "--neg_sample_size", "32", "--log_interval", "1000"])
    assert len(out) == 2
    for r in (0, 1):
        assert out[r]["last_loss"] < 0.85 * out[r]["first_loss"], out[r]


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
