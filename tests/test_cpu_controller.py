"""Lookahead controller: heap invariants and the read-your-updates contract with ranks impersonated by threads."""
import json
import random
import threading

import pytest
import torch


def test_indexed_heap_random_ops_keep_invariants():
    from recstore_b200.controller import IndexedPriorityQueue
    pq = IndexedPriorityQueue()
    rnd = random.Random(0)
    ref = {}
    for it in range(20000):
        op = rnd.random()
        k = rnd.randrange(500)
        if op < 0.6:
            p = rnd.randrange(10000)
            pq.upsert(k, p); ref[k] = p
        elif op < 0.8:
            assert pq.erase(k) == (k in ref); ref.pop(k, None)
        elif ref:
            i, p = pq.pop()
            assert p == min(ref.values()) and ref[i] == p
            del ref[i]
        if it % 997 == 0:
            assert pq.CheckConsistency() and len(pq) == len(ref)
    assert pq.CheckConsistency()


@pytest.mark.parametrize("mode", ["CppSync", "CppAsyncV2", "CppAsync", "CppAsync/omp0", "CppAsync/omp2", "CppAsync/nodetect",
                                  "CppAsyncV2/omp2", "CppAsyncV2/detect"])
def test_controller_read_sees_all_previous_updates(mode):
    """4 'ranks' (threads sharing one controller, as the reference's VirtualEnvironment test does) read ids,
    produce gradients and call the AfterBackward protocol; at every read the table row must equal the
    value a fully synchronous SGD would have produced."""
    from recstore_b200.controller import KGCacheController, BasePerfSampler
    ranks, N, D, L, steps, per = 4, 2000, 8, 5, 40, 64
    clr = 0.5
    mode, _, variant = mode.partition("/")
    cfg = {"num_gpus": ranks, "L": L, "clr": clr, "dim": D, "backwardMode": mode, "nr_background_threads": 2,
           "full_emb_capacity": N, "cache_ratio": 0.05}
    if variant.startswith("omp"):
        cfg["update_pq_use_omp"] = int(variant[3:])       # how a step's keys enter the queue: serial / per rank / per shard group
    if variant == "nodetect":
        cfg["use_detect_thread"] = 0
    if variant == "detect":
        cfg["use_detect_thread"] = 1
    ctrl = KGCacheController.Init(json.dumps(cfg))
    table = torch.zeros(N, D)
    c = int(N * 0.05)
    caches = [torch.zeros(c, D) for _ in range(ranks)]
    ctrl.RegTensorsPerProcess(table, caches)
    oracle = torch.zeros(N, D)
    samplers = [BasePerfSampler(r, L, per, N, mode, ctrl, seed=3) for r in range(ranks)]
    for s in samplers:
        s.Prefill()
    barrier = threading.Barrier(ranks)
    errors = []
    keys_of = [None] * ranks
    grads_of = [None] * ranks

    def read(ids):
        out = table[ids].clone()
        cached = ids < c * ranks
        if cached.any():
            ci = ids[cached]
            own = ci // c
            out[cached] = torch.stack([caches[int(o)][int(i - o * c)] for i, o in zip(ci, own)])
        return out

    def worker(r):
        try:
            for step in range(steps):
                ids = next(samplers[r])
                got = read(ids)
                if not torch.allclose(got, oracle[ids], atol=1e-5):
                    errors.append((step, r, (got - oracle[ids]).abs().max().item()))
                g = torch.full((per, D), float(r + 1)) * (1 + step % 3)
                keys_of[r], grads_of[r] = ids, g
                ctrl.SetStepInput(r, ids, g)
                barrier.wait()
                if r == 0:
                    ctrl.ProcessOneStep(step)
                    for rr in range(ranks):                      # synchronous oracle
                        oracle.index_add_(0, keys_of[rr], -clr * grads_of[rr])
                    ctrl.BlockToStepN(step + 1)
                barrier.wait()
        except Exception as e:  # pragma: no cover
            errors.append(("exc", r, repr(e)))
            barrier.abort()

    ts = [threading.Thread(target=worker, args=(r,)) for r in range(ranks)]
    [t.start() for t in ts]
    [t.join(120) for t in ts]
    assert not errors, errors[:5]
    assert "pq:" in ctrl.PrintPq()
    ctrl.Drain()
    ctrl.StopThreads()
    assert ctrl.PendingCount() == 0
    # the strategies really differ: the first one flushes id by id and reads announcements through mailboxes + a detect
    # thread, the second one swaps whole buckets out; the upsert variant that was asked for is the one that ran
    st = ctrl.Stats()
    if mode == "CppAsync":
        assert st["bucket_swaps"] == 0 and st["flushed"] > 0
        assert (st["mailed_announcements"] > 0) == (variant != "nodetect")
    elif mode == "CppAsyncV2":
        assert st["bucket_swaps"] > 0 and (st["mailed_announcements"] > 0) == (variant == "detect")
    if mode != "CppSync":
        want = {"omp0": "upsert_serial", "omp2": "upsert_per_shard_group"}.get(variant, "upsert_per_rank")
        assert st[want] == steps and sum(st[k] for k in ("upsert_serial", "upsert_per_rank", "upsert_per_shard_group")) == steps, st
    full = table.clone()
    for r in range(ranks):
        full[r * c:(r + 1) * c] = caches[r]
    assert torch.allclose(full, oracle, atol=1e-4)


def test_sampler_ring_pops_the_batch_announced_for_the_current_step():
    """``next()`` pushes batch t + L (announcing its reads for step t + L) and pops batch t: the ids a rank reads at step t
    must be exactly the ones it announced for step t, L steps earlier (a ring of only L slots would hand out batch
    t + L instead, and every read would come L steps before its announcement)."""
    from recstore_b200.controller import BasePerfSampler

    class Recorder:
        def __init__(self):
            self.by_step = {}

        def PublishReads(self, rank, step, ids):
            self.by_step[step] = ids.clone()

    for L in (1, 2, 5):
        rec = Recorder()
        s = BasePerfSampler(0, L, 16, 1000, "CppAsyncV2", rec, seed=4)
        s.Prefill()
        assert sorted(rec.by_step) == list(range(L))
        for step in range(12):
            ids = next(s)
            assert torch.equal(ids, rec.by_step[step]), (L, step)
            assert max(rec.by_step) == step + L                 # the lookahead window stays L steps deep


def test_wrapper_after_backward_protocol():
    from recstore_b200.controller import KGCacheControllerWrapperBase, TestPerfSampler
    N, D = 100, 4
    cfg = json.dumps({"num_gpus": 1, "L": 3, "clr": 1.0, "dim": D, "backwardMode": "CppAsyncV2", "full_emb_capacity": N})
    w = KGCacheControllerWrapperBase.FactoryNew("RecStore", cfg, 0, 1)
    table = torch.zeros(N, D)
    w.init(table)
    smp = TestPerfSampler(0, 3, 10, N, "CppAsyncV2", w.controller)
    smp.Prefill()
    expect = torch.zeros(N, D)
    for step in range(10):
        ids = next(smp)
        assert torch.allclose(table[ids], expect[ids])
        g = torch.ones(10, D)
        w.controller.SetStepInput(0, ids, g)
        expect.index_add_(0, ids, -g)
        w.AfterBackward()
    w.GraceFullyStopThreads()
    assert torch.allclose(table, expect)
    d = KGCacheControllerWrapperBase.FactoryNew("Dummy", cfg)
    d.AfterBackward(); d.StopThreads()


def test_controller_refuses_hostile_configs_and_ranks():
    """Sizes from the JSON config size vectors and start threads; out-of-range values and rank arguments are errors,
    not crashes."""
    from recstore_b200 import _lib
    from recstore_b200.controller import KGCacheController
    good = {"num_gpus": 2, "L": 5, "clr": 0.1, "dim": 8, "full_emb_capacity": 100, "backwardMode": "CppSync", "cache_ratio": 0.1}
    for bad in ({"num_gpus": 0}, {"num_gpus": -3}, {"num_gpus": 100000}, {"L": -1}, {"dim": 0}, {"full_emb_capacity": -1},
                {"cache_ratio": 5.0}, {"backwardMode": "Nope"}, {"nr_background_threads": -4}, {"nr_background_threads": 100000}):
        with pytest.raises(_lib.RecStoreError):
            KGCacheController(json.dumps({**good, **bad}))
    ctrl = KGCacheController(json.dumps(good))
    table = torch.zeros(100, 8)
    caches = [torch.zeros(5, 8), torch.zeros(5, 8)]
    ctrl.RegTensorsPerProcess(table, caches)
    ids, g = torch.arange(4), torch.ones(4, 8)
    for rank in (-1, 2, 99):
        with pytest.raises(_lib.RecStoreError):
            ctrl.SetStepInput(rank, ids, g)
        with pytest.raises(_lib.RecStoreError):
            ctrl.PublishReads(rank, 0, ids)
    ctrl.SetStepInput(0, ids, g); ctrl.SetStepInput(1, ids, g)
    ctrl.ProcessOneStep(0)
    ctrl.StopThreads()
    # still alive after the refused calls: ids 0..3 live in rank 0's cache and took both ranks' gradients
    assert torch.allclose(caches[0][:4], torch.full((4, 8), -0.2)) and float(caches[1].abs().sum()) == 0.0
