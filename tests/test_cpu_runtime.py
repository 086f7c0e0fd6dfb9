"""Host runtime (no GPU): shared tensors, barrier, timers, Zipf, KV engines, DistTensor / optimizers."""
import math
import os
import multiprocessing as mp

import numpy as np
import pytest
import torch


@pytest.fixture(autouse=True)
def _ns():
    from recstore_b200 import ipc, kvstore
    ipc.set_namespace(f"pytest{os.getpid()}")
    ipc.IPCTensorFactory.ClearIPCMemory()
    kvstore.kvreset()
    yield
    ipc.IPCTensorFactory.ClearIPCMemory()
    ipc.MultiProcessBarrierFactory.ClearIPCMemory()
    kvstore.kvreset()


def _child_mutate(ns, q):
    from recstore_b200 import ipc
    ipc.set_namespace(ns)
    t = ipc.IPCTensorFactory.FindIPCTensorFromName("shared_a")
    t[1] = 7.0
    s = ipc.IPCTensorFactory.GetSlicedIPCTensorFromName("ring")
    s.Copy_(torch.arange(5, dtype=torch.int64))
    b = ipc.MultiProcessBarrierFactory.Create("b0", 2)
    b.Wait()
    q.put(("ok", ipc.IPCTensorFactory.ListIPCTensors()))


def test_ipc_tensor_shared_between_processes():
    from recstore_b200 import ipc
    ns = f"pytest{os.getpid()}"
    t = ipc.IPCTensorFactory.NewIPCTensor("shared_a", (4, 3), torch.float32)
    assert t is not None and t.abs().sum() == 0
    assert ipc.IPCTensorFactory.NewIPCTensor("shared_a", (4, 3), torch.float32) is None   # name taken
    ring = ipc.IPCTensorFactory.NewSlicedIPCTensor("ring", (16,), torch.int64)
    assert len(ring) == 0
    b = ipc.MultiProcessBarrierFactory.Create("b0", 2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_child_mutate, args=(ns, q))
    p.start()
    b.Wait()
    msg, names = q.get(timeout=60)
    p.join(60)
    assert msg == "ok" and set(names) >= {"shared_a", "ring"}
    assert torch.equal(t[1], torch.full((3,), 7.0))
    assert torch.equal(ring.GetSlicedTensor(), torch.arange(5))
    assert ipc.IPCTensorFactory.ClearIPCMemory() >= 2


def test_barrier_timeout_is_an_error_not_a_hang():
    from recstore_b200 import ipc, _lib
    b = ipc.MultiProcessBarrierFactory.Create("lonely", 2, timeout_ms=100)
    with pytest.raises(_lib.RecStoreError) as e:
        b.Wait()                       # the second party never arrives
    assert e.value.code == _lib.ERR_TIMEOUT


def test_timers_and_counters():
    from recstore_b200.utils import timer as T
    T.Reporter.Clear()
    t = T.Timer("unit:sleep")
    for _ in range(5):
        with t:
            pass
    T.Timer.ManualRecordNs("unit:manual", 2_000_000)
    T.PerfCounter.Record("unit:hit_ratio", 0.75)
    s = T.stats("unit:manual")
    assert s["count"] == 1 and abs(s["mean"] - 2e6) < 1
    assert T.stats("unit:sleep")["count"] == 5
    rep = T.Reporter.Report()
    assert "unit:hit_ratio" in rep and "P99" in rep
    T.Reporter.StartReportThread(10_000)
    T.Reporter.StopReportThread()


def test_zipf_native_matches_python_and_is_skewed():
    import ctypes as C
    from recstore_b200 import _lib
    from recstore_b200.utils.data import zipf_from_uniform
    _lib.register_signatures({"rs_zipf_from_uniform": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_ulonglong, C.c_double]),
                              "rs_zipf_fill": (C.c_int, [C.c_void_p, C.c_longlong, C.c_ulonglong, C.c_double, C.c_ulonglong, C.c_int])})
    rng = np.random.default_rng(0)
    for alpha in (0.9, 1.0, 1.2, 1.3):
        u = rng.random(20000)
        ref = zipf_from_uniform(u, 1_000_000, alpha)
        out = np.empty(20000, dtype=np.int64)
        _lib.call("rs_zipf_from_uniform", u.ctypes.data, out.ctypes.data, 20000, 1_000_000, alpha)
        assert (out == ref).mean() > 0.9999          # libm vs numpy pow may differ in the last ulp
        assert ref.min() >= 0 and ref.max() < 1_000_000
    ids = np.empty(100000, dtype=np.int64)
    _lib.call("rs_zipf_fill", ids.ctypes.data, 100000, 1000, 1.2, 7, 1)
    assert ids.min() >= 1 and ids.max() <= 1000
    assert (ids == 1).mean() > 0.1                    # heavy head


@pytest.mark.parametrize("engine", ["KVEngineMap", "KVEngineExtendibleHash", "KVEngineChunkHash", "KVEnginePoolMap"])
def test_kv_engine_put_get_mirror(engine):
    """Random put / get / erase against a Python dict mirror (the reference's client consistency test,
    src/grpc_ps/python_client/python_client_test.py:9-44, applied to every engine)."""
    from recstore_b200.storage import BaseKV, list_engines
    assert engine in list_engines()
    kv = BaseKV(engine, {"capacity": 50000, "value_size": 32})
    rng = np.random.default_rng(1)
    mirror = {}
    for rnd in range(30):
        keys = rng.integers(0, 20000, size=500)
        vals = torch.from_numpy(rng.standard_normal((500, 8)).astype(np.float32))
        kv.BatchPut(keys, vals)
        for k, v in zip(keys.tolist(), vals):
            mirror[k] = v
        q = rng.integers(0, 25000, size=400)
        got, found = kv.BatchGet(q)
        for i, k in enumerate(q.tolist()):
            if k in mirror:
                assert found[i] and torch.equal(got[i], mirror[k])
            else:
                assert not found[i] and got[i].abs().sum() == 0
        for k in rng.integers(0, 20000, size=50).tolist():
            assert kv.Erase(k) == (k in mirror)
            mirror.pop(k, None)
        assert len(kv) == len(mirror)
    assert set(kv.keys().tolist()) == set(mirror.keys())
    if engine == "KVEngineExtendibleHash":
        assert kv.check_consistency()
    kv.clear()
    assert len(kv) == 0 and kv.Get(int(next(iter(mirror)))) is None
    kv.BulkLoad(1000)                                  # key -> [key] * dim
    got, found = kv.BatchGet(torch.arange(1000))
    assert found.all() and torch.equal(got[:, 0], torch.arange(1000, dtype=torch.float32))
    assert "size=1000" in kv.DebugInfo()


def test_chunkhash_crash_recovery_and_hot_migration(tmp_path):
    from recstore_b200.storage import BaseKV
    cfg = {"capacity": 20000, "value_size": 16, "path": str(tmp_path / "kv"), "num_shards": 4}
    kv = BaseKV("KVEngineChunkHash", cfg)
    keys = torch.arange(0, 12000)
    kv.BatchPut(keys, keys.float().unsqueeze(1).repeat(1, 4))
    for k in range(0, 12000, 7):
        kv.Erase(k)
    n_live = len(kv)
    moved = kv.migrate_hot(keys[:2000])
    assert moved >= 0
    # "crash": drop the handle without Flush -> files stay marked dirty; reopen must rebuild the index
    kv._l.rs_kv_destroy  # noqa: B018  (destructor flushes; emulate a crash by reopening while still open)
    kv2 = BaseKV("KVEngineChunkHash", cfg)
    recovered, clean = kv2.recovery_state()
    assert recovered and not clean
    assert len(kv2) == n_live
    got, found = kv2.BatchGet(keys)
    exp = torch.ones(12000, dtype=torch.bool)
    exp[::7] = False
    assert torch.equal(found, exp)
    assert torch.equal(got[found][:, 0], keys[found].float())
    kv2.BatchPut(torch.arange(0, 12000, 7), torch.zeros(len(range(0, 12000, 7)), 4))   # free list was rebuilt
    assert len(kv2) == 12000
    kv2.close()
    kv.close()
    kv3 = BaseKV("KVEngineChunkHash", cfg)
    assert kv3.recovery_state() == (True, True) and len(kv3) == 12000


def test_dist_tensor_embedding_and_optimizers(tmp_path):
    import recstore_b200 as rs
    from recstore_b200.dist_tensor import DistTensor, DistEmbedding
    from recstore_b200 import dist_opt
    rs.kvinit()
    a = DistTensor((10, 3), torch.float32, name="a", persistent=True)
    a[1] = torch.tensor([1.0, 2.0, 3.0])
    assert torch.equal(a[torch.tensor([1])], torch.tensor([[1.0, 2.0, 3.0]]))
    assert len(a) == 10 and a.shape == (10, 3) and a.name == "a"

    def init(t, shape, dtype):
        t.copy_(torch.arange(shape[0], dtype=dtype).unsqueeze(1).expand(shape))   # row i == i
    emb = DistEmbedding(50, 4, name="emb", init_func=init)
    idx = torch.tensor([3, 3, 7, 9, 3])
    # --- SparseSGD: mean over duplicates
    opt = dist_opt.SparseSGD([emb], lr=0.5)
    e = emb(idx)
    (e * torch.arange(5.0).unsqueeze(1)).sum().backward()
    opt.step(); opt.zero_grad()
    w = emb.weight
    assert torch.allclose(w[3], torch.full((4,), 3 - 0.5 * (0 + 1 + 4) / 3))
    assert torch.allclose(w[7], torch.full((4,), 7 - 0.5 * 2)) and torch.allclose(w[9], torch.full((4,), 9 - 0.5 * 3))
    # --- row-wise Adagrad: reference semantics against a hand-written loop
    emb2 = DistEmbedding(50, 4, name="emb2", init_func=init)
    opt2 = dist_opt.SparseRowWiseAdaGrad([emb2], lr=0.1, eps=1e-10)
    w_ref = emb2.weight.clone(); s_ref = torch.zeros(50)
    for step in range(3):
        e = emb2(idx)
        g = torch.randn(5, 4, generator=torch.Generator().manual_seed(step))
        e.backward(g)
        opt2.step(); opt2.zero_grad()
        for i, k in enumerate(idx.tolist()):
            s_ref[k] += g[i].pow(2).mean()
        for i, k in enumerate(idx.tolist()):
            w_ref[k] -= 0.1 * g[i] / (s_ref[k].sqrt() + 1e-10)
    assert torch.allclose(emb2.weight, w_ref, atol=1e-5)
    # --- element-wise Adagrad runs (disabled upstream)
    emb3 = DistEmbedding(20, 4, name="emb3", init_func=init)
    opt3 = dist_opt.SparseAdagrad([emb3], lr=0.1)
    e = emb3(torch.tensor([1, 1, 2])); e.sum().backward(); opt3.step(); opt3.zero_grad()
    assert torch.allclose(emb3.weight[1], torch.full((4,), 1 - 0.1 * 1 / (1 + 1e-10)))
    # --- checkpoint round trip in the per-rank file format
    f = str(tmp_path / "opt.ckpt")
    opt2.save(f)
    assert os.path.exists(f + "_0")
    sd = torch.load(f + "_0", weights_only=False)
    assert set(sd) == {"params", "emb_states"} and sd["params"]["world_size"] == 1 and "_lr" in sd["params"]
    name = "emb2_SparseRowWiseAdaGrad_sum"
    assert torch.equal(sd["emb_states"]["emb2"]["states"][name], s_ref[sd["emb_states"]["emb2"]["ids"]].to(torch.float32)) or \
        torch.allclose(sd["emb_states"]["emb2"]["states"][name], s_ref[sd["emb_states"]["emb2"]["ids"]], atol=1e-6)
    opt2._state["emb2"].get_shm_tensor().zero_()
    opt2.load(f)
    assert torch.allclose(opt2._state["emb2"].get_shm_tensor(), s_ref, atol=1e-6)
    # scale-in: a 2-rank checkpoint loaded by 1 rank picks up both files
    sd0 = opt2.local_state_dict(); sd1 = opt2.local_state_dict()
    ids = torch.arange(50)
    sd0["params"]["world_size"] = 2; sd1["params"]["world_size"] = 2
    sd0["emb_states"]["emb2"] = {"ids": ids[0::2], "states": {name: torch.full((25,), 5.0)}}
    sd1["emb_states"]["emb2"] = {"ids": ids[1::2], "states": {name: torch.full((25,), 9.0)}}
    torch.save(sd0, f + "2_0"); torch.save(sd1, f + "2_1")
    opt2.load(f + "2")
    st = opt2._state["emb2"].get_shm_tensor()
    assert torch.equal(st[0::2], torch.full((25,), 5.0)) and torch.equal(st[1::2], torch.full((25,), 9.0))
    with pytest.warns(UserWarning):
        opt2.load(str(tmp_path / "missing"))


def test_renumbering_narrow_and_zipf_filler():
    from recstore_b200 import torch_op
    d = torch.empty(20, dtype=torch.int64)
    hot = [torch.tensor([5, 7, 19]), torch.tensor([0, 3])]
    torch_op.construct_renumbering_dict_op(d, 2, hot)
    assert d[[5, 7, 19]].tolist() == [0, 1, 2] and d[[0, 3]].tolist() == [3, 4]
    cold = [i for i in range(20) if i not in (5, 7, 19, 0, 3)]
    assert d[cold].tolist() == list(range(5, 20))                    # cold ids keep their relative order
    assert sorted(d.tolist()) == list(range(20))                     # a permutation
    with pytest.raises(Exception):
        torch_op.construct_renumbering_dict_op(d, 2, [torch.tensor([1]), torch.tensor([1])])
    buf = torch.zeros(1000, 100)
    v = torch_op.NarrowShapeTensor_op(buf, (7, 3), torch.int64)
    v.fill_(5)
    assert v.shape == (7, 3) and v.data_ptr() == buf.data_ptr()
    t = torch.empty(10000, dtype=torch.int64)
    torch_op.ZipfianTorchFiller(1000, 0.99).fillArrayTorch(t)
    assert t.min() >= 1 and t.max() <= 1000 and (t <= 10).float().mean() > 0.2


@pytest.mark.parametrize("sanitizer", ["thread", "address", "undefined"])
def test_host_runtime_under_sanitizers(tmp_path, sanitizer):
    """The host runtime (KV engines, parameter server + clients, lookahead controller with its background threads) built
    with -fsanitize=thread / address (+ leak check) and driven from several threads by the stand-alone stress driver: no
    sanitizer report, no broken invariant."""
    import os
    import subprocess
    import pytest
    from recstore_b200.build import build_host_stress
    try:
        exe = build_host_stress(sanitizer, out_dir=tmp_path)
    except RuntimeError as e:
        if "sanitizer runtime" in str(e):
            pytest.skip(str(e))
        raise
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66 report_signal_unsafe=0",
               ASAN_OPTIONS="detect_leaks=1 exitcode=67", UBSAN_OPTIONS="halt_on_error=1 exitcode=68 print_stacktrace=1")
    p = subprocess.run([str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert p.returncode == 0 and "host_stress: ok" in p.stdout and "Sanitizer" not in p.stdout and "runtime error" not in p.stdout, p.stdout[-3000:]


def test_kv_factory_refuses_out_of_range_configs_and_survives_junk_json():
    """Sizes that would wrap around in a cast are refused; arbitrary text as the JSON config never crashes the factory."""
    import ctypes as C
    import random
    from recstore_b200 import _lib
    lib = _lib.lib()
    h = C.c_void_p()
    for cfg in (b'{"capacity": 1e30, "value_size": 16}', b'{"capacity": -5, "value_size": 16}',
                b'{"capacity": 1024, "value_size": 99999999999}', b'{"capacity": 1024, "value_size": 0}'):
        assert lib.rs_kv_create(b"KVEngineChunkHash", cfg, C.byref(h)) != 0, cfg
    assert lib.rs_kv_create(b"NoSuchEngine", b'{"capacity": 16, "value_size": 16}', C.byref(h)) != 0
    rnd = random.Random(1)
    alphabet = '{}[]",:0123456789.eE-+ truefalsn\\abc\n'
    for _ in range(500):
        s = "".join(rnd.choice(alphabet) for _ in range(rnd.randrange(0, 60)))
        if rnd.random() < 0.5:
            s = '{"capacity": 1024, "value_size": 16, ' + s
        if lib.rs_kv_create(b"KVEngineMap", s.encode(), C.byref(h)) == 0:
            lib.rs_kv_destroy(h)


def test_foreign_or_damaged_shm_objects_are_refused():
    """A shared-memory object that is not one of ours, or whose header describes more data than is mapped, is an error
    at open time (readers trust the header afterwards)."""
    import os
    import struct
    import uuid
    from recstore_b200 import _lib, ipc
    ns = "t" + uuid.uuid4().hex[:8]
    ipc.set_namespace(ns)
    try:
        t = ipc.IPCTensorFactory.NewIPCTensor("good", (4, 3))
        t.fill_(2.0)
        assert ipc.IPCTensorFactory.FindIPCTensorFromName("good").sum().item() == 24.0
        good_path = f"/dev/shm/rsb200.{os.getuid()}.{ns}.good"
        raw = open(good_path, "rb").read()
        cases = {"junk": os.urandom(8192), "short": raw[:100], "empty": b""}
        pos = raw.find(struct.pack("<Q", 48))            # data_bytes of a 4 x 3 float tensor
        if pos >= 0:
            cases["oversized"] = raw[:pos] + struct.pack("<Q", 1 << 40) + raw[pos + 8:]
        for name, blob in cases.items():
            with open(f"/dev/shm/rsb200.{os.getuid()}.{ns}.{name}", "wb") as f:
                f.write(blob)
            with pytest.raises(_lib.RecStoreError):
                ipc.IPCTensorFactory.FindIPCTensorFromName(name)
    finally:
        ipc.IPCTensorFactory.ClearIPCMemory()
        for name in ("junk", "short", "empty", "oversized"):
            try:
                os.unlink(f"/dev/shm/rsb200.{os.getuid()}.{ns}.{name}")
            except OSError:
                pass
        ipc.set_namespace(f"pytest{os.getpid()}")         # what the fixture of this file set


def test_persist_slab_pool_allocates_frees_and_recovers(tmp_path):
    """Slabs of mixed sizes keep their bytes, freed slabs are reused, empty chunks return to the pool, and a reopened file
    has exactly the slabs that were live (the reference's PersistMemoryPool::Recovery, src/memory/persist_malloc.h)."""
    from recstore_b200.storage import PersistSlabPool
    path = str(tmp_path / "pool.bin")
    P = PersistSlabPool(path, 64 * 65536, chunk_bytes=65536)
    assert not P.recovered
    assert [P.class_size(s) for s in (1, 16, 17, 256, 257, 300, 1000, 1025)] == [16, 16, 32, 256, 320, 320, 1024, 1280]
    rng = np.random.default_rng(0)
    live = {}
    for i in range(3000):
        size = int(rng.choice([8, 24, 100, 152, 700, 5000]))
        off = P.malloc(size)
        assert off != 0 and off not in live and P.slab_size(off) >= size
        data = bytes([i % 251]) * size
        P.write(off, data)
        live[off] = data
        if i % 3 == 0:
            victim = list(live)[int(rng.integers(len(live)))]
            P.free(victim)
            assert P.slab_size(victim) == 0
            P.free(victim)                                  # a double free is ignored
            del live[victim]
    st = P.stats()
    assert st["slabs_in_use"] == len(live) and sorted(P.allocated()) == sorted(live)
    assert st["bytes_in_use"] <= st["bytes_reserved"] <= 64 * 65536
    for off, data in live.items():
        assert P.read(off, len(data)) == data
    with pytest.raises(Exception):
        P.write(next(iter(live)), b"x" * 70000)            # larger than the slab
    assert P.malloc(70000) == 0                            # larger than a chunk
    # "crash": a second mapping of the file while the first is still open sees the same live set
    Q = PersistSlabPool(path, 64 * 65536, chunk_bytes=65536)
    assert Q.recovered and sorted(Q.allocated()) == sorted(live) and Q.stats()["slabs_in_use"] == len(live)
    for off, data in list(live.items())[:200]:
        assert Q.read(off, len(data)) == data
    fresh = Q.malloc(152)
    assert fresh != 0 and fresh not in live                 # the rebuilt free lists do not hand out a live slab
    Q.free(fresh)
    Q.close()
    for off in list(live):
        P.free(off)
    assert P.stats()["slabs_in_use"] == 0 and P.stats()["chunks_in_use"] == 0
    # exhaustion: 64 chunks of 65536 bytes hold fewer than 64 * 16 slabs of 5000 (class 5120) bytes
    got = []
    while True:
        off = P.malloc(5000)
        if off == 0:
            break
        got.append(off)
    assert 64 * 11 <= len(got) <= 64 * 12 and len(set(got)) == len(got)
    P.close()
    R = PersistSlabPool(path, 64 * 65536, chunk_bytes=65536)
    assert R.recovered and R.stats()["slabs_in_use"] == len(got)
    R.close()
    assert not PersistSlabPool(path, 32 * 65536, chunk_bytes=32768).recovered     # another geometry: formatted anew


def test_epoch_manager_defers_frees_past_protected_regions():
    """A retired slab stays allocated while a reader that could have seen it is inside a protected region, and goes back
    to the pool afterwards (Protect / UnProtect / BumpCurrentEpoch / IsSafeToReclaim of src/memory/epoch_manager.h)."""
    import threading
    from recstore_b200.storage import EpochManager, PersistSlabPool
    P, E = PersistSlabPool(None, 16 * 65536, chunk_bytes=65536), EpochManager()
    e0 = E.current()
    assert E.safe_to_reclaim(e0)                            # nobody is protected
    inside, leave = threading.Event(), threading.Event()

    def reader():
        with E:
            inside.set()
            leave.wait(10)
    t = threading.Thread(target=reader)
    t.start()
    assert inside.wait(10)
    off = P.malloc(100)
    E.retire_slab(P, off)                                   # unlinked at epoch e0, the reader published e0
    assert not E.safe_to_reclaim(e0) and E.safe_to_reclaim(e0 - 1)
    E.bump()
    assert E.collect() == 0 and E.pending() == 1 and P.slab_size(off) != 0
    with E:                                                 # a reader that starts after the bump does not hold it up
        off2 = P.malloc(100)
        E.retire_slab(P, off2)
        assert E.collect() == 0                             # ... but protects what is unlinked during its own region
    leave.set()
    t.join()
    assert E.collect() == 2 and E.pending() == 0 and P.slab_size(off) == 0 and P.slab_size(off2) == 0
    with E:
        with E:                                             # regions nest
            pass
        assert not E.safe_to_reclaim(E.current())
    assert E.safe_to_reclaim(E.current())
    E.close()
    P.close()


def test_pool_map_engine_concurrent_readers_never_see_torn_or_freed_values(tmp_path):
    """Writers replace values out of place while readers copy them without the shard lock: every value a reader gets is
    one complete version, superseded records return to the pool (bounded slab count), and a reopen after a 'crash' keeps
    the newest sealed version of every key and forgets erased keys."""
    import threading
    from recstore_b200.storage import BaseKV
    cfg = {"capacity": 4096, "value_size": 256, "path": str(tmp_path / "pm")}
    kv = BaseKV("KVEnginePoolMap", cfg)
    keys = torch.arange(2000)
    kv.BatchPut(keys, torch.zeros(2000, 64))
    stop, bad = threading.Event(), []

    def writer(seed):
        g = torch.Generator().manual_seed(seed)
        v = 1
        try:
            while not stop.is_set():
                ks = torch.randint(0, 2000, (256,), generator=g)
                kv.BatchPut(ks, torch.full((256, 64), float(seed * 100000 + v)))
                v += 1
        except Exception as e:                              # a refused write (engine "full" of unreclaimed records) is a failure
            bad.append((seed, repr(e)))

    def reader(seed):
        g = torch.Generator().manual_seed(100 + seed)
        while not stop.is_set():
            ks = torch.randint(0, 2000, (512,), generator=g)
            got, found = kv.BatchGet(ks)
            if not bool(found.all()) or not bool((got == got[:, :1]).all()):
                bad.append((seed, got[(got != got[:, :1]).any(1)][:2]))
                return
    ts = [threading.Thread(target=writer, args=(i + 1,)) for i in range(2)] + [threading.Thread(target=reader, args=(i,)) for i in range(3)]
    for t in ts:
        t.start()
    import time
    time.sleep(1.5)
    stop.set()
    for t in ts:
        t.join()
    assert not bad, bad
    kv.Flush()                                              # what still waited for a reader's epoch is reclaimed now
    info = kv.DebugInfo()
    slabs = int(info.split("slabs=")[1].split()[0])
    assert len(kv) == 2000 and 2000 <= slabs <= 2000 + 4096 // 4 + 64 + 300, info     # old versions were reclaimed
    for k in range(0, 2000, 5):
        kv.Erase(k)
    final, _ = kv.BatchGet(keys)
    kv2 = BaseKV("KVEnginePoolMap", cfg)                    # reopened while the first is still mapped: a crash image
    rec, _clean = kv2.recovery_state()
    assert rec and len(kv2) == 1600
    got, found = kv2.BatchGet(keys)
    exp = torch.ones(2000, dtype=torch.bool)
    exp[::5] = False
    assert torch.equal(found, exp) and torch.equal(got[found], final[found])
    kv2.close()
    kv.close()


@pytest.mark.parametrize("engine", ["KVEngineChunkHash", "KVEnginePoolMap"])
def test_hash_api_adapter_semantics(engine):
    """find / insert / update / remove as a hash-evaluation harness calls them (PiBenchWrapper.cc of the reference)."""
    from recstore_b200.storage import HashAPI
    h = HashAPI(engine, {"capacity": 1000, "value_size": 16})
    one, two = torch.full((4,), 1.0), torch.full((4,), 2.0)
    assert h.find(5) is None and not h.update(5, one) and not h.remove(5)
    assert h.insert(5, one) and not h.insert(5, two) and torch.equal(h.find(5), one)
    assert h.update(5, two) and torch.equal(h.find(5), two) and len(h) == 1
    assert h.remove(5) and h.find(5) is None and len(h) == 0
    h.close()


def test_slab_recyclers_direct_delayed_and_epoch():
    """The three policies for returning a freed slab to its pool (DirectRecycle / DelayedRecycle / ShmEpochRecycle of
    src/memory/malloc.h:34-152)."""
    import time
    from recstore_b200.storage import EpochManager, PersistSlabPool, SlabRecycler
    P, E = PersistSlabPool(None, 16 * 65536, chunk_bytes=65536), EpochManager()
    with pytest.raises(ValueError):
        SlabRecycler(P, "sometimes")
    with pytest.raises(Exception):
        SlabRecycler(P, "epoch")                            # no epoch manager

    R = SlabRecycler(P, "direct")
    off = P.malloc(64)
    assert R.recycle(off) == 1 and P.slab_size(off) == 0 and R.pending() == 0 and R.recycle(0) == 0

    R = SlabRecycler(P, "delayed", delay_s=1.0)
    offs = [P.malloc(64) for _ in range(5)]
    assert sum(R.recycle(o) for o in offs) == 0 and R.pending() == 5 and all(P.slab_size(o) for o in offs)
    time.sleep(1.2)
    late = P.malloc(64)
    assert R.recycle(late) == 5 and R.pending() == 1          # the five are due, the new one waits
    assert all(P.slab_size(o) == 0 for o in offs) and P.slab_size(late) != 0
    R.set_delay(0.0)
    assert R.recycle(0) == 1 and R.pending() == 0
    R.set_delay(60.0)
    o = P.malloc(64)
    R.recycle(o)
    assert R.clear() == 1 and P.slab_size(o) == 0              # clear frees what is not due yet

    R = SlabRecycler(P, "epoch", epochs=E, bump_every=4)
    E.protect()                                             # this thread may still read what is unlinked from now on
    offs = [P.malloc(64) for _ in range(8)]
    assert sum(R.recycle(o) for o in offs) == 0 and R.pending() == 8
    E.unprotect()
    assert R.recycle(0) == 8 and R.pending() == 0 and all(P.slab_size(o) == 0 for o in offs)
    o = P.malloc(64)
    R.recycle(o)
    R.close()                                               # closing frees what is left
    assert P.slab_size(o) == 0 and P.stats()["slabs_in_use"] == 0
    E.close()
    P.close()


@pytest.mark.parametrize("engine", ["KVEngineMap", "KVEngineExtendibleHash", "KVEngineChunkHash", "KVEnginePoolMap"])
def test_load_db_helper_warms_one_shard_and_checks_it(engine):
    """Warm-up of a PS shard: the keys that the partition function gives this server, value = float(key) repeated, then
    the check that counts them (LoadDBHelper::PreLoadDB / CheckDBLoad, src/storage/kv_engine/load_db.h:13-165)."""
    from recstore_b200.ps.client import ShardManager
    from recstore_b200.storage import BaseKV, LoadDBHelper
    N, S = 20000, 3
    owner = ShardManager.KeyPartition(torch.arange(1, N + 1), S)
    total = 0
    for sid in range(S):
        kv = BaseKV(engine, {"capacity": N, "value_size": 32})
        h = LoadDBHelper(kv, sid, S, warm_thread_count=4, warm_capacity=N)
        mine = int((owner == sid).sum())
        assert h.PreLoadDB(shuffle_load=(sid == 1)) == mine and len(kv) == mine
        assert h.CheckDBLoad() == (mine, mine)
        k = int((owner == sid).nonzero()[0]) + 1
        assert torch.equal(kv.Get(k), torch.full((8,), float(k)))
        other = int((owner != sid).nonzero()[0]) + 1
        assert kv.Get(other) is None
        kv.Put(k, torch.zeros(8))                           # a damaged row is counted as wrong, not as missing
        assert h.CheckDBLoad() == (mine - 1, mine)
        total += mine
        kv.close()
    assert total == N
    small = BaseKV("KVEngineMap", {"capacity": 100, "value_size": 32})
    with pytest.raises(Exception):
        LoadDBHelper(small, 0, 1, 2, 1000).PreLoadDB()      # more keys than the engine holds: an error, not a silent cut
    small.close()


def test_histogram_percentiles_merge_and_report():
    """Whole-run distribution of a measurement (Histogram of src/base/timer.h:102-204)."""
    from recstore_b200.utils.timer import Histogram
    h = Histogram()
    assert h.summary()["count"] == 0 and h.Percentile(50) == 0.0
    v = torch.arange(1, 10001, dtype=torch.float64)
    h.Add(v)
    s = h.summary()
    assert s["count"] == 10000 and s["min"] == 1.0 and s["max"] == 10000.0 and abs(s["mean"] - 5000.5) < 1e-6
    assert abs(s["stddev"] - float(v.std(unbiased=False))) < 1e-3
    for p in (1, 25, 50, 90, 99, 99.9):
        exact = float(torch.quantile(v, p / 100.0))
        assert abs(h.Percentile(p) - exact) <= exact / 16 + 1, (p, h.Percentile(p), exact)
    assert h.Percentile(0) >= 1.0 and h.Percentile(100) == 10000.0 and h.Median() == h.Percentile(50)
    g = Histogram()
    g.Add(0.25)
    g.Add(3e6)
    g.Add(-5.0)                                             # counted as zero
    h.Merge(g)
    s = h.summary()
    assert s["count"] == 10003 and s["min"] == 0.0 and s["max"] == 3e6
    text = h.ToString()
    assert text.startswith("Count: 10003") and "Median" in text and "#" in text and text.count("\n") > 10
    h.Clear()
    assert h.summary()["count"] == 0
    h.close()
    g.close()


@pytest.mark.parametrize("engine", ["KVEngineChunkHash", "KVEnginePoolMap"])
def test_reinit_tool_wipes_a_persistent_engine_directory(tmp_path, engine):
    """`python -m recstore_b200.storage --command reinit --path DIR` (role of src/memory/pm_command.cc)."""
    import subprocess, sys
    from recstore_b200.storage import BaseKV
    d = tmp_path / "kv"
    cfg = {"capacity": 1000, "value_size": 16, "path": str(d), "num_shards": 2}
    kv = BaseKV(engine, cfg)
    kv.Put(7, torch.ones(4))
    kv.Flush()
    kv.close()
    (d / "notes.txt").write_text("keep me")
    kv = BaseKV(engine, cfg)
    assert len(kv) == 1                                      # the directory brings the data back
    kv.close()
    r = subprocess.run([sys.executable, "-m", "recstore_b200.storage", "--command", "reinit", "--path", str(d)],
                       capture_output=True, text=True, timeout=300, cwd=os.path.dirname(os.path.dirname(__file__)))
    assert r.returncode == 0 and "removed" in r.stdout, r.stderr
    assert (d / "notes.txt").exists()
    kv = BaseKV(engine, cfg)
    assert len(kv) == 0 and kv.Get(7) is None
    kv.close()


def test_index_ring_coarse_clock_and_core_binding():
    """Ring of free indices (src/base/lf_list.h), coarse clock (src/base/async_time.h), thread pinning
    (src/base/bind_core.cc)."""
    import threading, time
    from recstore_b200.utils.host import IndexRing, bind_core, coarse_now_ns, numa_node_cores, steady_now_ns
    r = IndexRing(8)
    assert len(r) == 0 and r.pop(4).size == 0
    assert r.push([1, 2, 3, 4, 5]) and not r.push([6, 7, 8, 9]) and len(r) == 5      # a batch that does not fit is refused whole
    assert r.pop(2).tolist() == [1, 2] and r.push([6, 7, 8, 9]) and len(r) == 7       # ... and fits once there is room (wraps)
    assert r.pop(100).tolist() == [3, 4, 5, 6, 7, 8, 9] and len(r) == 0
    r.push([1, 2])
    r.clear()
    assert len(r) == 0
    big, got, lock = IndexRing(1 << 12), [], threading.Lock()
    done = threading.Event()

    def consumer():
        mine = []
        while not (done.is_set() and len(big) == 0):
            mine.extend(big.pop(7).tolist())
        with lock:
            got.extend(mine)
    ts = [threading.Thread(target=consumer) for _ in range(3)]
    [t.start() for t in ts]
    nxt = 0
    while nxt < 30000:
        if big.push(range(nxt, nxt + 100)):
            nxt += 100
    done.set()
    [t.join() for t in ts]
    assert sorted(got) == list(range(30000))
    a = coarse_now_ns()
    time.sleep(0.05)
    b, exact = coarse_now_ns(), steady_now_ns()
    assert a < b <= exact and exact - b < 1_000_000_000
    cores = sorted(os.sched_getaffinity(0))
    t = threading.Thread(target=lambda: (bind_core(cores[-1]), got.append(os.sched_getaffinity(0))))
    t.start()
    t.join()
    assert got[-1] == {cores[-1]}
    n0 = numa_node_cores(0)
    assert isinstance(n0, list) and all(isinstance(c, int) for c in n0)
    with pytest.raises(Exception):
        bind_core(1 << 20)


def test_closing_a_pool_or_an_epoch_manager_first_settles_what_depends_on_it():
    """Shutdown in any order: a pool that closes first has its recyclers closed and its epoch managers drained (their
    pending frees would otherwise touch an unmapped pool); an epoch manager that closes first closes the recyclers that
    consult it."""
    from recstore_b200.storage import EpochManager, PersistSlabPool, SlabRecycler
    P, E = PersistSlabPool(None, 16 * 65536, chunk_bytes=65536), EpochManager()
    R1 = SlabRecycler(P, "delayed", delay_s=60.0)
    R2 = SlabRecycler(P, "epoch", epochs=E)
    offs = [P.malloc(64) for _ in range(6)]
    R1.recycle(offs[0]); R1.recycle(offs[1])
    E.protect()
    R2.recycle(offs[2]); R2.recycle(offs[3])
    E.retire_slab(P, offs[4]); E.retire_slab(P, offs[5])
    E.unprotect()
    assert R1.pending() == 2 and R2.pending() == 2 and E.pending() == 2
    P.close()                                               # recyclers closed, manager drained, then the pool unmapped
    assert R1._h is None and R2._h is None and E.pending() == 0
    assert E.collect() == 0                                 # nothing left that could touch the pool
    R1.close(); R2.close()                                  # closing again is harmless
    P2 = PersistSlabPool(None, 16 * 65536, chunk_bytes=65536)
    R3 = SlabRecycler(P2, "epoch", epochs=E)
    o = P2.malloc(64)
    E.protect(); R3.recycle(o); E.unprotect()
    E.close()                                               # the manager goes first: its recycler is closed (and frees o)
    assert R3._h is None and P2.slab_size(o) == 0
    P2.close()


def test_symmetric_allocator_is_deterministic_reuses_and_merges():
    """The offset allocator of the peer heap: same calls, same layout (that is what lets every rank run it alone);
    freed blocks are reused lowest-address first and merge with free neighbours."""
    import random
    from recstore_b200.parallel.peer import SymmetricAllocator
    a = SymmetricAllocator(10 * 256 + 100)                  # rounded down to whole alignment units
    assert a.nbytes == 2560 and a.largest_free == 2560
    x, y, z = a.alloc(1), a.alloc(512), a.alloc(300)
    assert (x, y, z) == (0, 256, 768) and a.bytes_in_use == 256 + 512 + 512
    assert a.alloc(4096) is None and a.alloc(1281) is None and a.bytes_in_use == 1280
    a.free(y)
    assert a.alloc(600) == 1280                             # 600 -> 768 bytes: too big for the 512-byte hole, placed in the tail
    a2 = SymmetricAllocator(2560)
    for n in (1, 512, 300):
        a2.alloc(n)
    a2.free(256)
    assert a2.alloc(512) == 256                             # exact hole reused
    a2.free(0); a2.free(256)
    assert (0, 768, "free") in a2.layout()                  # neighbours merged into one block
    a2.free(768)
    assert a2.layout() == [(0, 2560, "free")] and a2.bytes_in_use == 0
    with pytest.raises(ValueError):
        a2.free(768)
    # two "ranks" replay one random script: identical offsets throughout, no overlap, everything inside the heap
    script, rng, live = [], random.Random(5), []
    for i in range(2000):
        if live and rng.random() < 0.45:
            script.append(("free", live.pop(rng.randrange(len(live)))))
        else:
            script.append(("alloc", rng.randrange(1, 40000)))
            live.append(len(script) - 1)
    def replay():
        h, got, out = SymmetricAllocator(1 << 20), {}, []
        for i, (op, v) in enumerate(script):
            if op == "alloc":
                got[i] = h.alloc(v)
                out.append(got[i])
            elif got.get(v) is not None:
                h.free(got.pop(v))
            used = sorted((o, s) for o, s, k in h.layout() if k == "used")
            assert all(o1 + s1 <= o2 for (o1, s1), (o2, _) in zip(used, used[1:])) and (not used or used[-1][0] + used[-1][1] <= 1 << 20)
        return out
    r0, r1 = replay(), replay()
    assert r0 == r1 and sum(o is not None for o in r0) > 500
