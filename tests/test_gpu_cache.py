"""GPU hash table, set-associative cache, unique, merge / range-cache ops against CPU mirrors."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from recstore_b200 import _lib
    _lib.lib()
    return torch.device("cuda:0")


def test_hash_table_insert_lookup_erase_dump(dev):
    from recstore_b200.cache import GpuHashTable
    g = torch.Generator().manual_seed(0)
    ht = GpuHashTable(capacity=1 << 16, max_rows=30000, device=dev)
    keys = torch.randint(0, 1 << 40, (20000,), generator=g)
    keys = torch.cat([keys, keys[:5000]])                      # duplicates inside one launch
    rows = ht.insert(keys).cpu()
    uniq = torch.unique(keys)
    assert (rows >= 0).all() and rows.max() < 30000
    m = {}
    for k, r in zip(keys.tolist(), rows.tolist()):
        assert m.setdefault(k, r) == r                          # same key -> same row
    assert len(set(m.values())) == len(m) == uniq.numel()       # distinct keys -> distinct rows
    live, size, bad = ht.check()
    assert live == size == uniq.numel() and bad == 0
    q = torch.cat([keys[:100], torch.arange(1 << 41, (1 << 41) + 50)])
    got = ht.lookup(q).cpu()
    assert torch.equal(got[:100], rows[:100]) and (got[100:] == -1).all()
    gone = uniq[::3]
    ht.erase(gone)
    assert (ht.lookup(gone).cpu() == -1).all()
    live, size, bad = ht.check()
    assert live == size == uniq.numel() - gone.numel() and bad == 0
    r2 = ht.insert(gone[:100]).cpu()                            # freed rows are reused
    assert (r2 >= 0).all() and r2.max() < 30000
    dk, dr = ht.dump()
    assert set(dk.cpu().tolist()) == (set(uniq.tolist()) - set(gone.tolist())) | set(gone[:100].tolist())
    assert ht.status.item() == 0
    # row store exhaustion is reported, not fatal
    small = GpuHashTable(capacity=1024, max_rows=10, device=dev)
    r = small.insert(torch.arange(100)).cpu()
    assert (r >= 0).sum().item() == 10 and small.status.item() != 0
    ht.clear()
    assert ht.check()[0] == 0


def test_unique_keys(dev):
    from recstore_b200.cache import unique_keys
    g = torch.Generator().manual_seed(1)
    keys = torch.randint(0, 5000, (100000,), generator=g).to(dev)
    st = torch.zeros(1, dtype=torch.int64, device=dev)
    u, inv = unique_keys(keys, st)
    assert st.item() == 0
    assert torch.equal(torch.sort(u).values, torch.unique(keys))
    assert torch.equal(u[inv], keys)


def test_reserved_keys_are_refused_not_miscounted(dev):
    """-1 (empty marker) and -2 (tombstone) mixed into a batch: unique() gives them inverse -1 and does not count
    them, erase() frees nothing for them, and both say so in the status word.  Compared with a CPU oracle."""
    from recstore_b200 import _lib
    from recstore_b200.cache import GpuHashTable, unique_keys
    g = torch.Generator().manual_seed(5)
    keys = torch.randint(0, 300, (4000,), generator=g)
    keys[::7] = -1
    keys[3::11] = -2
    st = torch.zeros(1, dtype=torch.int64, device=dev)
    u, inv = unique_keys(keys.to(dev), st)
    u, inv = u.cpu(), inv.cpu()
    real = keys >= 0
    assert st.item() & _lib.DEV_BAD_ARG
    assert torch.equal(torch.sort(u).values, torch.unique(keys[real]))          # count and contents: CPU oracle
    assert (inv[~real] == -1).all()
    assert torch.equal(u[inv[real]], keys[real])
    ht = GpuHashTable(capacity=1 << 12, max_rows=1000, device=dev)
    ht.insert(torch.arange(100))
    assert ht.status.item() == 0
    r = ht.erase(torch.tensor([-1, -2, 5, -1])).cpu()
    assert r[0] == -1 and r[1] == -1 and r[3] == -1 and r[2] >= 0
    assert ht.status.item() & _lib.DEV_BAD_ARG
    live, size, bad = ht.check()
    assert live == size == 99 and bad == 0                                      # only key 5 went away; free stack intact
    assert (ht.lookup(torch.tensor([-1, -2])).cpu() == -1).all()
    r2 = ht.insert(torch.tensor([1000, 1001])).cpu()
    assert (r2 >= 0).all() and r2.max() < 1000 and len(set(r2.tolist())) == 2


def test_gpu_cache_query_replace_update_dump(dev):
    from recstore_b200.cache import GpuCache, merge_op
    D = 32
    cache = GpuCache(4096, D, device=dev)
    table = torch.arange(100000, dtype=torch.float32, device=dev).unsqueeze(1).repeat(1, D)   # row i == i
    g = torch.Generator().manual_seed(2)
    mirror = set()
    for it in range(20):
        keys = torch.randint(0, 3000, (2000,), generator=g).to(dev)
        vals = torch.full((2000, D), -1.0, device=dev)
        res = cache.Query(keys, vals)
        hit = torch.ones(2000, dtype=torch.bool, device=dev)
        hit[res.missing_index] = False
        assert torch.equal(vals[hit][:, 0], keys[hit].float())                 # hits carry the right rows
        assert (vals[~hit] == -1).all()                                         # misses untouched
        assert torch.equal(torch.sort(res.missing_keys).values, torch.sort(keys[~hit]).values)
        for k in keys[hit].unique().tolist():
            assert k in mirror
        fetched = table[res.missing_keys]
        merge_op(vals, fetched, res.missing_index)
        assert torch.equal(vals[:, 0], keys.float())
        cache.Replace(res.missing_keys, fetched)
        mirror |= set(res.missing_keys.tolist())
    dumped = set(cache.Dump().tolist())
    assert dumped <= mirror and len(dumped) >= min(len(mirror), 2000)
    # everything fits (3000 keys < 4096 slots, ~23 per 32-way set on average): the hit rate is high now
    keys = torch.arange(3000, device=dev)
    res = cache.Query(keys)
    assert res.missing_keys.numel() < 300
    # Update overwrites cached rows only
    cache.Update(torch.tensor([1, 2, 999999], device=dev), torch.full((3, D), 5.0, device=dev))
    res = cache.Query(torch.tensor([1, 2, 999999], device=dev))
    assert 999999 in res.missing_keys.tolist()
    hitmask = torch.ones(3, dtype=torch.bool); hitmask[res.missing_index.cpu()] = False
    assert (res.values.cpu()[hitmask] == 5.0).all()
    assert cache.status.item() == 0
    # LRU: a set that overflows evicts the least recently used key
    c2 = GpuCache(32, 4, device=dev)                                           # one set
    c2.Replace(torch.arange(32, device=dev), torch.zeros(32, 4, device=dev))
    c2.Query(torch.arange(1, 32, device=dev))                                  # touch all but key 0
    c2.Replace(torch.tensor([100], device=dev), torch.ones(1, 4, device=dev))
    assert 0 not in c2.Dump().tolist() and 100 in c2.Dump().tolist()


def test_range_cache_query(dev):
    from recstore_b200.cache import uva_cache_query_op
    D = 12                                                   # not a multiple of 4: scalar path
    host = torch.arange(1000, dtype=torch.float32).unsqueeze(1).repeat(1, D).pin_memory()
    start, end = 100, 300
    hbm = (host[start:end] + 0.5).to(dev)                    # cached copy is distinguishable
    ids = torch.tensor([0, 100, 299, 300, 999, 150], device=dev)
    out = torch.zeros(6, D, device=dev)
    st = torch.zeros(1, dtype=torch.int64, device=dev)
    uva_cache_query_op(out, ids, hbm, host, start, end, st)
    torch.cuda.synchronize()
    assert torch.equal(out[:, 0].cpu(), torch.tensor([0, 100.5, 299.5, 300, 999, 150.5]))
    assert st.item() == 0


def test_sharded_table_single_gpu(dev):
    """The row-sharded table degenerates to a local gather / update on one GPU (same kernels, local windows)."""
    from recstore_b200.parallel.peer import PeerContext
    from recstore_b200.parallel.sharded_table import ShardedEmbeddingTable
    from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update, sgd_update
    ctx = PeerContext(0, 1, device=dev)
    N, D, n = 2000, 16, 4096
    for opt in ("rowwise_adagrad", "sgd"):
        tab = ShardedEmbeddingTable(ctx, f"solo_{opt}", N, D, max_keys=n, lr=0.1, eps=1e-8, optimizer=opt, init="row_index")
        W = torch.arange(N, device=dev, dtype=torch.float32).unsqueeze(1).repeat(1, D)
        S = torch.zeros(N, device=dev)
        g = torch.Generator(device=dev).manual_seed(3)
        for step in range(3):
            ids = torch.randint(0, N, (n,), device=dev, generator=g)
            rows = tab.lookup(ids)
            assert torch.allclose(rows, W[ids], atol=1e-4)
            grads = torch.randn(n, D, device=dev, generator=g)
            tab.update(grads)
            if opt == "sgd":
                sgd_update(W, ids, grads, 0.1)
            else:
                rowwise_adagrad_update(W, S, ids, grads, 0.1, 1e-8)
        torch.cuda.synchronize()
        ctx.check_status()
        assert torch.allclose(tab.weight, W, atol=2e-3, rtol=2e-3)


def _key_init_rows(keys, D, scale):
    """CPU mirror of the hash-table shard's first-touch initial row (a function of key and column only)."""
    import numpy as np
    M = np.uint64(0xFFFFFFFFFFFFFFFF)
    with np.errstate(over="ignore"):
        k = np.asarray(keys, dtype=np.uint64)[:, None] * np.uint64(0x9E3779B97F4A7C15) + (np.arange(D, dtype=np.uint64)[None, :] + np.uint64(1))
        k ^= k >> np.uint64(33); k *= np.uint64(0xff51afd7ed558ccd)
        k ^= k >> np.uint64(33); k *= np.uint64(0xc4ceb9fe1a85ec53)
        k ^= k >> np.uint64(33)
    u = (k >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return torch.from_numpy((u * np.float32(2.0) - np.float32(1.0)) * np.float32(scale))


@pytest.mark.parametrize("dedup", [True, False])
def test_hashed_shard_first_touch_lookup_update_dump(dev, dedup):
    """A shard whose storage is the HBM hash table: arbitrary 64-bit keys, inserted when first looked up with a row
    derived from the key, updated in place by row-wise Adagrad, enumerated by dump().  Against a dict on the CPU."""
    from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update
    from recstore_b200.parallel.peer import PeerContext
    from recstore_b200.parallel.sharded_table import ShardedEmbeddingTable
    ctx = PeerContext(0, 1, device=dev)
    D, n, scale = 32, 3000, 0.05
    tab = ShardedEmbeddingTable(ctx, f"hashed{int(dedup)}", 8000, D, max_keys=n, lr=0.1, eps=1e-8, dedup=dedup, hashed=True,
                                init_scale=scale)
    g = torch.Generator().manual_seed(11)
    pool = torch.randint(1 << 40, 1 << 62, (4000,), generator=g)                # nothing like row numbers
    oracle_w, oracle_s = {}, {}
    for step in range(4):
        ids = pool[torch.randint(0, pool.numel(), (n,), generator=g)]
        ids[::7] = pool[5]                                                       # a hot key
        new = [k for k in set(ids.tolist()) if k not in oracle_w]
        if new:
            init = _key_init_rows(new, D, scale)
            for k, r in zip(new, init):
                oracle_w[k], oracle_s[k] = r.clone(), 0.0
        rows = tab.lookup(ids.to(dev)).cpu()
        ref = torch.stack([oracle_w[k] for k in ids.tolist()])
        assert torch.allclose(rows, ref, atol=1e-6), (step, (rows - ref).abs().max())
        grads = torch.randn(n, D, generator=g)
        tab.update(grads.to(dev))
        # oracle update on a dense copy of the touched keys
        uk = sorted(set(ids.tolist()))
        pos = {k: i for i, k in enumerate(uk)}
        W = torch.stack([oracle_w[k] for k in uk]); S = torch.tensor([oracle_s[k] for k in uk])
        rowwise_adagrad_update(W, S, torch.tensor([pos[k] for k in ids.tolist()]), grads, 0.1, 1e-8)
        for k, i in pos.items():
            oracle_w[k], oracle_s[k] = W[i], float(S[i])
    torch.cuda.synchronize()
    ctx.check_status()
    keys, vals = tab.dump()
    assert sorted(keys.cpu().tolist()) == sorted(oracle_w)                       # exactly the keys that were ever looked up
    ref = torch.stack([oracle_w[k] for k in keys.cpu().tolist()])
    assert torch.allclose(vals.cpu(), ref, atol=2e-4, rtol=2e-4)


def test_tiered_table_lookup_and_adagrad_on_both_tiers():
    from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update
    from recstore_b200.cache.tiered_table import TieredEmbeddingTable
    dev = torch.device("cuda:0")
    N, D = 5000, 32
    t = TieredEmbeddingTable(N, D, hbm_ratio=0.1, max_keys=4096, lr=0.05, device=dev, init="row_index")
    assert t.hot_rows == 500 and t.cold.is_pinned()
    g = torch.Generator(device=dev).manual_seed(0)
    ids = torch.randint(0, N, (3000,), device=dev, generator=g)
    ids[::4] = 7            # hot duplicate
    ids[1::9] = 4321        # cold duplicate
    out = t.lookup(ids)
    assert torch.equal(out[:, 0].cpu(), ids.float().cpu()) and torch.equal(out[:, -1].cpu(), ids.float().cpu())
    hs = t.hit_stats()
    assert hs["hbm_rows"] + hs["host_rows"] == torch.unique(ids).numel() and 0 < hs["hit_ratio"] < 1
    # two optimizer steps against the reference semantics on a dense copy of the table
    W = torch.arange(N, dtype=torch.float32, device=dev).unsqueeze(1).expand(-1, D).contiguous()
    S = torch.zeros(N, device=dev)
    for step in range(2):
        ids = torch.randint(0, N, (3000,), device=dev, generator=g)
        ids[::5] = 11
        ids[2::7] = 4000
        grads = torch.randn(3000, D, device=dev, generator=g)
        t.lookup(ids)
        t.update(grads)
        rowwise_adagrad_update(W, S, ids, grads, 0.05, 1e-10)
    torch.cuda.synchronize()
    full = torch.cat([t.hot.cpu(), t.cold])
    assert torch.allclose(full, W.cpu(), atol=1e-4, rtol=1e-5)
    assert torch.allclose(torch.cat([t.hot_state.cpu(), t.cold_state]), S.cpu(), atol=1e-5, rtol=1e-5)
    assert t.status.item() == 0


def test_tiered_table_lookahead_prefetch_is_exact():
    """The same id / gradient stream with and without staging the next batch one step ahead: identical rows out,
    identical tables at the end (the rows a step updates are re-read into the staged copy)."""
    from recstore_b200.cache.tiered_table import TieredEmbeddingTable
    dev = torch.device("cuda:0")
    N, D, n = 4000, 32, 2500
    mk = lambda: TieredEmbeddingTable(N, D, hbm_ratio=0.15, max_keys=4096, lr=0.05, device=dev, init="row_index")
    plain, ahead = mk(), mk()
    g = torch.Generator(device=dev).manual_seed(1)
    batches = []
    for _ in range(6):
        ids = torch.randint(0, N, (n,), device=dev, generator=g)
        ids[::6] = 5                  # hot duplicate shared by consecutive steps
        ids[1::11] = 3900             # cold duplicate shared by consecutive steps
        batches.append((ids, torch.randn(n, D, device=dev, generator=g)))
    outs_plain, outs_ahead = [], []
    for ids, gr in batches:
        outs_plain.append(plain.lookup(ids).clone())
        plain.update(gr)
    for i, (ids, gr) in enumerate(batches):
        outs_ahead.append(ahead.lookup(ids).clone())
        if i + 1 < len(batches):
            ahead.prefetch(batches[i + 1][0])
        ahead.update(gr)
    torch.cuda.synchronize()
    # (duplicate gradients are summed with atomics, so two runs agree to rounding, not bit for bit; a stale staged row
    # would be off by a whole optimizer step, ~1e-2 here)
    close = lambda x, y: torch.allclose(x, y, rtol=1e-5, atol=1e-5)
    for i, (a, b) in enumerate(zip(outs_plain, outs_ahead)):
        assert close(a, b), (i, (a - b).abs().max().item())
    assert close(plain.hot, ahead.hot) and close(plain.cold, ahead.cold)
    assert close(plain.cold_state, ahead.cold_state)
    st = ahead.hit_stats()
    assert st["prefetched_lookups"] == len(batches) - 1 and st["staged_rows_refreshed"] > 0
    assert ahead.status.item() == 0


def test_lookahead_cached_table_reads_its_own_updates(dev):
    """Host-resident table + write-back HBM cache fed by the lookahead window: batches are announced two steps ahead,
    their missing rows are gathered on the host and copied to the device on a side stream, inserted at the step that
    uses them (evicting and writing back dirty rows), read, and updated in the cache.  Every lookup must return what a
    plain table updated synchronously would hold; after a flush the host table equals it."""
    from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update
    from recstore_b200.cache import LookaheadCachedTable
    N, D, n, L, steps = 20000, 32, 512, 2, 40
    tab = LookaheadCachedTable(N, D, cache_rows=8192, max_keys=n, lr=0.1, eps=1e-8, device=dev, lookahead=L, init="row_index")
    W = torch.arange(N, dtype=torch.float32, device=dev).unsqueeze(1).repeat(1, D)
    S = torch.zeros(N, device=dev)
    g = torch.Generator(device=dev).manual_seed(21)
    batches = [torch.randint(0, N, (n,), device=dev, generator=g) for _ in range(steps + L)]
    for b in batches:
        b[::9] = 7                                       # a hot id in every batch
    for t in range(L):
        tab.prefetch(batches[t], t)
    for t in range(steps):
        tab.prefetch(batches[t + L], t + L)              # the sampler is L steps ahead
        ids = batches[t]
        rows = tab.lookup(ids, t)
        assert torch.allclose(rows, W[ids], atol=1e-3, rtol=1e-5), (t, (rows - W[ids]).abs().max().item())
        grads = torch.randn(n, D, device=dev, generator=g)
        tab.update(grads)
        rowwise_adagrad_update(W, S, ids, grads, 0.1, 1e-8)
    tab.check()
    st = tab.stats
    assert st["late_announcements"] == 0 and st["staged_rows"] > 0 and st["written_back_rows"] > 0, st   # rows did migrate both ways
    tab.flush()
    assert torch.allclose(tab.weights(), W.cpu(), atol=2e-3, rtol=1e-5)
    assert torch.allclose(tab.state(), S.cpu(), atol=1e-2, rtol=2e-3)
    # a batch that was never announced is fetched on demand (counted), and is still right
    extra = torch.randint(0, N, (n,), device=dev, generator=g)
    rows = tab.lookup(extra, steps + L)
    assert torch.allclose(rows, W[extra], atol=1e-3, rtol=1e-5) and tab.stats["late_announcements"] == 1
    tab.close()


def test_lookahead_cached_table_withheld_staging_and_undersized_cache(dev):
    """Failure paths made on the host: (a) the staging of an announced batch never arrives (the worker is told to hold
    it): the lookup gives up after its time limit with an error instead of hanging; (b) a cache too small for the window
    refuses inserts and says so through the status word."""
    from recstore_b200 import _lib
    from recstore_b200.cache import LookaheadCachedTable
    tab = LookaheadCachedTable(1000, 16, cache_rows=1024, max_keys=64, device=dev, lookahead=1, wait_timeout_s=0.3)
    ids = torch.arange(64, device=dev)
    tab._hold.set()
    tab.prefetch(ids, 0)
    with pytest.raises(_lib.RecStoreError) as e:
        tab.lookup(ids, 0)
    assert e.value.code == _lib.ERR_TIMEOUT
    assert torch.ones(4, device=dev).sum().item() == 4          # the context is fine
    tab.close()
    small = LookaheadCachedTable(100000, 16, cache_rows=64, max_keys=2048, device=dev, lookahead=1, init="row_index")
    ids = torch.arange(2048, device=dev) * 7
    small.prefetch(ids, 0)
    small.lookup(ids, 0)
    with pytest.raises(_lib.DeviceStatusError) as e2:
        small.check()
    assert "table_full" in str(e2.value)
    small.close()


def test_nvlink_parameter_client_verbs_on_one_gpu(dev, tmp_path):
    """The parameter-server verbs served by an HBM hash-table shard: absent keys read as zeros (and say so), put
    overwrites, update applies SGD on the owner, stats count, a checkpoint round-trips.  Against a dict."""
    from recstore_b200.parallel.peer import PeerContext
    from recstore_b200.ps.gpu_client import NvlinkParameterClient
    ctx = PeerContext(0, 1, device=dev)
    D = 16
    ps = NvlinkParameterClient(ctx, emb_dim=D, capacity=20000, max_batch=4096, lr=0.5, name="ps_test")
    g = torch.Generator().manual_seed(3)
    keys = torch.randperm(1 << 20, generator=g)[:3000] + (1 << 33)
    vals = torch.randn(3000, D, generator=g)
    rows, found = ps.GetParameterWithMask(keys[:100])
    assert not found.any() and rows.abs().sum().item() == 0
    ps.PutParameter(keys, vals)
    rows, found = ps.GetParameterWithMask(torch.cat([keys[:500], keys[:5] + 1]))
    assert found[:500].all() and not found[500:].any()
    assert torch.equal(rows[:500].cpu(), vals[:500])
    grads = torch.randn(1000, D, generator=g)
    idx = torch.randint(0, 200, (1000,), generator=g)                      # duplicates: folded before they travel
    ps.UpdateParameter(keys[idx], grads)
    ref = vals.clone()
    ref.index_add_(0, idx, -0.5 * grads)
    got = ps.GetParameter(keys[:200]).cpu()
    assert torch.allclose(got, ref[:200], atol=1e-5)
    ps.PutParameter(keys[:10], torch.ones(10, D))                           # put overwrites
    assert torch.equal(ps.GetParameter(keys[:10]).cpu(), torch.ones(10, D))
    assert ps.Stats()["keys_stored"] == 3000
    ps.SaveCkpt(str(tmp_path / "ps"))
    ps.ClearPS()
    assert ps.Stats()["keys_stored"] == 0 and not ps.GetParameterWithMask(keys[:50])[1].any()
    ps.LoadCkpt(emb_file_path=str(tmp_path / "ps"))
    assert ps.Stats()["keys_stored"] == 3000
    assert torch.allclose(ps.GetParameter(keys[10:200]).cpu(), ref[10:200], atol=1e-5)
    ps.LoadFakeData(1000)
    assert torch.equal(ps.GetParameter(torch.tensor([5, 999]))[:, 0].cpu(), torch.tensor([5.0, 999.0]))
    ctx.check_status()


@pytest.mark.parametrize("choice", ["LocalCachedEmbedding", "ShardedCachedEmbedding"])
def test_hash_cache_embeddings_stay_coherent_with_the_host_table(choice):
    """The on-demand hash-cache placements on one GPU: rows are filled from the host table on a miss, evicted under
    pressure (the cache holds 2 % of the table) and updated in backward, so every step's forward output equals a
    replicated ``nn.Embedding`` trained with the same gradients."""
    from recstore_b200.cli import perf_emb
    out = perf_emb.main(["--num_workers", "1", "--device", "cuda", "--run_steps", "30", "--diff_test", "--emb_choice", choice,
                         "--backwardMode", "CppSync", "--batch_size", "2000", "--num_embs", "20000", "--cache_ratio", "0.02",
                         "--log_interval", "1000"])
    assert len(out) == 1 and out[0][0] == 30 and out[0][1] < 1e-3, out


@pytest.mark.parametrize("D,alpha", [(32, 1.2), (128, 1.05), (32, 0.0), (400, 1.2)])
def test_segment_sum_of_duplicate_keys_matches_index_add(D, alpha):
    """Folding the gradients of duplicate keys (sum and sum of squared norms per unique key): skewed keys go through the
    CTA-level combine (hot keys meet in shared memory first), keys without duplicates and rows wider than 128 floats take
    the direct path; entries marked -1 are skipped.  Oracle: torch.index_add_ in fp64."""
    from recstore_b200 import _lib
    from recstore_b200._lib import ptr, stream_ptr
    from recstore_b200.parallel import sharded_table  # noqa: F401  (registers rs_segment_sum)
    from recstore_b200.utils.data import zipf_ids_torch
    dev = torch.device("cuda:0")
    n, U = 150_000, 20_000
    if alpha > 0:
        inv = zipf_ids_torch(n, U, alpha, device=dev).to(torch.int32)
    else:
        inv = torch.randperm(n, device=dev)[:n].to(torch.int32) % U      # every key at most three times
    inv[::97] = -1
    g = torch.randn(n, D, device=dev)
    ug = torch.zeros(U, D, device=dev)
    un = torch.zeros(U, device=dev)
    _lib.call("rs_segment_sum", ptr(g), ptr(inv), n, D, ptr(ug), ptr(un), stream_ptr())
    torch.cuda.synchronize()
    keep = inv >= 0
    ref = torch.zeros(U, D, device=dev, dtype=torch.float64).index_add_(0, inv[keep].long(), g[keep].double())
    refn = torch.zeros(U, device=dev, dtype=torch.float64).index_add_(0, inv[keep].long(), g[keep].double().pow(2).sum(1))
    assert (ug.double() - ref).abs().max().item() < 1e-3 * max(1.0, ref.abs().max().item())
    assert (un.double() - refn).abs().max().item() < 1e-4 * max(1.0, refn.abs().max().item())


@pytest.mark.parametrize("engine", ["KVEngineExtendibleHash", "KVEnginePoolMap"])
def test_lookahead_cached_table_over_a_hashed_host_tier(dev, engine):
    """The two-level table: HBM cache over a host KV engine.  Keys are sparse 40-bit ids; a key the engine has never seen
    reads as its initial value (a function of the key), updated rows reach the engine when they are evicted or flushed.
    Oracle: a dict of rows under row-wise Adagrad."""
    from recstore_b200.cache import LookaheadCachedTable
    D, n, L, steps = 16, 256, 2, 30
    tab = LookaheadCachedTable(50000, D, cache_rows=2048, max_keys=n, lr=0.1, eps=1e-8, device=dev, lookahead=L, init="uniform",
                               seed=4, host_engine=engine)
    g = torch.Generator().manual_seed(5)
    universe = torch.randint(1 << 20, 1 << 40, (3000,), generator=g)
    batches = [universe[torch.randint(0, 3000, (n,), generator=g)] for _ in range(steps + L)]
    for b in batches:
        b[::11] = universe[0]                            # a hot key in every batch
    W, S = {}, {}

    def row(k):
        if k not in W:
            W[k] = tab._initial_rows(torch.tensor([k]))[0, :D].clone()
            S[k] = 0.0
        return W[k]
    for t in range(L):
        tab.prefetch(batches[t].to(dev), t)
    for t in range(steps):
        tab.prefetch(batches[t + L].to(dev), t + L)
        ids = batches[t]
        rows = tab.lookup(ids.to(dev), t).cpu()
        exp = torch.stack([row(int(k)) for k in ids.tolist()])
        assert torch.allclose(rows, exp, atol=1e-4, rtol=1e-5), (t, (rows - exp).abs().max().item())
        grads = torch.randn(n, D, generator=g)
        tab.update(grads.to(dev))
        for k in set(ids.tolist()):                      # every occurrence adds mean(g^2); all apply with the post-step state
            sel = (ids == k)
            S[k] += float(grads[sel].pow(2).mean(1).sum())
            W[k] = W[k] - 0.1 * grads[sel].sum(0) / (S[k] ** 0.5 + 1e-8)
    tab.check()
    assert tab.stats["late_announcements"] == 0 and tab.stats["staged_rows"] > 0
    tab.flush()
    keys = torch.tensor(sorted(W)[:500])
    got = tab.host_rows(keys)
    assert torch.allclose(got[:, :D], torch.stack([W[int(k)] for k in keys]), atol=1e-3, rtol=1e-4)
    assert torch.allclose(got[:, D], torch.tensor([S[int(k)] for k in keys]), atol=1e-3, rtol=2e-3)
    assert len(tab.kv) <= len(W)                          # only keys that were written back are stored
    tab.close()
