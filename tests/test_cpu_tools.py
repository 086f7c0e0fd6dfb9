"""Device-pool allocators on host backing, the UVM interposer's exports, and the build outputs (CPU only)."""
import ctypes as C
import random

import pytest
import torch

from recstore_b200 import _lib
from recstore_b200.utils.device_pool import DevicePool


def test_pool_allocator_coalesces_and_respects_limit():
    p = DevicePool("pool", backing="host", initial_bytes=1 << 16, max_bytes=1 << 18)
    a = [p.alloc(10000) for _ in range(5)]
    assert len(set(a)) == 5 and all(x % 256 == 0 for x in a)
    s = p.stats()
    assert s["live_blocks"] == 5 and s["in_use_bytes"] == 5 * 10240
    for x in a:
        p.free(x)
    assert p.stats()["in_use_bytes"] == 0
    big = p.alloc(60000)            # only fits if the freed neighbours were merged back
    assert p.stats()["slabs"] <= 2
    p.free(big)
    with pytest.raises(_lib.RecStoreError):
        p.alloc(1 << 19)            # over the limit
    with pytest.raises(_lib.RecStoreError):
        p.free(12345 * 256)         # foreign pointer
    assert p.stats()["failures"] == 1
    with pytest.raises(_lib.RecStoreError):
        p.alloc((1 << 64) - 1)      # rounding this up to the block granularity would wrap to zero
    p.close()


def test_pool_random_alloc_free_never_overlaps():
    rnd = random.Random(0)
    p = DevicePool("binning", backing="host", initial_bytes=1 << 20, max_bytes=64 << 20, max_bin_bytes=1 << 14)
    live = {}
    for _ in range(3000):
        if live and rnd.random() < 0.45:
            ptr = rnd.choice(list(live))
            p.free(ptr)
            del live[ptr]
        else:
            n = rnd.choice([1, 100, 256, 1000, 5000, 20000, 70000])
            ptr = p.alloc(n)
            for q, m in live.items():
                assert ptr + n <= q or q + m <= ptr, "overlapping blocks"
            live[ptr] = n
    st = p.stats()
    assert st["live_blocks"] == len(live)
    for ptr in list(live):
        p.free(ptr)
    assert p.stats()["in_use_bytes"] == 0
    p.close()


def test_fixed_allocator_and_tensor_views():
    p = DevicePool("fixed", backing="host", initial_bytes=4096 * 4, max_bytes=4096 * 8, block_bytes=4096)
    t = p.tensor((32, 32), torch.float32)
    t.fill_(3.0)
    u = p.tensor((100,), torch.int64)
    u.copy_(torch.arange(100))
    assert t.sum().item() == 3.0 * 1024 and u[99].item() == 99
    assert p.stats()["live_blocks"] == 2
    with pytest.raises(_lib.RecStoreError):
        p.alloc(5000)               # larger than a block
    del t, u
    import gc
    gc.collect()
    assert p.stats()["live_blocks"] == 0
    blocks = [p.alloc(4096) for _ in range(8)]
    with pytest.raises(_lib.RecStoreError):
        p.alloc(1)                  # 8 blocks is the cap
    for b in blocks:
        p.free(b)
    p.close()


def test_uvm_interposer_exports_and_falls_back_without_cuda():
    from recstore_b200.build import build_preload_shims
    so = build_preload_shims()
    lib = C.CDLL(str(so))
    ptr = C.c_void_p()
    lib.cudaMalloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
    rc = lib.cudaMalloc(C.byref(ptr), 1024)        # no libcudart behind the shim in this process image: any error code, no crash
    assert isinstance(rc, int)
    out = (C.c_ulonglong * 3)()
    lib.rs_uvm_intercept_stats(out)
    assert out[0] >= 1


def test_uvm_baseline_trainer_runs_under_the_interposer():
    """The unified-memory baseline re-executes itself with the shim preloaded; on a host without a GPU the shim is
    loaded (its statistics symbol resolves) and simply sees no device allocation."""
    from recstore_b200.baseline import uvm_trainer
    r = uvm_trainer.main(["--vocab_size", "2000", "--embed_size", "8", "--batch_size", "128", "--sample_number", "4", "--device", "cpu"])
    assert r["uvm"] is True and r["intercepted"]["cudaMalloc_calls"] == 0 and r["ms_per_step"] > 0
    r = uvm_trainer.main(["--vocab_size", "2000", "--embed_size", "8", "--batch_size", "128", "--sample_number", "4", "--device", "cpu",
                          "--no_uvm"])
    assert r["uvm"] is False and r["intercepted"] is None


def test_create_mini_dataset_truncates_and_recounts(tmp_path):
    import numpy as np
    from recstore_b200.utils import dlrm_data as Dd
    rng = np.random.default_rng(0)
    lines = ["\t".join([str(rng.integers(0, 2))] + [str(rng.integers(0, 9)) for _ in range(Dd.NUM_INT)] +
                       [format(int(rng.integers(0, 40)), "x") for _ in range(Dd.NUM_CAT)]) for _ in range(60)]
    full = Dd.criteo_preprocess(lines, str(tmp_path / "full.npz"))
    assert Dd.create_mini_dataset(str(tmp_path / "full.npz"), str(tmp_path / "mini.npz"), 25) == 25
    mini = np.load(tmp_path / "mini.npz")
    assert mini["y"].shape == (25,) and np.array_equal(mini["X_cat"], full["X_cat"][:25])
    assert np.all(mini["counts"] <= full["counts"]) and np.all(mini["counts"] == mini["X_cat"].max(0) + 1)
    ds = Dd.CriteoDataset(str(tmp_path / "mini.npz"), batch=5, test_frac=0.2)
    assert len(ds) == 4 and len(next(iter(ds)).ids) == Dd.NUM_CAT


def test_table_placement_policies():
    """Round robin by index, and the greedy by ids per sample: equal costs reproduce round robin, the multi-hot
    configuration is levelled as far as its heaviest table allows."""
    from recstore_b200.parallel.placement import place_tables, placement_stats
    hot = [3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1]
    rows = list(range(1000, 1026))
    for w in (1, 2, 3, 4, 8):
        assert place_tables([1] * 26, rows, w, "balanced") == place_tables([1] * 26, rows, w) == [t % w for t in range(26)]
        rr, bal = place_tables(hot, rows, w), place_tables(hot, rows, w, "balanced")
        assert sorted(set(bal)) == list(range(min(w, 26))) and len(bal) == 26
        assert placement_stats(bal, hot, w)["imbalance"] <= placement_stats(rr, hot, w)["imbalance"] + 1e-9
    assert placement_stats(place_tables(hot, rows, 2, "balanced"), hot, 2)["lookups_per_rank"] == [107, 107]
    assert max(placement_stats(place_tables(hot, rows, 8, "balanced"), hot, 8)["lookups_per_rank"]) == 100     # the 100-hot table alone
    with pytest.raises(ValueError):
        place_tables(hot, rows, 2, "nope")
