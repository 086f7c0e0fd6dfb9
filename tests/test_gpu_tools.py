"""Bandwidth probes and the device pool on a real GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bandwidth_probes_return_plausible_numbers():
    from recstore_b200.bench.bandwidth import probe
    n = 256 << 20
    hbm = probe("copy_kernel", n, iters=5)
    d2d = probe("d2d", n, iters=5)
    h2d = probe("h2d", 64 << 20, iters=3)
    uva = probe("uva_read", 64 << 20, iters=3)
    assert hbm > 1000 and d2d > 500, (hbm, d2d)          # HBM3e: several TB/s
    assert 5 < h2d < 500 and 5 < uva < 500, (h2d, uva)    # host link: tens of GB/s


def test_device_pool_tensors_are_usable_by_kernels():
    from recstore_b200.utils.device_pool import DevicePool
    p = DevicePool("binning", backing="device", initial_bytes=8 << 20, max_bytes=256 << 20)
    a = p.tensor((1024, 128), torch.float32)
    b = p.tensor((1024, 128), torch.bfloat16)
    a.fill_(2.0)
    b.copy_(a)
    assert a.is_cuda and b.is_cuda and b.float().sum().item() == 2.0 * 1024 * 128
    s = p.stats()
    assert s["live_blocks"] == 2 and s["reserved_bytes"] >= s["in_use_bytes"] > 0
    ptr = a.data_ptr()
    del a
    import gc
    gc.collect()
    torch.cuda.synchronize()
    c = p.tensor((1024, 128), torch.float32)             # the freed block is reused, no new slab
    assert c.data_ptr() == ptr
    del b, c
    gc.collect()
    p.close()


def test_engine_checkpoint_loads_into_pytorch_restatement_and_back(tmp_path):
    from recstore_b200.baseline.dlrm_torch import TorchDLRM
    from recstore_b200.models.checkpoint import load_checkpoint
    from recstore_b200.models.dlrm import DLRM, DLRMConfig
    from recstore_b200.utils.data import DLRMBatchSource
    rows, B, D = [500, 37, 2000], 256, 64
    kw = dict(emb_dim=D, bottom_mlp=(128, D), top_mlp=(128, 64, 1))
    eng = DLRM(DLRMConfig(table_rows=rows, batch=B, seed=3, **kw))
    src = DLRMBatchSource(rows, [1, 1, 1], B, seed=4)
    for _ in range(4):
        b = src.next()
        eng.train_step(eng.make_pinned_batch(b.dense, b.ids, b.labels))
    eng.save_checkpoint(str(tmp_path / "ck"), step=4)
    ora = TorchDLRM(rows, B, device="cuda:0", seed=77, **kw)
    meta = load_checkpoint(ora, str(tmp_path / "ck"))
    assert meta["step"] == 4 and meta["table_rows"] == rows
    b = src.next()
    p_eng = eng.predict(eng.make_pinned_batch(b.dense, b.ids, b.labels)).float().view(-1)
    p_ora = ora.predict(b.dense, b.ids).float().view(-1).to(p_eng.device)
    assert (p_eng - p_ora).abs().max().item() < 2e-2          # bf16 MLPs against fp32
    eng2 = DLRM(DLRMConfig(table_rows=rows, batch=B, seed=99, **kw))
    eng2.load_checkpoint(str(tmp_path / "ck"))
    p2 = eng2.predict(eng2.make_pinned_batch(b.dense, b.ids, b.labels)).float().view(-1)
    assert torch.equal(p_eng, p2)


def test_uvm_baseline_trainer_allocates_managed_memory():
    """Under the interposer the trainer's device allocations (the embedding table among them) become managed memory and
    training still runs; without it nothing is redirected."""
    from recstore_b200.baseline import uvm_trainer
    args = ["--vocab_size", "200000", "--embed_size", "32", "--batch_size", "4096", "--sample_number", "5"]
    r = uvm_trainer.main(args)
    assert r["device"].startswith("cuda") and r["uvm"] is True
    assert r["intercepted"]["made_managed"] > 0 and r["intercepted"]["bytes"] >= 200000 * 32 * 4
    r0 = uvm_trainer.main(args + ["--no_uvm"])
    assert r0["uvm"] is False and abs(r0["first_loss"] - r["first_loss"]) < 1e-3 * max(1.0, abs(r["first_loss"]))


def test_device_id_generators_match_the_host_formula():
    """Uniform and Zipf ids drawn on the device: reproducible from (seed, counter), independent of how a stream is cut into
    calls, inside the range, and equal to the host generator's closed form fed with the same uniforms."""
    import ctypes as C
    import numpy as np
    from recstore_b200 import _lib
    from recstore_b200.utils.data import device_uniform_ids, device_zipf_ids, spread_permutation, zipf_from_uniform
    dev = torch.device("cuda:0")
    n, N = 20000, 86_054_151
    a = device_zipf_ids(n, N, 1.3, 7, 0, device=dev)
    b = torch.cat([device_zipf_ids(n // 2, N, 1.3, 7, 0, device=dev), device_zipf_ids(n // 2, N, 1.3, 7, n // 2, device=dev)])
    assert torch.equal(a, b) and int(a.min()) >= 0 and int(a.max()) < N
    draw = _lib.lib().rs_gen_draw
    u = np.array([draw(7, i) >> 11 for i in range(n)], dtype=np.float64) / 9007199254740992.0
    ref = torch.from_numpy(zipf_from_uniform(u, N, 1.3))
    assert (a.cpu() != ref).float().mean().item() < 1e-3                 # the last ulp of pow() may flip a floor
    pa, pb = spread_permutation(N)
    s = device_zipf_ids(n, N, 1.3, 7, 0, device=dev, spread=True).cpu()
    assert torch.equal(s, torch.tensor([(int(k) * pa + pb) % N for k in a.cpu().tolist()]))
    un = device_uniform_ids(200000, 1000, 3, 0, device=dev)
    cnt = torch.bincount(un, minlength=1000).float()
    assert int(un.min()) >= 0 and int(un.max()) < 1000 and (cnt - 200).abs().max().item() < 80      # ~5.6 sigma
    # popularity: P(rank 0) = (2^-0.3 - 1) / ((N + 1)^-0.3 - 1) = 0.1885 for this N
    top = (a == 0).float().mean().item()
    assert 0.17 < top < 0.21


def test_peer_context_symmetric_heap_slices_reuse_and_fallback():
    """Windows carved out of one pre-exchanged heap: addresses follow from the heap's base, freed bytes are reused,
    a request that does not fit gets a window of its own, and tearing down frees only what owns memory."""
    from recstore_b200.parallel.peer import PeerContext
    ctx = PeerContext(0, 1, heap_bytes=1 << 20)
    heap = ctx.windows["__heap__"]
    a = ctx.alloc("a", 1000)                                # rounded to 1024
    b = ctx.alloc("b", 4096)
    assert a.heap_offset == 0 and b.heap_offset == 1024 and a.ptrs[0] == heap.ptrs[0] and b.ptrs[0] == heap.ptrs[0] + 1024
    assert int(b.table[0].item()) == b.local_ptr
    a.view(torch.float32, (256,)).fill_(3.0)
    b.view(torch.int32, (1024,)).copy_(torch.arange(1024, dtype=torch.int32, device="cuda:0"))
    raw = heap.view(torch.float32, (256,))
    assert torch.equal(raw, torch.full((256,), 3.0, device="cuda:0"))              # the slice IS heap memory
    assert torch.equal(b.peer_view(0, torch.int32, (1024,)).cpu(), torch.arange(1024, dtype=torch.int32))
    st = ctx.heap_stats()
    assert st["in_use"] == 1024 + 4096 and st["windows_in_heap"] == 2
    ctx.free("a")
    c = ctx.alloc("c", 512)
    assert c.heap_offset == 0 and "a" not in ctx.windows                           # the freed bytes are reused
    big = ctx.alloc("big", 2 << 20)                                                # larger than the heap: its own window
    assert big.heap_offset is None and big.nbytes == 2 << 20
    big.view(torch.uint8, (16,)).fill_(7)
    ctx.free("big")
    with pytest.raises(ValueError):
        ctx.free("__heap__")
    with pytest.raises(KeyError):
        ctx.free("a")
    ctx.free_all()
    assert ctx.windows == {}
    plain = PeerContext(0, 1)                                                      # without a heap nothing changes
    w = plain.alloc("w", 4096)
    assert w.heap_offset is None and plain.heap_stats()["heap_bytes"] == 0
    plain.free("w")
    plain.free_all()
