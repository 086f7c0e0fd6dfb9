"""Bags over PS rows, load generation, dataset replay and the native engine benchmark (CPU only)."""
import json

import numpy as np
import pytest
import torch

from recstore_b200.ps import ParameterClient, ParameterServer
from recstore_b200.ps.embedding_bag import PSEmbeddingBagModule, pool_rows
from recstore_b200.ps.load_generator import DatasetReplay, PoissonLoadGenerator, zipf_key_source


@pytest.mark.parametrize("mode", ["sum", "mean", "max"])
@pytest.mark.parametrize("padding_idx", [None, 3])
def test_pool_rows_matches_torch_embedding_bag(mode, padding_idx):
    g = torch.Generator().manual_seed(0)
    N, D = 20, 8
    w = torch.randn(N, D, generator=g)
    idx = torch.randint(0, N, (37,), generator=g)
    idx[::5] = 3
    offsets = torch.tensor([0, 4, 4, 9, 20, 30])            # one empty bag
    psw = torch.rand(37, generator=g) if mode == "sum" else None
    ref_mod = torch.nn.EmbeddingBag(N, D, mode=mode, padding_idx=padding_idx)
    with torch.no_grad():
        ref_mod.weight.copy_(w)
    ref = ref_mod(idx, offsets, per_sample_weights=psw)
    rows = w[idx].clone().requires_grad_(True)
    out = pool_rows(rows, idx, offsets, mode, psw, padding_idx)
    assert torch.allclose(out, ref, atol=1e-6)
    # gradients w.r.t. the table agree once row gradients are scattered back
    ref.sum().backward()
    out.sum().backward()
    gt = torch.zeros(N, D).index_add(0, idx, rows.grad)
    assert torch.allclose(gt, ref_mod.weight.grad, atol=1e-6)


def test_pool_rows_matrix_and_last_offset():
    w = torch.arange(40, dtype=torch.float32).view(10, 4)
    idx2 = torch.tensor([[1, 2, 3], [4, 5, 6]])
    out = pool_rows(w[idx2.reshape(-1)], idx2, None, "sum")
    assert torch.equal(out, w[idx2].sum(1))
    idx = torch.tensor([0, 1, 2, 3, 4])
    out = pool_rows(w[idx], idx, torch.tensor([0, 2, 5]), "mean", include_last_offset=True)
    assert torch.allclose(out, torch.stack([w[:2].mean(0), w[2:5].mean(0)]))


def test_ps_bag_module_updates_rows_on_server():
    srv = ParameterServer("KVEngineMap", {"capacity": 1000, "dim": 4, "optimizer": "sgd", "lr": 0.5})
    port = srv.serve(0)
    c = ParameterClient("127.0.0.1", port, 0, 4)
    try:
        keys = torch.arange(10)
        c.PutParameter(keys + 100, torch.ones(10, 4))
        bag = PSEmbeddingBagModule(c, 10, 4, mode="sum", padding_idx=0, key_offset=100)
        out = bag(torch.tensor([0, 1, 2, 2]), torch.tensor([0, 2]))
        assert torch.allclose(out, torch.tensor([[1.0] * 4, [2.0] * 4]))
        out.sum().backward()
        assert bag.step() == 3                                 # the padding row is neither read into the sum nor updated
        after = c.GetParameter(keys + 100)
        assert torch.allclose(after[0], torch.ones(4)) and not torch.allclose(after[2], torch.ones(4))
    finally:
        c.close()
        srv.close()


def test_dataset_replay_and_poisson_generator(tmp_path):
    p = tmp_path / "trace.txt"
    p.write_text("1 2 3\n4,5\n\n6\n")
    rep = DatasetReplay(str(p), loop=False)
    assert [b.tolist() for b in rep] == [[1, 2, 3], [4, 5], [6]]
    np.save(tmp_path / "ids.npy", np.arange(12))
    np.save(tmp_path / "off.npy", np.array([0, 5, 12]))
    rep = DatasetReplay(str(tmp_path / "ids.npy"), str(tmp_path / "off.npy"), loop=False)
    assert [b.numel() for b in rep] == [5, 7]
    srv = ParameterServer("KVEngineMap", {"capacity": 5000, "dim": 8})
    srv.LoadFakeData(2000)
    port = srv.serve(0)
    try:
        gen = PoissonLoadGenerator(lambda: ParameterClient("127.0.0.1", port, 0, 8), zipf_key_source(2000, 16, 0.9), rate=400,
                                   senders=2, seed=1)
        s = gen.run(0.5).summary()
        assert s["completed"] == s["sent"] > 50 and s["lat_ms_p99"] >= s["lat_ms_p50"] > 0
    finally:
        srv.close()


def test_native_engine_benchmark_and_zipf_check():
    from recstore_b200.bench.kv_engine import run_engine, zipf_check
    r = run_engine("KVEngineMap", threads=2, seconds=0.2, batch=32, alpha=0.9, read_ratio=0.8, key_space=5000)
    assert r["get_mkvs"] > 0 and r["put_mkvs"] > 0 and 0.99 <= r["hit_ratio"] <= 1.0
    z = zipf_check(100000, 1.2, n=200000, top=10)
    assert abs(z["mass"] - z["expected"]) < 0.01
    json.dumps(r)


def _po_member(gid, port, q):
    import torch
    from recstore_b200.ps import AllShardsParameterClient, ParameterClient, ParameterServer
    from recstore_b200.ps.postoffice import Postoffice
    po = Postoffice(num_servers=2, num_clients=1, global_id=gid, store_port=port, timeout_s=30)
    if po.is_server:
        srv = ParameterServer("KVEngineMap", {"dim": 4, "capacity": 1000})
        po.publish_server("127.0.0.1", srv.serve(0))
        po.barrier("ready"); po.barrier("done")
        q.put(("server", po.server_id, len(srv)))
        srv.close()
    else:
        po.barrier("ready")
        cl = AllShardsParameterClient([ParameterClient(h, p, i, 4) for i, (h, p) in enumerate(po.all_servers())])
        keys = torch.arange(40)
        cl.PutParameter(keys, keys.float().unsqueeze(1).expand(-1, 4).contiguous())
        ok = torch.equal(cl.GetParameter(keys)[:, 0], keys.float())
        po.barrier("done")
        q.put(("client", po.client_id, ok))


def test_postoffice_roles_rendezvous_and_barrier():
    import multiprocessing as mp
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_po_member, args=(g, port, q)) for g in range(3)]
    for p in ps:
        p.start()
    got = sorted(q.get(timeout=60) for _ in range(3))
    for p in ps:
        p.join(30)
    assert got[0] == ("client", 0, True)
    assert got[1][0] == got[2][0] == "server" and got[1][2] + got[2][2] == 40 and min(got[1][2], got[2][2]) > 0


def test_binary_trace_roundtrip(tmp_path):
    from recstore_b200.ps.load_generator import read_binary_trace, write_binary_trace
    reqs = [[1, 2, 3], [], [2 ** 40 + 5]]
    p = str(tmp_path / "t.bin")
    write_binary_trace(p, reqs, dim=32)
    assert [r.tolist() for r in read_binary_trace(p)] == reqs
    assert (tmp_path / "t.bin").stat().st_size == 4 + 3 * 4 + 4 * 12
    rep = DatasetReplay(p, loop=False)
    assert [b.tolist() for b in rep] == reqs
    with open(p, "ab") as f:
        f.write(b"xx")
    with pytest.raises(ValueError):
        read_binary_trace(p)


def test_binary_trace_renumber_and_wordcount(tmp_path):
    """Trace tools of the PS benchmark: dense renumbering in order of first appearance (with the dim check) and key
    frequencies."""
    import numpy as np
    import pytest
    from recstore_b200.ps import load_generator as L
    src, dst = str(tmp_path / "a.bin"), str(tmp_path / "b.bin")
    reqs = [[50, 7, 50], [9, 7], [10 ** 12]]
    L.write_binary_trace(src, reqs, dim=32)
    assert L.renumber_trace(src, dst) == 4
    assert [x.tolist() for x in L.read_binary_trace(dst)] == [[0, 1, 0], [2, 1], [3]]
    keys, counts = L.trace_wordcount(src)
    assert dict(zip(keys.tolist(), counts.tolist())) == {50: 2, 7: 2, 9: 1, 10 ** 12: 1} and counts.tolist() == sorted(counts.tolist(), reverse=True)
    L.write_binary_trace(src, reqs, dim=12)
    with pytest.raises(ValueError):
        L.renumber_trace(src, dst)
    replay = L.DatasetReplay(dst, loop=False)
    assert sum(1 for _ in replay) == 3
    raw = open(dst, "rb").read()
    for cut in (0, 2, 4, 6, 10, len(raw) - 1):                      # truncated files say where they stop making sense
        (tmp_path / "t.bin").write_bytes(raw[:cut])
        with pytest.raises(ValueError, match="truncated|announces"):
            L.read_binary_trace(str(tmp_path / "t.bin"))
    (tmp_path / "t.bin").write_bytes(raw + b"xx")
    with pytest.raises(ValueError, match="trailing"):
        L.trace_wordcount(str(tmp_path / "t.bin"))


def test_ps_client_benchmark_with_several_processes(capsys):
    """Closed-loop load from two generator processes against one in-process server shard."""
    import json
    from recstore_b200.bench import ps_client
    ps_client.main(["--processes", "2", "--threads", "1", "--seconds", "0.6", "--key-space", "20000", "--batch", "200"])
    out = json.loads([ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")][-1])
    assert out["processes"] == 2 and len(out["per_process"]) == 2 and out["keys_per_s"] > 0
