"""Command-line drivers end to end on CPU (gloo, two worker processes each)."""
import numpy as np
import pytest


def test_perf_emb_differential_two_workers():
    from recstore_b200.cli import perf_emb
    out = perf_emb.main(["--num_workers", "2", "--device", "cpu", "--run_steps", "12", "--num_embs", "5000", "--emb_dim", "8",
                         "--batch_size", "200", "--L", "4", "--diff_test", "--log_interval", "100"])
    if out is not None:
        for r, v in dict(out).items():
            assert v[0] == 12 and v[1] < 1e-4, (r, v)


@pytest.mark.parametrize("mode", ["CppSync", "CppAsyncV2"])
def test_perf_rec_model_matches_golden(mode):
    from recstore_b200.cli import perf_rec_model
    out = perf_rec_model.main(["--num_workers", "2", "--device", "cpu", "--run_steps", "10", "--dataset", "avazu", "--num_embs", "8000",
                               "--emb_dim", "8", "--batch_size", "64", "--L", "3", "--diff_test", "--backwardMode", mode,
                               "--with_nn", "16,1", "--log_interval", "100"])
    assert len(out) == 2
    for r, (steps, worst, loss) in out.items():
        assert steps == 10 and worst < 1e-4 and np.isfinite(loss), (r, steps, worst, loss)


def test_rec_dataset_loader_reads_files_and_synthesises(tmp_path):
    from recstore_b200.utils.rec_dataset import RecDatasetLoader
    ids = np.random.default_rng(0).integers(0, 5, size=(50, 21))
    np.save(tmp_path / "avazu.npy", ids)
    np.save(tmp_path / "avazu_offsets.npy", np.arange(0, 22) * 5)
    l0 = RecDatasetLoader("avazu", 8, root=str(tmp_path), rank=0, world=2)
    l1 = RecDatasetLoader("avazu", 8, root=str(tmp_path), rank=1, world=2)
    b0, b1 = l0.next_batch(), l1.next_batch()
    assert b0.shape == (8, 21) and l0.num_embeddings == 105
    assert (b0.numpy() == ids[0:8] + np.arange(21) * 5).all() and (b1.numpy() == ids[8:16] + np.arange(21) * 5).all()
    s = RecDatasetLoader("criteo", 16, synthetic_total=10000)
    b = s.next_batch()
    assert b.shape == (16, 26) and s.synthetic and int(b.max()) < s.num_embeddings
    assert (b.numpy() >= s.offsets[:-1]).all() and (b.numpy() < s.offsets[1:]).all()


def test_dlrm_main_trains_saves_and_resumes(tmp_path):
    import torch
    from recstore_b200.cli import dlrm_main
    ck = str(tmp_path / "ck")
    common = ["--arch-sparse-feature-size", "8", "--arch-embedding-size", "50-20-300", "--arch-mlp-bot", "5-16-8",
              "--arch-mlp-top", "14-16-1", "--mini-batch-size", "64", "--print-freq", "0", "--data-generation", "synthetic"]
    a = dlrm_main.main(common + ["--num-batches", "40", "--save-model", ck])
    assert a["steps"] == 40 and a["mean_last_10"] < a["first_loss"]
    b = dlrm_main.main(common + ["--num-batches", "5", "--load-model", ck, "--test-freq", "5"])
    assert abs(b["first_loss"] - a["mean_last_10"]) < 0.2 and b["test_accuracy"] is not None
    # wrong architecture is refused
    with pytest.raises((ValueError, SystemExit)):
        dlrm_main.main(["--arch-sparse-feature-size", "8", "--arch-embedding-size", "50-20", "--arch-mlp-bot", "5-16-8",
                        "--mini-batch-size", "64", "--num-batches", "1", "--load-model", ck, "--print-freq", "0"])
    with pytest.raises(SystemExit):
        dlrm_main.main(["--arch-sparse-feature-size", "8", "--arch-mlp-bot", "5-16-4", "--num-batches", "1"])


def test_checkpoint_roundtrip_preserves_predictions(tmp_path):
    import torch
    from recstore_b200.baseline.dlrm_torch import TorchDLRM
    from recstore_b200.models.checkpoint import load_checkpoint, save_checkpoint
    from recstore_b200.utils.data import DLRMBatchSource
    rows = [30, 200, 17]
    kw = dict(emb_dim=8, bottom_mlp=(16, 8), top_mlp=(16, 1), num_dense=4, seed=1)
    m = TorchDLRM(rows, 32, **kw)
    src = DLRMBatchSource(rows, [1, 1, 1], 32, num_dense=4, seed=2)
    for _ in range(5):
        b = src.next()
        m.train_step(b.dense, b.ids, b.labels)
    save_checkpoint(m, str(tmp_path / "c"), step=5)
    m2 = TorchDLRM(rows, 32, **dict(kw, seed=99))
    meta = load_checkpoint(m2, str(tmp_path / "c"))
    b = src.next()
    assert meta["step"] == 5 and torch.allclose(m.predict(b.dense, b.ids), m2.predict(b.dense, b.ids))
    assert torch.equal(m.states[1], m2.states[1])


def test_criteo_parser_random_dataset_and_trace_tools(tmp_path):
    import torch
    from recstore_b200.utils.dlrm_data import CriteoDataset, RandomDataset, criteo_preprocess, trace_generate, trace_profile
    rng = np.random.default_rng(0)
    lines = []
    for i in range(200):
        ints = [str(int(x)) if rng.random() > 0.1 else "" for x in rng.integers(0, 50, 13)]
        cats = ["%08x" % int(x) if rng.random() > 0.05 else "" for x in rng.integers(0, 7, 26)]
        lines.append("\t".join([str(int(rng.random() < 0.3))] + ints + cats) + "\n")
    lines.append("garbage line\n")
    d = criteo_preprocess(lines, str(tmp_path / "c.npz"))
    assert d["y"].shape == (200,) and d["X_cat"].shape == (200, 26) and int(d["counts"].max()) <= 8
    assert (d["X_cat"].max(0) < d["counts"]).all()
    ds = CriteoDataset(str(tmp_path / "c.npz"), batch=32)
    b = next(iter(ds))
    assert b.dense.shape == (32, 13) and len(b.ids) == 26 and b.ids[3].shape == (32,) and len(ds) == 5 and len(ds.table_rows) == 26
    assert torch.all(b.dense >= 0)
    rb = next(iter(RandomDataset([10, 1000], 4, 16, 2, num_indices_per_lookup=5, fixed=False, alpha=1.1, seed=1)))
    assert rb.offsets[0][0] == 0 and rb.ids[1].numel() >= 16 and int(rb.ids[0].max()) < 10
    trace = np.array([1, 2, 1, 3, 2, 1, 4, 1, 2, 3] * 30)
    uniq, dist, p = trace_profile(trace)
    assert uniq == [1, 2, 3, 4] and abs(p.sum() - 1) < 1e-12 and dist[0] == 0
    syn = trace_generate(uniq, dist, p, 3000, seed=2)
    _, d2, p2 = trace_profile(syn)
    common = {int(a): b for a, b in zip(dist, p)}
    for a, b in zip(d2, p2):
        if int(a) in common and common[int(a)] > 0.1:
            assert abs(b - common[int(a)]) < 0.05          # the reuse distribution is reproduced
    assert set(syn.tolist()) <= {1, 2, 3, 4}


def test_dlrm_driver_reference_flags():
    """Learning-rate policy, alternative losses, gaussian ids, inference-only and refused flags of the DLRM driver."""
    import pytest
    from recstore_b200.cli import dlrm_main
    lr = [dlrm_main.lr_at(s, 1.0, 4, 8, 4) for s in range(14)]
    assert lr[:4] == [0.25, 0.5, 0.75, 1.0] and lr[6] == 1.0                  # warm-up, then constant
    assert lr[7] == 1.0 and abs(lr[8] - (3 / 4) ** 2) < 1e-12 and lr[10] == (1 / 4) ** 2 and lr[11] == 1e-7 and lr[13] == 1e-7
    base = ["--arch-embedding-size", "50-30-20", "--arch-sparse-feature-size", "8", "--arch-mlp-bot", "4-16-8", "--mini-batch-size", "64",
            "--print-freq", "0"]
    out = dlrm_main.main(base + ["--num-batches", "0", "--data-size", "640", "--loss-function", "wbce", "--loss-weights", "0.5-2.0",
                                 "--lr-num-warmup-steps", "3", "--lr-decay-start-step", "6", "--lr-num-decay-steps", "4",
                                 "--rand-data-dist", "gaussian", "--rand-data-sigma", "0.2", "--round-targets", "--print-time",
                                 "--max-ind-range", "40"])
    assert out["steps"] == 10 and out["last_loss"] == out["last_loss"] and out["ms_per_iteration"] > 0
    out = dlrm_main.main(base + ["--num-batches", "5", "--loss-function", "mse"])
    assert 0 < out["last_loss"] < 1
    import torch
    g = torch.Generator().manual_seed(0)
    sc, yy = torch.randint(0, 10, (300,), generator=g).float(), (torch.rand(300, generator=g) < 0.4).float()
    pairs = (sc[yy > 0.5][:, None] > sc[yy < 0.5][None, :]).double() + 0.5 * (sc[yy > 0.5][:, None] == sc[yy < 0.5][None, :]).double()
    assert abs(dlrm_main.roc_auc(sc, yy) - pairs.mean().item()) < 1e-9             # AUC = P(score of a positive > score of a negative)
    import os
    import tempfile
    tb = tempfile.mkdtemp()
    out = dlrm_main.main(base + ["--num-batches", "6", "--test-freq", "3", "--tensor-board-filename", tb])
    assert 0.0 <= out["test_auc"] <= 1.0
    import json as _json
    rows = [_json.loads(ln) for ln in open(os.path.join(tb, "scalars.jsonl"))]
    assert sum("train_loss" in r for r in rows) == 6 and sum("test_accuracy" in r for r in rows) == 2
    out = dlrm_main.main(base + ["--num-batches", "3", "--inference-only", "--loss-threshold", "0.01"])
    assert out["steps"] == 0 and out["inference_batches"] == 3 and 0 <= out["test_accuracy"] <= 1
    import numpy as np
    tf = os.path.join(tempfile.mkdtemp(), "trace.txt")
    with open(tf, "w") as f:
        f.write(", ".join(str(int(x)) for x in np.random.default_rng(0).zipf(1.5, 400) % 40))
    out = dlrm_main.main(base + ["--num-batches", "3", "--data-generation", "synthetic", "--data-trace-file", tf])
    assert out["steps"] == 3 and out["last_loss"] == out["last_loss"]
    with pytest.raises(SystemExit):
        dlrm_main.main(base + ["--qr-flag"])
    with pytest.raises(SystemExit):
        dlrm_main.main(base + ["--quantize-emb-with-bit", "8"])


def test_dlrm_driver_trains_on_criteo_format_files(tmp_path):
    """--data-generation dataset: raw Criteo text is preprocessed (and cached as .npz), the table sizes come from the
    category counts, a second run reads the cache, negatives can be sub-sampled."""
    import numpy as np
    from recstore_b200.cli import dlrm_main
    rng = np.random.default_rng(0)
    raw = tmp_path / "day.txt"
    with open(raw, "w") as f:
        for _ in range(400):
            cat = [format(int(rng.integers(0, 30)), "x") for _ in range(26)]
            label = int(int(cat[0], 16) % 2 == 0)                           # learnable from the first categorical column
            f.write("\t".join([str(label)] + [str(int(rng.integers(0, 9))) for _ in range(13)] + cat) + "\n")
    base = ["--arch-sparse-feature-size", "8", "--arch-mlp-bot", "13-16-8", "--mini-batch-size", "40", "--print-freq", "0",
            "--data-generation", "dataset", "--raw-data-file", str(raw), "--processed-data-file", str(tmp_path / "day.npz"),
            "--nepochs", "6", "--num-batches", "0", "--test-freq", "9", "--learning-rate", "0.1"]
    out = dlrm_main.main(base)
    assert out["steps"] == 6 * 9 and out["mean_last_10"] < out["first_loss"] and (tmp_path / "day.npz").exists()
    assert out["test_accuracy"] is not None and 0 <= out["test_auc"] <= 1
    raw.unlink()                                                           # the cached file is enough now
    out2 = dlrm_main.main(base + ["--data-sub-sample-rate", "0.3", "--data-randomize", "none"])
    assert 0 < out2["steps"] <= 6 * 9


def test_perf_emb_eight_workers_smoke():
    """Eight worker processes (the reference's 8-process multi-card start-up check, src/executable/test/test_multicard.py)
    through the whole cached-embedding step on gloo: shared-memory table, controller on rank 0, all-to-alls among eight
    ranks, and the differential check against the replicated embedding."""
    from recstore_b200.cli import perf_emb
    out = perf_emb.main(["--num_workers", "8", "--device", "cpu", "--run_steps", "4", "--num_embs", "4000", "--emb_dim", "8",
                         "--batch_size", "64", "--L", "2", "--diff_test", "--log_interval", "100",
                         "--emb_choice", "KnownShardedCachedEmbedding"])
    assert len(out) == 8
    for r, v in dict(out).items():
        assert v[0] == 4 and v[1] < 1e-4, (r, v)


def test_profile_dir_writes_a_trace_and_an_operator_table(tmp_path):
    """`--profile_dir` on the KG driver: three steps under torch.profiler, a chrome trace and a per-operator table
    (the reference's torch.profiler windows: perf_emb.py:275-352, train_pytorch.py:185-236)."""
    import json
    import torch
    from recstore_b200.cli import kge_main
    d = tmp_path / "prof"
    out, _ = kge_main.main(["--max_step", "10", "--n_entities", "200", "--n_triples", "2000", "--hidden_dim", "8", "--batch_size", "32",
                            "--neg_sample_size", "8", "--log_interval", "1000", "--profile_dir", str(d)])
    assert out[0]["steps"] == 10
    trace = json.load(open(d / "trace_rank0.json"))
    assert len(trace["traceEvents"]) > 50
    table = (d / "ops_rank0.txt").read_text()
    assert "aten::" in table and "Self CPU" in table
    from recstore_b200.utils.profiling import StepProfiler
    p = StepProfiler(None)
    for _ in range(10):
        p.step()                                             # inert without a directory
    assert p.done and not p.enabled
    with StepProfiler(str(tmp_path / "early"), skip=1, active=100) as q:   # a run that ends inside the window still writes
        q.step()
        torch.ones(4).sum()
    assert (tmp_path / "early" / "trace_rank0.json").exists()


def test_cumulative_timer_adds_pieces_into_one_sample():
    import time
    from recstore_b200.utils.timer import Reporter, Timer, stats
    Reporter.Clear()
    t = Timer("cum.phase")
    for _ in range(3):                                       # three steps, each with two separate pieces of the phase
        for _ in range(2):
            t.CumStart(); time.sleep(0.01); t.CumEnd()
        t.CumReport()
    s = stats("cum.phase")
    assert s["count"] == 3 and 15e6 < s["mean"] < 2e9        # one sample per step, two sleeps of 10 ms each (in ns; a loaded box oversleeps)


def test_checkpoint_loader_refuses_torn_damaged_and_misfitting_saves(tmp_path):
    """A save interrupted half way (files of two steps), a truncated or bit-flipped file, a file that is not tensors,
    and a model of another shape are all refused with a message, and the model is left as it was."""
    import os
    import shutil
    import torch
    from recstore_b200.baseline.dlrm_torch import TorchDLRM
    from recstore_b200.models.checkpoint import load_checkpoint, save_checkpoint
    from recstore_b200.utils.data import DLRMBatchSource
    rows = [30, 200, 17]
    kw = dict(emb_dim=8, bottom_mlp=(16, 8), top_mlp=(16, 1), num_dense=4, seed=1)
    m = TorchDLRM(rows, 32, **kw)
    src = DLRMBatchSource(rows, [1, 1, 1], 32, num_dense=4, seed=2)
    step = lambda: (lambda b: m.train_step(b.dense, b.ids, b.labels))(src.next())
    step()
    old, new = str(tmp_path / "old"), str(tmp_path / "new")
    save_checkpoint(m, old, step=1)
    step()
    save_checkpoint(m, new, step=2)
    fresh = lambda: TorchDLRM(rows, 32, **dict(kw, seed=7))
    assert load_checkpoint(fresh(), new)["step"] == 2 and not (tmp_path / "new" / ".meta.json.tmp").exists()
    # torn: the save of step 2 was interrupted after table 1 -- meta.json and the rest are still those of step 1
    torn = str(tmp_path / "torn")
    shutil.copytree(old, torn)
    shutil.copy(tmp_path / "new" / "table_1.pt", tmp_path / "torn" / "table_1.pt")
    victim = fresh()
    before = [victim.table_weight(t).clone() for t in range(3)] + [v.clone() for v in victim.dense_state().values()]
    with pytest.raises(ValueError, match="torn checkpoint"):
        load_checkpoint(victim, torn)
    after = [victim.table_weight(t) for t in range(3)] + list(victim.dense_state().values())
    assert all(torch.equal(a, b) for a, b in zip(before, after))            # nothing was restored half way
    # damaged files
    for name, damage in (("table_0.pt", lambda b: b[: len(b) // 2]), ("dense.pt", lambda b: b[:100] + bytes([b[100] ^ 0xFF]) + b[101:len(b) // 3]),
                         ("table_2.pt", lambda b: b"this is not a tensor file")):
        d = tmp_path / ("bad_" + name)
        shutil.copytree(new, d)
        (d / name).write_bytes(damage((d / name).read_bytes()))
        with pytest.raises(ValueError, match="damaged|not a tensor"):
            load_checkpoint(fresh(), str(d))
    # pickled code is not executed: a file that would run something on load is refused
    import pickle

    class Boom:
        def __reduce__(self):
            return (os.system, ("true",))
    d = tmp_path / "evil"
    shutil.copytree(new, d)
    with open(d / "table_0.pt", "wb") as f:
        pickle.dump({"weight": Boom()}, f)
    with pytest.raises(ValueError):
        load_checkpoint(fresh(), str(d))
    # a model of another shape
    with pytest.raises(ValueError):
        load_checkpoint(TorchDLRM([30, 200, 18], 32, **kw), new)
    with pytest.raises(ValueError, match="dense.pt does not fit|written for"):
        load_checkpoint(TorchDLRM(rows, 32, **dict(kw, top_mlp=(32, 1))), new)
    d = tmp_path / "short_table"
    shutil.copytree(new, d)
    t = torch.load(d / "table_1.pt")
    torch.save({"weight": t["weight"][:100], "state": t["state"][:100], "save_step": t["save_step"]}, d / "table_1.pt")
    with pytest.raises(ValueError, match="table 1 holds"):
        load_checkpoint(fresh(), str(d))
    # a checkpoint of the older layout (no step stamps in the files) still loads
    d = tmp_path / "v1"
    shutil.copytree(new, d)
    for f in ("table_0.pt", "table_1.pt", "table_2.pt"):
        t = torch.load(d / f)
        t.pop("save_step")
        torch.save(t, d / f)
    assert load_checkpoint(fresh(), str(d))["step"] == 2


def test_sparse_reduce_helpers_and_rank_logging(capsys):
    """kv_to_sparse_tensor / reduce_sparse_tensor on one rank (the multi-rank gather is covered by the cached-embedding
    tests), and the logging helpers (src/python/pytorch/recstore/utils.py:183-219, 352-402)."""
    import logging
    import torch
    from recstore_b200.utils import comm
    from recstore_b200.utils.log import XLOG, cdebug, get_logger, print_rank0
    keys, vals = torch.tensor([5, 2, 5]), torch.tensor([[1.0, 1.0], [2.0, 2.0], [3.0, 3.0]])
    st = comm.kv_to_sparse_tensor(keys, vals, (8, 2))
    assert st.shape == (8, 2) and not st.is_coalesced()
    red = comm.reduce_sparse_tensor(st)
    assert red.is_coalesced() and red.indices().tolist() == [[2, 5]] and red.values().tolist() == [[2.0, 2.0], [4.0, 4.0]]
    assert torch.equal(red.to_dense()[5], torch.tensor([4.0, 4.0]))
    lg = get_logger()
    lg.setLevel(logging.DEBUG)
    records = []
    h = logging.Handler()
    h.emit = records.append
    lg.addHandler(h)
    try:
        cdebug("hello")
        XLOG.cdebug("again", colour=False)
        XLOG.info("plain")
    finally:
        lg.removeHandler(h)
        lg.setLevel(logging.INFO)
    assert [r.getMessage() for r in records] == ["\033[31mhello\033[0m", "again", "plain"]
    assert records[0].filename == "test_cpu_cli.py" and records[0].levelno == logging.DEBUG      # the caller's file, not log.py
    print_rank0("only once")
    assert capsys.readouterr().out == "only once\n"


def test_packaging_metadata_names_real_entry_points():
    """pyproject.toml: every console script points at a callable that exists."""
    import importlib
    import os
    import tomllib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tomllib.load(open(os.path.join(root, "pyproject.toml"), "rb"))
    assert cfg["project"]["name"] == "recstore_b200" and len(cfg["project"]["scripts"]) >= 8
    for name, target in cfg["project"]["scripts"].items():
        mod, fn = target.split(":")
        assert callable(getattr(importlib.import_module(mod), fn)), (name, target)


def test_migration_guide_names_things_that_exist():
    """Every `recstore_b200....` name and every `python -m recstore_b200....` module of the migration guide resolves."""
    import importlib
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "MIGRATION.md")).read()
    names = set(re.findall(r"`(recstore_b200(?:\.\w+)+)", text)) | set(re.findall(r"python -m (recstore_b200(?:\.\w+)+)", text))
    assert len(names) > 25
    for dotted in sorted(names):
        parts = dotted.split(".")
        obj = None
        for cut in range(len(parts), 0, -1):
            try:
                obj = importlib.import_module(".".join(parts[:cut]))
            except ModuleNotFoundError:
                continue
            for attr in parts[cut:]:
                assert hasattr(obj, attr), f"{dotted}: {'.'.join(parts[:cut])} has no {attr}"
                obj = getattr(obj, attr)
            break
        assert obj is not None, dotted
    for fn in re.findall(r"`(rs\.\w+)`?", text):
        import recstore_b200 as rs
        assert hasattr(rs, fn.split(".")[1]), fn


def test_checkpoint_written_by_three_ranks_loads_on_one_and_on_two(tmp_path):
    """Tables are filed by table index, not by rank: a save of three ranks restores on one rank and on two (each rank
    reads the tables it owns under the new placement)."""
    import torch
    from recstore_b200.baseline.dlrm_torch import TorchDLRM
    from recstore_b200.models.checkpoint import load_checkpoint, save_checkpoint
    rows = [30, 200, 17, 64, 9]
    kw = dict(emb_dim=8, bottom_mlp=(16, 8), top_mlp=(16, 1), num_dense=4)
    savers = [TorchDLRM(rows, 30, rank=r, world=3, seed=1, **kw) for r in range(3)]
    assert sorted(t for m in savers for t in m.local_tables) == list(range(5))
    for m in savers:
        for t in m.local_tables:
            m.table_weight(t).add_(t + 1.0)                  # make every table recognisable
            m.table_state(t).fill_(0.5 + t)
    for m in reversed(savers):                               # rank 0 (dense + meta.json) last, as after a barrier
        save_checkpoint(m, str(tmp_path / "ck"), step=9)
    truth = {t: (m.table_weight(t).clone(), m.table_state(t).clone()) for m in savers for t in m.local_tables}
    one = TorchDLRM(rows, 30, rank=0, world=1, seed=5, **kw)
    meta = load_checkpoint(one, str(tmp_path / "ck"))
    assert meta["step"] == 9 and meta["world_at_save"] == 3
    for t in range(5):
        assert torch.equal(one.table_weight(t), truth[t][0]) and torch.equal(one.table_state(t), truth[t][1])
    for k, v in savers[0].dense_state().items():
        assert torch.equal(one.dense_state()[k], v)
    for r in range(2):
        two = TorchDLRM(rows, 30, rank=r, world=2, seed=7, **kw)
        load_checkpoint(two, str(tmp_path / "ck"))
        assert all(torch.equal(two.table_weight(t), truth[t][0]) for t in two.local_tables) and len(two.local_tables) in (2, 3)
