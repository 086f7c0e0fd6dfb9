"""KG score functions against per-edge loops, datasets from fake files, partitions, pre-sampling, the driver (CPU)."""
import math

import numpy as np
import pytest
import torch

from recstore_b200.baseline.kge_torch import MODEL_NAMES, TorchKGE, chunk_neg_score, edge_score, projection_dim, relation_dim
from recstore_b200.utils import kg_data as K


def _naive(model, h, r, t, gamma, proj, emb_init):
    """One triple, scalar loops over the definition."""
    d = h.numel()
    if model in ("TransE", "TransE_l2"):
        return gamma - math.sqrt(sum((h[i] + r[i] - t[i]) ** 2 for i in range(d)))
    if model == "TransE_l1":
        return gamma - sum(abs(h[i] + r[i] - t[i]) for i in range(d))
    if model == "DistMult":
        return sum(h[i] * r[i] * t[i] for i in range(d))
    k = d // 2
    if model == "ComplEx":
        s = 0.0
        for i in range(k):
            a = complex(h[i], h[i + k]) * complex(r[i], r[i + k]) * complex(t[i], t[i + k]).conjugate()
            s += a.real
        return s
    if model == "RotatE":
        s = 0.0
        for i in range(k):
            ph = r[i] / (emb_init / math.pi)
            z = complex(h[i], h[i + k]) * complex(math.cos(ph), math.sin(ph)) - complex(t[i], t[i + k])
            s += abs(z)
        return gamma - s
    if model == "SimplE":
        s = sum(h[i] * r[i] * t[i + k] for i in range(k)) + sum(t[i] * r[i + k] * h[i + k] for i in range(k))
        return max(-20.0, min(20.0, s / 2))
    M = proj.view(d, -1)
    if model == "TransR":
        hp, tp = h @ M, t @ M
        return gamma - sum(abs(hp[i] + r[i] - tp[i]) for i in range(M.shape[1]))
    if model == "RESCAL":
        return float(h @ (M @ t))
    raise AssertionError(model)


@pytest.mark.parametrize("model", MODEL_NAMES)
def test_scores_match_per_edge_definition(model):
    g = torch.Generator().manual_seed(3)
    d, bs, chunk, ns, gamma, init = 8, 6, 3, 4, 5.0, 0.7
    rd = relation_dim(model, d)
    h, t = torch.randn(bs, d, generator=g, dtype=torch.float64), torch.randn(bs, d, generator=g, dtype=torch.float64)
    r = torch.randn(bs, rd, generator=g, dtype=torch.float64)
    pd = projection_dim(model, d)
    proj = torch.randn(bs, pd, generator=g, dtype=torch.float64) if pd else None
    neg = torch.randn(bs // chunk * ns, d, generator=g, dtype=torch.float64)
    pos = edge_score(model, h, r, t, gamma, proj, init)
    for i in range(bs):
        assert abs(pos[i].item() - _naive(model, h[i], r[i], t[i], gamma, None if proj is None else proj[i], init)) < 1e-9
    for corrupt_head in (False, True):
        sc = chunk_neg_score(model, h, r, t, neg, corrupt_head, chunk, gamma, proj, init)
        assert sc.shape == (bs, ns)
        for i in range(bs):
            for j in range(ns):
                n = neg[(i // chunk) * ns + j]
                hh, tt = (n, t[i]) if corrupt_head else (h[i], n)
                assert abs(sc[i, j].item() - _naive(model, hh, r[i], tt, gamma, None if proj is None else proj[i], init)) < 1e-9


@pytest.mark.parametrize("model", ["TransE_l1", "ComplEx", "RotatE"])
def test_trainer_learns_a_small_graph(model):
    g = torch.Generator().manual_seed(0)
    k = TorchKGE(150, 5, 16, model, gamma=6.0, lr=0.1, seed=1)
    h = torch.randint(0, 150, (48,), generator=g); r = torch.randint(0, 5, (48,), generator=g); t = (h * 5 + r) % 150
    first = last = None
    for s in range(150):
        last = k.train_step(h, r, t, torch.randint(0, 150, (3 * 8,), generator=g), chunk=16)
        first = first if first is not None else last
    assert last < 0.5 * first and k.evaluate(h, r, t, 64, g)["MRR"] > 0.5


def test_dataset_from_fake_files(tmp_path):
    (tmp_path / "train.tsv").write_text("a\tlikes\tb\nb\tlikes\tc\nc\thates\ta\n")
    (tmp_path / "valid.tsv").write_text("a\thates\tc\n")
    ds = K.KGDataset.load(str(tmp_path), ["train.tsv", "valid.tsv"], "raw_udd_hrt")
    assert (ds.n_entities, ds.n_relations) == (3, 2) and ds.train[0].tolist() == [0, 1, 2] and ds.train[2].tolist() == [1, 2, 0]
    assert ds.valid[1].tolist() == [1] and ds.test is None
    assert (tmp_path / "entities.tsv").read_text().splitlines() == ["0\ta", "1\tb", "2\tc"]
    # the same triples with columns in another order, then the id form with the dictionaries written above
    (tmp_path / "ids.tsv").write_text("0\t1\t2\n")
    d2 = K.KGDataset.load(str(tmp_path), ["entities.tsv", "relations.tsv", "ids.tsv"], "udd_hrt")
    assert d2.n_entities == 3 and d2.train[1].tolist() == [1]
    (tmp_path / "bad.tsv").write_text("0\t9\t2\n")
    with pytest.raises(ValueError):
        K.KGDataset.load(str(tmp_path), ["entities.tsv", "relations.tsv", "bad.tsv"], "udd_hrt")
    (tmp_path / "t2.tsv").write_text("a\tb\tlikes\n")           # (this load rewrites the dictionary files)
    assert K.KGDataset.load(str(tmp_path), ["t2.tsv"], "raw_udd_htr").train[1].tolist() == [0]


def test_partitions_cover_every_triple_once():
    ds = K.KGDataset.synthetic(500, 9, 6000, seed=1)
    rel = ds.train[1]
    for parts, cross in (K.balanced_relation_partition(rel, 4), K.soft_relation_partition(rel, 4, threshold=0.2)):
        allidx = np.concatenate(parts)
        assert np.array_equal(np.sort(allidx), np.arange(rel.size))
        for r in range(9):
            on = sum(1 for p in parts if (rel[p] == r).any())
            assert (on > 1) == bool(cross[r]) or (rel == r).sum() == 0
    bal, _ = K.balanced_relation_partition(rel, 4)
    assert max(p.size for p in bal) - min(p.size for p in bal) <= 1
    assert sum(p.size for p in K.random_partition(rel.size, 3)) == rel.size


def test_presample_hot_sets_and_renumbering():
    ds = K.KGDataset.synthetic(400, 4, 5000, seed=2)
    parts = K.random_partition(ds.train[0].size, 2)
    smp = [K.ChunkedNegativeSampler(tuple(x[p] for x in ds.train), 400, 32, 8, 8, seed=i) for i, p in enumerate(parts)]
    counts = K.presample(smp, 400, 10)
    assert all(int(c.sum()) == 10 * (32 * 2 + 32) for c in counts)
    hot = K.hot_sets(counts, 40)
    assert all(h.numel() <= 40 for h in hot) and not set(hot[0].tolist()) & set(hot[1].tolist())
    ds2, d = K.renumber_graph(ds, hot, 40)
    assert sorted(d.tolist()) == list(range(400))                      # a permutation
    for w, hs in enumerate(hot):
        assert ((d[hs] >= w * 40) & (d[hs] < (w + 1) * 40)).all()      # worker w's hot ids are its contiguous range
    assert np.array_equal(ds2.train[0], d.numpy()[ds.train[0]]) and np.array_equal(ds2.train[1], ds.train[1])


def test_driver_runs_on_cpu(tmp_path):
    from recstore_b200.cli import kge_main
    out, info = kge_main.main(["--model_name", "DistMult", "--max_step", "30", "--n_entities", "500", "--n_triples", "5000", "--hidden_dim", "16",
                               "--batch_size", "64", "--neg_sample_size", "16", "--soft_rel_part", "--cache_ratio", "0.2",
                               "--presample_steps", "5", "--test", "--save_path", str(tmp_path / "o"), "--log_interval", "1000"])
    r = out[0]
    assert r["steps"] == 30 and r["last_loss"] < r["first_loss"] and 0 < r["test"]["MRR"] <= 1
    assert info["presampled_hit_ratio"] > 0.1 and (tmp_path / "o" / "config.json").exists()


def test_driver_graph_partition_and_transr_checkpoint(tmp_path):
    """Edge-cut partition in the driver, and the TransR checkpoint with its per-relation projection file."""
    import numpy as np
    from recstore_b200.cli import kge_main
    out, info = kge_main.main(["--model_name", "TransR", "--max_step", "5", "--n_entities", "300", "--n_relations", "6", "--n_triples", "3000",
                               "--hidden_dim", "8", "--batch_size", "32", "--neg_sample_size", "8", "--num_proc", "2", "--graph_part",
                               "--save_path", str(tmp_path / "o"), "--log_interval", "1000"])
    assert 0.0 <= info["edge_cut"] <= 1.0 and out[0]["steps"] == 5
    proj = np.load(tmp_path / "o" / "synthetic_TransRprojection.npy")
    assert proj.shape == (6, 64)
    assert np.load(tmp_path / "o" / "synthetic_TransR_entity.npy").shape == (300, 8)
    # the inference loader reads the projection file too and scores with it
    import torch
    from recstore_b200.baseline.kge_torch import edge_score
    from recstore_b200.models.kge_infer import ScoreInfer
    inf = ScoreInfer.load(str(tmp_path / "o"))
    assert inf.projection is not None and inf.projection.shape == (6, 64)
    h, r, t = torch.tensor([1, 2]), torch.tensor([0, 5]), torch.tensor([7, 9])
    want = edge_score("TransR", inf.entity[h], inf.relation[r], inf.entity[t], inf.gamma, inf.projection[r], inf.emb_init)
    assert torch.allclose(inf._score(h, r, t), want)


def test_score_infer_modes_and_emb_similarity(tmp_path):
    from recstore_b200.models.kge_infer import EmbSimInfer, ScoreInfer
    g = torch.Generator().manual_seed(0)
    ent, rel = torch.randn(12, 8, generator=g), torch.randn(3, 8, generator=g)
    inf = ScoreInfer("DistMult", ent, rel)
    (h, r, t, s), = inf.topk(head=[0, 1], rel=[0, 2], tail=None, k=5, exec_mode="all")
    full = torch.stack([(ent[a] * rel[b] * ent[c]).sum() for a in (0, 1) for b in (0, 2) for c in range(12)])
    assert torch.allclose(s, torch.topk(full, 5).values, atol=1e-6)
    assert torch.allclose(s, (ent[h] * rel[r] * ent[t]).sum(1), atol=1e-6) and bool((s[:-1] >= s[1:]).all())
    per_head = inf.topk(head=[3, 4, 5], rel=[1], tail=[0, 1, 2, 3], k=2, exec_mode="batch_head")
    assert len(per_head) == 3 and all(x[0].unique().numel() == 1 for x in per_head)
    (h, r, t, s), = inf.topk([1, 2], [0, 1], [3, 4], k=10, exec_mode="triplet_wise")
    assert s.numel() == 2
    # checkpoints of the trainers load directly
    import json
    import numpy as np
    np.save(tmp_path / "d_DistMult_entity.npy", ent.numpy()); np.save(tmp_path / "d_DistMult_relation.npy", rel.numpy())
    (tmp_path / "config.json").write_text(json.dumps({"model_name": "DistMult", "gamma": 5.0, "emp_file": "d_DistMult_entity.npy",
                                                       "rmap_file": "d_DistMult_relation.npy"}))
    assert torch.equal(ScoreInfer.load(str(tmp_path)).entity, ent)
    sim = EmbSimInfer(ent, "cosine")
    (l, rr, v), = sim.topk(left=[0, 1, 2], right=None, k=3)
    assert torch.allclose(v, torch.ones(3), atol=1e-6) and torch.equal(l.sort().values, rr.sort().values)    # each id matches itself
    lists = EmbSimInfer(ent, "l2").topk(left=[5], right=[1, 5, 7], k=2, bcast=True)
    assert lists[0][1][0].item() == 5 and abs(lists[0][2][0].item()) < 1e-6
    for fn in ("l1", "dot", "ext_jaccard"):
        assert EmbSimInfer(ent, fn).topk([0, 1], [2, 3], k=1, pair_ws=True)[0][2].numel() == 1


def test_graph_cached_sampler_keeps_a_window_and_publishes_entity_ids():
    from recstore_b200.controller import GraphCachedSampler
    ds = K.KGDataset.synthetic(300, 4, 3000, seed=3)
    published = []

    class FakeController:
        def PublishReads(self, rank, step, ids):
            published.append((rank, step, ids.clone()))
    mk = lambda seed: K.ChunkedNegativeSampler(ds.train, 300, 16, 8, 8, seed=seed)
    cached = GraphCachedSampler.BatchCreateCachedSamplers(3, [mk(0), mk(1)], "CppAsyncV2", FakeController())
    assert len(published) == 6 and [p[1] for p in published if p[0] == 0] == [0, 1, 2]
    plain = mk(0)
    for step in range(4):
        got, want = next(cached[0]), next(plain)
        assert all(torch.equal(a, b) for a, b in zip(got[:4], want[:4])) and got[4] == want[4]     # same stream, L steps later
    mine = [p for p in published if p[0] == 0]
    assert [p[1] for p in mine] == list(range(7)) and mine[0][2].numel() == 16 * 2 + 16


def test_graph_partition_recovers_planted_blocks_and_balances():
    """Multilevel edge-cut partition (the METIS role of the reference's KG driver): a graph with 4 planted blocks and
    10 % of its edges rewired at random is cut close to those 10 %, far below a random assignment, with balanced
    parts; the result is deterministic and covers every triple exactly once."""
    import numpy as np
    from recstore_b200.utils import kg_data as K
    rng = np.random.default_rng(0)
    n, k, m = 8000, 4, 80000
    blk = rng.integers(0, k, n)
    members = [np.nonzero(blk == b)[0] for b in range(k)]
    h = rng.integers(0, n, m)
    t = np.empty(m, dtype=np.int64)
    for b in range(k):
        idx = np.nonzero(blk[h] == b)[0]
        t[idx] = rng.choice(members[b], idx.size)
    noise = rng.random(m) < 0.1
    t[noise] = rng.integers(0, n, int(noise.sum()))
    parts, part, st = K.graph_partition(h, t, n, k, seed=3)
    assert st["edge_cut"] < 0.15 and st["max_part"] < 1.06, st
    assert np.mean(rng.integers(0, k, n)[h] != rng.integers(0, k, n)[t]) > 0.6          # what a random assignment cuts
    allidx = np.sort(np.concatenate(parts))
    assert allidx.size == m and np.array_equal(allidx, np.arange(m))
    for p, idx in enumerate(parts):
        assert np.all(part[t[idx]] == p)
    parts2, part2, _ = K.graph_partition(h, t, n, k, seed=3)
    assert np.array_equal(part, part2)
    _, pn, stn = K.graph_partition(h, t, n, k, seed=3, balance="nodes")
    assert np.bincount(pn, minlength=k).max() <= 1.04 * n / k + 1
    _, p1, st1 = K.graph_partition(h, t, n, 1)
    assert not p1.any() and st1["edge_cut"] == 0.0
    import pytest
    with pytest.raises(Exception):
        K.graph_partition(np.array([0, n]), np.array([1, 2]), n, 2)


def test_loss_genres_match_their_definitions():
    """Criteria of the reference's loss generator (loss.py:10-99): label +1 for positives, -1 (0 for BCE) for negatives,
    negatives averaged or self-adversarially weighted, the two parts averaged."""
    import torch
    import torch.nn.functional as F
    from recstore_b200.baseline.kge_torch import kg_loss, logsigmoid_loss
    g = torch.Generator().manual_seed(0)
    pos, neg = torch.randn(16, generator=g) * 3, torch.randn(16, 7, generator=g) * 3
    assert torch.allclose(kg_loss(pos, neg), logsigmoid_loss(pos, neg))
    assert torch.allclose(kg_loss(pos, neg, "Logistic"), (F.softplus(-pos).mean() + F.softplus(neg).mean(-1).mean()) / 2)
    want = ((2.0 - pos).clamp_min(0).mean() + (2.0 + neg).clamp_min(0).mean(-1).mean()) / 2
    assert torch.allclose(kg_loss(pos, neg, "Hinge", margin=2.0), want)
    bce = (-torch.log(torch.sigmoid(pos)).mean() - torch.log(1 - torch.sigmoid(neg)).mean(-1).mean()) / 2
    assert torch.allclose(kg_loss(pos, neg, "BCE"), bce, atol=1e-5)
    w = torch.softmax(neg * 0.5, -1)
    adv = (-F.logsigmoid(pos).mean() + (w * -F.logsigmoid(-neg)).sum(-1).mean()) / 2
    assert torch.allclose(kg_loss(pos, neg, adversarial=True, temperature=0.5), adv)
    ew = torch.rand(16, generator=g)
    wl = ((-F.logsigmoid(pos) * ew).mean() + (-F.logsigmoid(-neg) * ew[:, None]).mean(-1).mean()) / 2
    assert torch.allclose(kg_loss(pos, neg, edge_weight=ew), wl)
    # the adversarial weights carry no gradient
    n2 = neg.clone().requires_grad_(True)
    kg_loss(pos, n2, adversarial=True).backward()
    direct = torch.autograd.grad((torch.softmax(neg, -1) * -F.logsigmoid(-n2)).sum(-1).mean() / 2, n2)[0]
    assert torch.allclose(n2.grad, direct)


def test_driver_reference_flags(tmp_path):
    """The rest of the reference's command line: loss options, degree-based negatives, validation during training,
    worker barriers, edge importance from a fourth column, --no_save_emb."""
    import numpy as np
    from recstore_b200.cli import kge_main
    rng = np.random.default_rng(0)
    with open(tmp_path / "train.tsv", "w") as f:
        for _ in range(600):
            f.write(f"e{rng.integers(0, 50)}|r{rng.integers(0, 4)}|e{rng.integers(0, 50)}|{rng.random():.3f}\n")
    out, info = kge_main.main(["--model_name", "ComplEx", "--dataset", "toy", "--data_path", str(tmp_path), "--data_files", "train.tsv",
                               "--format", "raw_udd_hrt", "--delimiter", "|", "--has_edge_importance", "--hidden_dim", "8", "--double_ent",
                               "--double_rel", "--batch_size", "32", "--neg_sample_size", "8", "--max_step", "12", "-lg", "Hinge",
                               "-m", "2.0", "-adv", "-a", "0.5", "-rc", "1e-6", "-rn", "3", "--neg_deg_sample", "--num_proc", "2",
                               "--force_sync_interval", "4", "--num_thread", "1", "--save_path", str(tmp_path / "o"), "--no_save_emb",
                               "--log_interval", "1000"])
    assert out[0]["steps"] == 12 and np.isfinite(out[0]["last_loss"]) and info["n_entities"] <= 50
    assert not (tmp_path / "o").exists()
    out, _ = kge_main.main(["--model_name", "DistMult", "--max_step", "20", "--n_entities", "300", "--n_triples", "3000", "--hidden_dim", "8",
                            "--batch_size", "32", "--neg_sample_size", "8", "--valid", "--eval_interval", "10", "--eval_percent", "0.5",
                            "--log_interval", "1000"])
    assert [v["step"] for v in out[0]["valid"]] == [10, 20] and 0 < out[0]["valid"][-1]["MRR"] <= 1
    import pytest
    with pytest.raises(SystemExit):
        kge_main.main(["--pairwise"])


def test_partition_files_for_multi_machine_runs(tmp_path):
    """Per-part directories: triples in global ids, owned entities first in the local-to-global map, halo entities after."""
    import json
    import numpy as np
    from recstore_b200.utils import kg_data as K
    ds = K.KGDataset.synthetic(300, 6, 3000, seed=2)
    parts, node, _ = K.graph_partition(ds.train[0], ds.train[2], 300, 3, seed=1)
    dirs = K.write_partition_files(str(tmp_path), ds, parts, node)
    seen = 0
    for p, d in enumerate(dirs):
        tri = np.loadtxt(f"{d}/train.txt", dtype=np.int64, ndmin=2)
        l2g = np.loadtxt(f"{d}/local_to_global.txt", dtype=np.int64, ndmin=1)
        book = np.loadtxt(f"{d}/partition_book.txt", dtype=np.int64, ndmin=1)
        meta = json.load(open(f"{d}/meta.json"))
        assert tri.shape == (parts[p].size, 3) and np.array_equal(tri[:, 0], ds.train[0][parts[p]])
        assert np.all(node[tri[:, 2]] == p)                                   # a triple lives with its tail
        assert np.all(book[: meta["n_owned_entities"]] == p) and np.all(book[meta["n_owned_entities"]:] != p)
        assert np.isin(np.unique(tri[:, [0, 2]]), l2g).all() and np.unique(l2g).size == l2g.size
        seen += tri.shape[0]
    assert seen == ds.train[0].size
    out = K._main(["-k", "2", "--out", str(tmp_path / "cli"), "--n_entities", "200", "--n_triples", "1500"])
    assert len(out["parts"]) == 2 and sum(out["triples_per_part"]) > 1000 and (tmp_path / "cli" / "part_0" / "meta.json").exists()
    # without a node partition the owner is the part holding most of the entity's triples
    rp = K.random_partition(ds.train[0].size, 2, 0)
    assert len(K.write_partition_files(str(tmp_path / "r"), ds, rp)) == 2


def test_distributed_trainer_against_ps_shards(tmp_path):
    """KVStore mode: two server shards with server-side row-wise Adagrad, two trainer processes on an edge-cut
    partition; the loss falls, every entity / relation key lives on exactly one shard, the checkpoint has the usual
    files."""
    import numpy as np
    from recstore_b200.cli import kge_dist
    out = kge_dist.main(["--model_name", "TransE_l2", "--num_servers", "2", "--num_clients", "2", "--max_step", "40", "--n_entities", "1500",
                         "--n_relations", "10", "--n_triples", "15000", "--hidden_dim", "16", "--batch_size", "64", "--neg_sample_size", "16",
                         "--gamma", "6", "--graph_part", "--test", "--save_path", str(tmp_path / "ck"), "--partition_dir", str(tmp_path / "parts")])
    assert sum(out["server_keys"]) == 1500 + 10 and min(out["server_keys"]) > 500
    for w in out["workers"]:
        assert w["last_loss"] < w["first_loss"]
    assert 0 < out["test"]["MRR"] <= 1 and 0 <= out["prepared"]["edge_cut"] <= 1
    assert np.load(tmp_path / "ck" / "synthetic_TransE_l2_entity.npy").shape == (1500, 16)
    assert np.load(tmp_path / "ck" / "synthetic_TransE_l2_relation.npy").shape == (10, 16)
    assert (tmp_path / "parts" / "part_1" / "train.txt").exists()
    # a second run trains straight from the directories the first one wrote
    out2 = kge_dist.main(["--model_name", "DistMult", "--num_servers", "1", "--max_step", "10", "--hidden_dim", "8", "--batch_size", "32",
                          "--neg_sample_size", "8", "--from_partition_dir", str(tmp_path / "parts")])
    assert len(out2["workers"]) == 2 and out2["prepared"]["n_entities"] == 1500 and sum(out2["server_keys"]) == 1510


def test_full_filtered_ranking_matches_brute_force_and_driver_flag():
    import torch
    from recstore_b200.baseline.kge_torch import TorchKGE, edge_score, known_triple_index
    m = TorchKGE(40, 3, 8, "TransE_l2", gamma=6, seed=1)
    h, r, t = torch.tensor([1, 2, 3, 1]), torch.tensor([0, 1, 2, 0]), torch.tensor([4, 5, 6, 9])
    raw = m.evaluate_full(h, r, t)
    known = known_triple_index((h, r, t))
    filt = m.evaluate_full(h, r, t, known)
    E, R = m.entity, m.relation
    pos = edge_score("TransE_l2", E[h], R[r], E[t], 6)
    ranks_raw, ranks_f = [], []
    for i in range(4):
        for side in ("tail", "head"):
            if side == "tail":
                sc = edge_score("TransE_l2", E[h[i]].expand(40, -1), R[r[i]].expand(40, -1), E, 6)
                truth, others = int(t[i]), [int(t[j]) for j in range(4) if int(h[j]) == int(h[i]) and int(r[j]) == int(r[i])]
            else:
                sc = edge_score("TransE_l2", E, R[r[i]].expand(40, -1), E[t[i]].expand(40, -1), 6)
                truth, others = int(h[i]), [int(h[j]) for j in range(4) if int(t[j]) == int(t[i]) and int(r[j]) == int(r[i])]
            sc = sc.clone(); sc[truth] = float("-inf")
            ranks_raw.append(1 + int((sc > pos[i]).sum()))
            sc[others] = float("-inf")
            ranks_f.append(1 + int((sc > pos[i]).sum()))
    assert abs(raw["MRR"] - sum(1 / x for x in ranks_raw) / 8) < 1e-6
    assert abs(filt["MRR"] - sum(1 / x for x in ranks_f) / 8) < 1e-6 and filt["MRR"] >= raw["MRR"]
    from recstore_b200.cli import kge_main
    out, _ = kge_main.main(["--model_name", "DistMult", "--max_step", "30", "--n_entities", "300", "--n_triples", "3000", "--hidden_dim", "8",
                            "--batch_size", "32", "--neg_sample_size", "8", "--test", "--neg_sample_size_eval", "-1", "--log_interval", "1000"])
    assert out[0]["test"]["candidates"] == 300 and 0 < out[0]["test"]["MRR"] <= 1


def test_renumber_by_partition_aligns_ids_with_cyclic_sharding():
    import numpy as np
    from recstore_b200.utils import kg_data as K
    ds = K.KGDataset.synthetic(1001, 5, 8000, seed=4)
    parts, node, _ = K.graph_partition(ds.train[0], ds.train[2], 1001, 4, seed=2, balance="nodes")
    ds2, new_id = K.renumber_by_partition(ds, node, 4)
    assert np.array_equal(np.sort(new_id), np.arange(1001))                       # a permutation
    assert np.mean(new_id % 4 == node) > 0.95                                     # all but the spill of oversized parts
    assert np.array_equal(ds2.train[0], new_id[ds.train[0]]) and np.array_equal(ds2.train[1], ds.train[1])
    assert np.array_equal(ds2.test[2], new_id[ds.test[2]])
    # triples of part p now mostly name entities with id % 4 == p
    local = np.mean([(np.mean(ds2.train[2][idx] % 4 == p)) for p, idx in enumerate(parts)])
    assert local > 0.9
    skew = np.zeros(1001, dtype=np.int32); skew[:700] = 0; skew[700:] = 1          # one oversized part spills
    _, nid = K.renumber_by_partition(ds, skew, 2)
    assert np.array_equal(np.sort(nid), np.arange(1001)) and np.mean(nid[700:] % 2 == 1) == 1.0


def test_async_entity_update_applies_every_gradient_and_reports_failures():
    """--async_update: a worker thread applies the entity updates behind the trainer.  With batches that touch disjoint
    rows the order of application cannot matter, so after finish_async_update() the tables equal the synchronous run's
    bit for bit; a failing update surfaces in the trainer; the driver flag trains."""
    from recstore_b200.baseline.kge_torch import TorchKGE
    from recstore_b200.cli import kge_main
    E, R, D, bs, ns = 4000, 7, 16, 32, 8
    a = TorchKGE(E, R, D, "DistMult", seed=3)
    b = TorchKGE(E, R, D, "DistMult", seed=3)
    b.create_async_update(max_pending=2)
    g = torch.Generator().manual_seed(1)
    perm = torch.randperm(E, generator=g)
    per = 2 * bs + ns * (bs // 8)                    # rows a step touches: heads, tails, chunked negatives
    for s in range(20):
        blk = perm[s * per:(s + 1) * per]
        h, t, n = blk[:bs], blk[bs:2 * bs], blk[2 * bs:]
        r = torch.randint(0, R, (bs,), generator=g)
        la = a.train_step(h, r, t, n, 8, corrupt_head=bool(s & 1))
        lb = b.train_step(h, r, t, n, 8, corrupt_head=bool(s & 1))
        assert la == lb                               # disjoint rows: a queued update cannot change this step's inputs
    b.finish_async_update()
    assert torch.equal(a.entity, b.entity) and torch.equal(a.state["entity"], b.state["entity"])
    assert torch.equal(a.relation, b.relation) and b._async_thread is None
    b.finish_async_update()                           # idempotent
    c = TorchKGE(E, R, D, "DistMult", seed=3)
    c.create_async_update()
    c.state["entity"] = torch.zeros(3)                # the worker's index_add_ goes out of range
    blk = perm[-per:]
    c.train_step(blk[:bs], torch.zeros(bs, dtype=torch.long), blk[bs:2 * bs], blk[2 * bs:], 8)
    with pytest.raises(RuntimeError, match="asynchronous entity update failed"):
        c.finish_async_update()
    out, _ = kge_main.main(["--device", "cpu", "--model_name", "TransE_l2", "--max_step", "150", "--n_entities", "500",
                            "--n_triples", "5000", "--hidden_dim", "32", "--batch_size", "128", "--neg_sample_size", "16",
                            "--async_update", "--log_interval", "1000", "--gamma", "6"])
    assert out[0]["last_loss"] < out[0]["first_loss"]


def test_link_predict_blocks_exclusion_and_model_objects(tmp_path):
    """Blocked top-k equals the one-shot ranking; `mask` / `exclude` treat triples of the attached graph as the
    reference's link_predict does (ke_model.py:205-455, 457-640); model objects load the trainers' checkpoints."""
    import json
    import numpy as np
    from recstore_b200.models import kge_infer as I
    g = torch.Generator().manual_seed(1)
    ent, rel = torch.randn(40, 8, generator=g), torch.randn(5, 8, generator=g)
    inf = I.ScoreInfer("TransE_l2", ent, rel, gamma=10.0)
    hs, ts = torch.arange(20), torch.arange(20, 40)          # disjoint, so no two candidates tie
    H, R, T = torch.meshgrid(hs, torch.arange(5), ts, indexing="ij")
    H, R, T = H.reshape(-1), R.reshape(-1), T.reshape(-1)
    full = 10.0 - (ent[H] + rel[R] - ent[T]).norm(dim=1)
    want = torch.topk(full, 25)
    for batch in (7, 1000, 1 << 16):                         # the block size does not change the answer
        (h, r, t, s), = inf.topk(hs, None, ts, k=25, exec_mode="all", batch_size=batch)
        assert torch.allclose(s, want.values, atol=1e-5)
        assert torch.equal(h, H[want.indices]) and torch.equal(r, R[want.indices]) and torch.equal(t, T[want.indices])
    # logsigmoid output keeps the order and changes the values
    (h2, r2, t2, s2), = I.ScoreInfer("TransE_l2", ent, rel, gamma=10.0, sfunc="logsigmoid").topk(hs, None, ts, k=25)
    assert torch.equal(h2, h) and torch.equal(t2, t) and torch.allclose(s2, torch.nn.functional.logsigmoid(want.values), atol=1e-5)
    # the ten best triples "exist": mask marks them, exclude returns the next ones
    inf.attach_graph(h[:10], r[:10], t[:10])
    (mh, mr, mt, ms, mask), = inf.topk(hs, None, ts, k=25, exclude_mode="mask")
    assert mask[:10].all() and not mask[10:].any() and torch.equal(mh, h)
    (eh, er, et, es), = inf.topk(hs, None, ts, k=12, exclude_mode="exclude")
    assert torch.equal(eh, h[10:22]) and torch.equal(er, r[10:22]) and torch.equal(et, t[10:22]) and torch.allclose(es, want.values[10:22], atol=1e-5)
    inf.attach_graph(H[:1990], R[:1990], T[:1990])           # nearly everything exists
    (eh, er, et, es), = inf.topk(hs, None, ts, k=25, exclude_mode="exclude")
    assert es.numel() == 10 and bool(((eh * 5 + er) * 20 + (et - 20) >= 1990).all())
    per_tail = inf.topk(head=[1, 2, 3], rel=[0, 1], tail=[7, 8], k=4, exec_mode="batch_tail", exclude_mode="mask")
    assert len(per_tail) == 2 and all(len(x) == 5 and x[2].unique().numel() == 1 for x in per_tail)
    with pytest.raises(AssertionError):
        I.ScoreInfer("TransE_l2", ent, rel).topk(k=3, exclude_mode="exclude")      # no graph attached
    with pytest.raises(ValueError):
        inf.topk(k=3, exec_mode="sideways")
    # model objects
    np.save(tmp_path / "d_DistMult_entity.npy", ent.numpy()); np.save(tmp_path / "d_DistMult_relation.npy", rel.numpy())
    (tmp_path / "config.json").write_text(json.dumps({"model_name": "DistMult", "gamma": 5.0, "emp_file": "d_DistMult_entity.npy",
                                                       "rmap_file": "d_DistMult_relation.npy"}))
    m = I.DistMultModel().load(str(tmp_path))
    assert m.model_name == "DistMult" and m.num_entity == 40 and m.num_rel == 5 and m.graph is None
    (h, r, t, s), = m.link_predict(head=[0, 1], rel=None, tail=None, topk=6)
    assert torch.allclose(s, (ent[h] * rel[r] * ent[t]).sum(1), atol=1e-6) and bool((s[:-1] >= s[1:]).all())
    m.attach_graph(h[:2], r[:2], t[:2])
    (h3, r3, t3, s3), = m.link_predict(head=[0, 1], topk=4, exclude_mode="exclude")
    assert torch.equal(h3, h[2:6]) and torch.equal(t3, t[2:6])
    (l, rr, v), = m.embed_sim(left=[0, 1, 2], embed_type="entity", topk=3)
    assert torch.allclose(v, torch.ones(3), atol=1e-6)
    lists = m.embed_sim(left=[0, 4], right=None, embed_type="relation", sfunc="l2", bcast=True, topk=2)
    assert len(lists) == 2 and lists[1][1][0].item() == 4
    np.save(tmp_path / "entity.npy", ent.numpy()); np.save(tmp_path / "relation.npy", rel.numpy())
    (tmp_path / "config.json").unlink()
    assert I.TransE_l1Model(gamma=3.0).load(str(tmp_path)).model_name == "TransE_l1"      # default file names, no config
    # RESCAL checkpoints that keep the matrices in the relation file
    mats = torch.randn(5, 64, generator=g)
    ri = I.ScoreInfer("RESCAL", ent, mats)
    got = ri._score(torch.tensor([1]), torch.tensor([2]), torch.tensor([3]))
    assert torch.allclose(got, ent[1] @ mats[2].view(8, 8) @ ent[3], atol=1e-5)
    # big pairwise similarity goes through blocks too
    big = torch.randn(3000, 4, generator=g)
    (l, rr, v), = I.EmbSimInfer(big, "dot").topk(k=5, batch_size=512)
    ref = torch.topk((big @ big.t()).reshape(-1), 5)
    assert torch.allclose(v, ref.values, atol=1e-5) and torch.equal(l * 3000 + rr, ref.indices)


def test_kge_infer_cli_score_emb_sim_eval_convert(tmp_path):
    """The four tools around a saved model (infer_score.py, infer_emb_sim.py, eval.py, convert.py of the reference)."""
    import json
    from recstore_b200.cli import kge_infer, kge_main
    ck = tmp_path / "ck"
    data = ["--n_entities", "200", "--n_relations", "5", "--n_triples", "4000"]
    kge_main.main(["--model_name", "DistMult", "--max_step", "60", "--hidden_dim", "16", "--batch_size", "64", "--neg_sample_size", "16",
                   "--save_path", str(ck), "--log_interval", "1000"] + data)
    # eval: one process and three processes rank the same triples, so the averages agree
    one = kge_infer.main(["eval", "--model_path", str(ck), "--json_out", str(tmp_path / "m.json")] + data, return_result=True)
    three = kge_infer.main(["eval", "--model_path", str(ck), "--num_proc", "3"] + data, return_result=True)
    assert one["filtered"] and one["processes"] == 1 and three["processes"] == 3 and one["triples"] == three["triples"] == 80
    for k in ("MRR", "MR", "HITS@10"):
        assert abs(one[k] - three[k]) < 1e-5, (k, one[k], three[k])
    assert 1.0 <= one["MR"] <= 200 and 0 < one["MRR"] <= 1 and json.load(open(tmp_path / "m.json"))["MRR"] == one["MRR"]
    raw = kge_infer.main(["eval", "--model_path", str(ck), "--no_eval_filter"] + data, return_result=True)
    assert not raw["filtered"] and raw["MR"] >= one["MR"]                       # filtering can only improve a rank
    sampled = kge_infer.main(["eval", "--model_path", str(ck), "--neg_sample_size_eval", "32"] + data, return_result=True)
    assert 1.0 <= sampled["MR"] <= 33
    # score: heads and relations listed, every tail a candidate
    (tmp_path / "h.list").write_text("3\n7\n")
    (tmp_path / "r.list").write_text("1\n")
    out = tmp_path / "res.tsv"
    assert kge_infer.main(["score", "--model_path", str(ck), "--format", "h_r_*", "--data_files", str(tmp_path / "h.list"), str(tmp_path / "r.list"),
                           "--exec_mode", "batch_head", "--topK", "4", "--output", str(out)]) == 0
    rows = [l.split("\t") for l in out.read_text().strip().split("\n")]
    assert rows[0] == ["head", "rel", "tail", "score"] and len(rows) == 1 + 2 * 4
    assert [r[0] for r in rows[1:]] == ["3"] * 4 + ["7"] * 4 and all(r[1] == "1" for r in rows[1:])
    ent, rel = np.load(ck / "synthetic_DistMult_entity.npy"), np.load(ck / "synthetic_DistMult_relation.npy")
    best = np.argsort(-(ent[3] * rel[1] * ent).sum(1))[:4]
    assert [int(r[2]) for r in rows[1:5]] == best.tolist()
    # ... by name, with the best candidate declared known and excluded
    (tmp_path / "e.map").write_text("".join(f"{i}\tent{i}\n" for i in range(200)))
    (tmp_path / "r.map").write_text("".join(f"{i}\trel{i}\n" for i in range(5)))
    (tmp_path / "hn.list").write_text("ent3\n")
    (tmp_path / "rn.list").write_text("rel1\n")
    (tmp_path / "known.tsv").write_text(f"3\t1\t{best[0]}\n")
    assert kge_infer.main(["score", "--model_path", str(ck), "--format", "h_r_*", "--data_files", str(tmp_path / "hn.list"), str(tmp_path / "rn.list"),
                           "--raw_data", "--entity_mfile", str(tmp_path / "e.map"), "--rel_mfile", str(tmp_path / "r.map"), "--topK", "3",
                           "--exclude_mode", "exclude", "--known_files", str(tmp_path / "known.tsv"), "--output", str(out)]) == 0
    rows = [l.split("\t") for l in out.read_text().strip().split("\n")][1:]
    assert [r[2] for r in rows] == [f"ent{i}" for i in best[1:4]] and rows[0][0] == "ent3" and rows[0][1] == "rel1"
    with pytest.raises(SystemExit):
        kge_infer.main(["score", "--model_path", str(ck), "--format", "h_r_t", "--data_files", str(tmp_path / "h.list")])
    # emb_sim: each listed id against everything; itself comes first
    assert kge_infer.main(["emb_sim", "--emb_file", str(ck / "synthetic_DistMult_entity.npy"), "--format", "l_*", "--data_files", str(tmp_path / "h.list"),
                           "--exec_mode", "batch_left", "--topK", "2", "--output", str(out)]) == 0
    rows = [l.split("\t") for l in out.read_text().strip().split("\n")]
    assert rows[0] == ["left", "right", "score"] and rows[1][:2] == ["3", "3"] and rows[3][:2] == ["7", "7"] and abs(float(rows[1][2]) - 1) < 1e-5
    # convert: names -> ids + dictionaries, column order as asked
    d = tmp_path / "raw"
    d.mkdir()
    (d / "train.tsv").write_text("a\tlikes\tb\nb\tlikes\tc\nc\tknows\ta\n")
    (d / "valid.tsv").write_text("a\tknows\tc\n")
    assert kge_infer.main(["convert", "--data_path", str(d), "--data_files", "train.tsv", "valid.tsv", "--output_format", "udd_htr",
                           "--output_path", str(tmp_path / "udd")]) == 0
    assert (tmp_path / "udd" / "train_output.txt").read_text() == "0\t1\t0\n1\t2\t0\n2\t0\t1\n"
    assert (tmp_path / "udd" / "valid_output.txt").read_text() == "0\t2\t1\n" and not (tmp_path / "udd" / "test_output.txt").exists()
    back = K.KGDataset.load(str(tmp_path / "udd"), ["entities.tsv", "relations.tsv", "train_output.txt", "valid_output.txt"], "udd_htr")
    assert back.n_entities == 3 and back.n_relations == 2 and back.train[1].tolist() == [0, 0, 1] and back.valid[2].tolist() == [2]


def test_external_embedding_trace_update_async_and_cross_relations(tmp_path):
    """The trainer's table object (tensor_models.py:217-476): traced lookups, row-wise Adagrad with duplicates,
    asynchronous update, relations shared across partitions, .npy round trip."""
    from recstore_b200.models.kg_embedding import ExternalEmbedding
    torch.manual_seed(0)
    e = ExternalEmbedding(50, 4, lr=0.5)
    e.init(0.3)
    assert float(e.emb.abs().max()) <= 0.3 and float(e.state_sum.abs().sum()) == 0
    w0 = e.emb.clone()
    idx = torch.tensor([3, 7, 3])
    rows = e(idx)
    assert rows.requires_grad and torch.equal(rows.detach(), w0[idx]) and torch.equal(e.curr_emb(), rows)
    assert not e(idx, trace=False).requires_grad and len(e.trace) == 1
    (rows * torch.tensor([[1.0], [2.0], [3.0]])).sum().backward()
    e.update()
    g = torch.tensor([[1.0] * 4, [2.0] * 4, [3.0] * 4])
    state = torch.zeros(50).index_add_(0, idx, (g * g).mean(1))
    want = w0.clone().index_add_(0, idx, -0.5 * g / (state[idx].sqrt() + 1e-10).unsqueeze(1))
    assert torch.allclose(e.emb, want, atol=1e-6) and torch.allclose(e.state_sum, state) and e.trace == [] and e.state_step == 1
    # asynchronous: the same updates, applied by the worker; after finish the table equals the synchronous one
    a, b = ExternalEmbedding(50, 4, lr=0.5), ExternalEmbedding(50, 4, lr=0.5)
    a.emb.copy_(w0); b.emb.copy_(w0)
    b.create_async_update()
    gen = torch.Generator().manual_seed(1)
    for _ in range(20):
        ids = torch.randint(0, 50, (16,), generator=gen)
        coef = torch.randn(16, 1, generator=gen)
        for t in (a, b):
            if t is b:
                t.wait_async_update()                # keep the two in lockstep so the results are comparable
            (t(ids) * coef).sum().backward()
            t.update()
    b.finish_async_update()
    assert torch.allclose(a.emb, b.emb, atol=1e-6) and torch.allclose(a.state_sum, b.state_sum, atol=1e-6)
    # relations 1 and 4 are shared by several partitions: their updates land in the global table, reads refresh from it
    glob, loc = ExternalEmbedding(6, 4, lr=0.5), ExternalEmbedding(6, 4, lr=0.5)
    glob.emb.fill_(1.0); loc.emb.fill_(2.0)
    loc.setup_cross_rels([1, 4], glob)
    assert loc.get_noncross_idx(torch.tensor([0, 1, 2, 4])).tolist() == [0, 2]
    r = loc(torch.tensor([1, 2]))
    assert torch.equal(r.detach(), torch.tensor([[1.0] * 4, [2.0] * 4]))          # row 1 came from the global table
    r.sum().backward()
    loc.update()
    assert float(glob.emb[1, 0]) == pytest.approx(1.0 - 0.5 / 1.0, abs=1e-6) and float(glob.emb[2, 0]) == 1.0
    assert float(loc.emb[2, 0]) == pytest.approx(2.0 - 0.5, abs=1e-6)
    e.save(str(tmp_path), "ent")
    f = ExternalEmbedding(50, 4)
    f.load(str(tmp_path), "ent")
    assert torch.equal(f.emb, e.emb)
    with pytest.raises(AssertionError):
        ExternalEmbedding(49, 4).load(str(tmp_path), "ent")


def test_custom_external_embedding_over_a_shared_table(tmp_path):
    """The RecStore-backed table object (cus_external_emb.py:20-215): DistEmbedding + cached embedding; update goes to
    the shared table; save / load work."""
    import os
    import recstore_b200 as rs
    from recstore_b200 import ipc
    from recstore_b200.models.kg_embedding import CustomExternalEmbedding
    ipc.set_namespace(f"pytest_cee_{os.getpid()}")
    rs.kvinit()
    c = CustomExternalEmbedding(40, 4, "cee_entity", lr=0.25, cached_emb_type="KGExternelEmbedding")
    c.init(0.0)
    assert float(c.emb.weight.abs().sum()) == 0
    c.init(0.2)
    w0 = c.emb.weight.clone()
    with pytest.raises(AssertionError):
        c(torch.tensor([1]))
    c.prepare_per_worker_process()
    idx = torch.tensor([5, 9, 5])
    rows = c(idx)
    assert torch.allclose(rows.detach(), w0[idx]) and torch.equal(c.curr_emb(), rows)
    rows.sum().backward()
    c.update()
    want = w0.clone().index_add_(0, idx, torch.full((3, 4), -0.25))
    assert torch.allclose(c.emb.weight, want, atol=1e-6) and c.trace == []
    c.save(str(tmp_path), "cee")
    c.emb.weight.zero_()
    c.load(str(tmp_path), "cee")
    assert torch.allclose(c.emb.weight, want, atol=1e-6)
    # the plain torch table as the "cache type": rows updated by a torch optimizer
    t = CustomExternalEmbedding(40, 4, "cee_entity2", lr=0.5, cached_emb_type="TorchNativeStdEmb")
    t.init(0.1)
    t.prepare_per_worker_process()
    before = t.cached_emb.weight.detach().clone()
    t(torch.tensor([2, 2, 3])).sum().backward()
    t.update()
    assert torch.allclose(t.cached_emb.weight.detach()[2], before[2] - 0.5 * 2, atol=1e-6)
    assert torch.allclose(t.cached_emb.weight.detach()[3], before[3] - 0.5, atol=1e-6)
    ipc.IPCTensorFactory.ClearIPCMemory()                    # leave nothing in shared memory


@pytest.mark.parametrize("model,floor", [("RotatE", 0.6), ("ComplEx", 0.5)])
def test_training_generalises_to_held_out_triples_of_a_planted_graph(model, floor):
    """Sampler -> scores -> loss -> sparse Adagrad -> filtered full ranking, end to end: on a graph whose relations are
    fixed shifts on a grid, held-out triples rank far above chance (MRR of a random table: ~0.02) after training."""
    from recstore_b200.baseline.kge_torch import known_triple_index
    ds = K.KGDataset.planted_grid(seed=0)
    assert ds.n_entities == 300 and ds.n_relations == 4 and ds.test[0].size == 104 and ds.train[0].size == 941
    m = TorchKGE(ds.n_entities, ds.n_relations, 16, model, gamma=6.0, lr=0.1, seed=0)
    known = known_triple_index(ds.train, ds.test)
    test = tuple(torch.from_numpy(x) for x in ds.test)
    before = m.evaluate_full(*test, known)["MRR"]
    train = tuple(torch.from_numpy(x) for x in ds.train)
    g = torch.Generator().manual_seed(1)
    for step in range(1500):
        b = torch.randint(0, train[0].numel(), (128,), generator=g)
        neg = torch.randint(0, ds.n_entities, (128,), generator=g)
        m.train_step(train[0][b], train[1][b], train[2][b], neg, 32, step % 2 == 1)
    after = m.evaluate_full(*test, known)
    assert before < 0.06 and after["MRR"] > floor and after["HITS@10"] > 0.8, (before, after)


def test_dataset_files_to_kvstore_trainers_to_checkpoint_to_eval_tool_generalises(tmp_path):
    """The whole chain on a graph with structure: id triples in files -> two trainer processes against two parameter-server
    shards (server-side row-wise Adagrad) -> checkpoint -> the stand-alone evaluation tool, which ranks the HELD-OUT
    triples against every entity (filtered).  Chance level is MRR ~0.02."""
    from recstore_b200.cli import kge_dist, kge_infer
    ds = K.KGDataset.planted_grid(seed=0)
    d = tmp_path / "grid"
    d.mkdir()
    (d / "entities.tsv").write_text("".join(f"{i}\te{i}\n" for i in range(ds.n_entities)))
    (d / "relations.tsv").write_text("".join(f"{i}\tr{i}\n" for i in range(ds.n_relations)))
    for name, split in (("train.txt", ds.train), ("valid.txt", ds.test), ("test.txt", ds.test)):
        (d / name).write_text("".join(f"{h}\t{r}\t{t}\n" for h, r, t in zip(*(x.tolist() for x in split))))
    files = ["entities.tsv", "relations.tsv", "train.txt", "valid.txt", "test.txt"]
    data = ["--dataset", "grid", "--data_path", str(d), "--data_files"] + files + ["--format", "udd_hrt"]
    out = kge_dist.main(["--model_name", "ComplEx", "--num_servers", "2", "--num_clients", "2", "--max_step", "1200", "--hidden_dim", "16",
                         "--batch_size", "128", "--neg_sample_size", "32", "--gamma", "6", "--lr", "0.1", "--save_path", str(tmp_path / "ck")] + data)
    assert sum(out["server_keys"]) == ds.n_entities + ds.n_relations
    res = kge_infer.main(["eval", "--model_path", str(tmp_path / "ck"), "--num_proc", "2"] + data, return_result=True)
    assert res["filtered"] and res["triples"] == 104 and res["model"] == "ComplEx"
    assert res["MRR"] > 0.4 and res["HITS@10"] > 0.7, res


def test_built_in_dataset_layouts_from_fake_files(tmp_path):
    """`--format built_in`: the directory layouts of the reference's named datasets, on hand-made files (its own tests
    use fake data files the same way: dgl-ke/tests/fake_data)."""
    d = tmp_path / "FB15k"
    d.mkdir()
    (d / "entities.dict").write_text("0\t/m/a\n1\t/m/b\n2\t/m/c\n")
    (d / "relations.dict").write_text("0\tlikes\n1\tknows\n")
    (d / "train.txt").write_text("/m/a\tlikes\t/m/b\n/m/b\tknows\t/m/c\n\n/m/c\tlikes\t/m/a\n")
    (d / "valid.txt").write_text("/m/a\tknows\t/m/c\n")
    ds = K.KGDataset.load_built_in(str(tmp_path), "FB15k")
    assert (ds.name, ds.n_entities, ds.n_relations) == ("FB15k", 3, 2) and ds.test is None
    assert [x.tolist() for x in ds.train] == [[0, 1, 2], [0, 1, 0], [1, 2, 0]] and [x.tolist() for x in ds.valid] == [[0], [1], [2]]
    assert ds.entity2id["/m/c"] == 2
    assert K.KGDataset.load(str(tmp_path), [], "built_in", name="FB15k").n_entities == 3      # through the general loader
    f = tmp_path / "Freebase"
    f.mkdir()
    (f / "entity2id.txt").write_text("5\n")
    (f / "relation2id.txt").write_text("3\n")
    (f / "train.txt").write_text("0\t4\t2\n3\t1\t0\n")                    # head, tail, relation
    (f / "test.txt").write_text("4\t0\t1\n")
    fb = K.KGDataset.load_built_in(str(tmp_path), "Freebase")
    assert (fb.n_entities, fb.n_relations) == (5, 3) and [x.tolist() for x in fb.train] == [[0, 3], [2, 0], [4, 1]]
    assert [x.tolist() for x in fb.test] == [[4], [1], [0]] and fb.valid is None
    (d / "test.txt").write_text("/m/a\tlikes\t/m/zzz\n")
    with pytest.raises(ValueError, match="not in the dictionaries"):
        K.KGDataset.load_built_in(str(tmp_path), "FB15k")
    (f / "train.txt").write_text("0\t9\t2\n")
    with pytest.raises(ValueError, match="outside"):
        K.KGDataset.load_built_in(str(tmp_path), "Freebase")
    with pytest.raises(FileNotFoundError, match="downloads nothing"):
        K.KGDataset.load_built_in(str(tmp_path), "wn18")
    with pytest.raises(ValueError, match="unknown built-in"):
        K.KGDataset.load_built_in(str(tmp_path), "imagenet")
    # the trainer's command line takes it
    (d / "test.txt").write_text("/m/b\tlikes\t/m/c\n")
    from recstore_b200.cli import kge_main
    out, info = kge_main.main(["--dataset", "FB15k", "--data_path", str(tmp_path), "--format", "built_in", "--max_step", "4", "--hidden_dim", "8",
                               "--batch_size", "2", "--neg_sample_size", "2", "--log_interval", "1000"])
    assert info["n_entities"] == 3 and out[0]["steps"] == 4


def test_kvstore_trainers_against_shards_that_run_already(tmp_path):
    """`--servers host:port ...`: the trainers use parameter-server processes started elsewhere (here: two stand-alone
    servers in threads) instead of starting their own -- the multi-machine form of the distributed trainer
    (dist_train.py / kvserver.py of the reference start servers and clients on the machines of an ip list)."""
    import queue, threading
    from recstore_b200.cli import kge_dist
    from recstore_b200.ps import server as ps_server
    stops, threads, ports = [], [], []
    for i in range(2):
        ev, ready = threading.Event(), queue.Queue()
        t = threading.Thread(target=ps_server.main, args=(["--port", "0", "--dim", "8", "--capacity", "65536", "--optimizer", "rowwise_adagrad",
                                                          "--lr", "0.1", "--workers", "2"], ev, ready.put))
        t.start()
        ports.append(ready.get(timeout=60))
        stops.append(ev); threads.append(t)
    assert len(ports) == 2
    out = kge_dist.main(["--model_name", "DistMult", "--servers", f"127.0.0.1:{ports[0]}", f"localhost:{ports[1]}", "--num_clients", "2",
                         "--max_step", "30", "--n_entities", "800", "--n_relations", "6", "--n_triples", "6000", "--hidden_dim", "8",
                         "--batch_size", "32", "--neg_sample_size", "8", "--lr", "0.1", "--test"])
    assert sum(out["server_keys"]) == 806 and min(out["server_keys"]) > 200
    assert all(w["last_loss"] < w["first_loss"] for w in out["workers"]) and 0 < out["test"]["MRR"] <= 1
    for ev in stops:
        ev.set()
    for t in threads:
        t.join(30)
    assert not any(t.is_alive() for t in threads)


def test_distributed_trainer_takes_the_loss_options():
    """Self-adversarial negatives, the other loss genres and the Lp penalty in the KVStore trainer (the reference's
    distributed mode takes the same CommonArgParser flags as its single-box trainer)."""
    from recstore_b200.cli import kge_dist
    base = ["--num_servers", "1", "--num_clients", "1", "--max_step", "40", "--n_entities", "400", "--n_relations", "5", "--n_triples", "4000",
            "--hidden_dim", "8", "--batch_size", "32", "--neg_sample_size", "8", "--gamma", "6"]
    for extra in (["-adv", "-a", "0.5"], ["--loss_genre", "Hinge", "--margin", "2.0"], ["-lg", "Logistic", "-rc", "1e-4", "-rn", "2"], ["-lg", "BCE"]):
        out = kge_dist.main(base + extra)
        w = out["workers"][0]
        assert w["last_loss"] < w["first_loss"] and w["last_loss"] == w["last_loss"], (extra, w)


def test_distributed_trainer_rotate_generalises_on_the_planted_graph(tmp_path):
    """RotatE through the KVStore trainer (relations use half of a shard row): held-out triples of the planted graph."""
    from recstore_b200.cli import kge_dist, kge_infer
    ds = K.KGDataset.planted_grid(seed=0)
    d = tmp_path / "grid"
    d.mkdir()
    (d / "entities.tsv").write_text("".join(f"{i}\te{i}\n" for i in range(ds.n_entities)))
    (d / "relations.tsv").write_text("".join(f"{i}\tr{i}\n" for i in range(ds.n_relations)))
    for name, split in (("train.txt", ds.train), ("valid.txt", ds.test), ("test.txt", ds.test)):
        (d / name).write_text("".join(f"{h}\t{r}\t{t}\n" for h, r, t in zip(*(x.tolist() for x in split))))
    data = ["--dataset", "grid", "--data_path", str(d), "--data_files", "entities.tsv", "relations.tsv", "train.txt", "valid.txt", "test.txt",
            "--format", "udd_hrt"]
    kge_dist.main(["--model_name", "RotatE", "--num_servers", "2", "--num_clients", "1", "--max_step", "1500", "--hidden_dim", "16",
                   "--batch_size", "128", "--neg_sample_size", "32", "--gamma", "6", "--lr", "0.1", "--save_path", str(tmp_path / "ck")] + data)
    import numpy as np
    assert np.load(tmp_path / "ck" / "grid_RotatE_relation.npy").shape == (4, 8)
    res = kge_infer.main(["eval", "--model_path", str(tmp_path / "ck")] + data, return_result=True)
    assert res["MRR"] > 0.5 and res["HITS@10"] > 0.8, res


@pytest.mark.parametrize("model", ["TransR", "RESCAL"])
def test_distributed_trainer_matrix_models(model, tmp_path):
    """TransR and RESCAL through the KVStore trainer: every relation's matrix is hidden_dim rows of the shards; the
    checkpoint has the projection file and the evaluation tool scores with it."""
    import numpy as np
    from recstore_b200.cli import kge_dist, kge_infer
    data = ["--n_entities", "300", "--n_relations", "4", "--n_triples", "3000"]
    out = kge_dist.main(["--model_name", model, "--num_servers", "2", "--num_clients", "2", "--max_step", "60", "--hidden_dim", "8",
                         "--batch_size", "32", "--neg_sample_size", "8", "--gamma", "6", "--lr", "0.1", "--test", "--save_path", str(tmp_path / "ck")] + data)
    assert sum(out["server_keys"]) == 300 + 4 + 4 * 8                       # entities, relation vectors, matrix rows
    assert all(w["last_loss"] < w["first_loss"] for w in out["workers"]) and 0 < out["test"]["MRR"] <= 1
    prj = np.load(tmp_path / "ck" / f"synthetic_{model}projection.npy")
    assert prj.shape == (4, 64) and np.abs(prj).sum() > 0
    res = kge_infer.main(["eval", "--model_path", str(tmp_path / "ck"), "--neg_sample_size_eval", "64"] + data, return_result=True)
    assert res["model"] == model and 1.0 <= res["MR"] <= 65


def test_planted_grid_by_name_through_trainer_and_eval_tool(tmp_path):
    """`--dataset planted_grid`: the demonstration graph straight from the command lines."""
    from recstore_b200.cli import kge_infer, kge_main
    out, info = kge_main.main(["--dataset", "planted_grid", "--model_name", "RotatE", "--hidden_dim", "16", "--gamma", "6", "--lr", "0.1",
                               "--batch_size", "128", "--neg_sample_size", "32", "--max_step", "1500", "--log_interval", "100000",
                               "--save_path", str(tmp_path / "ck")])
    assert info["n_entities"] == 300 and info["n_train"] == 941
    res = kge_infer.main(["eval", "--model_path", str(tmp_path / "ck"), "--dataset", "planted_grid"], return_result=True)
    assert res["triples"] == 104 and res["MRR"] > 0.5, res
