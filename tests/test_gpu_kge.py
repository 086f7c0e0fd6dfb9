"""KG scoring kernels + sharded tables against a PyTorch fp32 autograd reference (single GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_loss(model, gamma, h, r, t, neg, cs, ns, corrupt_head, emb_init):
    """Per-pair definition of every score function (the oracle of the PyTorch path)."""
    from recstore_b200.baseline.kge_torch import chunk_neg_score, edge_score, logsigmoid_loss
    pos = edge_score(model, h, r, t, gamma, None, emb_init)
    negs = chunk_neg_score(model, h, r, t, neg, corrupt_head, cs, gamma, None, emb_init)
    return logsigmoid_loss(pos, negs), pos, negs


@pytest.mark.parametrize("model", ["TransE_l2", "DistMult", "ComplEx", "SimplE", "TransE_l1", "RotatE"])
@pytest.mark.parametrize("corrupt_head", [False, True])
def test_kge_step_matches_autograd(model, corrupt_head):
    from recstore_b200.models.kge import KGEConfig, KGEModel
    from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update
    dev = torch.device("cuda:0")
    cfg = KGEConfig(n_entities=3000, n_relations=40, dim=400 if model in ("TransE_l2", "RotatE") else 64, model=model,
                    gamma=10.0, batch=512, neg_sample_size=128, neg_chunk_size=128, lr=0.1, seed=3)
    m = KGEModel(cfg)
    bs, ns, cs, D = cfg.batch, cfg.neg_sample_size, cfg.neg_chunk_size, cfg.dim
    g = torch.Generator(device=dev).manual_seed(1)
    # full copies for the oracle (world == 1: local rows are global rows)
    E = m.entity.weight[: cfg.n_entities].clone(); R = m.relation.weight[: cfg.n_relations].clone()
    SE = torch.zeros(cfg.n_entities, device=dev); SR = torch.zeros(cfg.n_relations, device=dev)
    for step in range(2):
        hi = torch.randint(0, 200, (bs,), device=dev, generator=g)              # few entities -> many duplicates
        ti = torch.randint(0, cfg.n_entities, (bs,), device=dev, generator=g)
        ri = torch.randint(0, cfg.n_relations, (bs,), device=dev, generator=g)
        ni = torch.randint(0, cfg.n_entities, (bs // cs * ns,), device=dev, generator=g)
        h = E[hi].clone().requires_grad_(True); t = E[ti].clone().requires_grad_(True)
        r = R[ri].clone().requires_grad_(True); n = E[ni].clone().requires_grad_(True)
        loss_ref, pos_ref, neg_ref = _ref_loss(model, cfg.gamma, h, r, t, n, cs, ns, corrupt_head, m.emb_init)
        loss_ref.backward()
        pos, negs = m.score_batch(hi, ri, ti, ni, corrupt_head)
        assert torch.allclose(pos, pos_ref, atol=2e-3, rtol=1e-3)
        assert torch.allclose(negs, neg_ref, atol=3e-2, rtol=2e-2)               # bf16 operands in the cross products
        loss = m.train_step(hi, ri, ti, ni, corrupt_head)
        assert abs(loss.item() - loss_ref.item()) < 5e-3 * max(1.0, abs(loss_ref.item()))
        # gradients as produced by the kernels vs autograd
        ge = torch.cat([h.grad, t.grad, n.grad])
        err = ((m.ent_grad - ge).norm() / ge.norm()).item()
        assert err < 3e-2, err
        err_r = ((m.rel_grad - r.grad).norm() / r.grad.norm()).item()
        assert err_r < 3e-2, err_r
        # the optimizer on the owners: exact semantics given the kernels' own gradients
        rowwise_adagrad_update(E, SE, torch.cat([hi, ti, ni]), m.ent_grad.clone(), cfg.lr, cfg.eps)
        rowwise_adagrad_update(R, SR, ri, m.rel_grad.clone(), cfg.lr, cfg.eps)
        torch.cuda.synchronize()
        assert torch.allclose(m.entity.weight[: cfg.n_entities], E, atol=2e-3, rtol=2e-3)
        assert torch.allclose(m.relation.weight[: cfg.n_relations], R, atol=2e-3, rtol=2e-3)
    m.ctx.check_status()


def test_kge_training_improves_mrr_and_checkpoints(tmp_path):
    from recstore_b200.models.kge import KGEConfig, KGEModel, KGSampler
    import numpy as np, json, os
    dev = torch.device("cuda:0")
    cfg = KGEConfig(n_entities=2000, n_relations=8, dim=64, model="TransE_l2", gamma=10.0, batch=512, neg_sample_size=64,
                    neg_chunk_size=64, lr=0.25, seed=1)
    m = KGEModel(cfg)
    smp = KGSampler(cfg, n_triples=4000, alpha=1.3, device=dev, seed=2)
    ev = (smp.h[:512], smp.r[:512], smp.t[:512])
    before = m.evaluate(*ev, generator=torch.Generator(device=dev).manual_seed(0))
    losses = []
    for step in range(300):
        h, r, t, neg = next(smp)
        losses.append(m.train_step(h, r, t, neg))
    after = m.evaluate(*ev, generator=torch.Generator(device=dev).manual_seed(0))
    m.ctx.check_status()
    assert losses[-1].item() < losses[0].item()
    assert after["MRR"] > before["MRR"] + 0.2 and after["HITS@10"] > before["HITS@10"]
    m.save(str(tmp_path))
    conf = json.load(open(os.path.join(tmp_path, "config.json")))
    assert conf["emp_file"] == "synthetic_TransE_l2_entity.npy" and conf["dim"] == 64
    ent = np.load(os.path.join(tmp_path, "synthetic_TransE_l2_entity.npy"))
    assert ent.shape == (2000, 64) and np.allclose(ent, m.entity.weight[:2000].cpu().numpy())
    m2 = KGEModel(cfg)
    m2.load(str(tmp_path))
    assert torch.equal(m2.entity.weight, m.entity.weight)


@pytest.mark.parametrize("corrupt_head", [False, True])
def test_rescal_step_matches_autograd_with_one_state_per_relation(corrupt_head):
    """RESCAL natively: scores, loss and gradients against autograd on h^T M_r t; the row-blocked relation table (D rows
    per relation) must move exactly like a [n_relations, D*D] table under row-wise Adagrad, i.e. with ONE accumulator
    value per relation, shared by its D rows."""
    from recstore_b200.models.kge import KGEConfig, KGEModel
    from recstore_b200.baseline.kge_torch import chunk_neg_score, edge_score, logsigmoid_loss
    from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update
    dev = torch.device("cuda:0")
    cfg = KGEConfig(n_entities=2000, n_relations=12, dim=32, model="RESCAL", gamma=10.0, batch=256, neg_sample_size=64,
                    neg_chunk_size=64, lr=0.1, seed=3)
    m = KGEModel(cfg)
    bs, ns, cs, D = cfg.batch, cfg.neg_sample_size, cfg.neg_chunk_size, cfg.dim
    g = torch.Generator(device=dev).manual_seed(1)
    E = m.entity.weight[: cfg.n_entities].clone()
    M = m.relation.weight[: cfg.n_relations * D].clone().view(cfg.n_relations, D * D)
    SE = torch.zeros(cfg.n_entities, device=dev); SM = torch.zeros(cfg.n_relations, device=dev)
    dummy_r = torch.zeros(bs, D, device=dev)
    for step in range(2):
        hi = torch.randint(0, 150, (bs,), device=dev, generator=g)
        ti = torch.randint(0, cfg.n_entities, (bs,), device=dev, generator=g)
        ri = torch.randint(0, cfg.n_relations, (bs,), device=dev, generator=g)             # 12 relations: many duplicates
        ni = torch.randint(0, cfg.n_entities, (bs // cs * ns,), device=dev, generator=g)
        h = E[hi].clone().requires_grad_(True); t = E[ti].clone().requires_grad_(True)
        P = M[ri].clone().requires_grad_(True); n = E[ni].clone().requires_grad_(True)
        pos_ref = edge_score("RESCAL", h, dummy_r, t, cfg.gamma, P)
        neg_ref = chunk_neg_score("RESCAL", h, dummy_r, t, n, corrupt_head, cs, cfg.gamma, P)
        loss_ref = logsigmoid_loss(pos_ref, neg_ref)
        loss_ref.backward()
        pos, negs = m.score_batch(hi, ri, ti, ni, corrupt_head)
        assert torch.allclose(pos, pos_ref, atol=2e-3, rtol=1e-3)
        assert torch.allclose(negs, neg_ref, atol=3e-2, rtol=2e-2)
        loss = m.train_step(hi, ri, ti, ni, corrupt_head)
        assert abs(loss.item() - loss_ref.item()) < 5e-3 * max(1.0, abs(loss_ref.item()))
        ge = torch.cat([h.grad, t.grad, n.grad])
        assert ((m.ent_grad - ge).norm() / ge.norm()).item() < 3e-2
        assert ((m.rel_grad - P.grad).norm() / P.grad.norm()).item() < 3e-2
        rowwise_adagrad_update(E, SE, torch.cat([hi, ti, ni]), m.ent_grad.clone(), cfg.lr, cfg.eps)
        rowwise_adagrad_update(M, SM, ri, m.rel_grad.clone(), cfg.lr, cfg.eps)
        torch.cuda.synchronize()
        assert torch.allclose(m.entity.weight[: cfg.n_entities], E, atol=2e-3, rtol=2e-3)
        got = m.relation.weight[: cfg.n_relations * D].view(cfg.n_relations, D * D)
        assert torch.allclose(got, M, atol=2e-3, rtol=2e-3), (got - M).abs().max().item()
        st = m.relation.state[: cfg.n_relations * D].view(cfg.n_relations, D)
        assert torch.allclose(st, SM.view(-1, 1).expand_as(st), atol=1e-6, rtol=2e-3)       # one value per relation
    m.ctx.check_status()


def test_rescal_trains_with_graph_replay_and_keeps_the_reference_checkpoint_shape(tmp_path):
    """RESCAL through the graph-replayed step: the loss falls, and the relation file has the reference's
    [n_relations, D*D] shape and loads back into the row-blocked table."""
    from recstore_b200.models.kge import KGEConfig, KGEModel, KGSampler
    import numpy as np, os
    dev = torch.device("cuda:0")
    cfg = KGEConfig(n_entities=2000, n_relations=8, dim=32, model="RESCAL", gamma=10.0, batch=256, neg_sample_size=64,
                    neg_chunk_size=64, lr=0.1, seed=1, use_cuda_graph=True)
    m = KGEModel(cfg)
    smp = KGSampler(cfg, n_triples=4000, alpha=1.3, device=dev, seed=2)
    losses = []
    for step in range(200):
        h, r, t, neg = next(smp)
        losses.append(m.train_step(h, r, t, neg))
    m.ctx.check_status()
    first, last = torch.stack(losses[:10]).mean().item(), torch.stack(losses[-10:]).mean().item()
    assert last < 0.8 * first, (first, last)
    m.save(str(tmp_path))
    rel = np.load(os.path.join(tmp_path, "synthetic_RESCAL_relation.npy"))
    assert rel.shape == (8, 32 * 32)
    assert np.allclose(rel.reshape(8 * 32, 32), m.relation.weight[: 8 * 32].cpu().numpy())
    m2 = KGEModel(cfg)
    m2.load(str(tmp_path))
    assert torch.equal(m2.relation.weight[: 8 * 32], m.relation.weight[: 8 * 32])


@pytest.mark.parametrize("corrupt_head", [False, True])
def test_transr_on_the_hbm_plane_matches_the_per_pair_definition(corrupt_head, tmp_path):
    """TransR with its tables on the sharded HBM plane (entities, relation vectors, row-blocked projection matrices) and
    batched-GEMM scoring: scores, loss and one optimizer step against the per-pair definition under autograd, with ONE
    Adagrad state per projection matrix; the projection checkpoint has the reference's name and shape."""
    from recstore_b200.models.kge import KGEConfig, KGEModel
    from recstore_b200.baseline.kge_torch import chunk_neg_score, edge_score, logsigmoid_loss
    from recstore_b200.baseline.dlrm_torch import rowwise_adagrad_update
    import numpy as np, os
    dev = torch.device("cuda:0")
    cfg = KGEConfig(n_entities=1500, n_relations=10, dim=16, model="TransR", gamma=8.0, batch=128, neg_sample_size=32,
                    neg_chunk_size=32, lr=0.1, seed=3)
    m = KGEModel(cfg)
    bs, ns, cs, D = cfg.batch, cfg.neg_sample_size, cfg.neg_chunk_size, cfg.dim
    g = torch.Generator(device=dev).manual_seed(1)
    E = m.entity.weight[: cfg.n_entities].clone(); R = m.relation.weight[: cfg.n_relations].clone()
    P = m.proj.weight[: cfg.n_relations * D].clone().view(cfg.n_relations, D * D)
    SE = torch.zeros(cfg.n_entities, device=dev); SR = torch.zeros(cfg.n_relations, device=dev); SP = torch.zeros(cfg.n_relations, device=dev)
    for step in range(2):
        hi = torch.randint(0, 100, (bs,), device=dev, generator=g)
        ti = torch.randint(0, cfg.n_entities, (bs,), device=dev, generator=g)
        ri = torch.randint(0, cfg.n_relations, (bs,), device=dev, generator=g)
        ni = torch.randint(0, cfg.n_entities, (bs // cs * ns,), device=dev, generator=g)
        h = E[hi].clone().requires_grad_(True); t = E[ti].clone().requires_grad_(True); n = E[ni].clone().requires_grad_(True)
        r = R[ri].clone().requires_grad_(True); M = P[ri].clone().requires_grad_(True)
        pos_ref = edge_score("TransR", h, r, t, cfg.gamma, M)
        neg_ref = chunk_neg_score("TransR", h, r, t, n, corrupt_head, cs, cfg.gamma, M)
        loss_ref = logsigmoid_loss(pos_ref, neg_ref)
        loss_ref.backward()
        pos, negs = m.score_batch(hi, ri, ti, ni, corrupt_head)
        assert torch.allclose(pos, pos_ref, atol=1e-4, rtol=1e-4) and torch.allclose(negs, neg_ref, atol=1e-4, rtol=1e-4)
        loss = m.train_step(hi, ri, ti, ni, corrupt_head)
        assert abs(loss.item() - loss_ref.item()) < 1e-4 * max(1.0, abs(loss_ref.item()))
        ge = torch.cat([h.grad, t.grad, n.grad])
        assert ((m.ent_grad - ge).norm() / ge.norm()).item() < 1e-3
        assert ((m.proj_grad.view(bs, D * D) - M.grad).norm() / M.grad.norm()).item() < 1e-3
        rowwise_adagrad_update(E, SE, torch.cat([hi, ti, ni]), ge.detach(), cfg.lr, cfg.eps)
        rowwise_adagrad_update(R, SR, ri, r.grad.detach(), cfg.lr, cfg.eps)
        rowwise_adagrad_update(P, SP, ri, M.grad.detach(), cfg.lr, cfg.eps)
        torch.cuda.synchronize()
        assert torch.allclose(m.entity.weight[: cfg.n_entities], E, atol=2e-3, rtol=2e-3)
        assert torch.allclose(m.relation.weight[: cfg.n_relations], R, atol=2e-3, rtol=2e-3)
        assert torch.allclose(m.proj.weight[: cfg.n_relations * D].view(cfg.n_relations, D * D), P, atol=2e-3, rtol=2e-3)
        st = m.proj.state[: cfg.n_relations * D].view(cfg.n_relations, D)
        assert torch.allclose(st, SP.view(-1, 1).expand_as(st), atol=1e-6, rtol=2e-3)
    m.ctx.check_status()
    m.save(str(tmp_path))
    prj = np.load(os.path.join(tmp_path, "synthetic_TransRprojection.npy"))
    assert prj.shape == (10, D * D)
    m2 = KGEModel(cfg)
    m2.load(str(tmp_path))
    assert torch.equal(m2.proj.weight[: 10 * D], m.proj.weight[: 10 * D])


@pytest.mark.parametrize("model,floor", [("ComplEx", 0.4), ("RotatE", 0.5)])
def test_native_training_generalises_to_held_out_triples_of_a_planted_graph(model, floor):
    """The native step (fused scoring kernels + sharded HBM tables + row-wise Adagrad) learns structure, not just its
    training triples: relations are fixed shifts on a grid, held-out triples are ranked against every entity
    (filtered) by the fp32 PyTorch scorer on the trained tables.  Chance level: MRR ~0.02."""
    from recstore_b200.baseline.kge_torch import TorchKGE, known_triple_index
    from recstore_b200.models.kge import KGEConfig, KGEModel
    from recstore_b200.utils.kg_data import KGDataset
    dev = torch.device("cuda:0")
    ds = KGDataset.planted_grid(seed=0)
    cfg = KGEConfig(n_entities=ds.n_entities, n_relations=ds.n_relations, dim=64, model=model, gamma=6.0, batch=128,
                    neg_sample_size=32, neg_chunk_size=32, lr=0.1, seed=0)
    m = KGEModel(cfg)
    train = tuple(torch.from_numpy(x).to(dev) for x in ds.train)
    known = known_triple_index(ds.train, ds.test)
    test = tuple(torch.from_numpy(x) for x in ds.test)

    def held_out_mrr():
        scorer = TorchKGE(2, 2, cfg.dim, model, cfg.gamma)
        scorer.entity = torch.from_numpy(m._gather_table(m.entity)).float()
        scorer.relation = torch.from_numpy(m._gather_table(m.relation)).float()
        scorer.emb_init = (cfg.gamma + 2.0) / cfg.dim
        return scorer.evaluate_full(*test, known)
    before = held_out_mrr()["MRR"]
    g = torch.Generator(device=dev).manual_seed(1)
    for step in range(1500):
        b = torch.randint(0, train[0].numel(), (cfg.batch,), device=dev, generator=g)
        neg = torch.randint(0, ds.n_entities, (cfg.batch // cfg.neg_chunk_size * cfg.neg_sample_size,), device=dev, generator=g)
        m.train_step(train[0][b], train[1][b], train[2][b], neg)
    m.ctx.check_status()
    after = held_out_mrr()
    assert before < 0.06 and after["MRR"] > floor and after["HITS@10"] > 0.7, (before, after)
