"""The fused training step against a PyTorch fp32 implementation of the same step."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("CUDA device required", allow_module_level=True)

from dice_embeddings_b200.data.datasets import KvsAll, OnevsAllDataset
from dice_embeddings_b200.data.synthetic import zipf_kg
from dice_embeddings_b200.models import initialize_model
from dice_embeddings_b200.ops.fused_step import FusedKvsAllEngine, build_fused_engine

DEV = torch.device("cuda:0")


def _make(name, D, optim, lr, NE=700, NR=15, smoothing=0.1, seed=0, scoring="KvsAll"):
    tr = zipf_kg(NE, NR, 4000, seed=seed)
    ds = (KvsAll(tr, NE, NR, label_smoothing_rate=smoothing) if scoring == "KvsAll" else OnevsAllDataset(tr, NE)).to(DEV)
    torch.manual_seed(seed)
    args = dict(model=name, embedding_dim=D, num_entities=NE, num_relations=NR, optim=optim, learning_rate=lr,
                scoring_technique=scoring, p=0, q=1)
    m1, _ = initialize_model(dict(args))
    m2, _ = initialize_model(dict(args))
    m2.load_state_dict(m1.state_dict())
    for m in (m1, m2):
        m.to(DEV)
        with torch.no_grad():
            m.entity_embeddings.weight.mul_(0.3)
            m.relation_embeddings.weight.mul_(0.3)
            if name == "Keci":
                m.q_coefficients.weight.fill_(0.5)
    return ds, m1, m2


@pytest.mark.parametrize("name,label_mode", [("DistMult", "mask"), ("ComplEx", "mask"), ("ComplEx", "sparse"),
                                             ("QMult", "mask"), ("OMult", "sparse"), ("Keci", "mask")])
@pytest.mark.parametrize("D", [64, 256])
def test_one_sgd_step_matches_autograd(name, label_mode, D):
    """With SGD the parameter change is the gradient itself, so this checks every gradient path."""
    lr = 50.0  # gradients of a mean over B x |E| logits are tiny
    ds, ref, fused = _make(name, D, "SGD", lr)
    B = 384
    idx = torch.randperm(len(ds), device=DEV)[:B]
    x, y = ds.make_batch(idx)
    opt = ref.configure_optimizers()
    loss_ref = ref.training_step((x, y))
    loss_ref.backward()
    opt.step()
    eng = FusedKvsAllEngine(fused, ds, batch_size=B, lr=lr, device=DEV, use_graph=False, label_mode=label_mode)
    loss = eng.step((x, idx))
    eng.sync_to_model()
    assert abs(float(loss) - float(loss_ref.detach())) < 1e-2 * abs(float(loss_ref.detach()))
    for (n, p_ref), (_, p) in zip(ref.named_parameters(), fused.named_parameters()):
        upd_ref = p_ref.detach() - 0  # after step
        # compare parameter *changes*: start values are identical copies
        start = p_ref.detach() + lr * p_ref.grad
        d_ref, d = upd_ref - start, p.detach() - start
        scale = d_ref.abs().max().clamp_min(1e-12)
        assert (d - d_ref).abs().max() / scale < 5e-2, n


@pytest.mark.parametrize("name,extra", [("ConEx", {}), ("AConEx", {}), ("ConvQ", {}), ("AConvO", {}), ("DualE", {}),
                                        ("ComplEx", {"normalization": "LayerNorm"}),
                                        ("QMult", {"normalization": "BatchNorm1d"}),
                                        ("Keci", {"p": 1, "q": 2}), ("DeCaL", {"p": 3, "q": 3, "r": 1}),
                                        ("TransE", {}), ("CoKE", {})])
@pytest.mark.parametrize("D", [64, 256])
def test_external_query_engine_matches_autograd(name, extra, D):
    """Models whose query vector comes out of PyTorch modules (convolutional gates, normalisers, dual quaternions),
    models with a per-query scalar next to the dot product (general Clifford algebras) and the distance model: one SGD step through the tensor-core scoring function against the same step in plain autograd on dense labels."""
    from dice_embeddings_b200.ops.hybrid_step import ExternalQueryEngine, build_hybrid_engine, hybrid_supported
    lr = 50.0
    NE, NR = 700, 15
    tr = zipf_kg(NE, NR, 4000, seed=0)
    ds = KvsAll(tr, NE, NR, label_smoothing_rate=0.1).to(DEV)
    torch.manual_seed(0)
    args = dict(model=name, embedding_dim=D, num_entities=NE, num_relations=NR, optim="SGD", learning_rate=lr,
                scoring_technique="KvsAll", num_of_output_channels=2, kernel_size=3, **extra)
    ref, _ = initialize_model(dict(args))
    hyb, _ = initialize_model(dict(args))
    hyb.load_state_dict(ref.state_dict())
    for m in (ref, hyb):
        m.to(DEV)
        with torch.no_grad():
            m.entity_embeddings.weight.mul_(0.3)
            m.relation_embeddings.weight.mul_(0.3)
            for n, p in m.named_parameters():
                if "coefficients" in n:
                    p.fill_(0.7)           # the interaction terms (and with them the per-query bias) are switched on
        m.train()
        for mod in m.modules():            # the transformer's dropout would draw different masks in the two runs
            if isinstance(mod, torch.nn.Dropout):
                mod.p = 0.0
            if isinstance(getattr(mod, "dropout", None), float):
                mod.dropout = 0.0
    assert hybrid_supported(hyb)
    B = 384
    idx = torch.randperm(len(ds), device=DEV)[:B]
    x, y = ds.make_batch(idx)
    start = {n: p.detach().clone() for n, p in ref.named_parameters()}
    opt = ref.configure_optimizers()
    loss_ref = ref.training_step((x, y))
    loss_ref.backward()
    opt.step()
    eng = build_hybrid_engine(hyb, ds, type("A", (), dict(scoring_technique="KvsAll", batch_size=B, lr=lr))(), DEV)
    assert isinstance(eng, ExternalQueryEngine)
    loss = eng.step((x, idx))
    eng.sync_to_model()
    assert abs(float(loss) - float(loss_ref.detach())) < 1e-2 * abs(float(loss_ref.detach()))
    moved = 0
    for (n, p_ref), (_, p) in zip(ref.named_parameters(), hyb.named_parameters()):
        d_ref, d = p_ref.detach() - start[n], p.detach() - start[n]
        scale = d_ref.abs().max()
        if n == "conv2d.bias" or scale < 1e-5 * start[n].abs().max().clamp_min(1e-3):
            continue   # the batch norm behind the convolution removes its bias: that gradient is rounding noise
        moved += 1
        assert (d - d_ref).abs().max() < 6e-2 * scale + 1e-6, n
    assert moved >= 2


@pytest.mark.parametrize("optim", ["Adam", "Adopt"])
def test_loss_trajectory_with_graph_replay(optim):
    ds, ref, fused = _make("ComplEx", 128, optim, 0.02)
    B = 256
    opt = ref.configure_optimizers()
    eng = FusedKvsAllEngine(fused, ds, batch_size=B, lr=0.02, device=DEV, use_graph=True)
    g = torch.Generator(device="cpu").manual_seed(0)
    ref_losses, losses = [], []
    for _ in range(6):
        idx = torch.randperm(len(ds), generator=g)[:B].to(DEV)
        x, y = ds.dense_batch(idx)
        opt.zero_grad()
        l = ref.training_step((x, y))
        l.backward()
        opt.step()
        ref_losses.append(float(l.detach()))
        losses.append(float(eng.step((x, idx))))
    eng.sync_to_model()
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 3e-2 * abs(b), (losses, ref_losses)
    assert losses[-1] < losses[0]


def test_one_vs_all_and_host_step():
    ds, ref, fused = _make("DistMult", 64, "Adam", 0.05, scoring="1vsAll")
    B = 200
    idx = torch.arange(B, device=DEV)
    x, y = ds.make_batch(idx)
    loss_ref = float(ref.training_step((x, y)).detach())
    eng = FusedKvsAllEngine(fused, ds, batch_size=B, lr=0.05, device=DEV)
    loss = eng.step_from_host(x.cpu().pin_memory(), idx.cpu().pin_memory())
    assert abs(loss - loss_ref) < 1e-2 * abs(loss_ref)


def test_trainer_uses_fused_engine(tmp_path):
    from dice_embeddings_b200 import Execute, KGE, Namespace
    from dice_embeddings_b200.data.synthetic import make_planted_kg
    kg = make_planted_kg(str(tmp_path / "kg"), num_entities=300, num_relations=10, seed=1)
    a = Namespace(dataset_dir=kg, model="ComplEx", scoring_technique="KvsAll", embedding_dim=64, num_epochs=100,
                  batch_size=256, lr=0.1, optim="Adam", path_to_store_single_run=str(tmp_path / "run"), gpus=0,
                  kernel_backend="cuda", trainer="torchCPUTrainer")
    rep = Execute(a).start()
    assert rep["Train"]["MRR"] > 0.9
    k = KGE(path=str(tmp_path / "run"))
    assert len(k.predict_topk(h=[next(iter(k.entity_to_idx))], r=[next(iter(k.relation_to_idx))], topk=3)[0]) == 3


@pytest.mark.parametrize("model,extra", [("TransE", {}), ("Keci", {"p": 1, "q": 2}), ("ConEx", {"num_of_output_channels": 2})])
def test_trainer_uses_external_query_engine(tmp_path, model, extra):
    """The distance model, a Clifford model with per-query scalar terms and a convolutional model train through
    ``Execute`` on the tensor-core scoring function and learn the planted graph."""
    from dice_embeddings_b200 import Execute, Namespace
    from dice_embeddings_b200.data.synthetic import make_planted_kg
    from dice_embeddings_b200.ops.hybrid_step import ExternalQueryEngine
    kg = make_planted_kg(str(tmp_path / "kg"), num_entities=300, num_relations=10, seed=1)
    a = Namespace(dataset_dir=kg, model=model, scoring_technique="KvsAll", embedding_dim=64, num_epochs=150,
                  batch_size=256, lr=0.05, optim="Adam", path_to_store_single_run=str(tmp_path / "run"), gpus=0,
                  kernel_backend="cuda", trainer="torchCPUTrainer", **extra)
    ex = Execute(a)
    rep = ex.start()
    assert isinstance(ex.trainer.trainer.engine, ExternalQueryEngine)
    assert rep["Train"]["MRR"] > 0.5, rep["Train"]


def test_pipelined_host_steps_return_the_same_losses():
    ds, m1, m2 = _make("ComplEx", 64, "Adam", 0.05)
    B = 256
    e1 = FusedKvsAllEngine(m1, ds, batch_size=B, lr=0.05, device=DEV)
    e2 = FusedKvsAllEngine(m2, ds, batch_size=B, lr=0.05, device=DEV)
    g = torch.Generator().manual_seed(3)
    pairs = ds.train_data.cpu()
    a, b = [], []
    for _ in range(6):
        idx = torch.randperm(len(ds), generator=g)[:B]
        x, dp = pairs[idx].contiguous().pin_memory(), idx.contiguous().pin_memory()
        a.append(e1.step_from_host(x, dp))
        b.append(e2.step_from_host_pipelined(x, dp))
    b = b[1:] + [e2.last_loss()]
    assert all(abs(u - v) < 1e-6 * max(1.0, abs(u)) for u, v in zip(a, b)), (a, b)
