"""Device sampling kernels and the fused sampled-candidate training step against PyTorch autograd."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("CUDA device required", allow_module_level=True)

from dice_embeddings_b200.data.datasets import OnevsSample, TriplePredictionDataset
from dice_embeddings_b200.data.synthetic import zipf_kg
from dice_embeddings_b200.models import initialize_model
from dice_embeddings_b200.ops import kernels as K
from dice_embeddings_b200.ops import sampling
from dice_embeddings_b200.ops.sampled_step import FusedSampledEngine

DEV = torch.device("cuda:0")


def test_uniform_int_range_reproducibility_and_spread():
    a = sampling.uniform_int(1000, (200001,), DEV, seed=7)
    b = sampling.uniform_int(1000, (200001,), DEV, seed=7)
    c = sampling.uniform_int(1000, (200001,), DEV, seed=8)
    assert a.min() >= 0 and a.max() < 1000 and torch.equal(a, b) and not torch.equal(a, c)
    counts = torch.bincount(a, minlength=1000).float()
    assert counts.min() > 120 and counts.max() < 290          # expectation 200, sd 14
    big = sampling.uniform_int(10 ** 12, (1000,), DEV, seed=1)
    assert big.max() > 10 ** 10 and big.max() < 10 ** 12


@pytest.mark.parametrize("per_negative", [False, True])
def test_neg_sample_layout_and_semantics(per_negative):
    B, k, NE = 500, 4, 3000
    pos = torch.stack((torch.randint(0, NE, (B,)), torch.randint(0, 9, (B,)), torch.randint(0, NE, (B,))), 1).to(DEV)
    x = torch.zeros(B * (1 + k), 3, dtype=torch.int64, device=DEV)
    y = torch.zeros(B * (1 + k), device=DEV)
    h, r, t = (torch.zeros(B * (1 + k), dtype=torch.int64, device=DEV) for _ in range(3))
    step = torch.tensor([3], device=DEV)
    K.neg_sample(pos, k, NE, 11, 0, y, x=x, hrt=(h, r, t), label_pos=0.9, label_neg=0.1,
                 per_negative_coin=per_negative, step=step)
    assert torch.equal(x[:B], pos) and torch.equal(torch.stack((h, r, t), 1), x)
    assert torch.allclose(y[:B], torch.full((B,), 0.9, device=DEV)) and torch.allclose(y[B:], torch.full((B * k,), 0.1, device=DEV))
    neg = x[B:].reshape(k, B, 3)
    assert (neg[:, :, 1] == pos[:, 1]).all()
    head_changed = neg[:, :, 0] != pos[:, 0]
    tail_changed = neg[:, :, 2] != pos[:, 2]
    assert not (head_changed & tail_changed).any()
    if per_negative:
        assert 0.3 < head_changed.float().mean() < 0.7
    else:
        assert head_changed.float().mean() > 0.95 or tail_changed.float().mean() > 0.95
    assert x.min() >= 0 and x[:, [0, 2]].max() < NE
    # same (seed, offset + step) -> same draw; another step -> another draw
    x2 = torch.zeros_like(x)
    K.neg_sample(pos, k, NE, 11, 3, y, x=x2, per_negative_coin=per_negative)
    assert torch.equal(x, x2)
    K.neg_sample(pos, k, NE, 11, 4, y, x=x2, per_negative_coin=per_negative)
    assert not torch.equal(x, x2)


def _pair(name, D, NE=600, NR=12, scoring="NegSample"):
    torch.manual_seed(1)
    args = dict(model=name, embedding_dim=D, num_entities=NE, num_relations=NR, optim="SGD", learning_rate=1.0,
                scoring_technique=scoring, p=0, q=1)
    m1, _ = initialize_model(dict(args))
    m2, _ = initialize_model(dict(args))
    m2.load_state_dict(m1.state_dict())
    for m in (m1, m2):
        m.to(DEV)
        if name == "Keci":
            with torch.no_grad():
                m.q_coefficients.weight.fill_(0.5)
    return m1, m2


def _compare_updates(ref, fused, lr):
    for (n, p_ref), (_, p) in zip(ref.named_parameters(), fused.named_parameters()):
        if p_ref.grad is None:
            continue
        start = p_ref.detach() + lr * p_ref.grad
        d_ref, d = p_ref.detach() - start, p.detach() - start
        scale = d_ref.abs().max().clamp_min(1e-12)
        assert (d - d_ref).abs().max() / scale < 1e-3, n


@pytest.mark.parametrize("name,D", [("DistMult", 64), ("ComplEx", 128), ("QMult", 64), ("OMult", 256), ("Keci", 96),
                                    ("TransE", 100)])
def test_negsample_step_matches_autograd(name, D):
    lr = 5.0
    ref, fused = _pair(name, D)
    tr = zipf_kg(600, 12, 5000, seed=2)
    ds = TriplePredictionDataset(tr, 600, 12, neg_sample_ratio=3, label_smoothing_rate=0.05).to(DEV)
    x, y = ds.make_batch(torch.arange(400, device=DEV))
    opt = torch.optim.SGD(ref.parameters(), lr=lr)
    loss_ref = ref.training_step((x, y))
    loss_ref.backward()
    opt.step()
    eng = FusedSampledEngine(fused, "NegSample", lr=lr, device=DEV, neg_ratio=3, label_smoothing=0.05, use_graph=False)
    loss = eng.step((x, y))
    eng.sync_to_model()
    assert abs(float(loss) - float(loss_ref)) < 1e-4 * abs(float(loss_ref))
    _compare_updates(ref, fused, lr)


def test_one_vs_sample_step_matches_autograd():
    lr = 5.0
    ref, fused = _pair("ComplEx", 64, scoring="1vsSample")
    tr = zipf_kg(600, 12, 5000, seed=3)
    ds = OnevsSample(tr, 600, 12, neg_sample_ratio=20, label_smoothing_rate=0.1).to(DEV)
    batch = ds.make_batch(torch.arange(256, device=DEV))
    opt = torch.optim.SGD(ref.parameters(), lr=lr)
    loss_ref = ref.training_step(batch)
    loss_ref.backward()
    opt.step()
    eng = FusedSampledEngine(fused, "1vsSample", lr=lr, device=DEV, use_graph=False)
    loss = eng.step(batch)
    eng.sync_to_model()
    assert abs(float(loss) - float(loss_ref)) < 1e-4 * abs(float(loss_ref))
    _compare_updates(ref, fused, lr)


def test_negsample_training_with_device_sampling_learns(umls_like_dir, tmp_path):
    """End to end through the trainer: graph replay, corruptions drawn inside the step, the model learns."""
    from dice_embeddings_b200 import Execute, Namespace
    rep = Execute(Namespace(dataset_dir=umls_like_dir, path_to_store_single_run=str(tmp_path / "run"),
                            model="ComplEx", scoring_technique="NegSample", neg_ratio=8, embedding_dim=32,
                            num_epochs=150, batch_size=1024, lr=0.1, gpus=0, kernel_backend="cuda",
                            trainer="torchCPUTrainer", eval_model="train_val_test")).start()
    assert rep["Train"]["MRR"] > 0.35, rep["Train"]


@pytest.mark.parametrize("kind,name", [(0, "Adam"), (2, "SGD")])
def test_sparse_rows_optimizer_updates_only_flagged_rows(kind, name):
    torch.manual_seed(0)
    rows, D = 1000, 128
    p = torch.randn(rows, D, device=DEV)
    g = torch.randn(rows, D, device=DEV)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    touched = (torch.rand(rows, device=DEV) < 0.3).to(torch.uint8)
    step = torch.zeros(1, dtype=torch.int64, device=DEV)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.Adam([ref], lr=0.01) if kind == 0 else torch.optim.SGD([ref], lr=0.01)
    ref.grad = g * touched[:, None].float()
    opt.step()
    p0, sel = p.clone(), touched.bool().clone()
    K.sparse_rows_optimizer(kind, p, g, m, v, None, touched, step, 0.01, 0.9, 0.999, 1e-8, 0.0)
    torch.cuda.synchronize()
    assert torch.equal(p[~sel], p0[~sel])                       # untouched rows are not even read
    assert torch.allclose(p[sel], ref.detach()[sel], atol=1e-5, rtol=1e-4)
    assert int(touched.sum()) == 0 and float(g[sel].abs().sum()) == 0.0 and float(g[~sel].abs().sum()) > 0


def test_uniform_int_into_column_block():
    cand = torch.full((300, 9), -1, dtype=torch.int64, device=DEV)
    K.uniform_int(cand[:, 1:], 50, seed=3)
    assert (cand[:, 0] == -1).all() and cand[:, 1:].min() >= 0 and cand[:, 1:].max() < 50
    flat = torch.empty(300 * 8, dtype=torch.int64, device=DEV)
    K.uniform_int(flat, 50, seed=3)
    assert torch.equal(flat.view(300, 8), cand[:, 1:])
