"""Query generator, experiment summary and the vector-search service."""
import os

import numpy as np
import pytest

from dice_embeddings_b200 import Execute, KGE, Namespace
from dice_embeddings_b200.data.query_generator import QUERY_STRUCTS, QueryGenerator


@pytest.fixture(scope="module")
def run_dir(umls_like_dir, tmp_path_factory):
    out = tmp_path_factory.mktemp("exp")
    for i, m in enumerate(["DistMult", "ComplEx"]):
        Execute(Namespace(dataset_dir=umls_like_dir, path_to_store_single_run=str(out / f"r{i}"), model=m,
                          embedding_dim=16, num_epochs=15, batch_size=256, save_embeddings_as_csv=True)).start()
    return str(out)


def test_query_generator_and_answering(umls_like_dir, run_dir):
    k = KGE(path=os.path.join(run_dir, "r1"))
    e2i = {e: i for e, i in k.entity_to_idx.items()}
    r2i = {r: i for r, i in k.relation_to_idx.items() if not r.endswith("_inverse")}
    r2i = {r: i for i, r in enumerate(sorted(r2i))}
    qg = QueryGenerator(umls_like_dir + "/train.txt", umls_like_dir + "/valid.txt", umls_like_dir + "/test.txt",
                        ent2id=e2i, rel2id=r2i, seed=3)
    for name in QUERY_STRUCTS:
        qs, tp, fp, fn = qg.get_queries(name, 2)
        assert len(qs) >= 1, name
        for q in qs:
            assert len(fn[q]) >= 1                      # a test query needs held-out edges
            scores = k.answer_multi_hop_query(query_type=name, query=q, tnorm="min", k=5, only_scores=True)
            assert scores.shape[0] == k.num_entities
    small, full = qg._get_graphs()
    qs, tp, fp, fn = qg.ground_queries(QUERY_STRUCTS["2p"], 3)
    for q in qs:
        assert qg.achieve_answer(q, full) == tp[q] | fn[q]


def test_analyse_experiments(run_dir):
    from dice_embeddings_b200.scripts.analyse_experiments import analyse
    df = analyse(run_dir, ["model", "trainMRR", "testMRR"])
    assert len(df) == 2 and os.path.isfile(os.path.join(run_dir, "summary.csv"))
    assert df["testMRR"].is_monotonic_decreasing


def test_vector_search_service(run_dir):
    from fastapi.testclient import TestClient
    from dice_embeddings_b200.scripts.index_serve import create_app, load_entity_embeddings
    path = os.path.join(run_dir, "r0")
    names, vecs = load_entity_embeddings(path)
    try:
        client = TestClient(create_app(path))
    except Exception as e:  # httpx missing
        pytest.skip(str(e))
    r = client.get("/api/search", params={"q": names[0], "k": 3}).json()
    assert len(r["results"]) == 3 and names[0] not in [h["hit"] for h in r["results"]]
    v = client.get("/api/get", params={"q": names[1]}).json()["vector"]
    assert np.allclose(v, vecs[1], atol=1e-5)
    b = client.post("/api/search_batch", json={"queries": names[:2], "k": 2}).json()
    assert set(b["results"]) == set(names[:2])


def test_multi_hop_evaluate_matches_loop_definition():
    """The vectorised filtered ranking of query answers equals the definition: rank of each hard answer among all
    entities after removing every other answer."""
    from dice_embeddings_b200 import evaluate
    rng = np.random.default_rng(0)
    ents = {f"e{i}": i for i in range(50)}
    scores, easy, hard = {}, {}, {}
    for q in range(6):
        s = rng.normal(size=50)
        ans = rng.choice(50, size=8, replace=False)
        scores[q], easy[q], hard[q] = s, {f"e{i}" for i in ans[:5]}, {f"e{i}" for i in ans[5:]}
    mrr, h1, h3, h10 = evaluate(ents, scores, easy, hard)
    exp = []
    for q in range(6):
        s = scores[q]
        rr = []
        for a in hard[q]:
            i = ents[a]
            others = {ents[e] for e in (easy[q] | hard[q])} - {i}
            rank = 1 + sum(1 for j in range(50) if j not in others and j != i and s[j] > s[i])
            rr.append(1.0 / rank)
        exp.append(np.mean(rr))
    assert abs(mrr - np.mean(exp)) < 1e-12 and 0 <= h1 <= h3 <= h10 <= 1


def test_helper_functions(tmp_path):
    import dice_embeddings_b200 as d
    from dice_embeddings_b200.trainer.callbacks import compute_convergence, estimate_q
    a = np.arange(12).reshape(4, 3)
    d.save_numpy_ndarray(data=a, file_path=str(tmp_path / "a.npy"))
    assert (d.load_numpy(str(tmp_path / "a.npy")) == a).all()
    assert d.numpy_data_type_changer(a, 100).dtype == np.int8 and d.numpy_data_type_changer(a, 70000).dtype == np.int32
    w = d.exponential_function(np.arange(5), 0.5)
    assert abs(float(w.sum()) - 1) < 1e-6 and w[0] < w[-1]
    assert 0 < estimate_q(np.array([1, .5, .25, .125, .0625]) * 0.1 + 1e-3) < 2
    assert compute_convergence(np.array([.9, .5, .3, .2, .15, .12]), 5) > 0
    import pandas as pd
    df = d.create_recipriocal_triples(pd.DataFrame({"subject": ["a"], "relation": ["r"], "object": ["b"]}))
    assert df.iloc[1].tolist() == ["b", "r_inverse", "a"]


def test_pseudo_labelling_callback_grows_training_set():
    import torch
    from types import SimpleNamespace
    from dice_embeddings_b200.trainer.callbacks import PseudoLabellingCallback

    class M(torch.nn.Module):
        device = torch.device("cpu")

        def forward(self, x):
            return torch.where(x[:, 0] % 2 == 0, torch.tensor(5.0), torch.tensor(-5.0))

    kg = SimpleNamespace(unlabelled_set=np.stack([np.arange(100), np.zeros(100, int), np.arange(100)], 1),
                         num_entities=100, num_relations=1)
    dm = SimpleNamespace(train_set_idx=np.zeros((3, 3), dtype=np.int64))
    cb = PseudoLabellingCallback(dm, kg, batch_size=40)
    cb.on_train_epoch_end(SimpleNamespace(current_epoch=0), M())
    assert len(dm.train_set_idx) > 3 and (dm.train_set_idx[3:, 0] % 2 == 0).all()
