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
