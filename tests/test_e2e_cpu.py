"""End-to-end runs on CPU: executor, trainers, callbacks, evaluation invariants, interactive API, layout."""
import json
import os

import numpy as np
import pytest
import torch

from dice_embeddings_b200 import KGE, ContinuousExecute, Execute, Namespace
from dice_embeddings_b200.cli import get_default_arguments
from dice_embeddings_b200.evaluation import (evaluate_link_prediction_performance,
                                              evaluate_link_prediction_performance_with_reciprocals)
from dice_embeddings_b200.io.checkpoint import load_pickle


def _args(kg, out, **kw):
    base = dict(dataset_dir=kg, path_to_store_single_run=str(out), model="Keci", scoring_technique="KvsAll",
                embedding_dim=32, num_epochs=60, batch_size=256, lr=0.1, optim="Adam", trainer="torchCPUTrainer",
                random_seed=1)
    base.update(kw)
    return Namespace(**base)


@pytest.fixture(scope="module")
def trained(umls_like_dir, tmp_path_factory):
    out = tmp_path_factory.mktemp("run_keci")
    rep = Execute(_args(umls_like_dir, out, save_embeddings_as_csv=True)).start()
    return str(out), rep


def test_layout_and_metric_band(trained):
    path, rep = trained
    files = set(os.listdir(path))
    for f in ("configuration.json", "report.json", "model.pt", "entity_to_idx.csv", "relation_to_idx.csv", "train_set.npy",
              "valid_set.npy", "test_set.npy", "eval_report.json", "epoch_losses.csv", "er_vocab.p", "re_vocab.p",
              "ee_vocab.p", "memory_map_train_set.npy", "memory_map_details.json", "Keci_entity_embeddings.csv",
              "Keci_relation_embeddings.csv"):
        assert f in files, f
    assert rep["Train"]["MRR"] > 0.8 and rep["Test"]["MRR"] > 0.15 and rep["Train"]["H@10"] >= rep["Train"]["H@3"] >= rep["Train"]["H@1"]
    report = json.load(open(os.path.join(path, "report.json")))
    for k in ("num_train_triples", "num_entities", "num_relations", "EstimatedSizeMB", "NumParam", "Runtime"):
        assert k in report
    sd = torch.load(os.path.join(path, "model.pt"), map_location="cpu")
    assert set(sd) == {"entity_embeddings.weight", "relation_embeddings.weight", "q_coefficients.weight"}
    ev = json.load(open(os.path.join(path, "eval_report.json")))
    assert set(ev) == {"Train", "Val", "Test"}
    assert isinstance(load_pickle(os.path.join(path, "er_vocab.p")), dict)


def test_report_equals_standalone_evaluation(trained):
    path, rep = trained
    k = KGE(path=path)
    idx_to_e, idx_to_r = k.idx_to_entity, k.idx_to_relations
    test = np.load(os.path.join(path, "test_set.npy"))
    triples = [(idx_to_e[h], idx_to_r[r], idx_to_e[t]) for h, r, t in test.tolist()]
    er = load_pickle(os.path.join(path, "er_vocab.p"))
    out = evaluate_link_prediction_performance_with_reciprocals(k, triples, er)
    for m in ("MRR", "H@1", "H@3", "H@10"):
        assert abs(out[m] - rep["Test"][m]) < 1e-9


def test_kge_predict_api(trained):
    path, _ = trained
    k = KGE(path=path)
    ents, rels = list(k.entity_to_idx), [r for r in k.relation_to_idx if not r.endswith("_inverse")]
    h, r = ents[3], rels[0]
    scores = k.predict(h=[h], r=[r])
    assert scores.shape == (k.num_entities,)
    top = k.predict_topk(h=[h], r=[r], topk=5)
    assert len(top) == 1 and len(top[0]) == 5
    best = torch.sigmoid(scores).topk(5)
    assert [e for e, _ in top[0]] == [k.idx_to_entity[i] for i in best.indices.tolist()]
    assert all(abs(p - q) < 1e-6 for (_, p), q in zip(top[0], best.values.tolist()))
    # batch-size invariance and determinism
    a = k.predict_topk(h=ents[:7], r=[r], topk=3, batch_size=2)
    b = k.predict_topk(h=ents[:7], r=[r], topk=3, batch_size=64)
    for ra, rb in zip(a, b):
        assert [e for e, _ in ra] == [e for e, _ in rb]
        assert all(abs(x - y) < 1e-6 for (_, x), (_, y) in zip(ra, rb))
    # missing head (rewritten through the inverse relation) and missing relation
    t = ents[5]
    heads = k.predict_topk(r=[r], t=[t], topk=4)
    assert len(heads[0]) == 4
    relp = k.predict_topk(h=[h], t=[t], topk=2)
    assert relp[0][0][0] in k.relation_to_idx
    s = k.triple_score(h=[h], r=[r], t=[t])
    assert 0.0 <= float(s) <= 1.0
    assert torch.allclose(k.predict(h=[h], r=[r], t=[t]), k.triple_score(h=[h], r=[r], t=[t], logits=True))
    # a training triple must be found among the top predictions of its (h, r)
    tr = np.load(os.path.join(path, "train_set.npy"))[0]
    res = k.predict_topk(h=[k.idx_to_entity[int(tr[0])]], r=[k.idx_to_relations[int(tr[1])]], topk=10)[0]
    assert k.idx_to_entity[int(tr[2])] in [e for e, _ in res]


def test_multi_hop_queries(trained):
    path, _ = trained
    k = KGE(path=path)
    e = list(k.entity_to_idx)
    r = [x for x in k.relation_to_idx if not x.endswith("_inverse")]
    q = {"1p": (e[0], (r[0],)), "2p": (e[0], (r[0], r[1])), "3p": (e[0], (r[0], r[1], r[2])),
         "2i": ((e[0], (r[0],)), (e[1], (r[1],))), "3i": ((e[0], (r[0],)), (e[1], (r[1],)), (e[2], (r[2],))),
         "ip": (((e[0], (r[0],)), (e[1], (r[1],))), (r[2],)), "pi": ((e[0], (r[0], r[1])), (e[1], (r[2],))),
         "2in": ((e[0], (r[0],)), (e[1], (r[1], "n"))), "3in": ((e[0], (r[0],)), (e[1], (r[1],)), (e[2], (r[2], "n"))),
         "inp": (((e[0], (r[0],)), (e[1], (r[1], "n"))), (r[2],)), "pin": ((e[0], (r[0], r[1])), (e[1], (r[2], "n"))),
         "pni": ((e[0], (r[0], r[1], "n")), (e[1], (r[2],))), "2u": ((e[0], (r[0],)), (e[1], (r[1],)), ("u",)),
         "up": (((e[0], (r[0],)), (e[1], (r[1],)), ("u",)), (r[2],))}
    for name, query in q.items():
        s = k.answer_multi_hop_query(query_type=name, query=query, tnorm="min", k=5, only_scores=True)
        assert s.shape == (k.num_entities,), name
    ranked = k.answer_multi_hop_query(query_type="2p", query=q["2p"], tnorm="prod", k=5)
    assert len(ranked) == 5 and ranked[0][1] >= ranked[-1][1]


@pytest.mark.parametrize("model,st,kw", [
    ("ComplEx", "NegSample", dict(neg_ratio=8, num_epochs=150)), ("DistMult", "1vsAll", {}),
    ("QMult", "KvsSample", dict(neg_ratio=20)), ("TransE", "1vsSample", dict(neg_ratio=30, lr=0.02, num_epochs=100)),
    ("OMult", "AllvsAll", dict(num_epochs=30)), ("ConEx", "KvsAll", dict(num_of_output_channels=2)),
    ("DeCaL", "KvsAll", dict(p=1, q=1, r=1, embedding_dim=32)), ("CoKE", "KvsAll", dict(lr=0.01, num_epochs=30)),
])
def test_models_and_techniques_learn(umls_like_dir, tmp_path, model, st, kw):
    rep = Execute(_args(umls_like_dir, tmp_path / "r", model=model, scoring_technique=st, **kw)).start()
    assert rep["Train"]["MRR"] > {"TransE": 0.2, "CoKE": 0.03}.get(model, 0.35), rep["Train"]
    if st == "NegSample":
        k = KGE(path=str(tmp_path / "r"))
        test = np.load(tmp_path / "r" / "test_set.npy")
        tr = [(k.idx_to_entity[h], k.idx_to_relations[r], k.idx_to_entity[t]) for h, r, t in test.tolist()]
        out = evaluate_link_prediction_performance(k, tr, load_pickle(str(tmp_path / "r" / "er_vocab.p")),
                                                   load_pickle(str(tmp_path / "r" / "re_vocab.p")))
        assert abs(out["MRR"] - rep["Test"]["MRR"]) < 1e-9


def test_adopt_and_other_optimizers(umls_like_dir, tmp_path):
    for i, opt in enumerate(["Adopt", "AdamW", "SGD", "NAdam", "Adagrad", "ASGD"]):
        rep = Execute(_args(umls_like_dir, tmp_path / f"o{i}", optim=opt, num_epochs=20, model="DistMult",
                            lr=0.1 if opt != "SGD" else 1.0)).start()
        assert np.isfinite(rep["Train"]["MRR"])


def test_continual_learning_and_cli(umls_like_dir, tmp_path):
    out = tmp_path / "c"
    a = get_default_arguments(["--dataset_dir", umls_like_dir, "--path_to_store_single_run", str(out), "--model", "ComplEx",
                               "--scoring_technique", "KvsAll", "--trainer", "torchCPUTrainer", "--num_epochs", "5",
                               "--batch_size", "256", "--optim", "Adam", "--embedding_dim", "32"])
    r1 = Execute(a).start()
    b = get_default_arguments(["--continual_learning", str(out), "--num_epochs", "40"])
    r2 = ContinuousExecute(b).continual_start()
    assert r2["Train"]["MRR"] > r1["Train"]["MRR"]


def test_kfold_cv_and_reuse_dir(umls_like_dir, tmp_path):
    ex = Execute(_args(umls_like_dir, tmp_path / "cv", num_folds_for_cv=3, num_epochs=5, model="DistMult",
                       eval_model="train"))
    rep = ex.start()
    assert set(ex.evaluator.report) == {"MRR", "H@1", "H@3", "H@10"} and len(ex.evaluator.report["MRR"]) == 3
    p = tmp_path / "keep"
    Execute(_args(umls_like_dir, p, num_epochs=1)).start()
    (p / "marker.txt").write_text("x")
    Execute(_args(umls_like_dir, p, num_epochs=1, reuse_existing_run_dir=True)).start()
    assert (p / "marker.txt").exists()
    Execute(_args(umls_like_dir, p, num_epochs=1)).start()
    assert not (p / "marker.txt").exists()
