"""Byte-pair-encoded / byte-level paths, literal regression, the remaining models of the zoo, pickling, ensembles."""
import os
import pickle

import numpy as np
import pandas as pd
import pytest
import torch

from dice_embeddings_b200 import Execute, KGE, Namespace


def _args(kg, out, **kw):
    base = dict(dataset_dir=kg, path_to_store_single_run=str(out), model="Keci", scoring_technique="KvsAll",
                embedding_dim=32, num_epochs=40, batch_size=256, lr=0.1, optim="Adam", trainer="torchCPUTrainer",
                random_seed=1)
    base.update(kw)
    return Namespace(**base)


@pytest.fixture(scope="module")
def worded_kg(umls_like_dir, tmp_path_factory):
    """The planted KG with entity names replaced by random 8-letter words: a sub-word model composes an entity from
    its characters, so names need enough distinct characters to tell 120 entities apart."""
    rng = np.random.default_rng(5)
    out = tmp_path_factory.mktemp("worded")
    names = {}
    for split in ("train", "valid", "test"):
        df = pd.read_csv(os.path.join(umls_like_dir, f"{split}.txt"), sep=r"\s+", header=None)
        for col in (0, 2):
            for e in df[col].unique():
                if e not in names:
                    names[e] = "".join(rng.choice(list("abcdefghijklmnopqrstuvwxyz"), 8))
            df[col] = df[col].map(names)
        df.to_csv(os.path.join(out, f"{split}.txt"), sep="\t", header=False, index=False)
    return str(out)


@pytest.mark.parametrize("st", ["KvsAll", "NegSample"])
def test_byte_pair_encoded_training_and_inductive_prediction(worded_kg, tmp_path, st):
    kw = dict(neg_ratio=8, num_epochs=150) if st == "NegSample" else dict(num_epochs=150)
    rep = Execute(_args(worded_kg, tmp_path / "r", byte_pair_encoding=True, scoring_technique=st, p=0, q=1, **kw)).start()
    assert rep["Train"]["MRR"] > 0.3, rep["Train"]
    k = KGE(path=str(tmp_path / "r"))
    df = pd.read_csv(os.path.join(worded_kg, "train.txt"), sep=r"\s+", header=None)
    seen = k.predict(h=df[0].iloc[0], r=df[1].iloc[0], t=df[2].iloc[0], logits=True)
    unseen = k.predict(h="Demir", r="loves", t="Embeddings", logits=True)   # strings never seen in training
    assert torch.isfinite(seen).all() and torch.isfinite(unseen).all()
    if st == "NegSample":    # the triple path is the trained path only there (KvsAll normalises heads and relations)
        assert float(seen) > float(unseen)


def test_byte_level_language_model_path(umls_like_dir, tmp_path):
    rep = Execute(_args(umls_like_dir, tmp_path / "r", model="BytE", byte_pair_encoding=True, num_epochs=3,
                        embedding_dim=16, batch_size=128, lr=0.01)).start()
    assert np.isfinite(rep["Train"]["Perplexity"]) and 0 <= rep["Train"]["NextTokenAcc"] <= 1
    assert rep["Train"]["Perplexity"] < 200          # far below the uniform 256


@pytest.mark.parametrize("model,kw", [
    ("Shallom", {}), ("Pyke", dict(scoring_technique="NegSample", neg_ratio=2)), ("DualE", dict(embedding_dim=32)),
    ("ConvQ", dict(num_of_output_channels=2)), ("AConvQ", dict(num_of_output_channels=2)),
    ("ConvO", dict(num_of_output_channels=2)), ("AConvO", dict(num_of_output_channels=2)),
    ("AConEx", dict(num_of_output_channels=2)), ("CKeci", dict(p=0, q=1)), ("LFMult", dict(embedding_dim=8, scoring_technique="NegSample", neg_ratio=2)),
    ("OMult", dict(scoring_technique="NegSample", neg_ratio=2)),
])
def test_rest_of_model_zoo_trains_saves_and_loads(umls_like_dir, tmp_path, model, kw):
    rep = Execute(_args(umls_like_dir, tmp_path / "r", model=model, num_epochs=8, **kw)).start()
    assert np.isfinite(rep["Train"]["MRR"]) and rep["Train"]["MRR"] > 0
    k = KGE(path=str(tmp_path / "r"))
    assert k.model.name == model
    x = torch.as_tensor(np.load(tmp_path / "r" / "train_set.npy")[:5]).long()
    assert torch.isfinite(k.model(x)).all()


def test_trained_models_pickle(umls_like_dir, tmp_path):
    for model in ("DistMult", "TransE", "QMult"):
        ex = Execute(_args(umls_like_dir, tmp_path / model, model=model, scoring_technique="NegSample", neg_ratio=1,
                           num_epochs=2, embedding_dim=16))
        ex.start()
        blob = pickle.dumps(ex.trained_model)
        m = pickle.loads(blob)
        assert m.name == model


def test_literal_regression_round_trip(umls_like_dir, tmp_path):
    Execute(_args(umls_like_dir, tmp_path / "r", num_epochs=20)).start()
    k = KGE(path=str(tmp_path / "r"))
    ents = list(k.entity_to_idx)[:40]
    rng = np.random.default_rng(0)
    rows = [(e, "age", float(20 + 3 * (i % 10) + rng.normal())) for i, e in enumerate(ents)] + \
           [(e, "height", float(150 + (i % 7) * 5)) for i, e in enumerate(ents)]
    lit_dir = tmp_path / "lit"
    lit_dir.mkdir()
    pd.DataFrame(rows[:60]).to_csv(lit_dir / "train.txt", header=False, sep="\t", index=False)
    pd.DataFrame(rows[60:]).to_csv(lit_dir / "test.txt", header=False, sep="\t", index=False)
    k.train_literals(train_file_path=str(lit_dir / "train.txt"), num_epochs=150, lit_lr=0.05, batch_size=32)
    assert os.path.isfile(tmp_path / "r" / "literal_model.pt")
    preds = k.predict_literals(entity=[r[0] for r in rows[:5]], attribute=[r[1] for r in rows[:5]])
    assert preds.shape == (5,) and np.isfinite(preds).all()
    from dice_embeddings_b200.evaluation.literal_prediction import evaluate_literal_prediction
    err = evaluate_literal_prediction(k, eval_file_path=str(lit_dir / "test.txt"), return_attr_error_metrics=True)
    assert {"MAE", "RMSE"} <= set(err.columns) and np.isfinite(err["MAE"]).all()
    k2 = KGE(path=str(tmp_path / "r"))           # the literal model is found again in the run directory
    if k2.literal_model is not None:
        p2 = k2.predict_literals(entity=[rows[0][0]], attribute=[rows[0][1]])
        assert abs(float(p2[0]) - float(preds[0])) < 1e-4


def test_ensemble_of_runs_is_evaluated(umls_like_dir, tmp_path):
    from dice_embeddings_b200.evaluation.ensemble import evaluate_ensemble_link_prediction_performance
    from dice_embeddings_b200.io.checkpoint import load_pickle
    models = []
    for i, m in enumerate(["DistMult", "ComplEx"]):
        Execute(_args(umls_like_dir, tmp_path / f"r{i}", model=m, num_epochs=25)).start()
        models.append(KGE(path=str(tmp_path / f"r{i}")).model)
    triples = np.load(tmp_path / "r0" / "test_set.npy")[:100]
    er = load_pickle(str(tmp_path / "r0" / "er_vocab.p"))
    out = evaluate_ensemble_link_prediction_performance(models, triples=triples, er_vocab=er, weights=[0.5, 0.5])
    plain = evaluate_ensemble_link_prediction_performance(models, triples=triples, er_vocab=er,
                                                         weighted_averaging=False)
    for o in (out, plain):
        assert 0 < o["MRR"] <= 1 and o["H@10"] >= o["H@1"]


def test_online_learning_moves_scores(umls_like_dir, tmp_path):
    """A stored model is fine-tuned on single triples and on one (h, r) pair (reference tests/test_online_learning.py)."""
    rep = Execute(_args(umls_like_dir, tmp_path / "r", model="AConEx", scoring_technique="1vsSample", neg_ratio=1,
                        num_epochs=0, num_of_output_channels=2)).start()
    assert os.path.isdir(rep["path_experiment_folder"])
    k = KGE(path=rep["path_experiment_folder"])
    tr = np.load(tmp_path / "r" / "train_set.npy")
    h, r, t = k.idx_to_entity[int(tr[0, 0])], k.idx_to_relations[int(tr[0, 1])], k.idx_to_entity[int(tr[0, 2])]
    first = float(k.triple_score(h=[h], r=[r], t=[h]))
    k.train_triples(h=[h], r=[r], t=[h], labels=[0.0], iteration=3,
                    optimizer=torch.optim.Adam(params=k.parameters(), lr=0.01))
    assert float(k.triple_score(h=[h], r=[r], t=[h])) < first
    before = float(k.triple_score(h=[h], r=[r], t=[t]))
    k.train_k_vs_all(h=[h], r=[r], iteration=5, lr=0.01)
    assert float(k.triple_score(h=[h], r=[r], t=[t])) > before
    k.save()                                     # the fine-tuned weights can be stored next to the original run


@pytest.mark.parametrize("backend", ["pandas", "polars", "rdflib"])
def test_reading_backends(umls_like_dir, tmp_path, backend):
    """``polars`` falls back to the pandas reader when the package is absent; ``rdflib`` needs the package."""
    kw = {}
    if backend == "rdflib":
        pytest.importorskip("rdflib")
        import pandas as pd
        df = pd.read_csv(os.path.join(umls_like_dir, "train.txt"), sep=r"\\s+", header=None)
        nt = tmp_path / "kg.nt"
        with open(nt, "w") as f:
            for s, p, o in df.head(300).itertuples(index=False):
                f.write(f"<http://x/{s}> <http://x/{p}> <http://x/{o}> .\\n")
        kw = dict(dataset_dir=None, path_single_kg=str(nt))
    rep = Execute(_args(kw.pop("dataset_dir", umls_like_dir), tmp_path / "r", backend=backend, num_epochs=3,
                        **kw)).start()
    assert rep["num_train_triples"] > 0 and np.isfinite(rep["Train"]["MRR"])
