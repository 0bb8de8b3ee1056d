"""Small pieces of the reference's surface: relation domain / range constraints, the paged SPARQL reader against a
fake endpoint, validation of the knowledge-graph source, and the indexed-data sanity check."""
import json
import os

import numpy as np
import pytest

from dice_embeddings_b200 import Namespace
from dice_embeddings_b200.config import (dataset_sanity_checking, preprocess_args, sanity_check_callback_args,
                                         validate_knowledge_graph)
from dice_embeddings_b200.data import kg as kgmod
from dice_embeddings_b200.data.vocab import create_constraints


def test_create_constraints_equals_the_loop_definition():
    rng = np.random.default_rng(0)
    tr = np.stack([rng.integers(0, 30, 200), rng.integers(0, 4, 200), rng.integers(0, 30, 200)], axis=1).astype(np.int16)
    dc, rc, dom, ran = create_constraints(tr)
    ents = set(tr[:, 0].tolist()) | set(tr[:, 2].tolist())
    for r in set(tr[:, 1].tolist()):
        d = {int(h) for h, p, _ in tr if p == r}
        g = {int(t) for _, p, t in tr if p == r}
        assert dom[r] == d and ran[r] == g
        assert set(dc[r]) == ents - d and set(rc[r]) == ents - g


class _FakeResponse:
    def __init__(self, payload, ok=True):
        self._payload, self.ok, self.status_code = payload, ok, 200 if ok else 500

    def json(self):
        return self._payload

    def raise_for_status(self):
        if not self.ok:
            raise RuntimeError("HTTP 500")


def _fake_endpoint(triples, fail_offsets=()):
    calls = []

    def post(url, data=None, headers=None):
        q = data["query"]
        calls.append(q)
        if "COUNT" in q:
            return _FakeResponse({"results": {"bindings": [{"count": {"value": str(len(triples))}}]}})
        limit = int(q.split("LIMIT")[1].split()[0])
        offset = int(q.split("OFFSET")[1].split()[0])
        if offset in fail_offsets:
            return _FakeResponse({}, ok=False)
        rows = triples[offset:offset + limit]
        return _FakeResponse({"results": {"bindings": [{"subject": {"value": s}, "predicate": {"value": p},
                                                          "object": {"value": o}} for s, p, o in rows]}})
    return post, calls


def test_sparql_reader_pages_through_the_store(monkeypatch, tmp_path):
    import requests
    triples = [(f"s{i}", f"p{i % 3}", f"o{i % 7}") for i in range(53)]
    post, calls = _fake_endpoint(triples)
    monkeypatch.setattr(requests, "post", post)
    df = kgmod._read_sparql("http://fake/sparql", chunk_size=10, num_workers=4, cache_dir=str(tmp_path / "pages"))
    assert [tuple(r) for r in df.values.tolist()] == triples              # every page, in offset order
    assert sum("LIMIT 10 OFFSET" in c for c in calls) == 6
    assert len(os.listdir(tmp_path / "pages")) == 6
    n_calls = len(calls)
    again = kgmod._read_sparql("http://fake/sparql", chunk_size=10, cache_dir=str(tmp_path / "pages"))
    assert len(calls) == n_calls and [tuple(r) for r in again.values.tolist()] == triples   # served from the folder
    # a failing page is skipped, the others still arrive
    post, _ = _fake_endpoint(triples, fail_offsets=(20,))
    monkeypatch.setattr(requests, "post", post)
    part = kgmod._read_sparql("http://fake/sparql", chunk_size=10, num_workers=2)
    assert len(part) == 43 and ("s20", "p2", "o6") not in {tuple(r) for r in part.values.tolist()}


def test_knowledge_graph_source_validation(tmp_path, monkeypatch):
    folder = tmp_path / "kg"
    folder.mkdir()
    (folder / "train.txt").write_text("a\tr\tb\n")
    single = tmp_path / "one.txt"
    single.write_text("a\tr\tb\n")
    a = Namespace(dataset_dir=str(folder), path_single_kg=None, sparql_endpoint=None)
    validate_knowledge_graph(a)
    assert a.dataset_dir == str(folder)
    a = Namespace(dataset_dir=str(folder), path_single_kg=str(single))
    validate_knowledge_graph(a)                      # the single file wins, as in the reference
    assert a.dataset_dir is None and a.path_single_kg == str(single)
    (tmp_path / "empty").mkdir()
    with pytest.raises(ValueError):
        validate_knowledge_graph(Namespace(dataset_dir=str(tmp_path / "empty")))
    with pytest.raises(AssertionError):
        validate_knowledge_graph(Namespace(dataset_dir=str(tmp_path / "nowhere")))
    with pytest.raises(RuntimeError):
        validate_knowledge_graph(Namespace(dataset_dir=None, path_single_kg=None, sparql_endpoint=None))
    import requests
    post, _ = _fake_endpoint([("s", "p", "o")])
    monkeypatch.setattr(requests, "post", post)
    a = Namespace(dataset_dir=str(folder), sparql_endpoint="http://fake/sparql")
    validate_knowledge_graph(a)                      # a live endpoint wins over the folder
    assert a.dataset_dir is None and a.sparql_endpoint == "http://fake/sparql"


def test_multi_gpu_runs_need_a_run_folder(monkeypatch, tmp_path):
    monkeypatch.setenv("WORLD_SIZE", "2")
    with pytest.raises(NotImplementedError):
        sanity_check_callback_args(Namespace(trainer="torchDDP", path_to_store_single_run=None))
    sanity_check_callback_args(Namespace(trainer="torchDDP", path_to_store_single_run=str(tmp_path)))
    monkeypatch.setenv("WORLD_SIZE", "1")
    a = Namespace(trainer="torchCPUTrainer", swa=True, swa_start_epoch=None)
    sanity_check_callback_args(a)
    assert a.swa_start_epoch == 1


def test_dataset_sanity_checking():
    ok = np.array([[0, 0, 1], [2, 1, 0]], dtype=np.int8)
    dataset_sanity_checking(ok, 3, 2)
    with pytest.raises(AssertionError):
        dataset_sanity_checking(ok, 2, 2)
    with pytest.raises(AssertionError):
        dataset_sanity_checking(ok, 3, 1)
    with pytest.raises(AssertionError):
        dataset_sanity_checking(np.zeros((0, 3), dtype=np.int8), 3, 2)


def test_semantic_constraint_zeroes_impossible_triples(tmp_path):
    from dice_embeddings_b200 import KGE, Execute
    from dice_embeddings_b200.data.synthetic import make_planted_kg
    kg = make_planted_kg(str(tmp_path / "kg"), num_entities=60, num_relations=6, seed=3)
    out = tmp_path / "run"
    Execute(Namespace(dataset_dir=kg, path_to_store_single_run=str(out), model="DistMult", scoring_technique="KvsAll",
                      embedding_dim=16, num_epochs=2, batch_size=64, eval_model="None", trainer="torchCPUTrainer")).start()
    plain, strict = KGE(str(out)), KGE(str(out), apply_semantic_constraint=True)
    _, _, dom, rng = strict.semantic_constraints()
    inv_e = {v: k for k, v in strict.entity_to_idx.items()}
    inv_r = {v: k for k, v in strict.relation_to_idx.items()}
    r = next(iter(dom))
    h_in = next(iter(dom[r]))
    t_in = next(iter(rng[r]))
    t_out = next(e for e in range(strict.num_entities) if e not in rng[r])
    assert float(strict.triple_score(inv_e[h_in], inv_r[r], inv_e[t_in])) == \
        pytest.approx(float(plain.triple_score(inv_e[h_in], inv_r[r], inv_e[t_in])))
    assert float(strict.triple_score(inv_e[h_in], inv_r[r], inv_e[t_out])) == 0.0
    assert float(plain.triple_score(inv_e[h_in], inv_r[r], inv_e[t_out])) > 0.0


def test_dict_vocabularies_vectorised_and_written_by_the_helper_process(tmp_path):
    """The dict-of-lists filter vocabularies: the sort-based construction equals the per-triple loop (input order kept
    per key, absent keys give an empty list), and the helper process writes the three pickles of a run folder."""
    import pickle
    import subprocess
    import sys
    from collections import defaultdict

    import numpy as np

    from dice_embeddings_b200.data import vocab_writer
    from dice_embeddings_b200.data.vocab import get_ee_vocab, get_er_vocab, get_re_vocab
    rng = np.random.default_rng(0)
    d = np.stack([rng.integers(0, 60, 3000), rng.integers(0, 7, 3000), rng.integers(0, 60, 3000)], 1)
    for fn, (i, j, k) in ((get_er_vocab, (0, 1, 2)), (get_re_vocab, (1, 2, 0)), (get_ee_vocab, (0, 2, 1))):
        ref = defaultdict(list)
        for row in d.tolist():
            ref[(row[i], row[j])].append(row[k])
        got = fn(d)
        assert dict(got) == dict(ref)
        assert got[(10 ** 6, 0)] == []
    assert dict(get_er_vocab(np.zeros((0, 3), dtype=np.int64))) == {}
    src = tmp_path / "triples.npy"
    np.save(src, d)
    subprocess.run([sys.executable, vocab_writer.__file__, str(src), str(tmp_path)], check=True)
    assert not src.exists()
    with open(tmp_path / "re_vocab.p", "rb") as f:
        assert dict(pickle.load(f)) == dict(get_re_vocab(d))
