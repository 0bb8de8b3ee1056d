"""Out-of-core ingestion: the native indexer against the in-memory KG class and the pandas stand-in, the memory-mapped
triples, and the per-owner label CSR."""
import os

import numpy as np
import pytest

from dice_embeddings_b200.data import ingest
from dice_embeddings_b200.data.kg import KG
from dice_embeddings_b200.data.synthetic import uniform_kg, write_kg_folder


def _kg_file(tmp_path, n=3000):
    tr = uniform_kg(120, 9, n, seed=5)
    folder = write_kg_folder(str(tmp_path / "kg"), tr, entity_prefix="http://ex.org/e", relation_prefix="p")
    return os.path.join(folder, "train.txt"), tr


@pytest.mark.parametrize("use_native", [True, False])
@pytest.mark.parametrize("reciprocal", [False, True])
def test_indexer_matches_the_in_memory_kg(tmp_path, use_native, reciprocal):
    if use_native and ingest.native() is None:
        pytest.skip("no C++ compiler on this machine")
    path, _ = _kg_file(tmp_path)
    out = str(tmp_path / f"run_{use_native}_{reciprocal}")
    d = ingest.index_triple_file(path, out, reciprocal=reciprocal, use_native=use_native, chunk_rows=700)
    assert d["indexer"] == ("native" if use_native else "pandas")
    kg = KG(path_single_kg=path, add_reciprocal=reciprocal, eval_model="train" if reciprocal else None)
    mm = ingest.open_triples(out)
    assert mm.shape == (kg.train_set.shape[0], 3) and d["num_entities"] == kg.num_entities
    assert d["num_relations"] == kg.num_relations
    # same ids (alphabetical vocabularies) and the same multiset of triples (the order of reciprocals differs)
    import pandas as pd
    e2i = pd.read_csv(os.path.join(out, "entity_to_idx.csv"), index_col=0)["entity"].tolist()
    assert e2i == sorted(kg.entity_to_idx, key=kg.entity_to_idx.get)
    a = np.asarray(mm).astype(np.int64)
    b = np.asarray(kg.train_set).astype(np.int64)
    assert sorted(map(tuple, a.tolist())) == sorted(map(tuple, b.tolist()))


def test_indexer_handles_ntriples_dots_blank_lines_and_max_rows(tmp_path):
    if ingest.native() is None:
        pytest.skip("no C++ compiler on this machine")
    p = tmp_path / "g.nt"
    p.write_text("<a> <p> <b> .\n\n<b>\t<q>\t<c> .\r\n<a> <p> <c> .\n<c> <q> <a> .")
    d = ingest.index_triple_file(str(p), str(tmp_path / "o"))
    assert d["shape"] == [4, 3] and d["num_entities"] == 3 and d["num_relations"] == 2
    assert np.asarray(ingest.open_triples(str(tmp_path / "o"))).tolist() == [[0, 0, 1], [1, 1, 2], [0, 0, 2], [2, 1, 0]]
    d = ingest.index_triple_file(str(p), str(tmp_path / "o2"), max_rows=2)
    assert d["shape"] == [2, 3]
    bad = tmp_path / "bad.txt"
    bad.write_text("a b\n")
    with pytest.raises(RuntimeError):
        ingest.index_triple_file(str(bad), str(tmp_path / "o3"), use_native=True)


def test_owner_csr_from_a_memory_map(tmp_path):
    path, tr = _kg_file(tmp_path, n=4000)
    out = str(tmp_path / "run")
    d = ingest.index_triple_file(path, out, use_native=False, chunk_rows=900)
    mm = ingest.open_triples(out)
    NR = d["num_relations"]
    full_pairs, full_off, full_val = ingest.owner_csr(mm, NR, 1, 0, chunk_rows=1000)
    truth = {}
    for h, r, t in np.asarray(mm).tolist():
        truth.setdefault((h, r), set()).add(t)
    assert [tuple(p) for p in full_pairs.tolist()] == sorted(truth)
    for i, key in enumerate(sorted(truth)):
        assert full_val[full_off[i]:full_off[i + 1]].tolist() == sorted(truth[key])
    W = 3
    for rank in range(W):
        pairs, off, val = ingest.owner_csr(mm, NR, W, rank, chunk_rows=1000)
        assert np.array_equal(pairs, full_pairs)              # every rank sees every data point
        for i, key in enumerate(sorted(truth)):
            want = sorted(t // W for t in truth[key] if t % W == rank)
            assert val[off[i]:off[i + 1]].tolist() == want


def test_memmap_batches_cover_the_file(tmp_path):
    path, _ = _kg_file(tmp_path, n=1000)
    out = str(tmp_path / "run")
    ingest.index_triple_file(path, out, use_native=False)
    mm = ingest.open_triples(out)
    ds = ingest.MemmapTriples(mm, batch_size=128, seed=1)
    rows = [tuple(r) for b in ds for r in b.tolist()]
    assert len(ds) == 8 and all(len(b) == 128 for b in ds)
    assert set(rows) == set(map(tuple, np.asarray(mm).astype(np.int64).tolist()))
