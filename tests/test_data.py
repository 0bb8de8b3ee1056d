"""Ingestion, vocabularies, on-disk layout and the vectorised scoring-technique datasets."""
import os
import pickle

import numpy as np
import pandas as pd
import pytest
import torch

from dice_embeddings_b200.data.datasets import (AllvsAll, KvsAll, KvsSampleDataset, OnevsAllDataset, OnevsSample,
                                                TriplePredictionDataset, construct_dataset)
from dice_embeddings_b200.data.kg import KG
from dice_embeddings_b200.data.vocab import PairCSR, get_er_vocab, get_re_vocab
from dice_embeddings_b200.data.synthetic import uniform_kg, zipf_kg


def _write(tmp_path, rows, name="train.txt"):
    d = tmp_path / "kg"
    d.mkdir(exist_ok=True)
    (d / name).write_text("\n".join("\t".join(r) for r in rows) + "\n")
    return str(d)


def test_kg_sorted_vocab_reciprocals_and_layout(tmp_path):
    rows = [("b", "likes", "a"), ("a", "knows", "c"), ("c", "likes", "b")]
    d = _write(tmp_path, rows)
    _write(tmp_path, [("a", "likes", "b")], "valid.txt")
    _write(tmp_path, [("b", "knows", "c")], "test.txt")
    out = tmp_path / "run"
    kg = KG(dataset_dir=d, add_reciprocal=True, eval_model="train_val_test", path_for_serialization=str(out))
    assert list(kg.entity_to_idx) == ["a", "b", "c"]                       # alphabetical ids
    assert list(kg.relation_to_idx) == ["knows", "knows_inverse", "likes", "likes_inverse"]
    assert len(kg.train_set) == 6 and len(kg.valid_set) == 2 and len(kg.test_set) == 2
    assert kg.train_set.dtype == np.int8
    ent = pd.read_csv(out / "entity_to_idx.csv", index_col=0)
    assert ent["entity"].tolist() == ["a", "b", "c"] and ent.index.tolist() == [0, 1, 2]
    assert np.array_equal(np.load(out / "train_set.npy"), kg.train_set)
    # reload from disk
    kg2 = KG(path_for_deserialization=str(out), eval_model="train_val_test")
    assert kg2.entity_to_idx == kg.entity_to_idx and np.array_equal(kg2.test_set, kg.test_set)
    assert kg.exists("b", "likes", "a") and not kg.exists("a", "likes", "c")


def test_no_reciprocals_without_eval(tmp_path):
    d = _write(tmp_path, [("b", "likes", "a"), ("a", "knows", "c")])
    kg = KG(dataset_dir=d, add_reciprocal=True, eval_model=None)
    assert len(kg.train_set) == 2 and kg.num_relations == 2


def test_read_only_few_and_separator(tmp_path):
    d = tmp_path / "k"
    d.mkdir()
    (d / "train.txt").write_text("\n".join(f"e{i},r{i % 3},e{i + 1}" for i in range(50)))
    kg = KG(dataset_dir=str(d), add_reciprocal=True, eval_model="train", read_only_few=10, separator=",")
    assert len(kg.train_set) == 20


def test_csr_equals_dict_vocab():
    tr = uniform_kg(30, 5, 400, seed=1)
    csr = PairCSR.build(tr[:, 0], tr[:, 1], tr[:, 2], 5)
    ref = get_er_vocab(tr)
    d = csr.to_dict()
    assert set(d) == set(ref)
    for k, v in ref.items():
        assert sorted(v) == d[k]
        assert sorted(v) == csr.lookup(*k).tolist()
    a = torch.tensor([k[0] for k in list(ref)[:7]] + [29])
    b = torch.tensor([k[1] for k in list(ref)[:7]] + [4])
    rows, cols = csr.batch_rows_cols(a, b)
    for i in range(len(a)):
        assert sorted(cols[rows == i].tolist()) == sorted(ref.get((int(a[i]), int(b[i])), []))
    assert set(get_re_vocab(tr)) == {(int(r), int(t)) for _, r, t in tr}


def test_kvsall_labels_match_per_item_construction():
    tr = uniform_kg(25, 4, 200, seed=2)
    ds = KvsAll(tr, 25, 4, label_smoothing_rate=0.1)
    er = get_er_vocab(tr)
    assert len(ds) == len(er)
    x, y = ds.make_batch(torch.arange(len(ds)))
    for i in range(len(ds)):
        ref = torch.zeros(25)
        ref[er[(int(x[i, 0]), int(x[i, 1]))]] = 1.0
        ref = ref * 0.9 + 1.0 / 25              # the reference's smoothing: y(1-eps) + 1/|E|
        assert torch.allclose(y[i], ref)
    xi, yi = ds[3]
    assert torch.equal(xi, x[3]) and torch.allclose(yi, y[3])


def test_allvsall_and_onevsall():
    tr = uniform_kg(12, 3, 40, seed=3)
    ds = AllvsAll(tr, 12, 3)
    assert len(ds) == 36
    x, y = ds.make_batch(torch.arange(36))
    er = get_er_vocab(tr)
    for i in range(36):
        assert sorted(torch.nonzero(y[i]).flatten().tolist()) == sorted(set(er.get((int(x[i, 0]), int(x[i, 1])), [])))
    d1 = OnevsAllDataset(tr, 12)
    x, y = d1.make_batch(torch.arange(len(d1)))
    assert y.sum(1).eq(1).all() and torch.equal(y.argmax(1), d1.train_data[:, 2])


def test_negative_sampling_semantics():
    tr = uniform_kg(50, 5, 300, seed=4)
    ds = TriplePredictionDataset(tr, 50, 5, neg_sample_ratio=3, label_smoothing_rate=0.1)
    g = torch.Generator().manual_seed(0)
    seen = set()
    for _ in range(8):
        x, y = ds.make_batch(torch.arange(10), g)
        assert x.shape == (40, 3) and y.shape == (40,)
        assert torch.allclose(y[:10], torch.full((10,), 0.9)) and torch.allclose(y[10:], torch.full((30,), 0.1))
        pos = x[:10]
        neg = x[10:]
        assert torch.equal(neg[:, 1], pos[:, 1].repeat(3))
        heads_same = torch.equal(neg[:, 0], pos[:, 0].repeat(3))
        tails_same = torch.equal(neg[:, 2], pos[:, 2].repeat(3))
        assert heads_same != tails_same or (heads_same and tails_same)   # one side corrupted per batch
        seen.add("tail" if heads_same else "head")
    assert seen == {"head", "tail"}


def test_sampled_techniques():
    tr = zipf_kg(60, 4, 500, seed=5)
    ds = OnevsSample(tr, 60, 4, neg_sample_ratio=7)
    x, yi, yv = ds.make_batch(torch.arange(64), torch.Generator().manual_seed(0))
    assert yi.shape == (64, 8) and torch.equal(yi[:, 0], ds.train_data[:64, 2])
    for row in yi.tolist():
        assert len(set(row)) == 8 and max(row) < 60          # distinct, true tail not among the negatives
    assert yv[:, 0].eq(1).all() and yv[:, 1:].eq(0).all()
    ks = KvsSampleDataset(tr, 60, 4, neg_ratio=5)
    x, yi, yv = ks.make_batch(torch.arange(len(ks)), torch.Generator().manual_seed(1))
    er = get_er_vocab(tr)
    assert yi.shape[1] == ks.max_num_of_classes
    for i in range(len(ks)):
        pos = set(er[(int(x[i, 0]), int(x[i, 1]))])
        got_pos = set(yi[i][yv[i] == 1].tolist())
        neg = set(yi[i][yv[i] == 0].tolist())
        assert got_pos == pos and not (neg & pos) and max(neg) < 60 and min(neg) >= 0


def test_construct_dataset_routing_and_sharded_batches():
    tr = uniform_kg(20, 3, 100, seed=6)
    kw = dict(train_set=tr, entity_to_idx=range(20), relation_to_idx=range(3), form_of_labelling="EntityPrediction",
              neg_ratio=2, label_smoothing_rate=0.0)
    names = {"KvsAll": "KvsAll", "AllvsAll": "AllvsAll", "1vsAll": "OnevsAllDataset", "NegSample": "TriplePredictionDataset",
             "1vsSample": "OnevsSample", "KvsSample": "KvsSampleDataset"}
    for st, cls in names.items():
        assert type(construct_dataset(scoring_technique=st, **kw)).__name__ == cls
    ds = construct_dataset(scoring_technique="KvsAll", **kw)
    g0, g1 = torch.Generator().manual_seed(3), torch.Generator().manual_seed(3)
    b0 = [b[0] for b in ds.batches(8, True, g0, rank=0, world_size=2)]
    b1 = [b[0] for b in ds.batches(8, True, g1, rank=1, world_size=2)]
    assert len(b0) == len(b1)
    both = torch.cat(b0 + b1)
    assert len({tuple(r) for r in both.tolist()}) == len(ds)      # the two ranks cover every data point
