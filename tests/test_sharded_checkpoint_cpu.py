"""Sharded checkpoint: round trip, re-sharding to another world size, export to / import from ``model.pt``."""
import os

import pytest
import torch

from dice_embeddings_b200.io import sharded_checkpoint as sc


def _write(tmp, world, n=53, d=6):
    torch.manual_seed(0)
    E, m, v = torch.randn(n, d), torch.randn(n, d), torch.rand(n, d)
    R = torch.randn(7, d)
    for r in range(world):
        pad = torch.zeros(2, d)   # engines hold padded shards; the padding must not be stored
        sc.save_shard(str(tmp), r, world, n, {"E": torch.cat((E[r::world], pad)), "mE": torch.cat((m[r::world], pad)),
                                              "vE": torch.cat((v[r::world], pad))},
                      replicated={"relation_embeddings.weight": R, "m_R": R * 0} if r == 0 else None, step=41,
                      extra={"lr": 0.1})
    return E, m, v, R


@pytest.mark.parametrize("w_old,w_new", [(4, 4), (4, 3), (2, 8), (8, 1)])
def test_round_trip_and_resharding(tmp_path, w_old, w_new):
    E, m, v, R = _write(tmp_path, w_old)
    man = sc.read_manifest(str(tmp_path))
    assert man["world"] == w_old and man["step"] == 41 and man["extra"]["lr"] == 0.1
    for r in range(w_new):
        t = sc.load_shard(str(tmp_path), r, w_new)
        assert torch.equal(t["E"], E[r::w_new]) and torch.equal(t["mE"], m[r::w_new]) and torch.equal(t["vE"], v[r::w_new])
    assert torch.equal(sc.load_replicated(str(tmp_path))["relation_embeddings.weight"], R)


def test_export_and_import_single_file_layout(tmp_path):
    E, _, _, R = _write(tmp_path / "ck", 3)
    sd = sc.export_model_pt(str(tmp_path / "ck"), str(tmp_path / "model.pt"))
    assert set(sd) == {"entity_embeddings.weight", "relation_embeddings.weight"}
    back = torch.load(tmp_path / "model.pt")
    assert torch.equal(back["entity_embeddings.weight"], E) and torch.equal(back["relation_embeddings.weight"], R)
    sc.import_model_pt(str(tmp_path / "model.pt"), str(tmp_path / "ck2"), world=5)
    assert torch.equal(sc.assemble_table(str(tmp_path / "ck2")), E)
    assert float(sc.load_shard(str(tmp_path / "ck2"), 2, 5)["mE"].abs().sum()) == 0.0


def test_missing_or_corrupt_shard_is_reported(tmp_path):
    _write(tmp_path, 4)
    os.remove(sc.shard_file(str(tmp_path), 2))
    with pytest.raises(FileNotFoundError, match=r"\[2\]"):
        sc.read_manifest(str(tmp_path))
    _write(tmp_path, 4)
    with open(sc.shard_file(str(tmp_path), 1), "wb") as f:
        f.write(b"not a checkpoint")
    with pytest.raises(Exception):
        sc.load_shard(str(tmp_path), 1, 4)
