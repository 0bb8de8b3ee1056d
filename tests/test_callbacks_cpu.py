"""Weight averaging, periodic evaluation, LR schedules, perturbation and the TP trainer on CPU."""
import json
import os

import numpy as np
import pytest
import torch

from dice_embeddings_b200 import Execute, KGE, Namespace


def _args(kg, out, **kw):
    base = dict(dataset_dir=kg, path_to_store_single_run=str(out), model="ComplEx", scoring_technique="KvsAll",
                embedding_dim=32, num_epochs=30, batch_size=256, lr=0.1, optim="Adam", trainer="torchCPUTrainer",
                random_seed=1)
    base.update(kw)
    return Namespace(**base)


@pytest.mark.parametrize("flag", ["swa", "ema", "twa", "swag", "adaptive_swa"])
def test_weight_averaging_variants(umls_like_dir, tmp_path, flag):
    rep = Execute(_args(umls_like_dir, tmp_path / flag, swa_start_epoch=10, **{flag: True})).start()
    assert np.isfinite(rep["Test"]["MRR"]) and rep["Train"]["MRR"] > 0.1
    if flag == "adaptive_swa":
        assert os.path.isfile(tmp_path / flag / "aswa.pt")
    if flag == "swag":
        assert os.path.isfile(tmp_path / flag / "swag_eval_report.json")


def test_periodic_eval_keys_and_checkpoints(umls_like_dir, tmp_path):
    out = tmp_path / "pe"
    Execute(_args(umls_like_dir, out, num_epochs=12, eval_every_n_epochs=5, eval_at_epochs=[2], save_every_n_epochs=True,
                  n_epochs_eval_model="val_test", swa=True, swa_start_epoch=1)).start()
    rep = json.load(open(out / "eval_report_n_epochs.json"))
    assert set(rep) == {"epoch_2_eval", "epoch_5_eval", "epoch_10_eval"}
    assert set(rep["epoch_5_eval"]) == {"Val", "Test"}
    assert sorted(os.listdir(out / "models_n_epochs")) == ["model_at_epoch_10.pt", "model_at_epoch_2.pt",
                                                           "model_at_epoch_5.pt"]


@pytest.mark.parametrize("name", ["cca", "mmcclr", "deferred_cca", "deferred_mmcclr"])
def test_lr_scheduler_snapshots(umls_like_dir, tmp_path, name):
    out = tmp_path / name
    Execute(_args(umls_like_dir, out, num_epochs=20,
                  adaptive_lr={"scheduler_name": name, "lr_min": 0.01, "num_cycles": 4, "n_snapshots": 2,
                               "weighted_ensemble": True})).start()
    rep = json.load(open(out / "ensemble_eval_report.json"))
    assert rep["scheduler_name"] == name and rep["ensemble_eval_report"]["MRR"] > 0
    n = len(os.listdir(out / "snapshots"))
    assert n == (2 if name.startswith("deferred") else 4)


def test_lr_multiplier_shape():
    from dice_embeddings_b200.trainer.callbacks import LRScheduler
    import tempfile
    s = LRScheduler({"scheduler_name": "cca", "lr_min": 0.01, "num_cycles": 2, "n_snapshots": 2}, total_epochs=10,
                    experiment_dir=tempfile.mkdtemp(), eta_max=0.1)
    s._initialize_training_params(5)
    m = [s.lr_multiplier(i) for i in range(50)]
    assert abs(m[0] - 1.0) < 1e-9 and abs(m[25] - 1.0) < 1e-9 and min(m) >= 0.1 - 1e-9 and m[24] < m[1]


def test_perturb_krone_eval_ppe_callbacks(umls_like_dir, tmp_path):
    for i, cb in enumerate([{"Perturb": {"level": "input", "ratio": 0.2}},
                            {"Perturb": {"level": "param", "ratio": 0.1, "method": "GN", "scaler": 0.01}},
                            {"Perturb": {"level": "out", "ratio": 0.1, "method": "Soft", "scaler": 0.1}},
                            {"Eval": {"epoch_ratio": 5}}, {"PPE": {"last_percent_to_consider": 30}}]):
        out = tmp_path / f"cb{i}"
        rep = Execute(_args(umls_like_dir, out, num_epochs=10, callbacks=cb)).start()
        assert np.isfinite(rep["Train"]["MRR"])
        if "Eval" in cb:
            assert os.path.isfile(out / "evals_per_epoch")
        if "PPE" in cb:
            assert os.path.isfile(out / "trainer_checkpoint_main.pt")
    rep = Execute(_args(umls_like_dir, tmp_path / "kr", num_epochs=5, model="DistMult", scoring_technique="NegSample",
                        neg_ratio=2, embedding_dim=8, callbacks={"KronE": {}})).start()
    assert np.isfinite(rep["Train"]["MRR"])


def test_tensor_parallel_trainer_on_cpu_replicas(umls_like_dir, tmp_path, monkeypatch):
    from dice_embeddings_b200.trainer import tensor_parallel as tp
    orig = tp.TensorParallel.__init__
    monkeypatch.setattr(tp.TensorParallel, "__init__",
                        lambda self, args, callbacks=None, devices=None: orig(self, args, callbacks, ["cpu", "cpu"]))
    out = tmp_path / "tp"
    rep = Execute(_args(umls_like_dir, out, trainer="TP", num_epochs=40, model="Keci", save_embeddings_as_csv=False)).start()
    assert rep["Train"]["MRR"] > 0.5
    assert os.path.isfile(out / "model_partial_0.pt") and os.path.isfile(out / "model_partial_1.pt")
    from dice_embeddings_b200.io.checkpoint import write_csv_from_model_parallel
    write_csv_from_model_parallel(str(out))
    import pandas as pd
    assert pd.read_csv(out / "entity_embeddings.csv", index_col=0).shape[1] == 64


def test_gradient_accumulation_flag_and_label_smoothing(umls_like_dir, tmp_path):
    rep = Execute(_args(umls_like_dir, tmp_path / "ga", gradient_accumulation_steps=2, label_smoothing_rate=0.1,
                        num_epochs=10, input_dropout_rate=0.1, normalization="LayerNorm")).start()
    assert np.isfinite(rep["Train"]["MRR"])
