"""Training callbacks (reference ``dicee/callbacks.py``)."""
from __future__ import annotations

import datetime
import os
import time

import numpy as np
import pandas as pd
import torch

from .base import AbstractCallback


class AccumulateEpochLossCallback(AbstractCallback):
    """Writes ``epoch_losses.csv`` (column ``EpochLoss``) at the end of training (reference ``callbacks.py:27-46``)."""

    def __init__(self, path: str):
        self.path = path

    def on_fit_end(self, trainer, model) -> None:
        if getattr(trainer, "is_global_zero", True):
            pd.DataFrame(model.loss_history, columns=["EpochLoss"]).to_csv(os.path.join(self.path, "epoch_losses.csv"))


class PrintCallback(AbstractCallback):
    """Prints start time and total training time (reference ``callbacks.py:49-76``)."""

    def __init__(self):
        self.start_time = time.time()

    def on_fit_start(self, trainer, pl_module):
        self.start_time = time.time()
        print(f"\nTraining is starting {datetime.datetime.now()}...")

    def on_fit_end(self, trainer, pl_module):
        t = time.time() - self.start_time
        if t < 60:
            msg = f"{t:.3f} seconds."
        elif t < 3600:
            msg = f"{t / 60:.3f} minutes."
        else:
            msg = f"{t / 3600:.3f} hours."
        print(f"Training Runtime: {msg}\n")


class KGESaveCallback(AbstractCallback):
    """Stores ``model_at_{k}_epoch_<timestamp>.pt`` every ``every_x_epoch`` epochs (reference ``callbacks.py:79-107``)."""

    def __init__(self, every_x_epoch: int = None, max_epochs: int = None, path: str = None):
        self.every_x_epoch = every_x_epoch if every_x_epoch else max((max_epochs or 2) // 2, 1)
        self.max_epochs = max_epochs
        self.epoch_counter = 0
        self.path = path

    def on_train_epoch_end(self, trainer, model):
        from ..io.checkpoint import save_checkpoint_model
        if self.epoch_counter % self.every_x_epoch == 0 and self.epoch_counter > 1 and getattr(trainer, "is_global_zero", True):
            save_checkpoint_model(model, path=os.path.join(
                self.path, f"model_at_{self.epoch_counter}_epoch_{datetime.datetime.now()}.pt"))
        self.epoch_counter += 1


class PseudoLabellingCallback(AbstractCallback):
    """Self-training: after each epoch a random batch of unlabelled triples is scored and those with
    ``sigmoid(score) >= threshold`` are appended to the training triples (reference ``callbacks.py:110-147``)."""

    def __init__(self, data_module, kg, batch_size: int, threshold: float = 0.9):
        super().__init__()
        self.data_module, self.kg, self.batch_size, self.threshold = data_module, kg, int(batch_size), threshold
        self.unlabelled_size = len(self.kg.unlabelled_set)

    def create_random_data(self) -> torch.Tensor:
        e = torch.randint(0, self.kg.num_entities, (self.batch_size, 2))
        r = torch.randint(0, self.kg.num_relations, (self.batch_size,))
        return torch.stack((e[:, 0], r, e[:, 1]), dim=1)

    def on_epoch_end(self, trainer, model):
        return self.on_train_epoch_end(trainer, model)

    def on_train_epoch_end(self, trainer, model):
        model.eval()
        with torch.no_grad():
            pool = torch.as_tensor(np.asarray(self.kg.unlabelled_set)).long()
            batch = pool[torch.randint(0, self.unlabelled_size, (self.batch_size,))]
            conf = torch.sigmoid(model(batch.to(model.device))).cpu()
            chosen = batch[conf >= self.threshold]
        if len(chosen):
            self.data_module.train_set_idx = np.concatenate(
                (np.asarray(self.data_module.train_set_idx), chosen.numpy().astype(np.asarray(self.data_module.train_set_idx).dtype)), axis=0)
            if hasattr(self.data_module, "train_dataloader"):
                trainer.train_dataloader = self.data_module.train_dataloader()
            print(f"\tEpoch:{trainer.current_epoch}: Pseudo-labelling\t |D|= {len(self.data_module.train_set_idx)}")
        model.train()


def estimate_q(eps) -> float:
    """Rate of convergence ``q`` estimated from an error sequence (reference ``callbacks.py:150-156``)."""
    eps = np.asarray(eps, dtype=np.float64)
    x = np.arange(len(eps) - 1)
    y = np.log(np.abs(np.diff(np.log(eps))))
    return float(np.exp(np.polyfit(x, y, 1)[0]))


def compute_convergence(seq, i: int) -> float:
    assert len(seq) >= i > 0
    return estimate_q(np.asarray(seq[-i:], dtype=np.float64) / (np.arange(i) + 1))


class Eval(AbstractCallback):
    """Evaluates every ``epoch_ratio`` epochs and pickles the list of reports as ``evals_per_epoch``
    (reference ``callbacks.py:164-204``)."""

    def __init__(self, path, epoch_ratio: int = None):
        self.path = path
        self.reports = []
        self.epoch_ratio = epoch_ratio if epoch_ratio is not None else 1
        self.epoch_counter = 0

    def on_train_epoch_end(self, trainer, model):
        self.epoch_counter += 1
        if self.epoch_counter % self.epoch_ratio == 0 and getattr(trainer, "is_global_zero", True):
            model.eval()
            self.reports.append(trainer.evaluator.eval(dataset=trainer.dataset, trained_model=model,
                                                       form_of_labelling=trainer.form_of_labelling,
                                                       during_training=True))
            model.train()

    def on_fit_end(self, trainer, model):
        import pickle
        if getattr(trainer, "is_global_zero", True):
            with open(os.path.join(trainer.attributes.full_storage_path, "evals_per_epoch"), "wb") as f:
                pickle.dump(self.reports, f)


class KronE(AbstractCallback):
    """Augments every triple representation with the Kronecker product of its two halves
    (reference ``callbacks.py:207-253``)."""

    def __init__(self):
        self.f = None

    @staticmethod
    def batch_kronecker_product(a, b):
        return torch.einsum("bi,bj->bij", a, b).flatten(1)

    def get_kronecker_triple_representation(self, indexed_triple):
        assert indexed_triple.shape[1] == 3
        out = []
        for emb in self.f(indexed_triple):
            out.append(torch.cat((emb, self.batch_kronecker_product(*torch.hsplit(emb, 2))), dim=1))
        return tuple(out)

    def on_fit_start(self, trainer, model):
        from ..models.base import IdentityClass
        if not isinstance(model.normalize_head_entity_embeddings, IdentityClass):
            raise NotImplementedError("Normalizer should be reinitialized")
        self.f = model.get_triple_representation
        model.get_triple_representation = self.get_kronecker_triple_representation


class PPE(AbstractCallback):
    """Polyak parameter ensemble: uniform average of the weights of the last epochs (from ``epoch_to_start`` or the
    last ``last_percent_to_consider`` percent), kept in ``trainer_checkpoint_main.pt`` and loaded into the model at
    the end (reference ``dicee/abstracts.py:584-631``)."""

    def __init__(self, num_epochs, path, epoch_to_start=None, last_percent_to_consider=None):
        self.num_epochs, self.path = num_epochs, path
        self.epoch_count = 0
        self.sample_counter = 0
        if epoch_to_start is not None:
            assert epoch_to_start < num_epochs, f"--epoch_to_start {epoch_to_start} must be less than --num_epochs {num_epochs}"
            self.epoch_to_start = epoch_to_start
        elif last_percent_to_consider is None:
            self.epoch_to_start = 1
        else:
            self.epoch_to_start = num_epochs - int(num_epochs * last_percent_to_consider / 100)
        self.avg = None

    def on_train_epoch_end(self, trainer, model):
        self.epoch_count += 1
        if self.epoch_count < self.epoch_to_start or not getattr(trainer, "is_global_zero", True):
            return
        w = torch.nn.utils.parameters_to_vector([p.detach() for p in model.parameters()])
        self.sample_counter += 1
        if self.avg is None:
            self.avg = w.clone()
        else:
            self.avg.lerp_(w, 1.0 / self.sample_counter)

    def on_fit_end(self, trainer, model):
        if self.avg is None or not getattr(trainer, "is_global_zero", True):
            return
        with torch.no_grad():
            torch.nn.utils.vector_to_parameters(self.avg, list(model.parameters()))
        torch.save({k: v.cpu() for k, v in model.state_dict().items()}, os.path.join(self.path, "trainer_checkpoint_main.pt"))


class Perturb(AbstractCallback):
    """Three-level perturbation of a mini-batch before the step: ``input`` (replace heads or relations of a share of
    the rows by random ids), ``param`` (add Gaussian ``GN`` / uniform ``RN`` noise to the embeddings of the selected
    heads) or ``out`` (``Soft`` / ``Hard`` label flips).  Reference ``callbacks.py:256-376``."""

    def __init__(self, level: str = "input", ratio: float = 0.0, method: str = None, scaler: float = None,
                 frequency=None):
        assert level in {"input", "param", "out"}
        assert ratio >= 0.0
        self.level, self.ratio, self.method, self.scaler, self.frequency = level, ratio, method, scaler, frequency

    def on_train_batch_start(self, trainer, model, batch, batch_idx):
        x, y = batch[0], batch[-1]
        n = x.shape[0]
        k = int(n * self.ratio)
        if k == 0:
            return None
        dev = x.device
        sel = torch.randperm(n, device=dev)[:k]
        if self.level == "input":
            if float(torch.rand(1)) > 0.5:
                x[sel, 0] = torch.randint(0, model.num_entities, (k,), device=dev)
            else:
                x[sel, 1] = torch.randint(0, model.num_relations, (k,), device=dev)
        elif self.level == "param":
            rows = x[sel, 0]
            w = model.entity_embeddings.weight
            with torch.no_grad():
                if self.method == "GN":
                    w[rows] += torch.normal(0.0, self.scaler, size=(k, w.shape[1]), device=w.device)
                elif self.method == "RN":
                    w[rows] += torch.rand(k, w.shape[1], device=w.device) * self.scaler
                else:
                    raise RuntimeError(f"--method is given as {self.method}!")
        else:
            if self.method == "Soft":
                p = torch.rand(1, device=y.device) * self.scaler
                y[sel] = torch.where(y[sel] == 1.0, 1.0 - p, p)
            elif self.method == "Hard":
                y[sel] = torch.where(y[sel] == 1.0, 0.0, 1.0)
            else:
                raise NotImplementedError(f"{self.level}")
        return None


class PeriodicEvalCallback(AbstractCallback):
    """Evaluates at the given epochs on the splits named by ``n_epochs_eval_model``, stores the reports under
    ``epoch_{k}_eval`` in ``eval_report_n_epochs.json`` and optionally the evaluated weights as
    ``models_n_epochs/model_at_epoch_{k}.pt`` (reference ``callbacks.py:378-511``).  With a weight-averaging
    callback active the averaged model is evaluated."""

    def __init__(self, experiment_path: str, max_epochs: int, eval_every_n_epoch: int = 0, eval_at_epochs: list = None,
                 save_model_every_n_epoch: bool = True, n_epochs_eval_model: str = "val_test"):
        from collections import defaultdict
        self.experiment_dir, self.max_epochs = experiment_path, max_epochs
        self.epoch_counter = 0
        self.save_model_every_n_epoch = save_model_every_n_epoch
        self.reports = defaultdict(dict)
        self.n_epochs_eval_model = n_epochs_eval_model
        self.default_eval_model = None
        ep = set(eval_at_epochs or [])
        if eval_every_n_epoch and eval_every_n_epoch > 0:
            ep.update(range(eval_every_n_epoch, max_epochs + 1, eval_every_n_epoch))
        self.eval_epochs = ep
        if self.save_model_every_n_epoch:
            self.n_epochs_storage_path = os.path.join(self.experiment_dir, "models_n_epochs")
            os.makedirs(self.n_epochs_storage_path, exist_ok=True)

    def on_fit_end(self, trainer, model):
        import json
        if getattr(trainer, "is_global_zero", True):
            with open(os.path.join(self.experiment_dir, "eval_report_n_epochs.json"), "w") as f:
                json.dump(self.reports, f, indent=4)

    def on_train_epoch_end(self, trainer, model):
        import copy
        self.epoch_counter += 1
        if self.epoch_counter not in self.eval_epochs or not getattr(trainer, "is_global_zero", True):
            return
        if self.default_eval_model is None:
            self.default_eval_model = trainer.evaluator.args.eval_model
        if self.epoch_counter == self.max_epochs and self.default_eval_model:
            if set(self.n_epochs_eval_model.split("_")).issubset(set(self.default_eval_model.split("_"))):
                return  # the final evaluation covers these splits anyway
        args = getattr(model, "args", {}) or {}
        eval_model = None
        if any(args.get(k) for k in ("swa", "ema", "twa")) and getattr(trainer, "wa_model", None) is not None:
            eval_model = copy.deepcopy(trainer.wa_model)
        elif args.get("adaptive_swa") and os.path.isfile(os.path.join(self.experiment_dir, "aswa.pt")):
            eval_model = copy.deepcopy(model)
            eval_model.load_state_dict(torch.load(os.path.join(self.experiment_dir, "aswa.pt"), map_location="cpu",
                                                  weights_only=False))
        else:
            eval_model = copy.deepcopy(model)
        eval_model.eval()
        trainer.evaluator.args.eval_model = self.n_epochs_eval_model
        report = trainer.evaluator.eval(dataset=trainer.dataset, trained_model=eval_model,
                                        form_of_labelling=trainer.form_of_labelling, during_training=True)
        trainer.evaluator.args.eval_model = self.default_eval_model
        self.reports[f"epoch_{self.epoch_counter}_eval"] = report
        if self.save_model_every_n_epoch:
            torch.save({k: v.cpu() for k, v in eval_model.state_dict().items()},
                       os.path.join(self.n_epochs_storage_path, f"model_at_epoch_{self.epoch_counter}.pt"))
        del eval_model


class LRScheduler(AbstractCallback):
    """Cyclic learning-rate schedules with snapshot ensembles (reference ``callbacks.py:512-820``).

    ``scheduler_name``: ``cca`` (cosine annealing per step inside each of ``num_cycles`` cycles), ``mmcclr`` (the same
    per epoch), and ``deferred_*`` variants that keep the maximum rate for the first
    ``(num_cycles - n_snapshots) / num_cycles`` of training.  A snapshot of the weights is stored at the end of every
    cycle; after training the snapshots are evaluated as a (loss-weighted) ensemble on the test split and the
    result goes to ``ensemble_eval_report.json``."""

    VALID = ("cca", "mmcclr", "deferred_cca", "deferred_mmcclr")

    def __init__(self, adaptive_lr_config: dict, total_epochs: int, experiment_dir: str, eta_max: float = 0.1,
                 snapshot_dir: str = "snapshots"):
        import math
        from collections import defaultdict
        if not isinstance(adaptive_lr_config, dict):
            raise ValueError("adaptive_lr_config must be a dictionary")
        c = adaptive_lr_config
        self.scheduler_name = str(c.get("scheduler_name", "cca")).lower()
        if self.scheduler_name not in self.VALID:
            raise ValueError(f"Invalid scheduler_name '{self.scheduler_name}'. Must be one of: {list(self.VALID)}")
        self.eta_min = c.get("lr_min", 0.01)
        self.n_cycles = c.get("num_cycles", 10)
        self.weighted_ensemble = c.get("weighted_ensemble", True)
        self.n_snapshots = c.get("n_snapshots", 5)
        self.eta_max = eta_max
        if not (isinstance(self.eta_min, (int, float)) and 0 < self.eta_min < eta_max):
            raise ValueError(f"lr_min ({self.eta_min}) must be positive and less than eta_max ({eta_max})")
        if not (isinstance(self.n_cycles, (int, float)) and self.n_cycles > 0):
            raise ValueError(f"num_cycles must be a positive number, got: {self.n_cycles}")
        if not (isinstance(self.n_snapshots, int) and self.n_snapshots > 0):
            raise ValueError(f"n_snapshots must be a positive integer, got: {self.n_snapshots}")
        if not isinstance(self.weighted_ensemble, bool):
            raise ValueError(f"weighted_ensemble must be a boolean, got: {self.weighted_ensemble}")
        assert self.n_snapshots <= self.n_cycles
        self.total_epochs, self.experiment_dir = total_epochs, experiment_dir
        self.snapshot_dir = os.path.join(experiment_dir, snapshot_dir)
        os.makedirs(self.snapshot_dir, exist_ok=True)
        self.warmup_epochs = int((self.n_cycles - self.n_snapshots) / self.n_cycles * total_epochs) \
            if self.scheduler_name.startswith("deferred") else 0
        self.batches_per_epoch = self.total_steps = self.cycle_length = None
        self.warmup_steps = 0
        self.step_count = 0
        self.snapshot_loss = defaultdict(float)
        self._math = math

    # ------------------------------------------------------------------ schedule
    def _initialize_training_params(self, num_training_batches: int) -> None:
        self.batches_per_epoch = num_training_batches
        self.total_steps = self.total_epochs * num_training_batches
        self.cycle_length = int(self.total_steps // self.n_cycles)
        if self.cycle_length < 1:
            raise ValueError(f"Cycle length must be at least 1 (total steps {self.total_steps}, cycles {self.n_cycles})")
        self.warmup_steps = int(self.warmup_epochs * num_training_batches)
        if self.warmup_steps >= self.total_steps:
            raise ValueError("Warmup steps must be less than total steps")

    def lr_multiplier(self, step: int) -> float:
        m = self._math
        lo = self.eta_min / self.eta_max
        name = self.scheduler_name
        if name.startswith("deferred"):
            if step < self.warmup_steps:
                return 1.0
            step -= self.warmup_steps
            name = name[len("deferred_"):]
        if name == "cca":
            L = m.ceil(self.total_steps / self.n_cycles)
            frac = (step % L) / L
        else:
            L = max(int(self.total_epochs // self.n_cycles), 1)
            frac = ((step // self.batches_per_epoch) % L) / L
        return lo + (1.0 - lo) * 0.5 * (1 + m.cos(m.pi * frac))

    def _is_snapshot_step(self, step: int) -> bool:
        if self.scheduler_name.startswith("deferred"):
            if step < self.warmup_steps:
                return False
            interval = max((self.total_steps - self.warmup_steps) // self.n_snapshots, 1)
            return (step - self.warmup_steps + 1) % interval == 0
        return (step + 1) % self.cycle_length == 0

    def _set_lr(self, trainer, model, lr: float) -> None:
        opts = list(getattr(model, "optimizers", None) or getattr(trainer, "optimizers", None) or [])
        for o in opts:
            if o is None:
                continue
            for pg in o.param_groups:
                pg["lr"] = lr

    # ------------------------------------------------------------------ hooks
    def on_fit_start(self, trainer, model):
        loader = getattr(trainer, "train_dataloaders", None)
        n = len(loader) if loader is not None else getattr(trainer, "num_training_batches", 1)
        self._initialize_training_params(int(n))
        self.step_count = 0
        self._set_lr(trainer, model, self.eta_max * self.lr_multiplier(0))

    on_train_start = on_fit_start

    def on_train_batch_end(self, trainer, model, outputs=None, batch=None, batch_idx=None):
        if self.total_steps is None:
            return
        self.step_count += 1
        self._set_lr(trainer, model, self.eta_max * self.lr_multiplier(self.step_count))
        if self._is_snapshot_step(self.step_count) and getattr(trainer, "is_global_zero", True):
            eng = getattr(trainer, "engine", None)
            if eng is not None:
                eng.sync_to_model()
            name = f"snapshot_epoch_{trainer.current_epoch}.pt"
            torch.save({k: v.detach().cpu() for k, v in model.state_dict().items()}, os.path.join(self.snapshot_dir, name))
            loss = outputs["loss"] if isinstance(outputs, dict) else outputs
            self.snapshot_loss[name] = float(loss.detach() if hasattr(loss, "detach") else loss) if loss is not None else 0.0

    def _calculate_snap_weights(self):
        import numpy as np
        names = list(self.snapshot_loss.keys())
        losses = np.array([self.snapshot_loss[n] for n in names])
        raw = np.clip((losses.max() + losses.min()) - losses, a_min=0, a_max=None)
        w = raw / raw.sum() if raw.sum() > 0 else np.ones_like(raw) / len(raw)
        self.snapshot_weights = dict(zip(names, w.tolist()))

    def on_fit_end(self, trainer, model):
        import copy
        import json
        if not getattr(trainer, "is_global_zero", True):
            return
        from ..evaluation.ensemble import evaluate_ensemble_link_prediction_performance
        files = sorted(f for f in os.listdir(self.snapshot_dir) if f.endswith(".pt"))
        snaps = []
        for f in files:
            m = copy.deepcopy(model)
            m.load_state_dict(torch.load(os.path.join(self.snapshot_dir, f), map_location="cpu", weights_only=False))
            snaps.append(m.eval())
        weights = None
        if self.snapshot_loss and self.weighted_ensemble and files:
            self._calculate_snap_weights()
            weights = [self.snapshot_weights.get(f, 0.0) for f in files]
        ds = trainer.dataset
        report = None
        if snaps and getattr(ds, "test_set", None) is not None and getattr(ds, "er_csr", None) is not None:
            report = evaluate_ensemble_link_prediction_performance(
                models=snaps, triples=ds.test_set, er_vocab=ds.er_csr, weights=weights, batch_size=1024,
                weighted_averaging=bool(self.weighted_ensemble and weights is not None))
        self.ensemble_eval_report = {
            "scheduler_name": self.scheduler_name, "total_epochs": self.total_epochs, "num_cycles": self.n_cycles,
            "warmup_epochs": self.warmup_epochs, "lr_max": self.eta_max, "lr_min": self.eta_min,
            "batches_per_epoch": self.batches_per_epoch, "total_steps": self.total_steps,
            "cycle_length": self.cycle_length, "warmup_steps": self.warmup_steps,
            "weighted_ensemble": self.weighted_ensemble, "n_snapshots": self.n_snapshots,
            "ensemble_eval_report": report, "snapshot_loss": dict(self.snapshot_loss)}
        with open(os.path.join(self.experiment_dir, "ensemble_eval_report.json"), "w", encoding="utf-8") as f:
            json.dump(self.ensemble_eval_report, f, indent=4, ensure_ascii=False)
