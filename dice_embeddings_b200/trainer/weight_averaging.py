"""Weight-averaging callbacks: SWA, ASWA, SWAG, EMA and TWA.

Semantics follow reference ``dicee/weight_averaging.py`` (ASWA ``:13-146``, SWA ``:148-266``, SWAG ``:268-452``,
EMA ``:456-538``, TWA ``:540-685``).  All averages are kept as flat parameter vectors
(``parameters_to_vector``) on the model's device, so an update is one fused axpy instead of a Python loop over
parameter tensors, and the averaged weights are swapped into the trained model at ``on_fit_end``.
"""
from __future__ import annotations

import copy
import json
import os
from typing import List, Optional

import torch
import torch.nn as nn

from .base import AbstractCallback


def _flat(model) -> torch.Tensor:
    return nn.utils.parameters_to_vector([p.detach() for p in model.parameters()])


def _load_flat(model, vec: torch.Tensor) -> None:
    with torch.no_grad():
        nn.utils.vector_to_parameters(vec.to(next(iter(model.parameters())).device), list(model.parameters()))


def _swa_lr_factor(epoch: int, max_epochs: int, lr_init: float, swa_lr: float) -> float:
    """Constant until half of training, linear decay to ``swa_lr / lr_init`` at 90 %, constant afterwards."""
    t = epoch / max_epochs
    ratio = swa_lr / lr_init
    if t <= 0.5:
        return 1.0
    if t <= 0.9:
        return 1.0 - (1.0 - ratio) * (t - 0.5) / 0.4
    return ratio


def _optimizers(trainer, model) -> List:
    if hasattr(model, "optimizers") and getattr(model, "optimizers"):
        return list(model.optimizers)
    opts = getattr(trainer, "optimizers", None)
    return [o for o in (opts or []) if o is not None]


def _clone_model(model):
    return copy.deepcopy(model)


class _AveragingBase(AbstractCallback):
    """Shared bookkeeping: start epoch, update period, exposure of the averaged model to periodic evaluation."""

    def __init__(self, start_epoch: Optional[int], every: int = 1, max_epochs: Optional[int] = None):
        self.start_epoch = int(start_epoch) if start_epoch is not None else 0
        self.every = max(int(every or 1), 1)
        self.max_epochs = max_epochs
        self.current_epoch = -1
        self.avg: Optional[torch.Tensor] = None
        self.n_avg = 0
        self._wa_model = None

    def on_train_epoch_start(self, trainer, model):
        self.current_epoch = getattr(trainer, "current_epoch", self.current_epoch + 1)

    def _due(self) -> bool:
        return self.current_epoch >= self.start_epoch and (self.current_epoch - self.start_epoch) % self.every == 0

    def _expose(self, trainer, model) -> None:
        """Periodic evaluation callbacks evaluate ``trainer.wa_model`` when present."""
        args = getattr(model, "args", {}) or {}
        if self.avg is None or not ((args.get("eval_every_n_epochs") or 0) > 0 or args.get("eval_at_epochs") is not None):
            return
        if self._wa_model is None:
            self._wa_model = _clone_model(model)
        _load_flat(self._wa_model, self.avg)
        trainer.wa_model = self._wa_model

    def on_fit_end(self, trainer, model):
        if self.avg is not None and getattr(trainer, "is_global_zero", True):
            _load_flat(model, self.avg)


class SWA(_AveragingBase):
    """Stochastic weight averaging: running mean of the weights of every ``swa_c_epochs``-th epoch from
    ``swa_start_epoch`` on, with the SWA learning-rate schedule applied to the trainer's optimisers."""

    def __init__(self, swa_start_epoch, swa_c_epochs: int = 1, lr_init: float = 0.1, swa_lr: float = 0.05,
                 max_epochs: int = None):
        super().__init__(swa_start_epoch, swa_c_epochs, max_epochs)
        self.swa_start_epoch, self.swa_c_epochs = self.start_epoch, self.every
        self.lr_init, self.swa_lr = lr_init, swa_lr
        self.swa_n = 0

    @property
    def swa_model(self):
        return self._wa_model

    def on_train_epoch_start(self, trainer, model):
        super().on_train_epoch_start(trainer, model)
        if self.current_epoch < self.start_epoch:
            return
        f = _swa_lr_factor(self.current_epoch, self.max_epochs, self.lr_init, self.swa_lr)
        for opt in _optimizers(trainer, model):
            for pg in opt.param_groups:
                pg["lr"] = self.lr_init * f

    def on_train_epoch_end(self, trainer, model):
        if not getattr(trainer, "is_global_zero", True) or not self._due():
            return
        w = _flat(model)
        if self.avg is None:
            self.avg = w.clone()
        else:
            self.avg.lerp_(w, 1.0 / (self.swa_n + 1))
        self.swa_n += 1
        self.n_avg = self.swa_n
        self._expose(trainer, model)


class EMA(_AveragingBase):
    """Exponential moving average of the weights (``decay`` 0.999) from ``ema_start_epoch`` on."""

    def __init__(self, ema_start_epoch: int, decay: float = 0.999, max_epochs: int = None, ema_c_epochs: int = 1):
        super().__init__(ema_start_epoch, ema_c_epochs, max_epochs)
        self.ema_start_epoch, self.ema_c_epochs, self.decay = self.start_epoch, self.every, decay

    @property
    def ema_model(self):
        return self._wa_model

    def on_train_epoch_end(self, trainer, model):
        if not getattr(trainer, "is_global_zero", True) or not self._due():
            return
        w = _flat(model)
        if self.avg is None:
            self.avg = w.clone()
        self.avg.mul_(self.decay).add_(w, alpha=1.0 - self.decay)
        self.n_avg += 1
        self._expose(trainer, model)


class ASWA(AbstractCallback):
    """Adaptive SWA: after every epoch the running model and the candidate "ensemble + running model" average are
    ranked on the validation split; the running ensemble is restarted, extended or left alone depending on which
    validation MRR is best.  The ensemble lives in ``aswa.pt`` inside the run directory and replaces the model's
    weights at the end of training."""

    def __init__(self, num_epochs, path):
        self.path = path
        self.num_epochs = num_epochs
        self.initial_eval_setting = None
        self.epoch_count = 0
        self.alphas: List[float] = []
        self.val_aswa = -1.0

    def _file(self) -> str:
        return os.path.join(self.path, "aswa.pt")

    @staticmethod
    def compute_mrr(trainer, model) -> float:
        was_training = model.training
        model.eval()
        rep = trainer.evaluator.eval(dataset=trainer.dataset, trained_model=model,
                                     form_of_labelling=trainer.form_of_labelling, during_training=True)
        model.train(was_training)
        return rep["Val"]["MRR"]

    def get_aswa_state_dict(self, model):
        ens = torch.load(self._file(), map_location=next(iter(model.parameters())).device, weights_only=False)
        s = sum(self.alphas)
        with torch.no_grad():
            for k, prm in model.state_dict().items():
                if prm.dtype == torch.float:
                    ens[k] = (ens[k] * s + prm) / (1 + s)
        return ens

    def decide(self, running_state, ensemble_state, val_running, val_ensemble) -> bool:
        if val_running > val_ensemble and val_running > self.val_aswa:
            torch.save(running_state, self._file())      # restart the ensemble from the running model
            self.alphas.clear()
            self.val_aswa = val_running
            return True
        if val_ensemble > self.val_aswa:
            self.val_aswa = val_ensemble                 # accept the running model into the ensemble
            torch.save(ensemble_state, self._file())
            self.alphas.append(1.0)
            return True
        if self.val_aswa > val_ensemble:
            self.alphas.append(0)                        # reject: the ensemble would get worse
        return True

    def on_train_epoch_end(self, trainer, model):
        if not getattr(trainer, "is_global_zero", True):
            return
        self.epoch_count += 1
        if self.initial_eval_setting is None:
            self.initial_eval_setting = trainer.evaluator.args.eval_model
            trainer.evaluator.args.eval_model = "val"
        val_running = self.compute_mrr(trainer, model)
        if self.val_aswa == -1.0:
            torch.save(model.state_dict(), self._file())
            self.alphas.append(1.0)
            self.val_aswa = val_running
            return
        ens_state = self.get_aswa_state_dict(model)
        ens = _clone_model(model)
        ens.load_state_dict(ens_state)
        val_ens = self.compute_mrr(trainer, ens)
        del ens
        self.decide(model.state_dict(), ens_state, val_running, val_ens)

    def on_fit_end(self, trainer, model):
        if not getattr(trainer, "is_global_zero", True):
            return
        if self.initial_eval_setting:
            trainer.evaluator.args.eval_model = self.initial_eval_setting
        if os.path.isfile(self._file()):
            model.load_state_dict(torch.load(self._file(), map_location="cpu", weights_only=False))


class SWAG(_AveragingBase):
    """SWA-Gaussian: running first and second moments of the weight vector plus the last ``max_num_models``
    deviations; at the end ``max_num_models`` models are sampled from the fitted Gaussian, evaluated as an ensemble
    on the test split (``swag_eval_report.json``) and the mean weights are installed."""

    def __init__(self, swa_start_epoch, swa_c_epochs: int = 1, lr_init: float = 0.1, swa_lr: float = 0.05,
                 max_epochs: int = None, max_num_models: int = 20, var_clamp: float = 1e-30):
        super().__init__(swa_start_epoch, swa_c_epochs, max_epochs)
        self.swa_start_epoch, self.swa_c_epochs = self.start_epoch, self.every
        self.lr_init, self.swa_lr = lr_init, swa_lr
        self.max_num_models, self.var_clamp = max_num_models, var_clamp
        self.mean = None
        self.sq_mean = None
        self.deviations: List[torch.Tensor] = []
        self.gswa_n = 0

    def on_train_epoch_start(self, trainer, model):
        super().on_train_epoch_start(trainer, model)
        if self.current_epoch < self.start_epoch:
            return
        f = _swa_lr_factor(self.current_epoch, self.max_epochs, self.lr_init, self.swa_lr)
        for opt in _optimizers(trainer, model):
            for pg in opt.param_groups:
                pg["lr"] = self.lr_init * f

    def _collect_stats(self, model) -> None:
        vec = _flat(model).cpu()
        if self.mean is None:
            self.mean, self.sq_mean = vec.clone(), vec.clone() ** 2
        else:
            self.mean = (self.mean * self.gswa_n + vec) / (self.gswa_n + 1)
            self.sq_mean = (self.sq_mean * self.gswa_n + vec ** 2) / (self.gswa_n + 1)
        self.deviations.append((vec - self.mean).unsqueeze(1))
        if len(self.deviations) > self.max_num_models:
            self.deviations.pop(0)
        self.gswa_n += 1
        self.avg = self.mean

    def get_mean_and_var(self):
        if self.mean is None:
            return None, None
        return self.mean, torch.clamp(self.sq_mean - self.mean ** 2, min=self.var_clamp)

    def sample(self, base_model, scale: float = 0.5):
        if self.mean is None:
            raise RuntimeError("No SWAG stats collected yet.")
        mean, var = self.get_mean_and_var()
        vec = mean + scale * torch.sqrt(var) * torch.randn_like(mean)
        if self.deviations:
            D = torch.cat(self.deviations, dim=1)
            vec = vec + (D @ torch.randn(D.shape[1])) / max(1, len(self.deviations) - 1) ** 0.5
        _load_flat(base_model, vec)
        return base_model

    def on_train_epoch_end(self, trainer, model):
        if getattr(trainer, "is_global_zero", True) and self._due():
            self._collect_stats(model)

    def on_fit_end(self, trainer, model):
        if not getattr(trainer, "is_global_zero", True) or self.mean is None:
            return
        from ..evaluation.ensemble import evaluate_ensemble_link_prediction_performance
        ds = trainer.dataset
        test = getattr(ds, "test_set", None)
        if test is not None and getattr(ds, "er_csr", None) is not None:
            samples = [self.sample(_clone_model(model)).eval() for _ in range(self.max_num_models)]
            rep = evaluate_ensemble_link_prediction_performance(models=samples, triples=test, er_vocab=ds.er_csr,
                                                                weights=None, batch_size=1024,
                                                                weighted_averaging=False, normalize_scores=False)
            path = (getattr(model, "args", {}) or {}).get("full_storage_path") or getattr(trainer.attributes,
                                                                                         "full_storage_path", ".")
            with open(os.path.join(path, "swag_eval_report.json"), "w", encoding="utf-8") as f:
                json.dump(rep, f, indent=4, ensure_ascii=False)
        _load_flat(model, self.mean)


class TWA(_AveragingBase):
    """Trainable weight averaging: weight snapshots collected before ``twa_start_epoch`` span a low-dimensional
    subspace (SVD of the centred snapshots); afterwards the epoch-end gradient is projected onto that subspace and
    the coefficients ``beta`` take one (optionally regularised) gradient step per epoch."""

    def __init__(self, twa_start_epoch: int, lr_init: float, num_samples: int = 5, reg_lambda: float = 0.0,
                 max_epochs: int = None, twa_c_epochs: int = 1):
        super().__init__(twa_start_epoch, twa_c_epochs, max_epochs)
        self.twa_start_epoch, self.twa_c_epochs = self.start_epoch, self.every
        self.lr_init, self.num_samples, self.reg_lambda = lr_init, num_samples, reg_lambda
        self.weight_samples: List[torch.Tensor] = []
        self.base_weights = None
        self.P = None
        self.beta = None

    @property
    def twa_model(self):
        return self._wa_model

    def sample_weights(self, model) -> torch.Tensor:
        w = _flat(model).clone()
        self.weight_samples.append(w)
        if len(self.weight_samples) > self.num_samples:
            self.weight_samples.pop(0)
        return w

    @staticmethod
    def build_projection(weight_samples, k=None):
        W = torch.stack(weight_samples)
        mean_w = W.mean(dim=0)
        _, _, Vh = torch.linalg.svd(W - mean_w, full_matrices=False)
        V = Vh.T
        k = min(W.size(0), V.size(1)) if k is None else k
        return mean_w, V[:, :k]

    def on_train_epoch_end(self, trainer, model):
        if not getattr(trainer, "is_global_zero", True):
            return
        if self.current_epoch < self.start_epoch:
            self.sample_weights(model)
            return
        if not self._due():
            return
        if self.P is None:
            if not self.weight_samples:
                self.sample_weights(model)
            self.base_weights, self.P = self.build_projection(self.weight_samples)
            self.beta = torch.zeros(self.P.size(1), device=self.base_weights.device)
        grads = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1)
                           for p in model.parameters()]).to(self.P.device)
        with torch.no_grad():
            self.beta = (1 - self.lr_init * self.reg_lambda) * self.beta - self.lr_init * (self.P.t() @ grads)
            self.avg = self.base_weights + self.P @ self.beta
        self._expose(trainer, model)
