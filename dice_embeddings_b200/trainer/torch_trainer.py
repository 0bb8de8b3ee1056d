"""Single-device trainer (CPU or one GPU).

Counterpart of the reference's ``TorchTrainer`` (``dicee/trainer/torch_trainer.py:9-180``) with three
differences that matter on a B200: batches are built on the device from resident index tensors (no per-step
host→device copy of ``B × |E|`` labels), the loss stays on the device and is read back once per epoch instead
of once per step (the reference calls ``loss.item()`` every batch, ``:146-149``), and when the model is one of
the bilinear families trained with KvsAll / 1vsAll on a CUDA device the whole step is handed to the fused
sm_100a engine (:mod:`dice_embeddings_b200.ops.fused_step`); bilinear models whose query vector is produced by
PyTorch modules (convolutional gates, normalisers, dropout) keep those in autograd and score against the entity
table on the tensor cores through :mod:`dice_embeddings_b200.ops.hybrid_step`.

Gradient accumulation follows the reference literally: with ``gradient_accumulation_steps = k > 1`` the
gradients are only *zeroed* every ``k`` batches while the optimiser still steps every batch (``:50-58, 148``).
"""
from __future__ import annotations

import time
import torch

from .base import AbstractTrainer, BatchLoader


def _to_device(batch, device):
    return tuple(b.to(device, non_blocking=True) if isinstance(b, torch.Tensor) else b for b in batch)


class TorchTrainer(AbstractTrainer):
    def __init__(self, args, callbacks=None):
        super().__init__(args, callbacks)
        gpus = getattr(args, "gpus", None)
        if gpus is not None and gpus is not False and torch.cuda.is_available():
            self.device = torch.device(f"cuda:{int(gpus) if not isinstance(gpus, bool) else 0}")
        elif getattr(args, "trainer", None) == "PL" and torch.cuda.is_available():
            self.device = torch.device("cuda:0")
        else:
            self.device = torch.device("cpu")
        self.loss_function = None
        self.train_dataloaders = None
        self.engine = None

    # ------------------------------------------------------------------
    def _maybe_build_engine(self, model, loader):
        backend = getattr(self.attributes, "kernel_backend", "auto")
        if backend == "torch" or self.device.type != "cuda":
            return None
        try:
            from ..ops.fused_step import build_fused_engine
            from ..ops.sampled_step import SUPPORTED_SCORING as SAMPLED, build_sampled_engine
        except Exception:
            if backend == "cuda":
                raise
            return None
        ds = getattr(loader, "dataset", None)
        if getattr(self.attributes, "scoring_technique", None) in SAMPLED:
            return build_sampled_engine(model, ds, self.attributes, self.device, strict=(backend == "cuda"))
        # models whose query vector comes out of PyTorch modules (convolutional gates, normalisers, dropout, dual
        # quaternions) keep those in autograd and hand only the scoring against the table to the tensor-core kernels
        from ..ops.fused_step import fused_model_code
        from ..ops.hybrid_step import build_hybrid_engine
        if fused_model_code(model) is None:
            hybrid = build_hybrid_engine(model, ds, self.attributes, self.device)
            if hybrid is not None:
                return hybrid
        return build_fused_engine(model, ds, self.attributes, self.device, strict=(backend == "cuda"))

    def fit(self, *args, train_dataloaders, **kwargs) -> None:
        assert len(args) == 1
        model, = args
        self.model = model
        self.model.to(self.device)
        self.train_dataloaders = train_dataloaders
        ds = getattr(train_dataloaders, "dataset", None)
        if hasattr(ds, "to") and isinstance(train_dataloaders, BatchLoader):
            ds.to(self.device)
        self.loss_function = model.loss_function
        self.engine = self._maybe_build_engine(model, train_dataloaders)
        self.optimizer = self.engine.optimizer_view() if self.engine is not None else model.configure_optimizers()
        self.on_fit_start(self, self.model)
        n_epochs = self.attributes.num_epochs
        accum = getattr(self.attributes, "gradient_accumulation_steps", 0) or 0
        step = 0
        for epoch in range(n_epochs):
            self.current_epoch = epoch
            self.on_train_epoch_start(self, self.model)
            self.model.train()
            total = torch.zeros((), device=self.device)
            nb = 0
            t0 = time.time()
            for i, batch in enumerate(train_dataloaders):
                batch = _to_device(batch, self.device)
                self.on_train_batch_start(self, self.model, batch, i)
                if self.engine is not None:
                    loss = self.engine.step(batch)
                else:
                    if accum <= 1 or step % accum == 0:
                        self.optimizer.zero_grad(set_to_none=True)
                    loss = self.model.training_step(batch)
                    loss.backward()
                    self.optimizer.step()
                total += loss.detach()
                nb += 1
                step += 1
                self.on_train_batch_end(self, self.model, loss, batch, i)
            if self.engine is not None:
                self.engine.sync_to_model()
            epoch_loss = float(total) / max(nb, 1)
            self.model.loss_history.append(epoch_loss)
            print(f"Epoch:{epoch + 1} | Loss:{epoch_loss:.8f} | Runtime:{(time.time() - t0) / 60:.3f}mins")
            self.on_train_epoch_end(self, self.model)
        if self.engine is not None:
            self.engine.sync_to_model()
        self.on_fit_end(self, self.model)
