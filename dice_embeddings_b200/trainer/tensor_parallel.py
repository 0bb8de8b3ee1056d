"""Embedding-dimension parallel trainer (``--trainer TP``): an :class:`EnsembleKGE` of one replica per device whose
averaged logits are trained with a single BCE (reference ``dicee/trainer/model_parallelism.py:119-201``).

``auto_batch_finding`` grows the batch size while the *measured* peak memory of a probe step stays below a fixed
share of the device; it never runs a device out of memory on purpose (the reference probes until
``torch.OutOfMemoryError``, ``:28-116``)."""
from __future__ import annotations

import time

import torch

from ..models.ensemble import EnsembleKGE
from .base import AbstractTrainer, BatchLoader


def forward_backward_update_loss(batch, ensemble: EnsembleKGE) -> float:
    d0 = ensemble.devices[0]
    if len(batch) == 2:
        x, y = batch
        yhat = ensemble(x)
    else:
        x, y_idx, y = batch
        yhat = ensemble((x, y_idx))
    loss = torch.nn.functional.binary_cross_entropy_with_logits(yhat, y.to(d0))
    loss.backward()
    ensemble.step()
    return float(loss.detach())


def find_good_batch_size(loader: BatchLoader, ensemble: EnsembleKGE, memory_share: float = 0.6) -> int:
    """Largest power-of-two multiple of the configured batch size whose probe step keeps the peak memory of the
    first device under ``memory_share`` of its capacity (bounded: at most 12 doublings, never beyond the dataset)."""
    n = len(loader.dataset)
    bs = loader.batch_size
    d0 = ensemble.devices[0]
    if bs >= n or d0.type != "cuda":
        return min(bs, n)
    total = torch.cuda.get_device_properties(d0).total_memory
    best = bs
    for _ in range(12):
        torch.cuda.reset_peak_memory_stats(d0)
        batch = loader.dataset.make_batch(torch.arange(min(bs, n), device=loader.dataset.device))
        forward_backward_update_loss(batch, ensemble)
        peak = torch.cuda.max_memory_allocated(d0)
        if peak > memory_share * total:
            break
        best = bs
        # predicted peak of the doubled batch must also fit
        if bs * 2 > n or 2 * peak > memory_share * total:
            break
        bs *= 2
    return min(best, n)


class TensorParallel(AbstractTrainer):
    def __init__(self, args, callbacks=None, devices=None):
        super().__init__(args, callbacks)
        if devices is None:
            n = torch.cuda.device_count()
            devices = [torch.device(f"cuda:{i}") for i in range(n)] if n else [torch.device("cpu")]
        self.devices = [torch.device(d) for d in devices]

    def fit(self, *args, train_dataloaders, **kwargs):
        ensemble, = args
        assert isinstance(ensemble, EnsembleKGE), type(ensemble)
        self.model = ensemble
        loader = train_dataloaders
        if isinstance(loader, BatchLoader):
            loader.dataset.to(ensemble.devices[0])
        if getattr(self.attributes, "auto_batch_finding", False) and isinstance(loader, BatchLoader):
            loader.batch_size = find_good_batch_size(loader, ensemble)
            print(f"Selected batch size: {loader.batch_size}")
        self.on_fit_start(self, ensemble)
        for epoch in range(self.attributes.num_epochs):
            self.current_epoch = epoch
            ensemble.train()
            tot, nb, t0 = 0.0, 0, time.time()
            for i, batch in enumerate(loader):
                tot += forward_backward_update_loss(batch, ensemble)
                nb += 1
            ensemble.loss_history.append(tot / max(nb, 1))
            print(f"Epoch:{epoch + 1} | Loss:{tot / max(nb, 1):.8f} | Runtime:{(time.time() - t0) / 60:.3f}mins")
            self.on_train_epoch_end(self, ensemble)
        self.on_fit_end(self, ensemble)
        return ensemble
