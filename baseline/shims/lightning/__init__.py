"""Minimal stand-in for the ``lightning`` package so the unmodified reference can be imported on a machine
where Lightning is not installed.  Only what the reference touches at import time and on its non-Lightning
trainers exists: ``LightningModule`` (a ``torch.nn.Module`` with a no-op ``log`` and a ``device`` property),
``pytorch.callbacks.Callback`` / ``ModelSummary`` and a ``Trainer`` that refuses to run."""
import torch

from . import pytorch  # noqa: F401


class LightningModule(torch.nn.Module):
    def log(self, *args, **kwargs):
        return None

    @property
    def device(self):
        try:
            return next(self.parameters()).device
        except StopIteration:
            return torch.device("cpu")


class Trainer:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("pytorch-lightning is not installed on this machine; use --trainer torchCPUTrainer/torchDDP")
