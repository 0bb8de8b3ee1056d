"""Training callbacks (reference ``dicee/callbacks.py``)."""
from __future__ import annotations

import datetime
import os
import time

import pandas as pd

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
