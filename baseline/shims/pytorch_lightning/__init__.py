"""Stand-in for ``pytorch_lightning``: ``seed_everything`` and ``utilities.rank_zero_only`` only."""
import os
import random

import numpy as np
import torch

from . import utilities  # noqa: F401


def seed_everything(seed=None, workers=False):
    seed = int(seed or 0)
    os.environ["PL_GLOBAL_SEED"] = str(seed)
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    return seed
