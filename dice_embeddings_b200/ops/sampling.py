"""Device-side random index generation (counter-based Philox kernel; reproducible from ``(seed, offset)``).

Replaces the per-item ``torch.randint`` calls inside the reference's dataset ``__getitem__`` / ``collate_fn``
(``dicee/dataset_classes.py:699-750``) when the batch is assembled on the GPU."""
from __future__ import annotations

import itertools
from typing import Optional

import torch

from . import kernels

_counter = itertools.count(1)


def uniform_int(high: int, size, device, seed: Optional[int] = None, offset: int = 0) -> torch.Tensor:
    """int64 tensor of shape ``size`` with entries uniform in ``[0, high)``.  ``seed=None`` draws a fresh stream
    from a process-wide counter mixed with torch's seed."""
    device = torch.device(device)
    if seed is None:
        seed = (torch.initial_seed() * 0x9E3779B97F4A7C15 + next(_counter)) & (2 ** 64 - 1)
    shape = (size,) if isinstance(size, int) else tuple(size)
    out = torch.empty(shape, dtype=torch.int64, device=device)
    if device.type != "cuda":
        g = torch.Generator().manual_seed(int(seed) % (2 ** 63))
        return torch.randint(0, high, shape, generator=g)
    with torch.cuda.device(device):
        kernels.uniform_int(out, high, seed, offset)
    return out
