"""Ensemble link-prediction evaluation: per-query min–max normalised scores of several models are averaged
(optionally weighted) before filtered tail ranking (reference ``dicee/evaluation/ensemble.py:20-130``)."""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from .ranking import filter_coordinates, filtered_rank_from_scores, metrics_from_ranks


@torch.no_grad()
def evaluate_ensemble_link_prediction_performance(models: List, triples, er_vocab, weights: Optional[List[float]] = None,
                                                  batch_size: int = 512, weighted_averaging: bool = True,
                                                  normalize_scores: bool = True) -> Dict[str, float]:
    n_models = len(models)
    assert n_models > 0
    if weighted_averaging:
        assert weights is not None and len(weights) == n_models, "Number of weights must match number of models."
    for m in models:
        m.eval()
    dev = getattr(models[0], "device", torch.device("cpu"))
    w = torch.tensor(weights, dtype=torch.float32, device=dev).view(-1, 1, 1) if weighted_averaging else None
    triples = torch.as_tensor(np.asarray(triples)).long()
    ranks = []
    for i in range(0, triples.shape[0], batch_size):
        b = triples[i:i + batch_size].to(dev)
        preds = []
        for m in models:
            p = m(b[:, :2])
            if normalize_scores:
                lo, hi = p.min(dim=1, keepdim=True)[0], p.max(dim=1, keepdim=True)[0]
                p = (p - lo) / (hi - lo + 1e-8)
            preds.append(p)
        stack = torch.stack(preds, dim=0)
        avg = (stack * w).sum(0) if weighted_averaging else stack.mean(0)
        fr, fc = filter_coordinates(er_vocab, b[:, 0], b[:, 1])
        ranks.append(filtered_rank_from_scores(avg, b[:, 2], fr, fc).cpu())
    return metrics_from_ranks(torch.cat(ranks), divisor=triples.shape[0])
