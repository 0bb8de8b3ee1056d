"""Real-valued models: DistMult, TransE, Shallom, Pyke.

Score functions follow reference ``dicee/models/real.py:10-132``.
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import nn

from .base import BaseKGE


class DistMult(BaseKGE):
    """``f(h, r, t) = Σ h ∘ r ∘ t`` (reference ``real.py:10-49``)."""
    bilinear = True

    def compose(self, h, r):
        return self.hidden_dropout(self.hidden_normalizer(h * r)), None


class TransE(BaseKGE):
    """``f = margin − ‖h + r − t‖₂`` with margin 4 (reference ``real.py:52-76``).

    ``pairwise_distance`` adds ``eps = 1e-6`` to the difference before the norm; the all-entity
    form here expands ``‖q' − t‖² = ‖q'‖² + ‖t‖² − 2 q'·t`` with ``q' = h + r + eps`` so that it is a
    GEMM instead of the reference's ``B × |E| × d`` broadcast (``real.py:72-76``)."""

    def __init__(self, args):
        super().__init__(args)
        self._norm = 2
        self.margin = 4
        self._eps = 1e-6

    def score(self, head_ent_emb, rel_ent_emb, tail_ent_emb):
        return self.margin - torch.nn.functional.pairwise_distance(head_ent_emb + rel_ent_emb, tail_ent_emb,
                                                                   p=self._norm)

    def k_vs_all_score(self, emb_h, emb_r, emb_E):
        q = emb_h + emb_r + self._eps
        sq = (q * q).sum(1, keepdim=True) + (emb_E * emb_E).sum(1).unsqueeze(0) - 2.0 * (q @ emb_E.t())
        return self.margin - torch.sqrt(sq.clamp_min(0.0))

    def forward_k_vs_all(self, x):
        h, r = self.get_head_relation_representation(x)
        return self.k_vs_all_score(h, r, self.entity_embeddings.weight)

    def forward_k_vs_sample(self, x, target_entity_idx):
        h, r = self.get_head_relation_representation(x)
        t = self.entity_embeddings(target_entity_idx)
        diff = (h + r + self._eps).unsqueeze(1) - t
        return self.margin - diff.norm(p=2, dim=-1)


class Shallom(BaseKGE):
    """Relation prediction from a pair of entities with a two-layer MLP (reference ``real.py:79-113``)."""

    def __init__(self, args):
        super().__init__(args)
        width = int(2 * self.embedding_dim)
        self.shallom = nn.Sequential(nn.Dropout(self.input_dropout_rate),
                                     nn.Linear(self.embedding_dim * 2, width),
                                     self.normalizer_class(width),
                                     nn.ReLU(),
                                     nn.Dropout(self.hidden_dropout_rate),
                                     nn.Linear(width, self.num_relations))

    def get_embeddings(self) -> Tuple[torch.Tensor, None]:
        return self.entity_embeddings.weight.data.detach(), None

    def forward_k_vs_all(self, x) -> torch.Tensor:
        s, o = self.entity_embeddings(x[:, 0]), self.entity_embeddings(x[:, 1])
        return self.shallom(torch.cat((s, o), 1))

    def forward_triples(self, x) -> torch.Tensor:
        # one score per row: logit of the row's own relation (the reference indexes ``[:, x[:, 1]]`` and
        # flattens a B × B matrix, real.py:108-113; the per-row gather is what a triple score means)
        scores = self.forward_k_vs_all(x[:, [0, 2]])
        return scores.gather(1, x[:, 1:2]).flatten()


class Pyke(BaseKGE):
    """``f = 1 − (‖h − r‖ + ‖r − t‖) / 2`` on triples only (reference ``real.py:116-132``)."""

    def __init__(self, args):
        super().__init__(args)
        self.dist_func = nn.PairwiseDistance(p=2)
        self.margin = 1.0

    def forward_triples(self, x: torch.Tensor):
        h, r, t = self.get_triple_representation(x)
        return self.margin - (self.dist_func(h, r) + self.dist_func(r, t)) / 2
