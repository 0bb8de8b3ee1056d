"""Complex, quaternion, octonion and dual-quaternion multiplicative models.

* ComplEx — reference ``dicee/models/complex.py:223-287``
* QMult — ``dicee/models/quaternion.py:24-214``
* OMult — ``dicee/models/octonion.py:47-155``
* DualE — ``dicee/models/dualE.py:5-199``

Each is expressed through one query composition (see :mod:`.algebra`).
"""
from __future__ import annotations

import torch
from torch import nn

from . import algebra
from .base import BaseKGE, IdentityClass


class ComplEx(BaseKGE):
    bilinear = True

    def compose(self, h, r):
        return algebra.compose_complex(h, r), None


class QMult(BaseKGE):
    bilinear = True

    def __init__(self, args):
        super().__init__(args)
        self.explicit = True

    quaternion_normalizer = staticmethod(algebra.quaternion_normalizer)

    def compose(self, h, r):
        if isinstance(self.normalize_relation_embeddings, IdentityClass):
            r = algebra.quaternion_normalizer(r)
        return algebra.compose_quaternion(h, r), None


class OMult(BaseKGE):
    bilinear = True

    @staticmethod
    def octonion_normalizer(*parts):
        return algebra.octonion_normalizer(parts)

    def compose(self, h, r):
        norm = isinstance(self.normalize_relation_embeddings, IdentityClass)
        return algebra.compose_octonion(h, r, normalize_relation=norm), None

    def forward_k_vs_sample(self, *args, **kwargs):  # the reference has none for OMult
        raise ValueError(f"MODEL:{self.name} does not have forward_k_vs_sample function")


class DualE(BaseKGE):
    """Dual-quaternion embeddings; the score is the negative inner product."""
    bilinear = True

    def __init__(self, args):
        super().__init__(args)
        # the reference re-creates both tables with the default N(0, 1) init (dualE.py:10-11)
        self.entity_embeddings = nn.Embedding(self.num_entities, self.embedding_dim)
        self.relation_embeddings = nn.Embedding(self.num_relations, self.embedding_dim)
        self.num_ent = self.num_entities

    def compose(self, h, r):
        return -algebra.compose_duale(h, r), None

    def forward_k_vs_sample(self, *args, **kwargs):
        raise ValueError(f"MODEL:{self.name} does not have forward_k_vs_sample function")
