"""Clifford-algebra models Keci / CKeci (Cl_{p,q}) and DeCaL (Cl_{p,q,r}).

Reference: ``dicee/models/clifford.py:3-560`` (Keci), ``:563-576`` (CKeci), ``:579-1092`` (DeCaL).
All the partial einsums of the reference collapse into one query vector plus a per-query
scalar (:func:`algebra.compose_clifford`).  State-dict keys (``p_coefficients.weight [1, p]``,
``q_coefficients.weight [1, q]``, ``r_coefficients.weight [1, r]``) and their zero (Keci, DeCaL) /
one (CKeci, frozen) initialisation are kept.

Two behaviours of the reference are treated as defects and not reproduced: its triple score for
``p > 0`` contracts the tail over the whole batch (``'brp, erp -> b'``, ``clifford.py:463-464``), and
for ``p ≥ 2`` / ``q ≥ 2`` it broadcasts the σ scalars to ``[n, n]`` (``:478-490``).  Here the triple
score is the same function as the all-entity score restricted to the given tail.
"""
from __future__ import annotations

import torch
from torch import nn

from . import algebra
from .base import BaseKGE


class Keci(BaseKGE):
    bilinear = True

    def __init__(self, args):
        super().__init__(args)
        self.p = self.args.get("p", 0) or 0
        self.q = self.args.get("q", 0) or 0
        r = self.embedding_dim / (self.p + self.q + 1)
        if not float(r).is_integer():
            raise AssertionError(f"r = embedding_dim / (p + q+ 1) must be a whole number\n"
                                 f"Currently {r}={self.embedding_dim} / ({self.p}+ {self.q} +1)")
        self.r = int(r)
        self.requires_grad_for_interactions = True
        if self.p > 0:
            self.p_coefficients = nn.Embedding(num_embeddings=1, embedding_dim=self.p)
            nn.init.zeros_(self.p_coefficients.weight)
        if self.q > 0:
            self.q_coefficients = nn.Embedding(num_embeddings=1, embedding_dim=self.q)
            nn.init.zeros_(self.q_coefficients.weight)

    def _coeffs(self):
        pc = self.p_coefficients.weight if self.p > 0 else None
        qc = self.q_coefficients.weight if self.q > 0 else None
        return pc, qc

    def compose(self, h, r):
        pc, qc = self._coeffs()
        return algebra.compose_clifford(h, r, self.r, self.p, self.q, 0, pc, qc)

    # helpers kept for API parity with the reference (clifford.py:115-192)
    def construct_cl_multivector(self, x: torch.Tensor, r: int, p: int, q: int):
        a0, ap, aq, _ = algebra.split_multivector(x, r, p, q, 0)
        return a0, ap, aq

    def apply_coefficients(self, hp, hq, rp, rq):
        if self.p > 0:
            hp, rp = hp * self.p_coefficients.weight, rp * self.p_coefficients.weight
        if self.q > 0:
            hq, rq = hq * self.q_coefficients.weight, rq * self.q_coefficients.weight
        return hp, hq, rp, rq

    def clifford_multiplication(self, h0, hp, hq, r0, rp, rq):
        """Full product ``h · r`` in Cl_{p,q}: returns (σ0, σp, σq, σpp, σqq, σpq)."""
        sigma_0 = h0 * r0 + torch.sum(hp * rp, dim=2) - torch.sum(hq * rq, dim=2)
        sigma_p = h0.unsqueeze(-1) * rp + r0.unsqueeze(-1) * hp
        sigma_q = h0.unsqueeze(-1) * rq + r0.unsqueeze(-1) * hq

        def anti(a, b, m):
            if m < 2:
                return a.new_zeros(a.shape[0], a.shape[1], 0)
            o = a.unsqueeze(-1) * b.unsqueeze(-2) - b.unsqueeze(-1) * a.unsqueeze(-2)
            iu = torch.triu_indices(m, m, offset=1, device=a.device)
            return o[:, :, iu[0], iu[1]]

        sigma_pp = anti(hp, rp, self.p)
        sigma_qq = anti(hq, rq, self.q)
        sigma_pq = hp.unsqueeze(-1) * rq.unsqueeze(-2) - rp.unsqueeze(-1) * hq.unsqueeze(-2)
        return sigma_0, sigma_p, sigma_q, sigma_pp, sigma_qq, sigma_pq


class CKeci(Keci):
    """Keci without learned dimension scaling: coefficients fixed to one."""

    def __init__(self, args):
        super().__init__(args)
        self.requires_grad_for_interactions = False
        if self.p > 0:
            self.p_coefficients = nn.Embedding(1, self.p)
            nn.init.ones_(self.p_coefficients.weight)
            self.p_coefficients.weight.requires_grad_(False)
        if self.q > 0:
            self.q_coefficients = nn.Embedding(1, self.q)
            nn.init.ones_(self.q_coefficients.weight)
            self.q_coefficients.weight.requires_grad_(False)


class DeCaL(BaseKGE):
    """Cl_{p,q,r}: adds a nilpotent block of ``r`` base vectors."""
    bilinear = True

    def __init__(self, args):
        super().__init__(args)
        self.entity_embeddings = nn.Embedding(self.num_entities, self.embedding_dim)
        self.relation_embeddings = nn.Embedding(self.num_relations, self.embedding_dim)
        self.p = self.args.get("p", 0) or 0
        self.q = self.args.get("q", 0) or 0
        self.r = self.args.get("r", 0) or 0
        self.re = int(self.embedding_dim / (self.r + self.p + self.q + 1))
        if self.re * (self.r + self.p + self.q + 1) != self.embedding_dim:
            raise AssertionError("embedding_dim must be divisible by (1 + p + q + r)")
        for name, m in (("p", self.p), ("q", self.q), ("r", self.r)):
            if m > 0:
                emb = nn.Embedding(num_embeddings=1, embedding_dim=m)
                nn.init.zeros_(emb.weight)
                setattr(self, f"{name}_coefficients", emb)

    def _coeffs(self):
        return (self.p_coefficients.weight if self.p > 0 else None,
                self.q_coefficients.weight if self.q > 0 else None,
                self.r_coefficients.weight if self.r > 0 else None)

    def compose(self, h, r):
        pc, qc, kc = self._coeffs()
        return algebra.compose_clifford(h, r, self.re, self.p, self.q, self.r, pc, qc, kc)

    def score(self, h, r, t):
        # the reference's triple path leaves the coefficients out (clifford.py:601-619)
        q, bias = algebra.compose_clifford(h, r, self.re, self.p, self.q, self.r)
        s = (q * t).sum(dim=1)
        return s if bias is None else s + bias
