"""Function-space embeddings: entities and relations parameterise small functions and a triple is
scored by an integral over their product or composition.

``LFMult`` is the registered model (reference ``dicee/models/function_space.py:295-479``); ``FMult``,
``GFMult``, ``FMult2`` and ``LFMult1`` exist in the reference but are not reachable from its model
registry (``dicee/static_funcs.py:33-54``) — they are provided here under the same names.  All of them
score triples only.
"""
from __future__ import annotations

import numpy as np
import torch
from torch import nn

from .base import BaseKGE


def _fresh_tables(model: BaseKGE, init: bool = True) -> None:
    model.entity_embeddings = nn.Embedding(model.num_entities, model.embedding_dim)
    model.relation_embeddings = nn.Embedding(model.num_relations, model.embedding_dim)
    if init:
        model.param_init(model.entity_embeddings.weight.data)
        model.param_init(model.relation_embeddings.weight.data)


class _TwoLayerFunctions(BaseKGE):
    """An embedding of size ``2k²`` is two ``k × k`` matrices: ``f(x) = W2 · tanh(W1 · x)``."""

    def _setup(self, num_sample: int):
        _fresh_tables(self)
        self.k = int(np.sqrt(self.embedding_dim // 2))
        self.num_sample = num_sample

    def _mats(self, w: torch.Tensor):
        n = len(w)
        w1, w2 = torch.hsplit(w[:, : 2 * self.k * self.k], 2)
        return w1.reshape(n, self.k, self.k), w2.reshape(n, self.k, self.k)

    def compute_func(self, weights: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        w1, w2 = self._mats(weights)
        return w2 @ torch.tanh(w1 @ x)

    def chain_func(self, weights: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        w1, w2 = self._mats(weights)
        return torch.bmm(w2, torch.tanh(torch.bmm(w1, x)))


class FMult(_TwoLayerFunctions):
    """Monte-Carlo estimate of ``∫ ⟨r(h(x)), t(x)⟩ dx`` on 50 Gaussian points (reference ``:5-47``)."""

    def __init__(self, args):
        super().__init__(args)
        self._setup(50)
        self.register_buffer("gamma", torch.randn(self.k, self.num_sample), persistent=False)

    def forward_triples(self, idx_triple: torch.Tensor) -> torch.Tensor:
        h, r, t = self.get_triple_representation(idx_triple)
        h_x = self.compute_func(h, self.gamma)
        t_x = self.compute_func(t, self.gamma)
        return (self.chain_func(r, h_x) * t_x).sum(dim=1).mean(dim=1)


class GFMult(_TwoLayerFunctions):
    """Gauss–Legendre quadrature (250 nodes) of the same integrand (reference ``:50-93``)."""

    def __init__(self, args):
        super().__init__(args)
        self._setup(250)
        roots, weights = np.polynomial.legendre.leggauss(self.num_sample)
        self.register_buffer("roots", torch.from_numpy(roots).float().repeat(self.k, 1), persistent=False)
        self.register_buffer("weights", torch.from_numpy(weights).float().reshape(1, -1), persistent=False)

    def forward_triples(self, idx_triple: torch.Tensor) -> torch.Tensor:
        h, r, t = self.get_triple_representation(idx_triple)
        h_x = self.compute_func(h, self.roots)
        t_x = self.compute_func(t, self.roots)
        return ((self.chain_func(r, h_x) * t_x).sum(dim=1) * self.weights).mean(dim=1)


class FMult2(BaseKGE):
    """Three-layer residual functions composed head→relation and integrated against the tail's
    function with the trapezoid rule on ``[-1, 1]`` (reference ``:96-213``)."""

    def __init__(self, args):
        super().__init__(args)
        self.n_layers = 3
        while int(np.sqrt((self.embedding_dim - 1) / self.n_layers)) != np.sqrt((self.embedding_dim - 1) / self.n_layers):
            self.embedding_dim += 1
        self.k = int(np.sqrt((self.embedding_dim - 1) // self.n_layers))
        self.n = 50
        self.a, self.b = -1.0, 1.0
        self.score_func = "compositional"
        self.register_buffer("discrete_points", torch.linspace(self.a, self.b, steps=self.n).repeat(self.k, 1),
                             persistent=False)
        _fresh_tables(self)

    def build_func(self, vec: torch.Tensor):
        n = len(vec)
        W = [w.reshape(n, self.k, self.k) for w in torch.hsplit(vec[:, :-1], self.n_layers)]
        return W, vec[:, -1]

    def build_chain_funcs(self, vecs):
        Ws, bs = zip(*(self.build_func(v) for v in vecs))
        tail_layers = list(Ws[-1][1:])
        acc = None
        for i in range(len(Ws) - 1):
            for w in Ws[i]:
                acc = w if acc is None else w @ acc
            acc = acc + bs[i].reshape(-1, 1, 1)
        first = Ws[-1][0] @ acc / ((len(vecs) - 1) * self.k)
        return [first] + tail_layers, bs[-1]

    def compute_func(self, W, b, x) -> torch.Tensor:
        out = W[0] @ x
        for i, w in enumerate(W[1:]):
            out = out + (torch.tanh(w @ out) if i % 2 == 0 else w @ out)
        return out + b.reshape(-1, 1, 1)

    def trapezoid(self, list_W, list_b) -> torch.Tensor:
        x = self.discrete_points
        val = self.compute_func(list_W[0], list_b[0], x)
        for W, b in zip(list_W[1:], list_b[1:]):
            val = val * self.compute_func(W, b, x)
        return torch.trapezoid(val, x=x, dim=-1).sum(dim=-1)

    def forward_triples(self, idx_triple: torch.Tensor) -> torch.Tensor:
        h, r, t = self.get_triple_representation(idx_triple)
        if self.score_func == "vtp":
            (hW, hb), (rW, rb), (tW, tb) = self.build_func(h), self.build_func(r), self.build_func(t)
            return (-self.trapezoid([tW], [tb]) * self.trapezoid([hW, rW], [hb, rb])
                    + self.trapezoid([rW], [rb]) * self.trapezoid([tW, hW], [tb, hb]))
        if self.score_func == "compositional":
            tW, tb = self.build_func(t)
            cW, cb = self.build_chain_funcs([h, r])
            return self.trapezoid([cW, tW], [cb, tb])
        if self.score_func == "full-compositional":
            cW, cb = self.build_chain_funcs([h, r, t])
            return self.trapezoid([cW], [cb])
        (hW, hb), (rW, rb), (tW, tb) = self.build_func(h), self.build_func(r), self.build_func(t)
        return self.trapezoid([hW, rW, tW], [hb, rb, tb])


class LFMult1(BaseKGE):
    """Embeddings are coefficients of ``f(x) = Σ_k a_k e^{ikx}``; the score is the vector-triple-product
    form ``⟨h, t⟩_sinc · S(r) − ⟨r, t⟩_sinc · S(h)`` with ``⟨a, b⟩_sinc = Σ_{i,j} a_i b_j sinc(i − j)`` and
    ``S(a) = Σ_i a_i sinc(i)`` (reference ``:215-292``, evaluated per triple)."""

    def __init__(self, args):
        super().__init__(args)
        _fresh_tables(self, init=False)
        d = self.embedding_dim
        idx = torch.arange(d, dtype=torch.float32)
        diff = idx.unsqueeze(1) - idx.unsqueeze(0)
        kern = torch.where(diff == 0, torch.ones_like(diff), torch.sin(diff) / torch.where(diff == 0, torch.ones_like(diff), diff))
        s = torch.where(idx == 0, torch.ones_like(idx), torch.sin(idx) / torch.where(idx == 0, torch.ones_like(idx), idx))
        self.register_buffer("_kern", kern, persistent=False)
        self.register_buffer("_sinc", s, persistent=False)

    def vtp_score(self, h, r, t):
        ht = ((h @ self._kern) * t).sum(-1)
        rt = ((r @ self._kern) * t).sum(-1)
        return ht * (r * self._sinc).sum(-1) - rt * (h * self._sinc).sum(-1)

    def tri_score(self, h, r, t):
        d = self.embedding_dim
        i = torch.arange(d, device=h.device)
        s = (i.view(-1, 1, 1) + i.view(1, -1, 1) - i.view(1, 1, -1)).float()
        w = torch.where(s == 0, torch.ones_like(s), torch.sin(s) / torch.where(s == 0, torch.ones_like(s), s))
        return torch.einsum("bi,bj,bk,ijk->b", h, r, t, w)

    def forward_triples(self, idx_triple):
        h, r, t = self.get_triple_representation(idx_triple)
        return self.vtp_score(h, r, t)


class LFMult(BaseKGE):
    """Each embedding holds ``m = d / (degree + 1)`` small functions ``tanh(w x + b)``; the score is
    ``∫₀¹ Σ_m h_m(x) r_m(x) t_m(x) dx`` by the trapezoid rule on 100 points (reference ``:295-350``).
    With ``degree = 0`` there is no bias coefficient and ``b = 0`` is used."""

    def __init__(self, args):
        super().__init__(args)
        _fresh_tables(self, init=False)
        self.degree = self.args.get("degree", 0) or 0
        self.m = int(self.embedding_dim / (1 + self.degree))
        self.register_buffer("x_values", torch.linspace(0, 1, 100), persistent=False)

    def construct_multi_coeff(self, x: torch.Tensor) -> torch.Tensor:
        """``[n, d] → [n, m, degree + 1]``: coefficient ``j`` of function ``i`` is ``x[:, j·m + i]``."""
        return torch.stack(torch.hsplit(x[:, : self.m * (self.degree + 1)], self.degree + 1), dim=1).transpose(1, 2)

    def _functions(self, coeff: torch.Tensor) -> torch.Tensor:
        w = coeff[:, :, 0]
        b = coeff[:, :, 1] if coeff.shape[-1] > 1 else torch.zeros_like(w)
        return torch.tanh(w.unsqueeze(-1) * self.x_values + b.unsqueeze(-1))  # [n, m, 100]

    def poly_NN(self, x, coefh, coefr, coeft):
        return (self._functions(coefh) * self._functions(coefr) * self._functions(coeft)).sum(dim=1)

    def forward_triples(self, idx_triple):
        h, r, t = self.get_triple_representation(idx_triple)
        ch, cr, ct = (self.construct_multi_coeff(v) for v in (h, r, t))
        return torch.trapezoid(self.poly_NN(self.x_values, ch, cr, ct), self.x_values)

    # closed-form alternatives of the reference for polynomial embeddings ------------------
    def tri_score(self, coeff_h, coeff_r, coeff_t):
        """``Σ_{i,j,k} h_i r_j t_k / (1 + (i + j + k) mod degree)`` per function."""
        D = self.degree + 1
        i, j, k = torch.meshgrid(torch.arange(D), torch.arange(D), torch.arange(D), indexing="ij")
        s = i + j + k
        terms = 1.0 / (1 + (s % self.degree if self.degree else s)).float().to(coeff_h.device)
        return torch.einsum("...i,...j,...k,jik->...", coeff_h, coeff_r, coeff_t, terms)

    def polynomial(self, coeff, x, degree):
        return coeff @ (x.unsqueeze(1) ** degree).T

    def pop(self, coeff, x, degree):
        return (coeff.unsqueeze(1) * (x.unsqueeze(2) ** degree)).sum(dim=-1)

    def comp_func(self, h, r, t):
        deg = torch.arange(self.embedding_dim, dtype=torch.float32, device=h.device)
        r_emb = self.polynomial(r, self.x_values, deg)
        t_emb = self.polynomial(t, self.x_values, deg)
        return torch.trapezoid(self.pop(h, r_emb, deg) * t_emb, self.x_values)
