"""Query composition ``q = compose(h, r)`` for the multiplicative model families.

Every bilinear model of the zoo scores a triple as ``⟨compose(h, r), t⟩ (+ bias(h, r))``:
the head/relation interaction can be folded into one *query vector* so that scoring
against all entities is a single GEMM ``Q · Eᵀ`` instead of the 4 / 8 / 7 partial products
of the reference (``dicee/models/complex.py:254-264``, ``quaternion.py:152-156``,
``octonion.py:136-144``, ``clifford.py:269-287``).  Vectors use the reference's *block
layout*: ``[part0 | part1 | …]``, each block ``d/k`` wide (``torch.hsplit``).

These PyTorch functions are the framework's generic path and the numerical oracle for the
fused CUDA lookup+compose kernel.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

# ---------------------------------------------------------------------------------- real / complex


def compose_distmult(h: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    return h * r


def compose_complex(h: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    """``Re⟨h, r, conj t⟩`` as ``q·t`` with ``q = [h_re r_re − h_im r_im | h_re r_im + h_im r_re]``."""
    h_re, h_im = torch.hsplit(h, 2)
    r_re, r_im = torch.hsplit(r, 2)
    return torch.cat((h_re * r_re - h_im * r_im, h_re * r_im + h_im * r_re), dim=1)


# ---------------------------------------------------------------------------------- quaternion


def quaternion_mul(*, Q_1, Q_2):
    """Hamilton product of two quaternion tuples (reference ``models/static_funcs.py:4-18``)."""
    a_h, b_h, c_h, d_h = Q_1
    a_r, b_r, c_r, d_r = Q_2
    r_val = a_h * a_r - b_h * b_r - c_h * c_r - d_h * d_r
    i_val = a_h * b_r + b_h * a_r + c_h * d_r - d_h * c_r
    j_val = a_h * c_r - b_h * d_r + c_h * a_r + d_h * b_r
    k_val = a_h * d_r + b_h * c_r - c_h * b_r + d_h * a_r
    return r_val, i_val, j_val, k_val


def quaternion_normalizer(x: torch.Tensor) -> torch.Tensor:
    """L2-normalise *consecutive* groups of four components.

    The reference groups consecutive elements here while the Hamilton product works on block
    quarters (``quaternion.py:97-100`` vs ``:109-115``); the mismatch is kept because trained
    checkpoints depend on it."""
    shape = x.shape
    x = x.reshape(*shape[:-1], -1, 4)
    x = torch.nn.functional.normalize(x, p=2, dim=-1)
    return x.reshape(*shape)


def compose_quaternion(h: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    return torch.cat(quaternion_mul(Q_1=torch.hsplit(h, 4), Q_2=torch.hsplit(r, 4)), dim=1)


# ---------------------------------------------------------------------------------- octonion


def octonion_mul(*, O_1, O_2):
    """Octonion product (Cayley–Dickson sign table of reference ``octonion.py:5-17``)."""
    x0, x1, x2, x3, x4, x5, x6, x7 = O_1
    y0, y1, y2, y3, y4, y5, y6, y7 = O_2
    x = x0 * y0 - x1 * y1 - x2 * y2 - x3 * y3 - x4 * y4 - x5 * y5 - x6 * y6 - x7 * y7
    e1 = x0 * y1 + x1 * y0 + x2 * y3 - x3 * y2 + x4 * y5 - x5 * y4 - x6 * y7 + x7 * y6
    e2 = x0 * y2 - x1 * y3 + x2 * y0 + x3 * y1 + x4 * y6 + x5 * y7 - x6 * y4 - x7 * y5
    e3 = x0 * y3 + x1 * y2 - x2 * y1 + x3 * y0 + x4 * y7 - x5 * y6 + x6 * y5 - x7 * y4
    e4 = x0 * y4 - x1 * y5 - x2 * y6 - x3 * y7 + x4 * y0 + x5 * y1 + x6 * y2 + x7 * y3
    e5 = x0 * y5 + x1 * y4 - x2 * y7 + x3 * y6 - x4 * y1 + x5 * y0 - x6 * y3 + x7 * y2
    e6 = x0 * y6 + x1 * y7 + x2 * y4 - x3 * y5 - x4 * y2 + x5 * y3 + x6 * y0 - x7 * y1
    e7 = x0 * y7 - x1 * y6 + x2 * y5 + x3 * y4 - x4 * y3 - x5 * y2 + x6 * y1 + x7 * y0
    return x, e1, e2, e3, e4, e5, e6, e7


def octonion_normalizer(parts):
    """Divide every block by the per-position norm over the 8 blocks (reference ``octonion.py:53-66``)."""
    den = torch.sqrt(sum(p ** 2 for p in parts))
    return tuple(p / den for p in parts)


def compose_octonion(h: torch.Tensor, r: torch.Tensor, normalize_relation: bool = True) -> torch.Tensor:
    rp = torch.hsplit(r, 8)
    if normalize_relation:
        rp = octonion_normalizer(rp)
    return torch.cat(octonion_mul(O_1=torch.hsplit(h, 8), O_2=rp), dim=1)


# ---------------------------------------------------------------------------------- Clifford Cl(p, q[, r])


def split_multivector(x: torch.Tensor, r: int, p: int, q: int, k: int = 0):
    """Row layout of Keci / DeCaL vectors: ``[scalar(r) | p-part(r·p) | q-part(r·q) | nilpotent(r·k)]``
    with the vector parts viewed as ``[n, r, p]`` etc. (reference ``clifford.py:179-192, 1007-1025``)."""
    n = x.shape[0]
    a0 = x[:, :r]
    ap = x[:, r:r + r * p].reshape(n, r, p)
    aq = x[:, r + r * p:r + r * p + r * q].reshape(n, r, q)
    ak = x[:, r + r * p + r * q:r + r * (p + q + k)].reshape(n, r, k)
    return a0, ap, aq, ak


def _pair_antisym_sum(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``Σ_r Σ_{i<j} (a_i b_j − a_j b_i)`` for ``a, b`` of shape ``[n, r, m]`` → ``[n]``."""
    m = a.shape[-1]
    if m < 2:
        return a.new_zeros(a.shape[0])
    outer = a.unsqueeze(-1) * b.unsqueeze(-2) - b.unsqueeze(-1) * a.unsqueeze(-2)  # [n, r, m, m]: a_i b_j − a_j b_i
    iu = torch.triu_indices(m, m, offset=1, device=a.device)
    return outer[:, :, iu[0], iu[1]].sum(dim=(1, 2))


def _cross_sum(ha, hb, ra, rb) -> torch.Tensor:
    """``Σ_r Σ_{i,j} (ha_i rb_j − hb_j ra_i)`` → ``[n]`` (the σ_pq / σ_pr / σ_qr scalars)."""
    return (ha.sum(-1) * rb.sum(-1) - hb.sum(-1) * ra.sum(-1)).sum(dim=1)


def compose_clifford(h: torch.Tensor, r: torch.Tensor, re: int, p: int, q: int, k: int = 0,
                     p_coeff: Optional[torch.Tensor] = None, q_coeff: Optional[torch.Tensor] = None,
                     k_coeff: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Query vector and tail-independent bias of Keci (``k = 0``) and DeCaL.

    ``q = [h0 r0 + Σ_p hp rp − Σ_q hq rq | h0 rp + hp r0 | h0 rq + hq r0 | h0 rk + hk r0]`` and
    ``bias = σ_pp + σ_qq (+ σ_rr) + cross terms``, where each σ only exists for grade ≥ 2 and the
    cross terms need both grades ≥ 2 (reference ``clifford.py:258-305`` and ``:808-899``)."""
    n = h.shape[0]
    h0, hp, hq, hk = split_multivector(h, re, p, q, k)
    r0, rp, rq, rk = split_multivector(r, re, p, q, k)
    if p > 0 and p_coeff is not None:
        hp, rp = hp * p_coeff, rp * p_coeff
    if q > 0 and q_coeff is not None:
        hq, rq = hq * q_coeff, rq * q_coeff
    if k > 0 and k_coeff is not None:
        hk, rk = hk * k_coeff, rk * k_coeff
    s0 = h0 * r0
    parts = []
    if p > 0:
        s0 = s0 + (hp * rp).sum(-1)
        parts.append((h0.unsqueeze(-1) * rp + hp * r0.unsqueeze(-1)).reshape(n, re * p))
    if q > 0:
        s0 = s0 - (hq * rq).sum(-1)
        parts.append((h0.unsqueeze(-1) * rq + hq * r0.unsqueeze(-1)).reshape(n, re * q))
    if k > 0:
        parts.append((h0.unsqueeze(-1) * rk + hk * r0.unsqueeze(-1)).reshape(n, re * k))
    qv = torch.cat([s0] + parts, dim=1)
    bias = None
    terms = []
    if p >= 2:
        terms.append(_pair_antisym_sum(hp, rp))
    if q >= 2:
        terms.append(_pair_antisym_sum(hq, rq))
    if k >= 2:
        terms.append(_pair_antisym_sum(hk, rk))
    if p >= 2 and q >= 2:
        terms.append(_cross_sum(hp, hq, rp, rq))
    if p >= 2 and k >= 2:
        terms.append(_cross_sum(hp, hk, rp, rk))
    if q >= 2 and k >= 2:
        terms.append(_cross_sum(hq, hk, rq, rk))
    if terms:
        bias = sum(terms)
    return qv, bias


# ---------------------------------------------------------------------------------- dual quaternion (DualE)


def duale_normalize_relation(parts):
    """Unit-normalise the real quaternion and orthogonalise the dual part against it
    (reference ``dualE.py:31-44``)."""
    r1, r2, r3, r4, r5, r6, r7, r8 = parts
    den0 = r1 ** 2 + r2 ** 2 + r3 ** 2 + r4 ** 2
    den1 = torch.sqrt(den0)
    cross = r5 * r1 + r6 * r2 + r7 * r3 + r8 * r4
    r5 = r5 - cross / den0 * r1
    r6 = r6 - cross / den0 * r2
    r7 = r7 - cross / den0 * r3
    r8 = r8 - cross / den0 * r4
    return r1 / den1, r2 / den1, r3 / den1, r4 / den1, r5, r6, r7, r8


def compose_duale(h: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    """Dual-quaternion product ``h ⊗ r̂`` in 8 blocks (reference ``dualE.py:16-28``); the model's
    score is the *negative* inner product with the tail."""
    a0, a1, a2, a3, b0, b1, b2, b3 = torch.hsplit(h, 8)
    c0, c1, c2, c3, d0, d1, d2, d3 = duale_normalize_relation(torch.hsplit(r, 8))
    h0 = a0 * c0 - a1 * c1 - a2 * c2 - a3 * c3
    g0 = a0 * d0 + b0 * c0 - a1 * d1 - b1 * c1 - a2 * d2 - b2 * c2 - a3 * d3 - b3 * c3
    h1 = a0 * c1 + a1 * c0 + a2 * c3 - a3 * c2
    g1 = a0 * d1 + b0 * c1 + a1 * d0 + b1 * c0 + a2 * d3 + b2 * c3 - a3 * d2 - b3 * c2
    h2 = a0 * c2 - a1 * c3 + a2 * c0 + a3 * c1
    g2 = a0 * d2 + b0 * c2 - a1 * d3 - b1 * c3 + a2 * d0 + b2 * c0 + a3 * d1 + b3 * c1
    h3 = a0 * c3 + a1 * c2 - a2 * c1 + a3 * c0
    g3 = a0 * d3 + b0 * c3 + a1 * d2 + b1 * c2 - a2 * d1 - b2 * c1 + a3 * d0 + b3 * c0
    return torch.cat((h0, h1, h2, h3, g0, g1, g2, g3), dim=1)
