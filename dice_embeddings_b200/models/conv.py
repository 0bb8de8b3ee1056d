"""Convolutional gate models: ConEx / AConEx, ConvQ / AConvQ, ConvO / AConvO.

All six stack the ``k`` blocks of the head and of the relation as a ``1 × 2k × d/k`` image,
apply one ``conv2d`` (padding 1) → BatchNorm2d → ReLU → Dropout2d → Linear → normaliser →
ReLU, and use the result either multiplicatively (``gate ∘ product``) or additively
(``gate + product``) on the algebra's product before the inner product with the tail.

References: ConEx ``dicee/models/complex.py:6-109``, AConEx ``:112-220``, ConvQ
``dicee/models/quaternion.py:217-321``, AConvQ ``:324-426``, ConvO ``dicee/models/octonion.py:158-313``,
AConvO ``:316-474``.  Sub-module names (``conv2d``, ``fc1``, ``norm_fc1``, ``bn_conv2d`` /
``bn_conv1``, ``bn_conv2``) are state-dict keys and therefore fixed.

One quirk of the additive variants is kept: on the triple path the reference sums the gate
itself (``Σ (gate + product ∘ t)``, e.g. ``quaternion.py:388-391``) whereas on the all-entity path it
adds the gate to the product before the dot product (``:421-424``).
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import nn

from . import algebra
from .base import BaseKGE, IdentityClass


class _ConvGate(BaseKGE):
    """Shared machinery; subclasses set ``_k`` (number of blocks) and the layer names."""
    bilinear = True
    _k = 2
    _gate_chunks = 2
    _fc_out_mult = 1
    _bn_conv_name = "bn_conv2d"
    _norm_fc_name = "norm_fc1"
    _recreate_embeddings = False
    fused_conv_gate = True   # on a B200: conv + batch norm + ReLU in the kernels of ops/conv_gate.py

    def __init__(self, args):
        super().__init__(args)
        if self._recreate_embeddings:
            self.entity_embeddings = nn.Embedding(self.num_entities, self.embedding_dim)
            self.relation_embeddings = nn.Embedding(self.num_relations, self.embedding_dim)
            self.param_init(self.entity_embeddings.weight.data)
            self.param_init(self.relation_embeddings.weight.data)
        C = self.num_of_output_channels
        self.conv2d = nn.Conv2d(in_channels=1, out_channels=C, kernel_size=(self.kernel_size, self.kernel_size),
                                stride=1, padding=1, bias=True)
        self.fc_num_input = self.embedding_dim * 2 * C
        out = self.embedding_dim * self._fc_out_mult
        self.fc1 = nn.Linear(self.fc_num_input, out)
        setattr(self, self._norm_fc_name, self.normalizer_class(out))
        setattr(self, self._bn_conv_name, nn.BatchNorm2d(C))
        self.feature_map_dropout = nn.Dropout2d(self.feature_map_dropout_rate)

    def residual_convolution(self, C_1: Tuple[torch.Tensor, ...], C_2: Tuple[torch.Tensor, ...]):
        """Gate vectors from the blocks of head (``C_1``) and relation (``C_2``)."""
        w = self.embedding_dim // self._k
        bn = getattr(self, self._bn_conv_name)
        x = None
        if C_1[0].is_cuda and self.fused_conv_gate and not (self.training and self.feature_map_dropout_rate):
            from ..ops import conv_gate
            image = torch.cat((*C_1, *C_2), dim=1)   # [B, 2k * w]: row i of the image is block i
            if conv_gate.supported(image, self.conv2d, bn, 2 * self._k, w):
                x = conv_gate.conv_gate_features(image, self.conv2d, bn, 2 * self._k, w)
        if x is None:
            x = torch.cat([p.reshape(-1, 1, 1, w) for p in (*C_1, *C_2)], dim=2)
            x = torch.relu(bn(self.conv2d(x)))
            x = self.feature_map_dropout(x)
            x = x.reshape(x.shape[0], -1)
        x = torch.relu(getattr(self, self._norm_fc_name)(self.fc1(x)))
        return torch.chunk(x, self._gate_chunks, dim=1)

    # subclasses: blocks of h / r (after any relation normalisation) and the algebra product
    def _blocks(self, h, r):
        return torch.hsplit(h, self._k), torch.hsplit(r, self._k)

    def _product(self, hb, rb):
        raise NotImplementedError


class _Multiplicative(_ConvGate):
    def compose(self, h, r):
        hb, rb = self._blocks(h, r)
        gate = torch.cat(self.residual_convolution(hb, rb), dim=1)
        return gate * torch.cat(self._product(hb, rb), dim=1), None


class _Additive(_ConvGate):
    def compose(self, h, r):
        hb, rb = self._blocks(h, r)
        gate = torch.cat(self.residual_convolution(hb, rb), dim=1)
        return gate + torch.cat(self._product(hb, rb), dim=1), None

    def score(self, h, r, t):
        hb, rb = self._blocks(h, r)
        gate = torch.cat(self.residual_convolution(hb, rb), dim=1)
        prod = torch.cat(self._product(hb, rb), dim=1)
        return gate.sum(dim=1) + (prod * t).sum(dim=1)


# ------------------------------------------------------------------------------ complex
class ConEx(_ConvGate):
    """``q = [a h_re r_re − b h_im r_im | a h_re r_im + b h_im r_re]`` with gates ``(a, b)``."""
    _k = 2
    _gate_chunks = 2

    def compose(self, h, r):
        (h_re, h_im), (r_re, r_im) = self._blocks(h, r)
        a, b = self.residual_convolution((h_re, h_im), (r_re, r_im))
        return torch.cat((a * h_re * r_re - b * h_im * r_im, a * h_re * r_im + b * h_im * r_re), dim=1), None


class AConEx(_ConvGate):
    """Additive ConEx with four gates ``(a, b, c, d)`` of width ``d/2``."""
    _k = 2
    _gate_chunks = 4
    _fc_out_mult = 2
    _normalize_sampled_tails = True

    def _terms(self, h, r):
        (h_re, h_im), (r_re, r_im) = self._blocks(h, r)
        a, b, c, d = self.residual_convolution((h_re, h_im), (r_re, r_im))
        return (a, b, c, d), (h_re * r_re, h_re * r_im, h_im * r_re, h_im * r_im)

    def compose(self, h, r):
        (a, b, c, d), (rr, ri, ir, ii) = self._terms(h, r)
        return torch.cat(((a + rr) - (d + ii), (b + ri) + (c + ir)), dim=1), None

    def score(self, h, r, t):
        (a, b, c, d), (rr, ri, ir, ii) = self._terms(h, r)
        t_re, t_im = torch.hsplit(t, 2)
        return ((a + rr * t_re).sum(1) + (b + ri * t_im).sum(1) + (c + ir * t_im).sum(1)
                - (d + ii * t_re).sum(1))


# ------------------------------------------------------------------------------ quaternion
class _QuaternionConv:
    _k = 4
    _gate_chunks = 4
    _bn_conv_name = "bn_conv1"
    _norm_fc_name = "bn_conv2"
    _recreate_embeddings = True

    def _product(self, hb, rb):
        return algebra.quaternion_mul(Q_1=hb, Q_2=rb)


class ConvQ(_QuaternionConv, _Multiplicative):
    pass


class AConvQ(_QuaternionConv, _Additive):
    pass


# ------------------------------------------------------------------------------ octonion
class _OctonionConv:
    _k = 8
    _gate_chunks = 8

    def _blocks(self, h, r):
        hb, rb = torch.hsplit(h, 8), torch.hsplit(r, 8)
        if isinstance(self.normalize_relation_embeddings, IdentityClass):
            rb = algebra.octonion_normalizer(rb)
        return hb, rb

    def _product(self, hb, rb):
        return algebra.octonion_mul(O_1=hb, O_2=rb)

    @staticmethod
    def octonion_normalizer(*parts):
        return algebra.octonion_normalizer(parts)


class ConvO(_OctonionConv, _Multiplicative):
    pass


class AConvO(_OctonionConv, _Additive):
    pass
