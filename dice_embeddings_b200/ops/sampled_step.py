"""Fused single-GPU training step for the sampled-candidate scoring techniques (NegSample, 1vsSample, KvsSample).

One step is the launch sequence

1. ``neg_sample``        (NegSample only) corrupted triples + labels from the counter-based device generator
2. ``lookup_compose``    gather ``E[h]``, ``R[r]`` and compose the query vectors in fp32
3. ``candidate_bce``     score each query against its own candidates, BCE-with-logits, ``dq`` and candidate-row grads
4. ``compose_backward``  chain rule of the composition into ``dE`` / ``dR``
5. ``optimizer_step`` ×k and ``finish_step``

replayed from a CUDA graph.  The reference runs the same step as ``forward_triples`` / ``forward_k_vs_sample`` +
``BCEWithLogitsLoss`` + autograd + ``torch.optim`` (``dicee/models/base_model.py:25-46, 331-344``), with the
negatives drawn on the host (``dicee/dataset_classes.py:699-750``).
"""
from __future__ import annotations

import os
from types import SimpleNamespace
from typing import Optional

import torch

from ..models.base import IdentityClass
from . import kernels as K
from .fused_step import _EngineOptimizer

SUPPORTED_SCORING = ("NegSample", "1vsSample", "KvsSample")
_DIM_MULTIPLE = {"DistMult": 4, "ComplEx": 8, "QMult": 16, "OMult": 32, "Keci": 8, "CKeci": 8, "TransE": 4}


def sampled_model_code(model) -> Optional[int]:
    name = type(model).__name__
    if name not in K.MODEL_CODE:
        return None
    if name in ("Keci", "CKeci") and not (model.p == 0 and model.q == 1):
        return None
    if model.input_dropout_rate or not isinstance(model.normalize_head_entity_embeddings, IdentityClass):
        return None
    d = model.embedding_dim
    if d % _DIM_MULTIPLE[name] or d > 512 or getattr(model, "byte_pair_encoding", False):
        return None
    if model.optimizer_name not in K.OPT_CODE:
        return None
    return K.MODEL_CODE[name]


def build_sampled_engine(model, dataset, args, device, strict: bool = False):
    reason = None
    st = getattr(args, "scoring_technique", None)
    if sampled_model_code(model) is None:
        reason = f"model {type(model).__name__} (dim {model.embedding_dim}, optim {model.optimizer_name}) is not covered"
    elif st not in SUPPORTED_SCORING:
        reason = f"scoring technique {st} is not covered"
    elif torch.cuda.get_device_capability(device)[0] != 10:
        reason = "device is not sm_100"
    if reason is not None:
        if strict:
            raise RuntimeError("kernel_backend=cuda requested but " + reason)
        return None
    if st == "NegSample" and hasattr(dataset, "defer_sampling"):
        dataset.defer_sampling = True   # the engine draws the corruptions itself, on the device
    return FusedSampledEngine(model, st, lr=args.lr, weight_decay=getattr(args, "weight_decay", 0.0) or 0.0,
                              device=device, neg_ratio=getattr(args, "neg_ratio", 0) or 0,
                              label_smoothing=getattr(args, "label_smoothing_rate", 0.0) or 0.0,
                              seed=getattr(args, "random_seed", 0) or 0)


class FusedSampledEngine:
    def __init__(self, model, scoring_technique: str, lr: float, weight_decay: float = 0.0, device=None,
                 neg_ratio: int = 0, label_smoothing: float = 0.0, seed: int = 0, use_graph: bool = True):
        self.model = model
        self.device = dev = torch.device(device or model.device)
        self.code = sampled_model_code(model)
        assert self.code is not None
        self.st = scoring_technique
        self.D, self.NE = model.embedding_dim, model.num_entities
        self.lr, self.weight_decay = float(lr), float(weight_decay)
        self.opt_kind = K.OPT_CODE[model.optimizer_name]
        self.betas = (0.9, 0.9999) if self.opt_kind == 3 else (0.9, 0.999)
        self.eps = 1e-6 if self.opt_kind == 3 else 1e-8
        self.use_graph = use_graph and os.environ.get("DICE_B200_NO_GRAPH") != "1"
        self.normalize = type(model).__name__ in ("QMult", "OMult")
        self.kind = 1 if self.code == 5 else 0
        self.margin = float(getattr(model, "margin", 0.0)) if self.kind else 0.0
        self.dist_eps = float(getattr(model, "_eps", 0.0)) if self.kind else 0.0
        self.neg_ratio, self.label_smoothing, self.seed = int(neg_ratio), float(label_smoothing), int(seed)

        self.E = model.entity_embeddings.weight.data
        self.R = model.relation_embeddings.weight.data
        assert self.E.is_cuda and self.E.is_contiguous() and self.E.dtype == torch.float32
        self.coeff, self.coeff_trainable = None, False
        if self.code == 4:
            self.coeff = model.q_coefficients.weight.data
            self.coeff_trainable = bool(model.q_coefficients.weight.requires_grad)
        self.gE, self.gR = torch.zeros_like(self.E), torch.zeros_like(self.R)
        self.mE, self.vE = torch.zeros_like(self.E), torch.zeros_like(self.E)
        self.mR, self.vR = torch.zeros_like(self.R), torch.zeros_like(self.R)
        if self.coeff is not None:
            self.gC, self.mC, self.vC = (torch.zeros_like(self.coeff) for _ in range(3))
        self.step_count = torch.zeros(1, dtype=torch.int64, device=dev)
        self.loss_acc = torch.zeros(1, dtype=torch.float64, device=dev)
        self.loss_out = torch.zeros(1, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ent_tab = K.pointer_table([self.E], dev)
        self.gent_tab = K.pointer_table([self.gE], dev)
        self._bufs = {}
        self._graphs = {}

    # ------------------------------------------------------------------ buffers
    def _buffers(self, key):
        """``key = (queries N, candidates C, positives B or 0)``."""
        if key not in self._bufs:
            N, C, B = key
            dev = self.device
            b = SimpleNamespace()
            b.h, b.r = (torch.zeros(N, dtype=torch.int64, device=dev) for _ in range(2))
            b.cand = torch.zeros(N, C, dtype=torch.int64, device=dev)
            b.labels = torch.zeros(N, C, dtype=torch.float32, device=dev)
            b.q = torch.zeros(N, self.D, dtype=torch.float32, device=dev)
            b.dq = torch.zeros(N, self.D, dtype=torch.float32, device=dev)
            b.pos = torch.zeros(max(B, 1), 3, dtype=torch.int64, device=dev)
            self._bufs[key] = b
        return self._bufs[key]

    def _launch_all(self, b, key) -> None:
        N, C, B = key
        if B:  # draw the corruptions on the device
            K.neg_sample(b.pos, self.neg_ratio, self.NE, self.seed, 0, b.labels, hrt=(b.h, b.r, b.cand),
                         label_pos=1.0 - self.label_smoothing, label_neg=self.label_smoothing, step=self.step_count)
        scale = 1.0 / float(N * C)
        K.lookup_compose(self.code, self.normalize, b.h, b.r, self.ent_tab, 1, self.NE, self.R, self.coeff, None, 0,
                         0, b.q, N, self.D, self.status)
        K.candidate_bce(b.q, b.cand, C, 1, C, b.labels, self.ent_tab, 1, self.gent_tab, b.dq, None, self.loss_acc,
                        scale, self.kind, self.margin, self.dist_eps)
        K.compose_backward(self.code, self.normalize, b.h, b.r, self.ent_tab, 1, self.R, self.coeff, b.dq,
                           self.gent_tab, self.gR, self.gC if self.coeff_trainable else None, N, self.D)
        b1, b2 = self.betas
        K.optimizer_step(self.opt_kind, self.E, self.gE, self.mE, self.vE, None, self.step_count, self.lr, b1, b2,
                         self.eps, self.weight_decay)
        K.optimizer_step(self.opt_kind, self.R, self.gR, self.mR, self.vR, None, self.step_count, self.lr, b1, b2,
                         self.eps, self.weight_decay)
        if self.coeff_trainable:
            K.optimizer_step(self.opt_kind, self.coeff, self.gC, self.mC, self.vC, None, self.step_count, self.lr,
                             b1, b2, self.eps, self.weight_decay)
        K.finish_step(self.loss_acc, self.loss_out, 1.0, self.step_count)

    def launches_per_step(self, with_sampling: bool = True) -> int:
        return 6 + (1 if with_sampling and self.st == "NegSample" else 0) + (1 if self.coeff_trainable else 0)

    def _tensors(self):
        t = [self.E, self.R, self.mE, self.vE, self.mR, self.vR, self.gE, self.gR, self.step_count, self.loss_acc]
        if self.coeff is not None:
            t += [self.coeff, self.gC, self.mC, self.vC]
        return t

    def _run(self, b, key) -> None:
        gkey = (key, self.lr)
        if self.use_graph and gkey not in self._graphs and len({k[1] for k in self._graphs}) >= 3:
            self.use_graph = False
            self._graphs.clear()
        if not self.use_graph:
            self._launch_all(b, key)
            return
        if gkey not in self._graphs:
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            state = [(x, x.clone()) for x in self._tensors()]
            with torch.cuda.stream(s):
                self._launch_all(b, key)
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            K.check_status(self.status, "during sampled-step warm-up")
            for x, c in state:
                x.copy_(c)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch_all(b, key)
            self._graphs[gkey] = g
        self._graphs[gkey].replay()

    # ------------------------------------------------------------------ public
    def step(self, batch) -> torch.Tensor:
        """Accepted batches (device tensors):

        * NegSample: ``(x [N, 3], labels [N])`` as built by the dataset, or ``(positives [B, 3],)`` to have the
          corruptions drawn by the device generator;
        * 1vsSample / KvsSample: ``(x [B, 2], candidate ids [B, C], labels [B, C])``.
        """
        if self.st == "NegSample":
            if len(batch) == 1 or batch[1] is None:
                pos = batch[0]
                B = pos.shape[0]
                key = (B * (1 + self.neg_ratio), 1, B)
                b = self._buffers(key)
                b.pos.copy_(pos)
            else:
                x, y = batch[0], batch[1]
                key = (x.shape[0], 1, 0)
                b = self._buffers(key)
                b.h.copy_(x[:, 0])
                b.r.copy_(x[:, 1])
                b.cand.copy_(x[:, 2:3])
                b.labels.copy_(y.reshape(-1, 1))
        else:
            x, idx, y = batch[0], batch[1], batch[2]
            key = (x.shape[0], idx.shape[1], 0)
            b = self._buffers(key)
            b.h.copy_(x[:, 0])
            b.r.copy_(x[:, 1])
            b.cand.copy_(idx)
            b.labels.copy_(y)
        self._run(b, key)
        return self.loss_out[0]

    def sync_to_model(self) -> None:
        K.check_status(self.status, "in sampled training step")

    def optimizer_view(self):
        return _EngineOptimizer(self)
