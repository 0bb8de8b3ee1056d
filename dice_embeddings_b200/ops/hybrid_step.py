"""Tensor-core scoring for every model whose score is ``compose(h, r) · t`` (+ a per-query scalar), or a distance.

:mod:`fused_step` covers the models whose composition is one of the algebra products the lookup kernel knows.  The
rest of the bilinear zoo produces its query vector with ordinary PyTorch modules: the convolutional gates of ConEx /
AConEx / ConvQ / AConvQ / ConvO / AConvO, DualE's dual-quaternion product, and any covered model once input dropout
or a normaliser sits between the embedding and the product.  For those the step is split:

* **autograd side** (PyTorch): gather ``E[h]``, ``R[r]``, dropout / normalisers / gates / product → ``Q [B, d]``;
* **kernel side** (:class:`FusedScoring`, one ``autograd.Function``): ``Q`` is scored against the whole entity table
  by the two tcgen05 launches of :func:`~dice_embeddings_b200.ops.kernels.kvsall_fused` — loss and dense ``dE`` with
  the table stationary, ``dQ`` with the queries stationary — with labels from the resident CSR as bit masks; nothing of
  size ``B × |E|`` exists.  ``backward`` hands ``dQ`` to autograd, which carries it through the gates to every other
  parameter;
* the entity table itself never meets autograd: the gathered head rows are a leaf whose gradient is scatter-added into
  the dense ``dE`` the kernel produced, and the table is updated by the fused optimiser kernel (bf16 shadow refreshed
  in the same sweep).  All other parameters are stepped by the model's own optimiser.

Two epilogue variants of the scoring kernel widen the contract.  Models whose score adds a scalar that depends on the
query only — the general Clifford models Keci / CKeci (p, q) and DeCaL (p, q, r), whose σ_pp / σ_qq / σ_pq / … terms
are summed into one number per (h, r) (``dicee/models/clifford.py:258-305``, ``:601-790``) — pass it as a per-query bias
(a column bias in the launch that keeps the table stationary, a row bias in the other, which also returns its
gradient).  TransE (``dicee/models/real.py:52-76``) uses the distance epilogue: ``margin − sqrt(‖q‖² + ‖e‖² − 2 q·e)``
from the same dot products, with the squared norms as per-row scalars; the kernel's second GEMM then yields
``Σ w e`` with ``w = dS / distance`` together with ``Σ w``, and the gradient is ``Σ w e − (Σ w) q``.

The reference runs these models as ``conv2d`` / ``Linear`` / four to eight ``torch.mm`` against the table plus
``BCEWithLogitsLoss`` on dense labels (``dicee/models/complex.py:33-62``, ``dicee/models/quaternion.py:242-319``,
``dicee/models/octonion.py:206-313``, ``dicee/models/dualE.py:102-127``, ``dicee/models/base_model.py:25-46``).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K
from .fused_step import SUPPORTED_DIMS, SUPPORTED_SCORING, _EngineOptimizer, fused_model_code


def hybrid_supported(model) -> bool:
    """Bilinear contract (with or without a per-query bias) or TransE's distance, a width the scoring kernel takes,
    ordinary index inputs."""
    if getattr(model, "byte_pair_encoding", False):
        return False
    if model.embedding_dim not in SUPPORTED_DIMS or model.optimizer_name not in K.OPT_CODE:
        return False
    if type(model).__name__ == "TransE":
        return True
    return bool(getattr(model, "bilinear", False)) and hasattr(model, "compose")


class FusedScoring(torch.autograd.Function):
    """``loss = mean BCE-with-logits(logits(Q, E), labels)`` with the gradient w.r.t. ``Q`` (and the per-query bias)
    computed in the same call.  ``mode`` 0: ``Q Eᵀ``; 1: ``Q Eᵀ + bias[:, None]``; 2: ``margin − cdist(Q, E)``."""

    @staticmethod
    def forward(ctx, q: torch.Tensor, bias: Optional[torch.Tensor], engine: "ExternalQueryEngine", dp: torch.Tensor,
                mode: int):
        n = q.shape[0]
        b = engine._buffers(n)
        scale = 1.0 / (float(n) * float(engine.NE))
        b.Q.copy_(q.detach())                                  # fp32 -> bf16 operand
        b.dQ.zero_()
        engine.loss_acc.zero_()
        b.mask_q.zero_()
        b.mask_e.zero_()
        K.build_label_masks(dp, engine.offsets, engine.values, n, 1, 0, b.mask_q, b.mask_e,
                            num_data_points=engine.num_data_points, num_local_rows=engine.NE, status=engine.status)
        common = dict(pos_delta=engine.pos_weight, score_mode=mode, margin=engine.margin)
        if mode == 0:
            e_kw, q_kw = {}, {}
        elif mode == 1:
            b.q_scalar[:n].copy_(bias.detach())
            b.q_sum.zero_()
            e_kw = dict(y_bias=b.q_scalar)
            q_kw = dict(x_bias=b.q_scalar, x_dsum=b.q_sum)
        else:
            # squared norms of the operands as the tensor cores see them (bf16-rounded)
            torch.sum(b.Q.float() ** 2, dim=1, out=b.q_scalar[:n])
            torch.sum(engine.E_bf16.float() ** 2, dim=1, out=engine.e_scalar[:engine.NE])
            b.q_sum.zero_()
            engine.e_sum.zero_()
            e_kw = dict(x_bias=engine.e_scalar, y_bias=b.q_scalar, x_dsum=engine.e_sum)
            q_kw = dict(x_bias=b.q_scalar, y_bias=engine.e_scalar, x_dsum=b.q_sum)
        K.kvsall_fused(engine.E_bf16, b.Q, engine.gE, engine.loss_acc, engine.status, engine.base, scale, True,
                       mask=b.mask_e, **common, **e_kw)
        K.kvsall_fused(b.Q, engine.E_bf16, b.dQ, None, engine.status, engine.base, scale, False,
                       mask=b.mask_q, **common, **q_kw)
        if mode == 2:
            # d logit / d x = (y − x) / distance: the kernels returned Σ w y and Σ w
            engine.gE.addcmul_(engine.e_sum[:, None], engine.E, value=-1.0)
            b.dQ.addcmul_(b.q_sum[:, None], q.detach(), value=-1.0)
        ctx.dq, ctx.dbias = b.dQ, (b.q_sum if mode == 1 else None)
        return (engine.loss_acc * scale).to(torch.float32).reshape(())

    @staticmethod
    def backward(ctx, grad_out):
        return grad_out * ctx.dq, (None if ctx.dbias is None else grad_out * ctx.dbias), None, None, None


class ExternalQueryEngine:
    def __init__(self, model, dataset, batch_size: int, lr: float, weight_decay: float = 0.0, device=None):
        assert hybrid_supported(model)
        self.model = model
        self.device = dev = torch.device(device or model.device)
        self.D, self.NE = model.embedding_dim, model.num_entities
        self.lr, self.weight_decay = float(lr), float(weight_decay)
        self.opt_kind = K.OPT_CODE[model.optimizer_name]
        self.betas = (0.9, 0.9999) if self.opt_kind == 3 else (0.9, 0.999)
        self.eps = 1e-6 if self.opt_kind == 3 else 1e-8
        self.E = model.entity_embeddings.weight.data
        assert self.E.is_cuda and self.E.is_contiguous() and self.E.dtype == torch.float32
        self.E_bf16 = torch.empty(self.NE, self.D, dtype=torch.bfloat16, device=dev)
        K.cast_bf16(self.E, self.E_bf16)
        self.gE = torch.zeros_like(self.E)
        self.mE, self.vE = torch.zeros_like(self.E), torch.zeros_like(self.E)
        self.step_count = torch.zeros(1, dtype=torch.int64, device=dev)
        self.loss_acc = torch.zeros(1, dtype=torch.float64, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        # every parameter but the entity table belongs to the model's own optimiser
        model.entity_embeddings.weight.requires_grad_(False)
        rest = [p for p in model.parameters() if p.requires_grad]
        self.rest_optimizer = model.configure_optimizers(rest) if rest else None
        if self.rest_optimizer is not None:
            for g in self.rest_optimizer.param_groups:
                g["lr"] = self.lr
        self.dataset = dataset
        dataset.sparse_labels = True
        if hasattr(dataset, "offsets"):
            self.offsets, self.values = dataset.offsets.to(dev).contiguous(), dataset.values.to(dev).contiguous()
            pos, base = dataset.label_constants()
        else:  # 1vsAll: one positive per data point
            pairs = dataset.train_data.to(dev)
            self.offsets = torch.arange(pairs.shape[0] + 1, dtype=torch.int64, device=dev)
            self.values = pairs[:, 2].contiguous()
            pos, base = 1.0, 0.0
        self.pos_weight, self.base = float(pos - base), float(base)
        self.distance = type(model).__name__ == "TransE"
        self.margin = float(getattr(model, "margin", 0.0)) if self.distance else 0.0
        if self.distance:
            self.e_scalar = torch.zeros(K.padded_rows(self.NE), device=dev)
            self.e_sum = torch.zeros(self.NE, device=dev)
        self.num_data_points = int(self.offsets.numel() - 1)
        self.label_mode = "mask"
        self._bufs = {}

    def _buffers(self, n: int):
        if n not in self._bufs:
            from types import SimpleNamespace
            dev = self.device
            b = SimpleNamespace()
            b.Q = torch.zeros(n, self.D, dtype=torch.bfloat16, device=dev)
            b.dQ = torch.zeros(n, self.D, dtype=torch.float32, device=dev)
            b.mask_q = torch.zeros(n, K.mask_stride(self.NE), dtype=torch.int32, device=dev)
            b.mask_e = torch.zeros(self.NE, K.mask_stride(n), dtype=torch.int32, device=dev)
            b.q_scalar = torch.zeros(K.padded_rows(n), device=dev)     # per-query bias or squared norm
            b.q_sum = torch.zeros(n, device=dev)
            self._bufs[n] = b
        return self._bufs[n]

    def step(self, batch) -> torch.Tensor:
        """``batch = (x [n, 2] int64, data-point ids [n] int64)`` on the device; returns the loss (device scalar)."""
        x, dp = batch[0], batch[1]
        m = self.model
        if self.rest_optimizer is not None:
            self.rest_optimizer.zero_grad(set_to_none=True)
        h_idx = x[:, 0].contiguous()
        head_rows = self.E[h_idx].requires_grad_(True)          # leaf: the table itself stays outside autograd
        h = m.normalize_head_entity_embeddings(m.input_dp_ent_real(head_rows))
        r = m.normalize_relation_embeddings(m.input_dp_rel_real(m.relation_embeddings(x[:, 1])))
        if self.distance:
            q, bias, mode = h + r + m._eps, None, 2
        else:
            q, bias = m.compose(h, r)
            mode = 0 if bias is None else 1
            if bias is not None:
                bias = bias.float().reshape(-1).contiguous()
        loss = FusedScoring.apply(q.float().contiguous(), bias, self, dp.contiguous(), mode)
        loss.backward()
        self.gE.index_add_(0, h_idx, head_rows.grad)           # row gradients of the lookups join the dense dE
        if self.rest_optimizer is not None:
            self.rest_optimizer.step()
        b1, b2 = self.betas
        K.optimizer_step(self.opt_kind, self.E, self.gE, self.mE, self.vE, self.E_bf16, self.step_count, self.lr, b1,
                         b2, self.eps, self.weight_decay)
        self.step_count += 1
        return loss.detach()

    def launches_per_step(self) -> int:
        return 5

    def sync_to_model(self) -> None:
        K.check_status(self.status, "in the external-query training step")

    def optimizer_view(self):
        return _HybridOptimizer(self)


class _HybridOptimizer(_EngineOptimizer):
    """LR-scheduling callbacks steer both halves: the kernel-side table update and the model's own optimiser."""

    def __init__(self, engine: ExternalQueryEngine):
        super().__init__(engine)
        self.param_groups = [_BothLr(engine)]


class _BothLr(dict):
    def __init__(self, engine):
        super().__init__(lr=engine.lr)
        self._e = engine

    def __setitem__(self, k, v):
        super().__setitem__(k, v)
        if k == "lr":
            self._e.lr = float(v)
            if self._e.rest_optimizer is not None:
                for g in self._e.rest_optimizer.param_groups:
                    g["lr"] = float(v)


def build_hybrid_engine(model, dataset, args, device) -> Optional[ExternalQueryEngine]:
    """An :class:`ExternalQueryEngine` when the fully fused engine does not cover the model but the bilinear contract
    holds; ``None`` otherwise."""
    if fused_model_code(model) is not None or not hybrid_supported(model):
        return None
    if getattr(args, "scoring_technique", None) not in SUPPORTED_SCORING:
        return None
    if dataset is None or not hasattr(dataset, "train_data") or torch.cuda.get_device_capability(device)[0] != 10:
        return None
    mask_bytes = 2 * int(args.batch_size) * model.num_entities / 8
    if mask_bytes > (1 << 30):
        return None
    return ExternalQueryEngine(model, dataset, batch_size=args.batch_size, lr=args.lr,
                               weight_decay=getattr(args, "weight_decay", 0.0) or 0.0, device=device)
