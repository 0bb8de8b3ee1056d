"""Row-sharded training step for the sampled-candidate scoring techniques (NegSample, 1vsSample, KvsSample) with a
row-wise sparse optimiser: the path for entity tables too large for one GPU whose steps touch only a small part of
the rows.

Every rank owns the rows ``rank, rank + W, ...`` of the entity table (fp32 master, moments and a gradient shard of
the same shape, all in the symmetric heap) and its own slice of the batch.  One step is

    S0  bounded device barrier           the previous step's updates are visible everywhere
        candidates                       ``layout="tails"``: candidate matrix ``[B, 1 + k]`` = true tail + k uniform
                                         entities per positive (one query vector per positive); ``layout="flat"``: the
                                         reference's corruption (heads or tails per batch, one coin) as ``B (1 + k)``
                                         independent triples
        lookup_compose                   head rows are *pulled* from their owners by peer loads, composed with the
                                         (replicated) relation rows
        candidate_bce                    candidate rows pulled by peer loads; scores, BCE-with-logits, dq; candidate-row
                                         gradients *pushed* to the owners by peer ``red.add``; owners' row flags set
        compose_backward                 head-row gradients pushed to the owners, relation gradients kept locally
    S1  bounded device barrier           every gradient has reached its owner
        sparse_rows_optimizer            Adam / AdamW / SGD on the flagged rows of the local shard only (lazy moments)
        optimizer_step (relations, ...)  reads all ranks' gradient buffers by peer loads: all-reduce folded into the update
        finish_step                      global mean loss

so the index dispatch / row gather / gradient combine of an embedding-parallel step never goes through a collective
library call, and rows that were not sampled cost nothing.  The reference trains these techniques with dense
``torch.optim`` updates of the whole table on every replica (``dicee/models/base_model.py:86-118``).
"""
from __future__ import annotations

import os
from types import SimpleNamespace
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops.sampled_step import sampled_model_code
from .sharded_engine import shard_rows, take_shard
from .symm import SymmetricHeap


class ShardedSampledEngine:
    def __init__(self, model, scoring_technique: str, batch_size: int, lr: float, neg_ratio: int = 0,
                 label_smoothing: float = 0.0, weight_decay: float = 0.0, device=None, group=None, seed: int = 0,
                 layout: str = "flat", use_graph: bool = True, entity_rows: Optional[torch.Tensor] = None):
        """``entity_rows``: this rank's rows of the entity table when the model does not hold the full table
        (tables larger than one GPU); otherwise the shard is cut from ``model.entity_embeddings``."""
        assert dist.is_initialized(), "ShardedSampledEngine needs an initialised process group"
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.W = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.model, self.st = model, scoring_technique
        self.device = dev = torch.device(device or model.device)
        self.code = sampled_model_code(model)
        assert self.code is not None, "model is not covered by the sampled-candidate kernels"
        assert layout in ("flat", "tails")
        self.layout = layout if scoring_technique == "NegSample" else "given"
        self.D, self.NE, self.NR = model.embedding_dim, model.num_entities, model.num_relations
        self.B, self.k = int(batch_size), int(neg_ratio)
        self.lr, self.weight_decay = float(lr), float(weight_decay)
        self.opt_kind = K.OPT_CODE[model.optimizer_name]
        assert self.opt_kind in (0, 1, 2), "the row-wise sparse optimiser covers Adam, AdamW and SGD"
        self.betas, self.eps = (0.9, 0.999), 1e-8
        self.normalize = type(model).__name__ in ("QMult", "OMult")
        self.kind = 1 if self.code == 5 else 0
        self.margin = float(getattr(model, "margin", 0.0)) if self.kind else 0.0
        self.dist_eps = float(getattr(model, "_eps", 0.0)) if self.kind else 0.0
        self.label_smoothing = float(label_smoothing)
        self.seed = int(seed) + 7919 * self.rank
        self.use_graph = use_graph and os.environ.get("DICE_B200_NO_GRAPH") != "1"
        W, D = self.W, self.D
        self.rows_pad = (self.NE + W - 1) // W
        self.rows = shard_rows(self.NE, self.rank, W)

        with torch.no_grad():  # replicated parameters start from rank 0's values
            for name, prm in model.named_parameters():
                if entity_rows is not None and name.startswith("entity_embeddings"):
                    continue
                dist.broadcast(prm.data, src=dist.get_global_rank(self.group, 0), group=self.group)
        self.coeff_trainable = self.code == 4 and bool(model.q_coefficients.weight.requires_grad)

        heap = SymmetricHeap(self.group, dev)
        heap.plan("E", (self.rows_pad, D), torch.float32)
        heap.plan("gE", (self.rows_pad, D), torch.float32)
        heap.plan("touched", (self.rows_pad + 16,), torch.uint8)
        heap.plan("gR", (self.NR, D), torch.float32)
        heap.plan("gC", (4,), torch.float32)
        heap.plan("loss", (2,), torch.float64)
        heap.plan("sig", (64,), torch.int32)
        heap.commit()
        self.heap = heap
        self.E, self.gE, self.touched = heap.local("E"), heap.local("gE"), heap.local("touched")
        self.gR, self.gC, self.loss_acc = heap.local("gR"), heap.local("gC"), heap.local("loss")
        if entity_rows is not None:
            self.E[: self.rows].copy_(entity_rows[: self.rows])
        else:
            self.E[: self.rows].copy_(take_shard(model.entity_embeddings.weight.data, self.rank, W))
        self.R = model.relation_embeddings.weight.data
        self.coeff = model.q_coefficients.weight.data if self.code == 4 else None
        self.mE, self.vE = torch.zeros_like(self.E), torch.zeros_like(self.E)
        self.mR, self.vR = torch.zeros_like(self.R), torch.zeros_like(self.R)
        if self.coeff is not None:
            self.mC, self.vC = torch.zeros_like(self.coeff), torch.zeros_like(self.coeff)
        self.step_count = torch.zeros(1, dtype=torch.int64, device=dev)
        self.loss_out = torch.zeros(1, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.barrier_count = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tab = SimpleNamespace(E=heap.table("E"), gE=heap.table("gE"), touched=heap.table("touched"),
                                   gR=heap.table("gR"), gC=heap.table("gC"), loss=heap.table("loss"),
                                   sig=heap.table("sig"))
        self._bufs = {}
        self._graphs = {}
        self._eager_done = set()
        heap.host_barrier()

    # ------------------------------------------------------------------ buffers
    def _buffers(self, key):
        """``key = (queries N, candidates C, positives B or 0)``."""
        if key not in self._bufs:
            N, C, B = key
            dev = self.device
            b = SimpleNamespace()
            b.pos = torch.zeros(max(B, 1), 3, dtype=torch.int64, device=dev)
            b.h, b.r = (torch.zeros(N, dtype=torch.int64, device=dev) for _ in range(2))
            b.cand = torch.zeros(N, C, dtype=torch.int64, device=dev)
            b.labels = torch.zeros(N, C, dtype=torch.float32, device=dev)
            b.q = torch.zeros(N, self.D, dtype=torch.float32, device=dev)
            b.dq = torch.zeros(N, self.D, dtype=torch.float32, device=dev)
            if self.layout == "tails":  # labels never change: the true tail first, then the corruptions
                b.labels.fill_(self.label_smoothing)
                b.labels[:, 0] = 1.0 - self.label_smoothing
            self._bufs[key] = b
        return self._bufs[key]

    def _barrier(self) -> None:
        K.p2p_barrier(self.tab.sig, self.rank, self.W, self.barrier_count, self.status)

    def _launch_all(self, b, key) -> None:
        N, C, B = key
        W, D = self.W, self.D
        scale = 1.0 / (float(N) * float(C) * float(W))
        self._barrier()                                          # S0
        self.gR.zero_()
        self.gC.zero_()
        self.loss_acc.zero_()
        if self.layout == "flat" and B:
            K.neg_sample(b.pos, self.k, self.NE, self.seed, 0, b.labels, hrt=(b.h, b.r, b.cand),
                         label_pos=1.0 - self.label_smoothing, label_neg=self.label_smoothing, step=self.step_count)
        elif self.layout == "tails":
            b.h.copy_(b.pos[:, 0])
            b.r.copy_(b.pos[:, 1])
            b.cand[:, 0].copy_(b.pos[:, 2])
            if C > 1:
                K.uniform_int(b.cand[:, 1:], self.NE, self.seed, 0, step=self.step_count)
        K.lookup_compose(self.code, self.normalize, b.h, b.r, self.tab.E, W, self.NE, self.R, self.coeff, None, 0, 0,
                         b.q, N, D, self.status)
        K.candidate_bce(b.q, b.cand, C, 1, C, b.labels, self.tab.E, W, self.tab.gE, b.dq, None, self.loss_acc[:1],
                        scale, self.kind, self.margin, self.dist_eps, touched_table=self.tab.touched)
        K.compose_backward(self.code, self.normalize, b.h, b.r, self.tab.E, W, self.R, self.coeff, b.dq, self.tab.gE,
                           self.gR, self.gC if self.coeff_trainable else None, N, D, touched_table=self.tab.touched)
        self._barrier()                                          # S1
        b1, b2 = self.betas
        a = (self.lr, b1, b2, self.eps, self.weight_decay)
        K.sparse_rows_optimizer(self.opt_kind, self.E, self.gE, self.mE, self.vE, None, self.touched[: self.rows_pad],
                                self.step_count, *a)
        K.optimizer_step(self.opt_kind, self.R, self.gR, self.mR, self.vR, None, self.step_count, *a,
                         grad_table=self.tab.gR, n_grad=W)
        if self.coeff_trainable:
            K.optimizer_step(self.opt_kind, self.coeff, self.gC[:1], self.mC, self.vC, None, self.step_count, *a,
                             grad_table=self.tab.gC, n_grad=W)
        K.finish_step(self.loss_acc, self.loss_out, 1.0, self.step_count, acc_table=self.tab.loss, n_acc=W)

    def launches_per_step(self) -> int:
        return 2 + 6 + (1 if self.layout in ("flat", "tails") else 0) + (1 if self.coeff_trainable else 0)

    def _run(self, b, key) -> None:
        gkey = (key, self.lr)
        if not self.use_graph:
            self._launch_all(b, key)
            return
        if gkey not in self._graphs:
            if key not in self._eager_done:   # first call with this shape: plain launches on every rank
                self._launch_all(b, key)
                self._eager_done.add(key)
                return
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch_all(b, key)
            self._graphs[gkey] = g
        self._graphs[gkey].replay()

    # ------------------------------------------------------------------ public
    def step(self, batch) -> torch.Tensor:
        """NegSample: ``(positives [B, 3],)`` of this rank (the corruptions are drawn on the device).
        1vsSample / KvsSample: ``(x [B, 2], candidate ids [B, C], labels [B, C])`` as built by the dataset.
        Every rank must call with the same shapes.  Returns the global mean loss (device scalar)."""
        if self.st == "NegSample":
            pos = batch[0]
            assert len(batch) == 1 or batch[1] is None, "pass the positives only (dataset.defer_sampling = True)"
            assert pos.shape[1] == 3, "the sharded NegSample step takes the positives; it draws the corruptions itself"
            B = pos.shape[0]
            key = (B, 1 + self.k, B) if self.layout == "tails" else (B * (1 + self.k), 1, B)
            b = self._buffers(key)
            b.pos.copy_(pos)
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

    def step_from_host(self, pos_pinned: torch.Tensor) -> float:
        """End-to-end NegSample step: host→device copy of the positives, the step, device→host read of the loss."""
        return float(self.step((pos_pinned.to(self.device, non_blocking=True),)).item())

    def check(self) -> None:
        K.check_status(self.status, f"on rank {self.rank} of the sharded sampled step")

    @torch.no_grad()
    def sync_to_model(self) -> None:
        """Gather the shards into the model's full entity table (collective; skipped when the model holds no full
        table, i.e. it was built with ``entity_rows``)."""
        self.check()
        full = self.model.entity_embeddings.weight.data
        if full.shape[0] != self.NE:
            return
        shards = [torch.empty_like(self.E) for _ in range(self.W)]
        dist.all_gather(shards, self.E.contiguous(), group=self.group)
        for r, s in enumerate(shards):
            full[r::self.W] = s[: shard_rows(self.NE, r, self.W)]

    def optimizer_view(self):
        from ..ops.fused_step import _EngineOptimizer
        return _EngineOptimizer(self)
