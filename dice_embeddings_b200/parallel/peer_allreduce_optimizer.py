"""Gradient all-reduce of a replicated model folded into its optimiser step, over peer memory.

For models outside the fused engines (convolutional, transformer, function-space ...) the multi-GPU trainer
replicates the model and averages gradients.  Instead of an NCCL all-reduce followed by ``optimizer.step()``
(reference: ``DistributedDataParallel`` + ``torch.optim``, ``dicee/trainer/torch_trainer_ddp.py:104-147``) every rank
copies its gradients, already divided by the world size, into a buffer of the symmetric heap; after one bounded device
barrier a single optimiser kernel per rank reads all ranks' buffers by peer loads, sums them on the fly and applies
Adam / AdamW / SGD / ADOPT to the (flattened) parameters.  All replicas apply the same update, so they stay identical
without a broadcast.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .symm import SymmetricHeap


class PeerAllReduceOptimizer:
    def __init__(self, model: torch.nn.Module, lr: float, weight_decay: float = 0.0, device=None, group=None):
        assert dist.is_initialized()
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.W = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device = dev = torch.device(device or next(model.parameters()).device)
        name = getattr(model, "optimizer_name", "Adam")
        assert name in K.OPT_CODE, f"optimiser {name} is not covered by the fused update"
        self.kind = K.OPT_CODE[name]
        self.betas = (0.9, 0.9999) if self.kind == 3 else (0.9, 0.999)
        self.eps = 1e-6 if self.kind == 3 else 1e-8
        self.lr, self.weight_decay = float(lr), float(weight_decay)
        self.params: List[torch.nn.Parameter] = [p for p in model.parameters() if p.requires_grad]
        assert all(p.dtype == torch.float32 for p in self.params)
        sizes = [p.numel() for p in self.params]
        self.offsets = [0]
        for n in sizes:
            self.offsets.append(self.offsets[-1] + n)
        total = self.offsets[-1]
        # parameters become views of one flat buffer, so one kernel launch updates the whole model
        self.flat = torch.empty(total, dtype=torch.float32, device=dev)
        for p, o, n in zip(self.params, self.offsets, sizes):
            self.flat[o:o + n].copy_(p.data.reshape(-1))
            p.data = self.flat[o:o + n].view_as(p.data)
        self.m, self.v = torch.zeros_like(self.flat), torch.zeros_like(self.flat)
        heap = SymmetricHeap(self.group, dev)
        heap.plan("g", (total,), torch.float32)
        heap.plan("sig", (64,), torch.int32)
        heap.commit()
        self.heap, self.g, self.g_table, self.sig_table = heap, heap.local("g"), heap.table("g"), heap.table("sig")
        self.step_count = torch.zeros(1, dtype=torch.int64, device=dev)
        self.barrier_count = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.param_groups = [{"lr": self.lr}]   # what learning-rate callbacks look at
        heap.host_barrier()

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            p.grad = None

    @torch.no_grad()
    def step(self) -> None:
        """Collective: every rank calls it once per training step, after ``backward``."""
        self.lr = float(self.param_groups[0]["lr"])
        inv = 1.0 / self.W
        K.p2p_barrier(self.sig_table, self.rank, self.W, self.barrier_count, self.status)   # peers finished reading g
        for p, o in zip(self.params, self.offsets):
            n = p.numel()
            if p.grad is None:
                self.g[o:o + n].zero_()
            else:
                torch.mul(p.grad.reshape(-1), inv, out=self.g[o:o + n])
        K.p2p_barrier(self.sig_table, self.rank, self.W, self.barrier_count, self.status)   # all gradients are in place
        b1, b2 = self.betas
        K.optimizer_step(self.kind, self.flat, self.g, self.m, self.v, None, self.step_count, self.lr, b1, b2, self.eps,
                         self.weight_decay, grad_table=self.g_table, n_grad=self.W)
        self.step_count += 1

    def check(self) -> None:
        K.check_status(self.status, f"on rank {self.rank} in the fused all-reduce + optimiser step")

    def state_dict(self):
        return {"step": int(self.step_count.item()), "lr": self.lr}

    def load_state_dict(self, sd) -> None:
        self.param_groups[0]["lr"] = float(sd.get("lr", self.lr))
