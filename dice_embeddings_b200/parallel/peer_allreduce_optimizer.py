"""Gradient all-reduce of a replicated model, overlapped with backward and fused with the optimiser step.

For models outside the sharded engines (convolutional, transformer, function-space ...) the multi-GPU trainer
replicates the model.  The reference wraps it in ``DistributedDataParallel`` (bucketed NCCL all-reduce from autograd
hooks) and then calls ``optimizer.step()`` (``dicee/trainer/torch_trainer_ddp.py:87-122``).  Here:

* parameters and gradients are two flat buffers in a symmetric heap that every rank maps (and that is bound to an
  NVSwitch multicast object where available); ``p.data`` and ``p.grad`` are views into them, so autograd accumulates
  gradients straight into the buffer the peers read: nothing is staged or copied;
* the flat vector is cut into buckets in the order in which backward produces gradients.  A post-accumulate hook
  counts the finished parameters of a bucket; when the last one arrives, the bucket is queued on a side stream, behind
  an event of the backward stream: a bounded device barrier over the ranks (on per-bucket signal slots) followed by
  ONE kernel that reduce-scatters the bucket (each rank sums its 1 / W slice over all ranks with
  ``multimem.ld_reduce`` or peer loads), applies Adam / AdamW / SGD / ADOPT to that slice and all-gathers the updated
  parameters (``multimem.st`` or peer stores).  Backward keeps running on its own stream meanwhile;
* :meth:`step` queues the buckets that did not fire (unused parameters), joins the side stream and closes with one
  barrier, after which every replica holds the same updated parameters.

A rank moves 1 / W of a bucket in each direction (two-shot) instead of reading W full copies.
"""
from __future__ import annotations

import os
from typing import List

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .symm import SymmetricHeap


class PeerAllReduceOptimizer:
    def __init__(self, model: torch.nn.Module, lr: float, weight_decay: float = 0.0, device=None, group=None,
                 bucket_bytes: int = 4 << 20, overlap: bool = True):
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
        self.overlap = bool(overlap) and os.environ.get("DICE_B200_NO_OVERLAP") != "1"
        params = [p for p in model.parameters() if p.requires_grad]
        assert all(p.dtype == torch.float32 for p in params)
        # gradients become ready roughly in reverse order of registration: lay the flat vector out in that order so
        # that a bucket is a contiguous range which completes early in backward
        self.params: List[torch.nn.Parameter] = list(reversed(params))
        align = 4 * self.W                       # every rank's slice of a bucket starts on a 16-byte boundary
        elems = max(bucket_bytes // 4, align)
        # buckets are runs of whole parameters (a parameter larger than bucket_bytes is a bucket of its own); a
        # bucket's range starts and ends on multiples of 4 * W elements, padding words stay zero
        self.offsets, self.buckets = [], []
        off, start, members = 0, 0, []
        for i, p in enumerate(self.params):
            self.offsets.append(off)
            off += (p.numel() + 3) // 4 * 4
            members.append(i)
            if off - start >= elems or i == len(self.params) - 1:
                off = (off + align - 1) // align * align
                self.buckets.append(dict(lo=start, hi=off, members=members))
                start, members = off, []
        total = self.total = off
        heap = SymmetricHeap(self.group, dev)
        heap.plan("p", (total,), torch.float32)
        heap.plan("g", (total,), torch.float32)
        heap.plan("sig", (len(self.buckets) + 1, 64), torch.int32)
        heap.commit()
        self.heap = heap
        self.flat, self.g = heap.local("p"), heap.local("g")
        for p, o in zip(self.params, self.offsets):
            n = p.numel()
            self.flat[o:o + n].copy_(p.data.reshape(-1))
            p.data = self.flat[o:o + n].view_as(p.data)
            p.grad = self.g[o:o + n].view_as(p.data)       # autograd accumulates in place into the shared buffer
        self.m, self.v = torch.zeros(total, device=dev), torch.zeros(total, device=dev)
        self.p_table, self.g_table = heap.table("p"), heap.table("g")
        use_mc = bool(heap.mc_base) and os.environ.get("DICE_B200_MULTIMEM", "1") != "0"
        self.multimem = use_mc
        self.p_mc = heap.mc_address("p") if use_mc else 0
        self.g_mc = heap.mc_address("g") if use_mc else 0
        sig_base = [heap.address("sig", r) for r in range(self.W)]
        self.sig_tables = [torch.tensor([b + 256 * k for b in sig_base], dtype=torch.int64, device=dev)
                           for k in range(len(self.buckets) + 1)]
        self.bar_counts = torch.zeros(len(self.buckets) + 1, dtype=torch.int32, device=dev)
        self.step_count = torch.zeros(1, dtype=torch.int64, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.param_groups = [{"lr": self.lr}]   # what learning-rate callbacks look at
        self._side = torch.cuda.Stream(device=dev)
        self._pending = [len(b["members"]) for b in self.buckets]
        self._launched = [False] * len(self.buckets)
        self._bucket_of = {}
        for k, b in enumerate(self.buckets):
            for i in b["members"]:
                self._bucket_of[id(self.params[i])] = k
        if self.overlap:
            for p in self.params:
                p.register_post_accumulate_grad_hook(self._on_grad)
        heap.host_barrier()

    # ------------------------------------------------------------------ bucket launch
    def _launch_bucket(self, k: int, lr: float) -> None:
        b = self.buckets[k]
        n = b["hi"] - b["lo"]
        per = n // self.W
        lo = b["lo"] + self.rank * per
        hi = b["hi"] if self.rank == self.W - 1 else lo + per
        b1, b2 = self.betas
        K.p2p_barrier(self.sig_tables[k], self.rank, self.W, self.bar_counts[k:k + 1], self.status)
        K.bucket_reduce_update(self.kind, self.p_table, self.p_mc, self.flat, self.g_table, self.g_mc, self.m, self.v,
                               self.step_count, lo, hi, self.W, lr, b1, b2, self.eps, self.weight_decay,
                               1.0 / self.W, self.status)
        self._launched[k] = True

    def _on_grad(self, param) -> None:
        k = self._bucket_of.get(id(param))
        if k is None:
            return
        self._pending[k] -= 1
        if self._pending[k] == 0 and not self._launched[k]:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))     # the stream backward runs on
            self._side.wait_event(ev)
            with torch.cuda.stream(self._side):
                self._launch_bucket(k, float(self.param_groups[0]["lr"]))

    # ------------------------------------------------------------------ optimiser interface
    def zero_grad(self, set_to_none: bool = True) -> None:
        """Gradients live in the shared buffer: they are cleared in place (one fill), never detached."""
        self.g.zero_()
        for p, o in zip(self.params, self.offsets):
            if p.grad is None or p.grad.data_ptr() != self.g.data_ptr() + 4 * o:
                p.grad = self.g[o:o + p.numel()].view_as(p.data)

    @torch.no_grad()
    def step(self) -> None:
        """Collective: every rank calls it once per training step, after ``backward``."""
        self.lr = float(self.param_groups[0]["lr"])
        main = torch.cuda.current_stream(self.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            for k in range(len(self.buckets)):
                if not self._launched[k]:
                    self._launch_bucket(k, self.lr)
            # every slice of every bucket has been written everywhere before anyone reads parameters again, and
            # everyone has finished reading gradients before they are cleared
            K.p2p_barrier(self.sig_tables[-1], self.rank, self.W, self.bar_counts[-1:], self.status)
        main.wait_stream(self._side)
        self.step_count += 1
        self._pending = [len(b["members"]) for b in self.buckets]
        self._launched = [False] * len(self.buckets)

    def check(self) -> None:
        K.check_status(self.status, f"on rank {self.rank} in the fused all-reduce + optimiser step")

    def state_dict(self):
        return {"step": int(self.step_count.item()), "lr": self.lr}

    def load_state_dict(self, sd) -> None:
        self.param_groups[0]["lr"] = float(sd.get("lr", self.lr))
