"""Data-parallel trainer: one process per device under ``torchrun`` (``--trainer torchDDP``).

The reference wraps the model in ``DistributedDataParallel`` after ``torch.compile`` and hard-codes fp16 autocast
(``dicee/trainer/torch_trainer_ddp.py:45-191``); every step all-reduces the dense gradient of the whole entity
table.  Here the name selects, in this order:

1. the row-sharded fused engine (:class:`ShardedKvsAllEngine`) when the model / scoring technique is covered and the
   ranks run on B200s — no replicated table, no dense-table all-reduce;
2. otherwise plain data parallelism: every rank holds a replica, processes its slice of each epoch and the
   gradients are averaged with one flat all-reduce per step.  This path also runs on CPU ranks (Gloo), which is
   how it is tested without GPUs.

Callbacks fire on global rank 0 at epoch end, as in the reference (``:188-191``); every rank then meets in a host-side
barrier, so that long callbacks (evaluation, checkpoints, weight averaging) never eat into the bounded waits of the
device-side barriers of the next step.  Ranks publish heartbeats through the process group's store and check their
peers between steps; a silent peer raises :class:`~dice_embeddings_b200.parallel.watchdog.RankFailure` before the next
launch instead of a device barrier time-out.  The process group is left alive for the executor to tear down.
"""
from __future__ import annotations

import os
import time

import torch
import torch.distributed as dist

from .base import AbstractTrainer, BatchLoader


class TorchDDPTrainer(AbstractTrainer):
    def __init__(self, args, callbacks=None):
        super().__init__(args, callbacks)
        if dist.is_initialized():
            self.global_rank, self.world_size = dist.get_rank(), dist.get_world_size()
        else:
            self.global_rank, self.world_size = 0, 1
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        self.is_global_zero = self.global_rank == 0
        if torch.cuda.is_available() and (not dist.is_initialized() or dist.get_backend() == "nccl"):
            self.device = torch.device(f"cuda:{self.local_rank}")
        else:
            self.device = torch.device("cpu")
        self.engine = None

    # ------------------------------------------------------------------
    def _maybe_sharded_engine(self, model, loader):
        backend = getattr(self.attributes, "kernel_backend", "auto")
        if backend == "torch" or self.device.type != "cuda" or self.world_size < 2:
            return None
        try:
            from ..ops.fused_step import SUPPORTED_SCORING, fused_model_code
            if fused_model_code(model) is None or self.attributes.scoring_technique not in SUPPORTED_SCORING \
                    or torch.cuda.get_device_capability(self.device)[0] != 10:
                if backend == "cuda":
                    raise RuntimeError("kernel_backend=cuda requested but the model / scoring technique is not covered")
                return None
            from ..parallel.sharded_engine import ShardedKvsAllEngine
            return ShardedKvsAllEngine(model, loader.dataset, batch_size=loader.batch_size, lr=self.attributes.lr,
                                       weight_decay=getattr(self.attributes, "weight_decay", 0.0) or 0.0,
                                       device=self.device, comm=getattr(self.attributes, "comm", "p2p"))
        except ImportError:
            if backend == "cuda":
                raise
            return None

    def _maybe_peer_optimizer(self, model):
        """Replicated model on B200s: the gradient all-reduce is folded into the optimiser kernel (peer loads)."""
        backend = getattr(self.attributes, "kernel_backend", "auto")
        if backend == "torch" or getattr(self.attributes, "comm", "p2p") != "p2p" or self.world_size < 2 \
                or self.device.type != "cuda" or torch.cuda.get_device_capability(self.device)[0] != 10:
            return None
        try:
            from ..ops import kernels as K
            from ..parallel.peer_allreduce_optimizer import PeerAllReduceOptimizer
            if getattr(model, "optimizer_name", None) not in K.OPT_CODE:
                return None
            if any(p.dtype != torch.float32 for p in model.parameters() if p.requires_grad):
                return None
            return PeerAllReduceOptimizer(model, lr=self.attributes.lr,
                                          weight_decay=getattr(self.attributes, "weight_decay", 0.0) or 0.0,
                                          device=self.device)
        except (ImportError, RuntimeError, OSError):
            if backend == "cuda":
                raise
            return None

    def _allreduce_grads(self, params) -> None:
        grads = [p.grad for p in params if p.grad is not None]
        if not grads or self.world_size == 1:
            return
        flat = torch._utils._flatten_dense_tensors(grads)
        dist.all_reduce(flat)
        flat.div_(self.world_size)
        for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
            g.copy_(f)

    def fit(self, *args, train_dataloaders, **kwargs) -> None:
        model, = args
        self.model = model
        model.to(self.device)
        loader = train_dataloaders
        if isinstance(loader, BatchLoader):
            loader.rank, loader.world_size = self.global_rank, self.world_size
            loader.dataset.to(self.device)
        if self.world_size > 1:  # identical start on every rank
            for p in model.parameters():
                dist.broadcast(p.data, src=0)
        if isinstance(loader, BatchLoader) and self.world_size > 1:
            # engines with a fixed batch size: never more than a rank's share of the data (the same number on every
            # rank), and the short final batch is filled by wrap-around instead of being dropped
            per_rank = -(-len(loader.dataset) // self.world_size)
            if per_rank < loader.batch_size:
                if self.is_global_zero:
                    print(f"batch_size {loader.batch_size} exceeds the {per_rank} data points per rank: using {per_rank}")
                loader.batch_size = per_rank
        self.engine = self._maybe_sharded_engine(model, loader)
        if self.engine is not None:
            loader.drop_last, loader.pad_last = False, True
            assert len(loader) >= 1, "no training step per epoch: the dataset is empty"
        self.peer_optimizer = None
        if self.engine is not None:
            self.optimizer = self.engine.optimizer_view()
        else:
            self.peer_optimizer = self._maybe_peer_optimizer(model)
            self.optimizer = self.peer_optimizer if self.peer_optimizer is not None else model.configure_optimizers()
        params = [p for p in model.parameters() if p.requires_grad]
        use_bf16 = getattr(self.attributes, "compute_dtype", "fp32") == "bf16" and self.device.type == "cuda"
        heartbeat = self._start_heartbeat()
        if self.is_global_zero:
            self.on_fit_start(self, model)
        self._host_barrier()
        for epoch in range(self.attributes.num_epochs):
            self.current_epoch = epoch
            if hasattr(loader, "set_epoch"):
                loader.set_epoch(epoch)
            model.train()
            total = torch.zeros((), device=self.device)
            nb = 0
            t0 = time.time()
            for i, batch in enumerate(loader):
                if heartbeat is not None:
                    heartbeat.raise_if_failed()   # a peer went silent: stop before the next launch
                batch = tuple(b.to(self.device, non_blocking=True) if isinstance(b, torch.Tensor) else b for b in batch)
                if self.engine is not None:
                    loss = self.engine.step(batch)
                else:
                    self.optimizer.zero_grad(set_to_none=True)
                    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=use_bf16):
                        loss = model.training_step(batch)
                    loss.backward()
                    if self.peer_optimizer is None:
                        self._allreduce_grads(params)
                    self.optimizer.step()   # the peer optimiser sums all ranks' gradients inside its update kernel
                total += loss.detach()
                nb += 1
            if self.engine is None and self.world_size > 1:
                dist.all_reduce(total)
                total /= self.world_size
            if self.engine is not None:
                self.engine.sync_to_model()
            if self.peer_optimizer is not None:
                self.peer_optimizer.check()
            epoch_loss = float(total) / max(nb, 1)
            model.loss_history.append(epoch_loss)
            if self.is_global_zero:
                print(f"Epoch:{epoch + 1} | Loss:{epoch_loss:.8f} | Runtime:{(time.time() - t0) / 60:.3f}mins")
                self.on_train_epoch_end(self, model)
            self._host_barrier()      # the other ranks wait here, on the host, while rank 0 runs its callbacks
        if self.is_global_zero:
            self.on_fit_end(self, model)
        self._host_barrier()
        if heartbeat is not None:
            heartbeat.stop()

    def _host_barrier(self) -> None:
        if self.world_size > 1 and dist.is_initialized():
            dist.barrier()

    def _start_heartbeat(self):
        """Background heartbeats through the default process group's store (``None`` for a single rank or when the
        store cannot be reached).  ``DICE_B200_HEARTBEAT_TIMEOUT`` (seconds, default 120; 0 switches it off) bounds how
        long a peer may stay silent; rank-0 callbacks may run longer than that only while the others sit in the host
        barrier, where heartbeats keep flowing from the background thread."""
        timeout = float(os.environ.get("DICE_B200_HEARTBEAT_TIMEOUT", "120"))
        if self.world_size < 2 or timeout <= 0 or not dist.is_initialized():
            return None
        try:
            from torch.distributed.distributed_c10d import _get_default_store
            from ..parallel.watchdog import Heartbeat
            return Heartbeat(_get_default_store(), self.global_rank, self.world_size, timeout=timeout,
                             interval=min(1.0, timeout / 4)).start()
        except Exception:   # noqa: BLE001 - the store is an implementation detail of the backend
            return None
