"""Row-sharded fused training step over several GPUs of one node (one process per GPU).

Entity row ``e`` lives on rank ``e % W`` at local row ``e // W``; relations (and the Keci coefficient) are
replicated.  With ``comm="p2p"`` every communication step happens *inside* the kernels through a symmetric heap that
is mapped on every rank and, where the fabric offers it, bound to an NVSwitch multicast object:

====  =====================================================  ==================================================
step  kernel                                                 traffic over NVLink
====  =====================================================  ==================================================
1     ``lookup_compose_vec``: pull ``E[h]`` from the owner,    peer loads of rows; one ``multimem.st`` per 16 bytes
      compose, publish the bf16 query row and the batch        of query row reaches every rank (the all-gather of
      indices on every rank                                    Q); without multicast, one store per rank
S1    ``p2p_barrier``
2     ``build_label_masks`` + ``kvsall_fused`` (query-         none (local shard × all queries; the label CSR is
      stationary): partial ``dQ`` of the local shard for       partitioned by owner when the engine is built; the
      all queries                                              partials of the whole batch stay local)
3m    main branch: ``kvsall_fused`` (entity-stationary):       none
      loss and dense ``dE`` of the local shard
3s    side branch, beside 3m.  ``S2``, then the *owner of      peer loads of the query-gradient rows of all ranks
      the head row* sums that query's partial ``dQ`` over      (the reduce-scatter of dQ, done by its consumer:
      all ranks, applies the chain rule and adds the row       inside ``compose_backward_owner``, or as the light
      gradient to its own gradient shard; ``S2b``; the         kernel ``dq_pull_owner`` in front of it);
      replicated tables are updated from the sum of all        peer loads of every rank's gradient buffer: the
      ranks' gradient buffers (``step_tail``); dQ cleared      all-reduce folded into the update.  No row gradient
                                                               crosses the fabric.
4     main joins the backward; ``optimizer_step`` over the     none
      local entity shard
S3    ``p2p_barrier``
5     main joins the side branch; ``finish_step`` sums the     peer loads of the loss partials
      loss partials
====  =====================================================  ==================================================

``S3`` also orders the next step's peer reads of the updated entity rows, so no barrier opens a step: three barriers
lie on the critical path, ``S2`` and ``S2b`` (on signal slots and a counter of their own, since they can be in flight
together with ``S3``) beside the entity-role launch.  ``DICE_B200_OVERLAP_BACKWARD=0`` and the sparse-label flavour keep
the serial order entity role → query role → ``S2`` → backward → update → ``S3`` → ``step_tail``.  Buffers
that peers read after a barrier (``gR``, loss partials) are cleared behind the *next* barrier, when every peer is
known to have read them.  Once a barrier times out the status word is set and every later kernel that would touch
peer memory returns at once; :meth:`check` reports it.

``comm="nccl"`` runs the same local kernels but moves data with ``torch.distributed`` collectives
(all-gather, reduce-scatter, all-reduce); it is the comparison pipeline.  Buffers are never handed to library
GEMMs as peer memory, and no load uses cluster multicast.
"""
from __future__ import annotations

import os
from types import SimpleNamespace
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops.fused_step import fused_model_code
from .symm import SymmetricHeap


def partition_csr(offsets: torch.Tensor, values: torch.Tensor, world: int, rank: int):
    """CSR restricted to the values owned by ``rank`` (``value % world == rank``), re-numbered as local rows
    (``value // world``); row ``i`` of the result lists the owned entries of row ``i`` of the input."""
    own = (values % world) == rank
    csum = torch.zeros(values.numel() + 1, dtype=torch.int64, device=values.device)
    torch.cumsum(own.to(torch.int64), 0, out=csum[1:])
    new_offsets = csum[offsets].contiguous()
    new_values = torch.div(values[own], world, rounding_mode="floor").contiguous()
    return new_offsets, new_values


def owner_of(e: torch.Tensor, world: int) -> torch.Tensor:
    return e % world


def local_row(e: torch.Tensor, world: int) -> torch.Tensor:
    return torch.div(e, world, rounding_mode="floor")


def shard_rows(num_rows: int, rank: int, world: int) -> int:
    """Number of valid rows of the cyclic shard of ``rank``."""
    return (num_rows - rank + world - 1) // world if num_rows > rank else 0


def take_shard(full: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    return full[rank::world]


def scatter_shard_back(full: torch.Tensor, shard: torch.Tensor, rank: int, world: int) -> None:
    full[rank::world] = shard[: shard_rows(full.shape[0], rank, world)]


class ShardedKvsAllEngine:
    def __init__(self, model, dataset, batch_size: int, lr: float, weight_decay: float = 0.0, device=None,
                 comm: str = "p2p", group=None, use_graph: bool = True, label_mode: Optional[str] = None,
                 multimem: Optional[bool] = None):
        assert dist.is_initialized(), "ShardedKvsAllEngine needs an initialised process group"
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.W = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.model = model
        self.device = dev = torch.device(device or model.device)
        self.code = fused_model_code(model)
        assert self.code is not None, "model is not covered by the fused kernels"
        assert comm in ("p2p", "nccl")
        self.comm = comm
        self.D, self.NE, self.NR = model.embedding_dim, model.num_entities, model.num_relations
        self.B = int(batch_size)
        self.lr, self.weight_decay = float(lr), float(weight_decay)
        self.opt_kind = K.OPT_CODE[model.optimizer_name]
        self.betas = (0.9, 0.9999) if self.opt_kind == 3 else (0.9, 0.999)
        self.eps = 1e-6 if self.opt_kind == 3 else 1e-8
        self.normalize = type(model).__name__ in ("QMult", "OMult")
        self.use_graph = use_graph and os.environ.get("DICE_B200_NO_GRAPH") != "1"
        W, B, D = self.W, self.B, self.D
        self.rows_pad = (self.NE + W - 1) // W
        self.rows = shard_rows(self.NE, self.rank, W)

        # every rank starts from rank 0's initial weights
        with torch.no_grad():
            for prm in model.parameters():
                dist.broadcast(prm.data, src=dist.get_global_rank(self.group, 0), group=self.group)
        self.coeff_trainable = self.code == 4 and bool(model.q_coefficients.weight.requires_grad)

        heap = SymmetricHeap(self.group, dev)
        heap.plan("E", (self.rows_pad, D), torch.float32)
        heap.plan("gR", (self.NR, D), torch.float32)
        heap.plan("gC", (4,), torch.float32)
        heap.plan("Q", (W * B, D), torch.bfloat16)
        heap.plan("dQ", (W * B, D), torch.float32)   # this rank's partial query gradients for the whole batch
        heap.plan("ids", (3, W * B), torch.int64)    # h | r | data point of every query of the global batch
        heap.plan("loss", (2,), torch.float64)
        heap.plan("sig", (64,), torch.int32)
        heap.commit()
        self.heap = heap
        want = os.environ.get("DICE_B200_MULTIMEM", "1") != "0" if multimem is None else bool(multimem)
        self.multimem = bool(want and heap.mc_base and comm == "p2p")
        self.E, self.gR, self.gC = heap.local("E"), heap.local("gR"), heap.local("gC")
        self.gE = torch.zeros(self.rows_pad, D, dtype=torch.float32, device=dev)   # row gradients never leave the owner
        self.Q, self.dQ, self.ids_all = heap.local("Q"), heap.local("dQ"), heap.local("ids")
        self.h_all, self.r_all, self.dp_all = self.ids_all[0], self.ids_all[1], self.ids_all[2]
        self.loss_acc = heap.local("loss")
        self.E[: self.rows].copy_(take_shard(model.entity_embeddings.weight.data, self.rank, W))
        self.R = model.relation_embeddings.weight.data
        self.coeff = model.q_coefficients.weight.data if self.code == 4 else None
        self.E_bf16 = torch.zeros(self.rows_pad, D, dtype=torch.bfloat16, device=dev)
        K.cast_bf16(self.E, self.E_bf16)
        self.mE, self.vE = torch.zeros_like(self.E), torch.zeros_like(self.E)
        self.mR, self.vR = torch.zeros_like(self.R), torch.zeros_like(self.R)
        if self.coeff is not None:
            self.mC, self.vC = torch.zeros_like(self.coeff), torch.zeros_like(self.coeff)
        self.step_count = torch.zeros(1, dtype=torch.int64, device=dev)
        self.loss_out = torch.zeros(1, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.barrier_count = torch.zeros(1, dtype=torch.int32, device=dev)
        self.barrier_count_side = torch.zeros(1, dtype=torch.int32, device=dev)
        self.owned_list = torch.zeros(W * batch_size, dtype=torch.int32, device=dev)   # batch rows whose head lives here
        self.owned_count = torch.zeros(1, dtype=torch.int32, device=dev)

        self.tab = SimpleNamespace(E=heap.table("E"), gR=heap.table("gR"), gC=heap.table("gC"),
                                   Q=heap.table("Q"), dQ=heap.table("dQ"), ids=heap.table("ids"),
                                   loss=heap.table("loss"), sig=heap.table("sig"))
        assert W <= 32, "the signal region holds two sets of 32 slots"
        self.sig_side = self.tab.sig + 128        # second half of every rank's 64-word signal region
        mm = self.multimem
        # Measured on B200s (owner-side backward of 4096 owned queries, d = 256): multimem.ld_reduce 30 us against 17 us
        # with peer loads at two ranks, 52 us against 25 us at four.  The 16-byte in-switch reductions of scattered
        # rows cost more than reading W - 1 peer copies, so the reduce-scatter of dQ and the all-reduce of the
        # replicated gradients use peer loads unless DICE_B200_MULTIMEM_REDUCE=1; the all-gather of Q keeps
        # multimem.st (one store instead of W).
        mm_red = mm and os.environ.get("DICE_B200_MULTIMEM_REDUCE") == "1"
        self.mc = SimpleNamespace(Q=heap.mc_address("Q") if mm else 0, dQ=heap.mc_address("dQ") if mm_red else 0,
                                  gR=heap.mc_address("gR") if mm_red else 0, gC=0)

        # dataset (replicated): pairs and CSR of known tails
        self.dataset = dataset
        dataset.sparse_labels = True
        self.pairs = dataset.train_data.to(dev)
        if hasattr(dataset, "offsets"):
            self.offsets, self.values = dataset.offsets.to(dev).contiguous(), dataset.values.to(dev).contiguous()
            pos, base = dataset.label_constants()
        else:
            n = self.pairs.shape[0]
            self.offsets = torch.arange(n + 1, dtype=torch.int64, device=dev)
            self.values = self.pairs[:, 2].contiguous()
            pos, base = 1.0, 0.0
        self.pos_weight, self.base = float(pos - base), float(base)
        self.num_data_points = int(self.offsets.numel() - 1)
        # the label CSR is partitioned by owner once: this rank keeps the known tails that live in its shard, as
        # local row numbers, so the label kernels of a step walk 1/W of the positives and filter nothing
        if comm == "p2p":
            self.offsets_loc, self.values_loc = partition_csr(self.offsets, self.values, W, self.rank)
        else:
            self.offsets_loc, self.values_loc = self.offsets, self.values

        self.dp = torch.zeros(B, dtype=torch.int64, device=dev)
        self.x_in = torch.zeros(B, 2, dtype=torch.int64, device=dev)
        self.h, self.r = self.x_in.view(-1), self.x_in.view(-1)[1:]   # read in place with stride 2 by the lookup
        # labels: "mask" (default while the masks fit 1 GiB) feeds bit masks of the positives to the scoring epilogues;
        # "sparse" applies the known tails by a correction kernel driven by the owner-partitioned CSR, beside the dense
        # scoring launches (tables of millions of rows)
        mask_bytes = 2.0 * W * B * self.rows_pad / 8
        self.label_mode = label_mode or os.environ.get("DICE_B200_LABELS") or \
            ("mask" if mask_bytes <= (1 << 30) else "sparse")
        assert self.label_mode in ("mask", "sparse")
        assert self.label_mode == "sparse" or mask_bytes <= (1 << 30), "label masks would exceed 1 GiB"
        if comm == "nccl":
            self.label_mode = "mask"   # the comparison pipeline keeps the mask flavour
        if self.label_mode == "mask":
            self.mask_q = torch.zeros(W * B, K.mask_stride(self.rows_pad), dtype=torch.int32, device=dev)
            self.mask_e = torch.zeros(self.rows_pad, K.mask_stride(W * B), dtype=torch.int32, device=dev)
        else:
            self.mask_q = self.mask_e = None
        self.first = torch.zeros(W * B + 1, dtype=torch.int32, device=dev)
        if comm == "nccl":
            self._init_nccl_buffers()
        self._graph = None
        self._graph_lr = None
        self._side = torch.cuda.Stream(device=dev)
        # Programmatic dependent launch (csrc/launch_pdl.cuh) is measured and tested on the single-GPU step only (1 %
        # there); the sharded step keeps ordinary stream-ordered launches unless DICE_B200_PDL=1 is set.
        os.environ.setdefault("DICE_B200_PDL", "0")
        # Reduce-scatter of dQ as a light kernel of its own (DICE_B200_DQ_PULL=1) or inside the backward kernel (=0).
        # Measured, ms per step at N = 2 / 8: 0.236 / 0.349 with the light kernel (it fits beside the scoring CTA, but
        # its 32-register budget keeps only a few of the W peer loads of a thread in flight, which costs more than the
        # overlap gains once W is large), 0.246 / 0.318 inside the backward kernel.  Default: the light kernel at W = 2.
        pull = os.environ.get("DICE_B200_DQ_PULL", "auto")
        self.dq_pull = (W <= 2) if pull == "auto" else pull == "1"
        # with the light kernel the graph is captured on a high-priority stream: kernel nodes inherit it, so where both
        # branches are ready the scoring launch gets its CTAs resident first and the side branch fills what is left
        self._capture_stream = torch.cuda.Stream(device=dev, priority=-1) if self.dq_pull else None
        # DICE_B200_OVERLAP_BACKWARD=0 keeps the serial order entity role -> query role -> S2 -> backward
        self.overlap_backward = os.environ.get("DICE_B200_OVERLAP_BACKWARD", "1") != "0"
        if comm == "p2p":
            segs = [dict(param=self.R, grad=self.gR, m=self.mR, v=self.vR, grad_table=self.tab.gR, grad_mc=self.mc.gR)]
            if self.coeff_trainable:
                segs.append(dict(param=self.coeff, grad=self.gC[:1], m=self.mC, v=self.vC, grad_table=self.tab.gC))
            self._tail = K.StepTail(self.opt_kind, segs, self.step_count, self.status, finish=True,
                                    loss_out=self.loss_out, acc_table=self.tab.loss, n_acc=W, n_grad=W)
            self._tail_rest = K.StepTail(self.opt_kind, segs, self.step_count, self.status, finish=False, n_grad=W)
        self._phase_events = [] if os.environ.get("DICE_B200_PHASE_TIMING") == "1" else None
        self._phase_names = []
        self._phase_slots = torch.zeros(32, dtype=torch.int64, device=dev)
        heap.host_barrier()

    # ------------------------------------------------------------------ the step, peer-memory flavour
    def _barrier(self, side: bool = False) -> None:
        """Bounded device barrier.  The barriers of the parallel branch (``side``) use their own signal slots and
        counter: they may be in flight at the same time as a barrier of the main branch."""
        if side:
            K.p2p_barrier(self.sig_side, self.rank, self.W, self.barrier_count_side, self.status)
        else:
            K.p2p_barrier(self.tab.sig, self.rank, self.W, self.barrier_count, self.status)

    def _optimizers_and_finish(self, scale: float) -> None:
        """Collective flavour: replicated gradients and the loss were already summed by library collectives."""
        b1, b2 = self.betas
        a = (self.lr, b1, b2, self.eps, self.weight_decay)
        K.optimizer_step(self.opt_kind, self.E, self.gE, self.mE, self.vE, self.E_bf16, self.step_count, *a)
        K.optimizer_step(self.opt_kind, self.R, self.gR, self.mR, self.vR, None, self.step_count, *a)
        if self.coeff_trainable:
            K.optimizer_step(self.opt_kind, self.coeff, self.gC[:1], self.mC, self.vC, None, self.step_count, *a)
        K.finish_step(self.loss_acc, self.loss_out, scale, self.step_count)

    def _mark(self, name: str) -> None:
        """Phase timing (``DICE_B200_PHASE_TIMING=1``): a one-thread kernel stores the GPU timer after each phase, so
        the times are device times also under graph replay; :meth:`phase_times` returns the microseconds per phase of
        the last step."""
        if self._phase_events is not None:
            if name not in self._phase_names:
                self._phase_names.append(name)
            K.timestamp(self._phase_slots, self._phase_names.index(name))

    def phase_times(self):
        torch.cuda.synchronize(self.device)
        t = self._phase_slots.cpu().tolist()
        out = {}
        for i in range(1, len(self._phase_names)):
            out[self._phase_names[i]] = (t[i] - t[i - 1]) / 1e6   # milliseconds
        return out

    def _launch_p2p(self) -> None:
        W, B, D, n = self.W, self.B, self.D, self.W * self.B
        scale = 1.0 / (float(n) * float(self.NE))
        b1, b2 = self.betas
        a = (self.lr, b1, b2, self.eps, self.weight_decay)
        self._mark("start")
        masks = self.label_mode == "mask"
        main = torch.cuda.current_stream(self.device)
        if masks:   # cleared on a parallel branch; joined before the masks are built
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                self.mask_q.zero_()
                self.mask_e.zero_()
        # head rows by peer loads, query rows and batch indices to every rank (multimem.st or one store per rank)
        K.lookup_compose_vec(self.code, self.normalize, self.h, self.r, self.dp, self.tab.E, W, self.NE, self.NR,
                             self.R, self.coeff, self.tab.Q, W, self.mc.Q, self.rank * B, None, self.tab.ids, n, B, D,
                             self.status, idx_stride=2 if self.comm == "p2p" else 1)
        self._mark("lookup+allgather")
        self._barrier()                                   # S1: all query rows have landed everywhere
        self._mark("S1")
        self.gR.zero_()                                   # every peer has read last step's partial sums by now
        self.gC.zero_()
        self.loss_acc.zero_()
        if self.dq_pull:
            self.owned_count.zero_()                      # (here: a fill kernel would not fit beside the scoring launch)
        if masks:
            main.wait_stream(self._side)
            K.build_label_masks(self.dp_all, self.offsets_loc, self.values_loc, n, 1, 0, self.mask_q, self.mask_e,
                                first=self.first, num_data_points=self.num_data_points, num_local_rows=self.rows_pad,
                                status=self.status)
            self._mark("masks")
        e_loc = self.E_bf16[: self.rows]
        if not masks:
            # label term of the positives whose tail lives in this shard (loss, dE rows here, partial dQ rows here; all
            # added atomically) on a parallel branch beside the two dense scoring launches
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                K.positive_scan(self.dp_all, self.offsets_loc, n, self.first)
                K.positive_correction(self.dp_all, self.offsets_loc, self.values_loc, self.first, self.Q, self.E_bf16,
                                      self.dQ, self.gE, self.loss_acc[:1], self.pos_weight, scale, n, D, 1, 0)
        if masks and self.overlap_backward:
            # query role first; then the barrier S2, the pull of the partial dQ rows over NVLink and the backward of the
            # composition run on a parallel branch BESIDE the entity-role launch, which needs none of them: the wait
            # for the slowest rank and the link latency of the pull hide behind tensor-core work
            K.kvsall_fused(self.Q, e_loc, self.dQ, self.loss_acc[:1], self.status, self.base, scale, True,
                           mask=self.mask_q, pos_delta=self.pos_weight, loss_share=1)
            self._mark("fused_Q")
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                if self.dq_pull:
                    K.owned_rows(self.h_all, n, W, self.rank, self.NE, self.owned_list, self.owned_count, self.status)
                self._barrier(side=True)                  # S2: every rank's partial dQ is complete
                if self.dq_pull:
                    # the reduce-scatter of dQ alone (light blocks that fit beside the scoring CTA of every SM: the
                    # NVLink transfer runs under the entity-role launch), then the backward on local memory
                    K.dq_pull_owner(self.owned_list, self.owned_count, self.tab.dQ, W, self.dQ, D, self.status)
                    K.compose_backward_owner(self.code, self.normalize, self.h_all, self.r_all, self.E, W, self.rank,
                                             self.NE, self.NR, self.R, self.coeff, self.dQ, None, 0, 0,
                                             self.gE, self.gR, self.gC if self.coeff_trainable else None, n, D,
                                             self.status)
                else:
                    # owner-side backward with the reduce-scatter inside it (peer loads or multimem.ld_reduce)
                    K.compose_backward_owner(self.code, self.normalize, self.h_all, self.r_all, self.E, W, self.rank,
                                             self.NE, self.NR, self.R, self.coeff, None, self.tab.dQ, W, self.mc.dQ,
                                             self.gE, self.gR, self.gC if self.coeff_trainable else None, n, D,
                                             self.status)
                backward_done = torch.cuda.Event()
                backward_done.record(self._side)
                # the branch goes on beside the entity update and S3: once every rank's backward is through (barrier
                # S2b) the replicated tables are updated from the sum of all ranks' gradient buffers, and dQ is cleared
                self._barrier(side=True)
                self._tail_rest.launch(*a, scale)
                self.dQ.zero_()
            K.kvsall_fused(e_loc, self.Q, self.gE, self.loss_acc[:1], self.status, self.base, scale, True,
                           mask=self.mask_e, pos_delta=self.pos_weight, loss_share=0)
            self._mark("fused_E")
            main.wait_event(backward_done)                # the row gradients of the lookups are in gE
            self._mark("backward joined")
            K.optimizer_step(self.opt_kind, self.E, self.gE, self.mE, self.vE, self.E_bf16, self.step_count, *a,
                             status=self.status)
            self._mark("optim_E")
            self._barrier()                               # S3: shards updated, loss partials complete everywhere
            self._mark("S3")
            main.wait_stream(self._side)
            self._mark("side branch joined")
            K.finish_step(self.loss_acc, self.loss_out, scale, self.step_count, acc_table=self.tab.loss, n_acc=W,
                          status=self.status)
            self._mark("finish")
            return
        self._score_then_backward(masks, main, e_loc, scale, W, n, D)
        K.optimizer_step(self.opt_kind, self.E, self.gE, self.mE, self.vE, self.E_bf16, self.step_count, *a,
                         status=self.status)
        self._mark("optim_E")
        self._barrier()                                   # S3: shards updated, partial sums complete, dQ pulls done
        self._mark("S3")
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            self.dQ.zero_()
        # one launch: the replicated tables are updated from the sum of all ranks' gradient buffers (multimem.ld_reduce
        # or peer loads: the all-reduce folded into the update) and the last block sums the loss partials
        self._tail.launch(*a, scale)
        main.wait_stream(self._side)
        self._mark("optim_R")

    def _score_then_backward(self, masks, main, e_loc, scale, W, n, D) -> None:
        """Serial order: entity role, query role, S2, owner-side backward."""
        # both launches add half of the loss terms each (the epilogue with loss costs several times the one without)
        K.kvsall_fused(e_loc, self.Q, self.gE, self.loss_acc[:1], self.status, self.base, scale, True,
                       mask=self.mask_e, pos_delta=self.pos_weight, loss_share=0)
        self._mark("fused_E")
        K.kvsall_fused(self.Q, e_loc, self.dQ, self.loss_acc[:1], self.status, self.base, scale, True,
                       mask=self.mask_q, pos_delta=self.pos_weight, loss_share=1)
        self._mark("fused_Q")
        if not masks:
            main.wait_stream(self._side)
        self._barrier()                                   # S2: every rank's partial dQ is complete
        self._mark("S2")
        # owner-side backward: dQ rows summed over the ranks inside the switch (or by peer loads), row gradients local
        K.compose_backward_owner(self.code, self.normalize, self.h_all, self.r_all, self.E, W, self.rank, self.NE,
                                 self.NR, self.R, self.coeff, None, self.tab.dQ, W, self.mc.dQ, self.gE, self.gR,
                                 self.gC if self.coeff_trainable else None, n, D, self.status)
        self._mark("backward+reduce_scatter")

    def launches_per_step(self) -> int:
        if self.comm != "p2p":
            return 9
        if self.label_mode == "mask" and self.overlap_backward:
            # four barriers + lookup, masks, two scoring launches, backward, replicated-table update, entity update,
            # loss sum (+ owned-row list and dQ pull)
            return 4 + 8 + (2 if self.dq_pull else 0)
        return 3 + (9 if self.label_mode == "mask" else 8)

    # ------------------------------------------------------------------ the step, collective flavour
    def _init_nccl_buffers(self) -> None:
        dev, W, B, D = self.device, self.W, self.B, self.D
        self.n_h_all = torch.zeros(W * B, dtype=torch.int64, device=dev)
        self.n_rows_all = torch.zeros(W * B, D, dtype=torch.float32, device=dev)
        self.n_hrows = torch.zeros(B, D, dtype=torch.float32, device=dev)
        self.n_Q = torch.zeros(B, D, dtype=torch.bfloat16, device=dev)
        self.n_Qall = torch.zeros(W * B, D, dtype=torch.bfloat16, device=dev)
        self.n_dp_all = torch.zeros(W * B, dtype=torch.int64, device=dev)
        self.n_dQall = torch.zeros(W * B, D, dtype=torch.float32, device=dev)
        self.n_dQ = torch.zeros(B, D, dtype=torch.float32, device=dev)
        self.n_dh = torch.zeros(B, D, dtype=torch.float32, device=dev)
        self.n_dh_all = torch.zeros(W * B, D, dtype=torch.float32, device=dev)
        self.n_arange = torch.arange(B, dtype=torch.int64, device=dev)
        self.n_h = torch.zeros(B, dtype=torch.int64, device=dev)
        self.n_r = torch.zeros(B, dtype=torch.int64, device=dev)
        self.n_tab_h = K.pointer_table([self.n_hrows], dev)
        self.n_tab_q = K.pointer_table([self.n_Q], dev)
        self.n_tab_dh = K.pointer_table([self.n_dh], dev)

    def _launch_nccl(self) -> None:
        W, B, D, n, g = self.W, self.B, self.D, self.W * self.B, self.group
        scale = 1.0 / (float(n) * float(self.NE))
        self.n_h.copy_(self.x_in[:, 0])
        self.n_r.copy_(self.x_in[:, 1])
        # lookup: all-gather the head ids, every owner contributes its rows, reduce-scatter back
        dist.all_gather_into_tensor(self.n_h_all, self.n_h, group=g)
        dist.all_gather_into_tensor(self.n_dp_all, self.dp, group=g)
        mine = (self.n_h_all % W) == self.rank
        self.n_rows_all.zero_()
        self.n_rows_all[mine] = self.E[torch.div(self.n_h_all[mine], W, rounding_mode="floor")]
        dist.reduce_scatter_tensor(self.n_hrows, self.n_rows_all, group=g)
        K.lookup_compose(self.code, self.normalize, self.n_arange, self.n_r, self.n_tab_h, 1, B, self.R, self.coeff,
                         self.n_tab_q, 1, 0, None, B, D, self.status)
        dist.all_gather_into_tensor(self.n_Qall, self.n_Q, group=g)
        self.mask_q.zero_()
        self.mask_e.zero_()
        self.n_dQall.zero_()
        K.build_label_masks(self.n_dp_all, self.offsets, self.values, n, W, self.rank, self.mask_q, self.mask_e)
        e_loc = self.E_bf16[: self.rows]
        K.kvsall_fused(e_loc, self.n_Qall, self.gE, self.loss_acc[:1], self.status, self.base, scale, True,
                       mask=self.mask_e, pos_delta=self.pos_weight)
        K.kvsall_fused(self.n_Qall, e_loc, self.n_dQall, None, self.status, self.base, scale, False,
                       mask=self.mask_q, pos_delta=self.pos_weight)
        dist.reduce_scatter_tensor(self.n_dQ, self.n_dQall, group=g)
        self.n_dh.zero_()
        K.compose_backward(self.code, self.normalize, self.n_arange, self.n_r, self.n_tab_h, 1, self.R, self.coeff,
                           self.n_dQ, self.n_tab_dh, self.gR, self.gC if self.coeff_trainable else None, B, D)
        dist.all_gather_into_tensor(self.n_dh_all, self.n_dh, group=g)
        self.gE.index_add_(0, torch.div(self.n_h_all[mine], W, rounding_mode="floor"), self.n_dh_all[mine])
        dist.all_reduce(self.gR, group=g)
        dist.all_reduce(self.gC, group=g)
        dist.all_reduce(self.loss_acc, group=g)
        self._optimizers_and_finish(scale)

    # ------------------------------------------------------------------ driving
    def _run(self) -> None:
        launch = self._launch_p2p if self.comm == "p2p" else self._launch_nccl
        if not self.use_graph or self.comm == "nccl":
            launch()
            return
        if self._graph is None or self._graph_lr != self.lr:
            if self._graph is None and self._graph_lr is None:
                # first call: plain launches (also sets kernel attributes); every rank does the same
                launch()
                self._graph_lr = -1.0
                return
            g = torch.cuda.CUDAGraph()
            with (torch.cuda.graph(g, stream=self._capture_stream) if self._capture_stream is not None
                  else torch.cuda.graph(g)):
                launch()
            self._graph, self._graph_lr = g, self.lr
        self._graph.replay()

    def step(self, batch) -> torch.Tensor:
        """``batch = (x [B, 2], data-point ids [B])`` of *this rank* on the device; returns the global mean loss."""
        x, dp = batch[0], batch[1]
        assert x.shape[0] == self.B, "the sharded step needs full batches of the configured size on every rank"
        self.x_in.copy_(x)
        self.dp.copy_(dp)
        self._run()
        return self.loss_out[0]

    def step_from_host(self, x_pinned: torch.Tensor, dp_pinned: torch.Tensor) -> float:
        self.x_in.copy_(x_pinned, non_blocking=True)
        self.dp.copy_(dp_pinned, non_blocking=True)
        self._run()
        return float(self.loss_out.item())

    def step_from_host_pipelined(self, x_pinned: torch.Tensor, dp_pinned: torch.Tensor) -> Optional[float]:
        """:meth:`step_from_host` without stalling the host on the step it has just queued: returns the loss of the
        previous step (``None`` first); :meth:`last_loss` waits for the newest.  Each step still has its own
        host→device input copy and device→host loss copy."""
        if not hasattr(self, "_loss_host"):
            self._loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
            self._loss_event = [torch.cuda.Event(), torch.cuda.Event()]
            self._loss_slot, self._loss_pending = 0, False
        prev = None
        if self._loss_pending:
            self._loss_event[self._loss_slot].synchronize()
            prev = float(self._loss_host[self._loss_slot][0])
        self.x_in.copy_(x_pinned, non_blocking=True)
        self.dp.copy_(dp_pinned, non_blocking=True)
        self._run()
        self._loss_slot ^= 1
        self._loss_host[self._loss_slot].copy_(self.loss_out, non_blocking=True)
        self._loss_event[self._loss_slot].record()
        self._loss_pending = True
        return prev

    def last_loss(self) -> Optional[float]:
        if not getattr(self, "_loss_pending", False):
            return None
        self._loss_event[self._loss_slot].synchronize()
        return float(self._loss_host[self._loss_slot][0])

    def check(self) -> None:
        K.check_status(self.status, f"on rank {self.rank} of the sharded step")

    @torch.no_grad()
    def sync_to_model(self) -> None:
        """Gather the shards into the model's full entity table on every rank (collective)."""
        self.check()
        shards = [torch.empty_like(self.E) for _ in range(self.W)]
        dist.all_gather(shards, self.E.contiguous(), group=self.group)
        full = self.model.entity_embeddings.weight.data
        for r, s in enumerate(shards):
            scatter_shard_back(full, s, r, self.W)

    # ------------------------------------------------------------------ checkpoint / resume
    def _replicated_state(self):
        rep = {"relation_embeddings.weight": self.R, "m_R": self.mR, "v_R": self.vR}
        if self.coeff is not None:
            rep.update({"q_coefficients.weight": self.coeff, "m_C": self.mC, "v_C": self.vC})
        return rep

    @torch.no_grad()
    def save_checkpoint(self, directory: str) -> None:
        """Collective: every rank writes its rows of the entity table and of the Adam moments, rank 0 the replicated
        parameters and the manifest (see :mod:`dice_embeddings_b200.io.sharded_checkpoint`)."""
        from ..io import sharded_checkpoint as sc
        self.check()
        torch.cuda.synchronize(self.device)
        sc.save_shard(directory, self.rank, self.W, self.NE, {"E": self.E, "mE": self.mE, "vE": self.vE},
                      replicated=self._replicated_state() if self.rank == 0 else None,
                      step=int(self.step_count.item()),
                      extra={"lr": self.lr, "optimizer": self.model.optimizer_name, "model": type(self.model).__name__})
        dist.barrier(group=self.group)

    @torch.no_grad()
    def load_checkpoint(self, directory: str) -> None:
        """Collective: resume from a sharded checkpoint written with any world size."""
        from ..io import sharded_checkpoint as sc
        man = sc.read_manifest(directory)
        assert man["num_entities"] == self.NE and man["dim"] == self.D, "checkpoint belongs to another table shape"
        t = sc.load_shard(directory, self.rank, self.W, self.device)
        for name, dst in (("E", self.E), ("mE", self.mE), ("vE", self.vE)):
            dst[: self.rows].copy_(t[name])
        rep = sc.load_replicated(directory, self.device)
        for k, dst in self._replicated_state().items():
            if k in rep:
                dst.copy_(rep[k])
        self.step_count.fill_(int(man["step"]))
        K.cast_bf16(self.E, self.E_bf16)   # the captured graph stays valid: all buffers keep their addresses
        dist.barrier(group=self.group)

    def optimizer_view(self):
        from ..ops.fused_step import _EngineOptimizer
        return _EngineOptimizer(self)
