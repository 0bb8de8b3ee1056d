"""Fused single-GPU training step for bilinear models trained against all entities (KvsAll, AllvsAll, 1vsAll).

One step is a short fixed sequence of kernel launches replayed from a CUDA graph:

1. ``lookup_compose_vec``  gather ``E[h]``, ``R[r]`` (fp32 masters), compose the query, write it as bf16
2. ``kvsall_fused`` (E)    X = bf16 entity table, Y = queries  →  dense part of ``dE`` and of the loss
3. ``kvsall_fused`` (Q)    X = queries, Y = entity table        →  dense part of ``dQ``
4. labels: either ``build_label_masks`` before 2–3 (bit masks of the batch's known tails in both orientations,
   read by the scoring epilogue) or, for tables too large for masks, ``positive_scan`` + ``positive_correction``
   after them (sparse label term from the CSR)
5. ``compose_backward_owner``  chain rule of the composition, row gradients added into ``dE`` / ``dR``
6. ``step_tail``           Adam / AdamW / SGD / ADOPT over E (refreshing the bf16 shadow), R and the coefficient in one
   launch whose last block closes the step: loss = accumulator / (B·|E|), accumulator = 0, step += 1

The ``[B, |E|]`` logit and label matrices of the reference's step (``dicee/models/base_model.py:25-46``:
forward, ``BCEWithLogitsLoss``, backward, optimiser) never exist; labels are the resident CSR.  The model's own
``nn.Parameter`` storage is updated in place, so evaluation and checkpointing see the trained weights.
"""
from __future__ import annotations

import os
from types import SimpleNamespace
from typing import Optional, Tuple

import torch

from ..models.base import IdentityClass
from . import kernels as K

SUPPORTED_DIMS = (64, 128, 256)
SUPPORTED_SCORING = ("KvsAll", "AllvsAll", "1vsAll")


def fused_model_code(model) -> Optional[int]:
    """Kernel model code, or ``None`` when the model is outside what the fused path covers."""
    name = type(model).__name__
    if name not in K.MODEL_CODE or name == "TransE":  # the translation model is not a dot product against E
        return None
    if name in ("Keci", "CKeci") and not (model.p == 0 and model.q == 1):
        return None
    if model.input_dropout_rate or not isinstance(model.normalize_head_entity_embeddings, IdentityClass):
        return None
    if model.embedding_dim not in SUPPORTED_DIMS or getattr(model, "byte_pair_encoding", False):
        return None
    if model.optimizer_name not in K.OPT_CODE:
        return None
    return K.MODEL_CODE[name]


def build_fused_engine(model, dataset, args, device, strict: bool = False):
    """Return a :class:`FusedKvsAllEngine` when model, dataset and optimiser qualify, else ``None``
    (or raise when ``strict``)."""
    reason = None
    if fused_model_code(model) is None:
        reason = f"model {type(model).__name__} (dim {model.embedding_dim}, optim {model.optimizer_name}) is not covered"
    elif getattr(args, "scoring_technique", None) not in SUPPORTED_SCORING:
        reason = f"scoring technique {getattr(args, 'scoring_technique', None)} is not covered"
    elif dataset is None or not hasattr(dataset, "train_data"):
        reason = "dataset does not expose its index tensors"
    elif torch.cuda.get_device_capability(device)[0] != 10:
        reason = "device is not sm_100"
    if reason is not None:
        if strict:
            raise RuntimeError("kernel_backend=cuda requested but " + reason)
        return None
    return FusedKvsAllEngine(model, dataset, batch_size=args.batch_size, lr=args.lr,
                             weight_decay=getattr(args, "weight_decay", 0.0) or 0.0, device=device)


class FusedKvsAllEngine:
    def __init__(self, model, dataset, batch_size: int, lr: float, weight_decay: float = 0.0, device=None,
                 use_graph: bool = True, label_mode: Optional[str] = None):
        self.model = model
        self.device = torch.device(device or model.device)
        self.code = fused_model_code(model)
        assert self.code is not None
        dev = self.device
        self.D = model.embedding_dim
        self.NE, self.NR = model.num_entities, model.num_relations
        self.B = int(batch_size)
        self.lr, self.weight_decay = float(lr), float(weight_decay)
        self.opt_kind = K.OPT_CODE[model.optimizer_name]
        self.betas = (0.9, 0.9999) if self.opt_kind == 3 else (0.9, 0.999)
        self.eps = 1e-6 if self.opt_kind == 3 else 1e-8
        self.use_graph = use_graph and os.environ.get("DICE_B200_NO_GRAPH") != "1"
        self.normalize = type(model).__name__ in ("QMult", "OMult")

        # parameters (updated in place) and their optimiser state
        self.E = model.entity_embeddings.weight.data
        self.R = model.relation_embeddings.weight.data
        assert self.E.is_cuda and self.E.is_contiguous() and self.E.dtype == torch.float32
        self.coeff = None
        self.coeff_trainable = False
        if self.code == 4:
            self.coeff = model.q_coefficients.weight.data
            self.coeff_trainable = bool(model.q_coefficients.weight.requires_grad)
        f32 = dict(dtype=torch.float32, device=dev)
        self.E_bf16 = torch.empty(self.NE, self.D, dtype=torch.bfloat16, device=dev)
        K.cast_bf16(self.E, self.E_bf16)
        self.gE, self.gR = torch.zeros_like(self.E), torch.zeros_like(self.R)
        self.mE, self.vE = torch.zeros_like(self.E), torch.zeros_like(self.E)
        self.mR, self.vR = torch.zeros_like(self.R), torch.zeros_like(self.R)
        if self.coeff is not None:
            self.gC, self.mC, self.vC = (torch.zeros_like(self.coeff) for _ in range(3))
        self.step_count = torch.zeros(1, dtype=torch.int64, device=dev)
        self.loss_acc = torch.zeros(1, dtype=torch.float64, device=dev)
        self.loss_out = torch.zeros(1, **f32)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

        # dataset: pairs, CSR of positives, label constants
        self.dataset = dataset
        dataset.sparse_labels = True
        self.pairs = dataset.train_data.to(dev)
        if hasattr(dataset, "offsets"):
            self.offsets, self.values = dataset.offsets.to(dev).contiguous(), dataset.values.to(dev).contiguous()
            pos, base = dataset.label_constants()
        else:  # 1vsAll: one positive per data point
            n = self.pairs.shape[0]
            self.offsets = torch.arange(n + 1, dtype=torch.int64, device=dev)
            self.values = self.pairs[:, 2].contiguous()
            pos, base = 1.0, 0.0
        self.pos_weight, self.base = float(pos - base), float(base)

        # Labels.  "mask" (default while both masks fit 1 GiB): bit masks of the batch's positives in both orientations,
        # read by the scoring epilogues, so the positives ride along in the tensor-core passes.  "sparse": the epilogues
        # use the label-free value everywhere and the known tails are applied by a sparse correction kernel that runs
        # beside the two scoring launches (BCE splits into a dense label-free term and a term over the positives); it
        # is the only option for tables of millions of rows, but its atomics on hot tail rows make it the slower one
        # on small graphs (measured: 0.280 against 0.228 ms per step on the 14 541-entity benchmark).
        mask_bytes = 2 * self.B * self.NE / 8
        self.label_mode = label_mode or os.environ.get("DICE_B200_LABELS") or \
            ("mask" if mask_bytes <= (1 << 30) else "sparse")
        assert self.label_mode in ("mask", "sparse")
        assert self.label_mode == "sparse" or mask_bytes <= (1 << 30), "label masks would exceed 1 GiB"
        self._bufs = {}
        self._graphs = {}
        self._side = torch.cuda.Stream(device=dev)
        self._phase_names = [] if os.environ.get("DICE_B200_PHASE_TIMING") == "1" else None
        self._phase_slots = torch.zeros(32, dtype=torch.int64, device=dev)
        segs = [dict(param=self.E, grad=self.gE, m=self.mE, v=self.vE, shadow=self.E_bf16),
                dict(param=self.R, grad=self.gR, m=self.mR, v=self.vR)]
        if self.coeff_trainable:
            segs.append(dict(param=self.coeff, grad=self.gC, m=self.mC, v=self.vC))
        self._tail = K.StepTail(self.opt_kind, segs, self.step_count, self.status, finish=True, acc=self.loss_acc,
                                loss_out=self.loss_out)
        # DICE_B200_FUSED_UPDATE=1: the launch order becomes query role -> backward -> entity role, and the entity update
        # rides inside the entity-role launch (the CTA that completes a 128-row tile of dE applies the optimiser to it).
        # Measured slower (112 us against 84 + 19 us: every tile completes at the very end of some CTA's range, where
        # one SM's memory bandwidth then bounds its update), so it is opt-in.  Running the backward of the composition on
        # a parallel branch beside the entity-role launch was measured too: the launch slows down by what the overlap
        # saves (96 us against 84 + 14 us), so the step stays serial.
        self.fuse_entity_update = self.label_mode == "mask" and os.environ.get("DICE_B200_FUSED_UPDATE", "0") == "1"
        if self.fuse_entity_update:
            self._tile_count = torch.zeros((self.NE + 127) // 128, dtype=torch.int32, device=dev)
            self._tail_rest_finish = K.StepTail(self.opt_kind, segs[1:], self.step_count, self.status, finish=True,
                                                acc=self.loss_acc, loss_out=self.loss_out)

    # ------------------------------------------------------------------ buffers per batch size
    def _buffers(self, n: int):
        if n not in self._bufs:
            dev = self.device
            b = SimpleNamespace()
            b.x_in = torch.zeros(n, 2, dtype=torch.int64, device=dev)   # the batch's (h, r) pairs as they arrive
            b.h, b.r = b.x_in.view(-1), b.x_in.view(-1)[1:]             # read in place with stride 2 by the kernels
            b.dp = torch.zeros(n, dtype=torch.int64, device=dev)
            b.Q = torch.zeros(n, self.D, dtype=torch.bfloat16, device=dev)
            b.dQ = torch.zeros(n, self.D, dtype=torch.float32, device=dev)
            b.first = torch.zeros(n + 1, dtype=torch.int32, device=dev)
            b.ent_tab = K.pointer_table([self.E], dev)
            b.gent_tab = K.pointer_table([self.gE], dev)
            b.q_tab = K.pointer_table([b.Q], dev)
            if self.label_mode == "mask":
                b.mask_q = torch.zeros(n, K.mask_stride(self.NE), dtype=torch.int32, device=dev)
                b.mask_e = torch.zeros(self.NE, K.mask_stride(n), dtype=torch.int32, device=dev)
            self._bufs[n] = b
        return self._bufs[n]

    def _mark(self, name: str) -> None:
        """Phase timing (``DICE_B200_PHASE_TIMING=1``): a one-thread kernel stores the GPU timer after each phase, also
        under graph replay; :meth:`phase_times` returns milliseconds per phase of the last step."""
        if self._phase_names is not None:
            if name not in self._phase_names:
                self._phase_names.append(name)
            K.timestamp(self._phase_slots, self._phase_names.index(name))

    def phase_times(self):
        torch.cuda.synchronize(self.device)
        t = self._phase_slots.cpu().tolist()
        return {self._phase_names[i]: (t[i] - t[i - 1]) / 1e6 for i in range(1, len(self._phase_names))}

    def _launch_all(self, b, n: int) -> None:
        scale = 1.0 / (float(n) * float(self.NE))
        main = torch.cuda.current_stream(self.device)
        self._mark("start")
        if self.label_mode == "mask":
            # the label masks depend on the data-point ids only: they are built on a side stream (a parallel branch
            # of the captured graph) while the main stream gathers and composes the queries
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                b.mask_q.zero_()
                b.mask_e.zero_()
                K.build_label_masks(b.dp, self.offsets, self.values, n, 1, 0, b.mask_q, b.mask_e, first=b.first)
        K.lookup_compose_vec(self.code, self.normalize, b.h, b.r, None, b.ent_tab, 1, self.NE, self.NR, self.R,
                             self.coeff, b.q_tab, 1, 0, 0, None, None, 0, n, self.D, self.status, idx_stride=2)
        self._mark("lookup")
        b1, b2 = self.betas
        if self.label_mode == "mask" and self.fuse_entity_update:
            main.wait_stream(self._side)
            self._mark("masks_join")
            K.kvsall_fused(b.Q, self.E_bf16, b.dQ, self.loss_acc, self.status, self.base, scale, True,
                           mask=b.mask_q, pos_delta=self.pos_weight, loss_share=1)
            self._mark("fused_Q")
            K.compose_backward_owner(self.code, self.normalize, b.h, b.r, self.E, 1, 0, self.NE, self.NR, self.R,
                                     self.coeff, b.dQ, None, 0, 0, self.gE, self.gR,
                                     self.gC if self.coeff_trainable else None, n, self.D, self.status, idx_stride=2)
            self._mark("backward")
            # relation table, coefficient and dQ clear on a parallel branch: they need nothing of the launch below
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                b.dQ.zero_()
            opt = K.fused_optimizer_args(self.opt_kind, self.E, self.mE, self.vE, self.E_bf16, self._tile_count,
                                         self.step_count, self.lr, b1, b2, self.eps, self.weight_decay)
            K.kvsall_fused(self.E_bf16, b.Q, self.gE, self.loss_acc, self.status, self.base, scale, True,
                           mask=b.mask_e, pos_delta=self.pos_weight, loss_share=0, opt=opt)
            self._mark("fused_E+update")
            self._tail_rest_finish.launch(self.lr, b1, b2, self.eps, self.weight_decay, scale)
            main.wait_stream(self._side)
            self._mark("tail")
            return
        if self.label_mode == "mask":
            main.wait_stream(self._side)
            self._mark("masks_join")
            # both launches add half of the loss terms each (the epilogue with loss costs several times the one without)
            K.kvsall_fused(self.E_bf16, b.Q, self.gE, self.loss_acc, self.status, self.base, scale, True,
                           mask=b.mask_e, pos_delta=self.pos_weight, loss_share=0)
            self._mark("fused_E")
            K.kvsall_fused(b.Q, self.E_bf16, b.dQ, self.loss_acc, self.status, self.base, scale, True,
                           mask=b.mask_q, pos_delta=self.pos_weight, loss_share=1)
            self._mark("fused_Q")
        else:
            # the label term of the known tails (loss, dE rows, dQ rows; all added atomically) runs on a parallel
            # branch next to the two dense scoring launches: it needs the queries and the entity table only
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                K.positive_scan(b.dp, self.offsets, n, b.first)
                K.positive_correction(b.dp, self.offsets, self.values, b.first, b.Q, self.E_bf16, b.dQ, self.gE,
                                      self.loss_acc, self.pos_weight, scale, n, self.D, 1, 0)
            # both launches add half of the loss terms each (the epilogue with loss costs several times the one without)
            K.kvsall_fused(self.E_bf16, b.Q, self.gE, self.loss_acc, self.status, self.base, scale, True, loss_share=0)
            K.kvsall_fused(b.Q, self.E_bf16, b.dQ, self.loss_acc, self.status, self.base, scale, True, loss_share=1)
            main.wait_stream(self._side)
        K.compose_backward_owner(self.code, self.normalize, b.h, b.r, self.E, 1, 0, self.NE, self.NR, self.R,
                                 self.coeff, b.dQ, None, 0, 0, self.gE, self.gR,
                                 self.gC if self.coeff_trainable else None, n, self.D, self.status, idx_stride=2)
        self._mark("backward")
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            b.dQ.zero_()
        # one launch: Adam / ADOPT / SGD over entities (refreshing the bf16 shadow), relations and the coefficient; its
        # last block turns the loss accumulator into the step's loss and advances the step counter
        self._tail.launch(self.lr, b1, b2, self.eps, self.weight_decay, scale)
        main.wait_stream(self._side)
        self._mark("tail")

    #: number of kernels of this library launched per step (for launch accounting)
    def launches_per_step(self) -> int:
        return 8 if self.label_mode == "mask" else 7   # kernels of this library

    def _run(self, b, n: int) -> None:
        key = (n, self.lr)
        if self.use_graph and key not in self._graphs and len({k[1] for k in self._graphs}) >= 3:
            # the learning rate is a launch argument; a per-step schedule would re-capture every step
            self.use_graph = False
            self._graphs.clear()
        if not self.use_graph:
            self._launch_all(b, n)
            return
        if key not in self._graphs:
            # warm-up launch outside capture (sets function attributes), then capture
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            state = self._snapshot()
            with torch.cuda.stream(s):
                self._launch_all(b, n)
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            K.check_status(self.status, "during fused-step warm-up")
            self._restore(state)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch_all(b, n)
            self._graphs[key] = g
        self._graphs[key].replay()

    def _snapshot(self):
        t = [self.E, self.R, self.E_bf16, self.mE, self.vE, self.mR, self.vR, self.gE, self.gR, self.step_count,
             self.loss_acc]
        if self.coeff is not None:
            t += [self.coeff, self.gC, self.mC, self.vC]
        return [(x, x.clone()) for x in t]

    @staticmethod
    def _restore(state):
        for x, c in state:
            x.copy_(c)

    # ------------------------------------------------------------------ public
    def step(self, batch) -> torch.Tensor:
        """``batch = (x [n, 2] int64, data-point ids [n] int64)`` on the device; returns the loss (device scalar)."""
        x, dp = batch[0], batch[1]
        n = x.shape[0]
        b = self._buffers(n)
        b.x_in.copy_(x)
        b.dp.copy_(dp)
        self._run(b, n)
        return self.loss_out[0]

    def step_from_host(self, x_pinned: torch.Tensor, dp_pinned: torch.Tensor) -> float:
        """End-to-end step: asynchronous host→device copies of the (pinned) index tensors, the fused step, and a
        device→host read of the loss."""
        n = x_pinned.shape[0]
        b = self._buffers(n)
        b.x_in.copy_(x_pinned, non_blocking=True)
        b.dp.copy_(dp_pinned, non_blocking=True)
        self._run(b, n)
        return float(self.loss_out.item())

    def step_from_host_pipelined(self, x_pinned: torch.Tensor, dp_pinned: torch.Tensor) -> Optional[float]:
        """Like :meth:`step_from_host` but without stalling the host on the step it has just queued: the loss is
        copied to pinned host memory in stream order and the call returns the loss of the *previous* step (``None``
        on the first call; :meth:`last_loss` waits for the newest one).  Every step still carries its own host→device
        input copy and device→host loss copy; the host merely runs one step ahead of the GPU."""
        n = x_pinned.shape[0]
        b = self._buffers(n)
        if not hasattr(self, "_loss_host"):
            self._loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
            self._loss_event = [torch.cuda.Event(), torch.cuda.Event()]
            self._loss_slot, self._loss_pending = 0, False
        prev = None
        if self._loss_pending:
            self._loss_event[self._loss_slot].synchronize()
            prev = float(self._loss_host[self._loss_slot][0])
        b.x_in.copy_(x_pinned, non_blocking=True)
        b.dp.copy_(dp_pinned, non_blocking=True)
        self._run(b, n)
        self._loss_slot ^= 1
        self._loss_host[self._loss_slot].copy_(self.loss_out, non_blocking=True)
        self._loss_event[self._loss_slot].record()
        self._loss_pending = True
        return prev

    def last_loss(self) -> Optional[float]:
        """Loss of the newest pipelined step (waits for it)."""
        if not getattr(self, "_loss_pending", False):
            return None
        self._loss_event[self._loss_slot].synchronize()
        return float(self._loss_host[self._loss_slot][0])

    def sync_to_model(self) -> None:
        """Parameters are updated in place; only kernel failures need surfacing."""
        K.check_status(self.status, "in fused training step")

    def optimizer_view(self):
        """Minimal optimiser façade (``param_groups[0]['lr']``) so LR-scheduling callbacks can steer the engine."""
        return _EngineOptimizer(self)


class _EngineOptimizer:
    def __init__(self, engine: FusedKvsAllEngine):
        self._e = engine
        self.param_groups = [_LrGroup(engine)]
        self.state = {}

    def zero_grad(self, set_to_none: bool = True):
        pass

    def step(self):
        pass

    def state_dict(self):
        e = self._e
        return {"step": int(e.step_count.item()), "lr": e.lr}

    def load_state_dict(self, sd):
        self._e.lr = float(sd.get("lr", self._e.lr))


class _LrGroup(dict):
    def __init__(self, engine):
        super().__init__(lr=engine.lr)
        self._e = engine

    def __setitem__(self, k, v):
        super().__setitem__(k, v)
        if k == "lr":
            self._e.lr = float(v)
