"""Typed Python wrappers over the ``extern "C"`` kernel entry points.

Every wrapper takes CUDA tensors, checks dtype / contiguity / device, passes raw pointers plus a stream and raises on
a non-zero return code.  The launch happens on the device that holds the operands, not on whatever device happens to
be current: the wrapper makes that device current for the call and uses *its* current stream, and it refuses operands
that live on different devices.  There is no silent fallback: if the library is missing or the launch is rejected
the call fails.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from . import _lib

MODEL_CODE = {"DistMult": 0, "ComplEx": 1, "QMult": 2, "OMult": 3, "Keci": 4, "CKeci": 4, "TransE": 5}
OPT_CODE = {"Adam": 0, "AdamW": 1, "SGD": 2, "Adopt": 3}

STATUS_TEXT = {0: "ok", 1: "producer wait timed out", 2: "mma wait timed out", 3: "epilogue wait timed out",
               4: "peer wait timed out", 5: "index out of range", 6: "inbox overflow", 7: "copy drain timed out"}


class KernelError(RuntimeError):
    pass


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _call(name: str, anchor: torch.Tensor, *args, others: Sequence[Optional[torch.Tensor]] = ()) -> None:
    """Launch entry point ``name`` on the device of ``anchor`` (made current for the call) and on that device's
    current stream, which is appended as the last argument.  ``others`` are further tensor operands that must live
    on the same device."""
    dev = anchor.device
    if dev.type != "cuda":
        raise KernelError(f"{name}: operands must be CUDA tensors, got {dev}")
    for t in others:
        if t is not None and t.device != dev:
            raise KernelError(f"{name}: operands on different devices ({dev} and {t.device})")
    with torch.cuda.device(dev):
        rc = getattr(_lib.lib(), name)(*args, torch.cuda.current_stream(dev).cuda_stream)
    _check(rc, name)


def _check(rc: int, what: str):
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def _req(t: torch.Tensor, dtype, name: str):
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise KernelError(f"{name}: expected contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}")


def pointer_table(tensors: Sequence[torch.Tensor], device) -> torch.Tensor:
    """Device int64 tensor holding the base addresses of ``tensors`` (an array of pointers for the kernels)."""
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=device)


def pair_kernel_enabled() -> bool:
    """``DICE_B200_PAIR=1`` routes d = 256 scoring launches to the CTA-pair kernel (``tcgen05.mma.cta_group::2``).
    Both kernels pass the same tests; measured on B200 they are within a few per cent of each other (the pair kernel
    wins the query role on large tables, the one-CTA kernel the loss role and the small benchmark shape), so the
    one-CTA kernel stays the default."""
    return os.environ.get("DICE_B200_PAIR", "0") == "1"


class FusedOptimizerArgs(ctypes.Structure):
    """``DiceFusedOptimizer`` of ``csrc/dice_b200.h``: the optimiser step of the rows of ``x`` applied inside
    :func:`kvsall_fused` by whichever CTA completes a 128-row tile of the gradient."""
    _fields_ = [("param", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p), ("shadow", ctypes.c_void_p),
                ("count", ctypes.c_void_p), ("step", ctypes.c_void_p), ("lr", ctypes.c_float), ("beta1", ctypes.c_float),
                ("beta2", ctypes.c_float), ("eps", ctypes.c_float), ("weight_decay", ctypes.c_float),
                ("kind", ctypes.c_int)]


def fused_optimizer_args(kind: int, param: torch.Tensor, m: torch.Tensor, v: torch.Tensor, shadow: torch.Tensor,
                         count: torch.Tensor, step: torch.Tensor, lr: float, beta1: float, beta2: float, eps: float,
                         weight_decay: float) -> FusedOptimizerArgs:
    _req(param, torch.float32, "param")
    _req(m, torch.float32, "m")
    _req(v, torch.float32, "v")
    _req(shadow, torch.bfloat16, "shadow")
    _req(count, torch.int32, "count")
    _req(step, torch.int64, "step")
    assert count.numel() >= (param.shape[0] + 127) // 128
    a = FusedOptimizerArgs(_ptr(param), _ptr(m), _ptr(v), _ptr(shadow), _ptr(count), _ptr(step), float(lr), float(beta1),
                           float(beta2), float(eps), float(weight_decay), int(kind))
    a._keep = (param, m, v, shadow, count, step)
    return a


def kvsall_fused(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor, loss_acc: Optional[torch.Tensor],
                 status: torch.Tensor, base: float, scale: float, with_loss: bool, num_ctas: int = 0,
                 mask: Optional[torch.Tensor] = None, pos_delta: float = 0.0,
                 trace: Optional[torch.Tensor] = None, loss_share: int = -1, score_mode: int = 0,
                 x_bias: Optional[torch.Tensor] = None, y_bias: Optional[torch.Tensor] = None,
                 x_dsum: Optional[torch.Tensor] = None, margin: float = 0.0,
                 opt: Optional[FusedOptimizerArgs] = None) -> None:
    """``out[x_rows, D] += scale · (sigmoid(X Yᵀ) − base) · Y`` and optionally
    ``loss_acc += Σ softplus(X Yᵀ) − base · X Yᵀ`` on the tcgen05 path.  ``x``/``y`` bf16, ``out`` fp32.

    ``score_mode`` 1 adds one scalar per row of ``x`` and of ``y`` to the logit (``x_bias``, ``y_bias``; fp32, padded
    with readable zeros to a multiple of 128 rows, see :func:`padded_rows`); ``x_dsum [x_rows]`` then receives
    ``scale · Σ_y dS``, the gradient of ``x_bias``.  ``score_mode`` 2 makes the logit
    ``margin − sqrt(x_bias + y_bias − 2 x·y)`` with the squared row norms as biases; ``out`` then holds
    ``scale · Σ_y w y`` with ``w = dS / distance`` and ``x_dsum`` the row sums of ``scale · w``: the gradient with
    respect to ``x`` is ``out − x_dsum[:, None] · x``.  Both modes need a label mask.

    ``opt`` (:func:`fused_optimizer_args`) fuses the optimiser step of the rows of ``x`` into the launch: ``out`` is
    then their gradient buffer, already holding every other contribution, and comes back cleared.

    ``loss_share`` splits the loss arithmetic between the two launches of a training step (the same pairs with the
    roles of ``x`` and ``y`` swapped): launch 0 and launch 1 each add the loss of one half of the ``(x, y)`` plane
    (256 x 256 blocks of alternating parity); ``-1`` keeps all of it in this launch.  The one-CTA kernel does not
    split: there share 0 takes everything and share 1 nothing."""
    pair = x.shape[1] == 256 and score_mode == 0 and opt is None and pair_kernel_enabled()
    if score_mode != 0:
        assert mask is not None and score_mode in (1, 2)
        for t, rows, nm in ((x_bias, x.shape[0], "x_bias"), (y_bias, y.shape[0], "y_bias")):
            if t is not None:
                _req(t, torch.float32, nm)
                assert t.numel() >= padded_rows(rows), f"{nm} must be padded to a multiple of 128 rows"
        if x_dsum is not None:
            _req(x_dsum, torch.float32, "x_dsum")
            assert x_dsum.numel() >= x.shape[0]
    if with_loss and loss_share >= 0 and not pair:
        if loss_share == 1:
            with_loss, loss_acc = False, None
        loss_share = -1
    _req(x, torch.bfloat16, "x")
    _req(y, torch.bfloat16, "y")
    D = x.shape[1]
    _req(out, torch.float32, "out")
    assert out.shape[0] >= x.shape[0] and out.shape[1] == D
    assert y.shape[1] == D
    if with_loss:
        _req(loss_acc, torch.float64, "loss_acc")
    if pair:
        # CTA-pair kernel (tcgen05.mma.cta_group::2): num_ctas counts CTAs, two per pair
        _call("dice_kvsall_pair", x, _ptr(x), x.shape[0], _ptr(y), y.shape[0], D, _ptr(out), _ptr(loss_acc),
              float(base), float(scale), int(with_loss), _ptr(status), int(num_ctas) // 2 if num_ctas > 1 else int(num_ctas),
              _ptr(mask), 0 if mask is None else mask.shape[1], float(pos_delta), int(loss_share), _ptr(trace),
              others=(y, out, loss_acc, status, mask, trace))
        return
    _call("dice_kvsall_fused", x, _ptr(x), x.shape[0], _ptr(y), y.shape[0], D, _ptr(out), _ptr(loss_acc),
          float(base), float(scale), int(with_loss), _ptr(status), int(num_ctas),
          _ptr(mask), 0 if mask is None else mask.shape[1], float(pos_delta), _ptr(trace),
          int(score_mode), _ptr(x_bias), _ptr(y_bias), _ptr(x_dsum), float(margin),
          ctypes.addressof(opt) if opt is not None else None,
          others=(y, out, loss_acc, status, mask, trace, x_bias, y_bias, x_dsum))


def padded_rows(n: int) -> int:
    """Length the per-row scalar vectors of :func:`kvsall_fused` need for ``n`` rows (whole 128-row tiles)."""
    return (int(n) + 127) // 128 * 128


def lookup_compose(model: int, normalize: bool, idx_h, idx_r, ent_table: torch.Tensor, W: int, num_entities: int,
                   rel: torch.Tensor, coeff: Optional[torch.Tensor], q_dst_table: Optional[torch.Tensor], n_dst: int,
                   q_row_offset: int, q_f32: Optional[torch.Tensor], B: int, D: int, status: torch.Tensor,
                   dp_src: Optional[torch.Tensor] = None, dp_dst_table: Optional[torch.Tensor] = None) -> None:
    _call("dice_lookup_compose", rel, model, int(normalize), _ptr(idx_h), _ptr(idx_r), _ptr(ent_table), W,
          int(num_entities), _ptr(rel), _ptr(coeff), _ptr(q_dst_table), n_dst, int(q_row_offset), _ptr(q_f32), B, D,
          _ptr(status), _ptr(dp_src), _ptr(dp_dst_table), others=(idx_h, idx_r, ent_table, status, q_f32))


def lookup_vec_supported(model: int, D: int) -> bool:
    """True when the vectorised lookup / backward kernels cover this model code and embedding width."""
    return bool(_lib.lib().dice_lookup_vec_supported(int(model), int(D)))


def lookup_compose_vec(model: int, normalize: bool, idx_h, idx_r, dp_src: Optional[torch.Tensor],
                       ent_table: torch.Tensor, W: int, num_entities: int, num_relations: int, rel: torch.Tensor,
                       coeff: Optional[torch.Tensor], q_dst_table: Optional[torch.Tensor], n_dst: int, q_mc: int,
                       q_row_offset: int, q_f32: Optional[torch.Tensor], ids_dst_table: Optional[torch.Tensor],
                       ids_stride: int, B: int, D: int, status: torch.Tensor, idx_stride: int = 1) -> None:
    """Head rows are pulled from their owners, composed with the relation rows, and the bf16 query rows are published
    either through the multicast address ``q_mc`` (one ``multimem.st`` per 16 bytes reaches every rank) or to the
    ``n_dst`` buffers of ``q_dst_table``.  ``ids_dst_table``: per-destination index buffers receiving ``h | r | dp``
    (three arrays of ``ids_stride`` entries each).  ``idx_stride``: distance between consecutive entries of ``idx_h`` /
    ``idx_r`` (2 with ``idx_r = idx_h[1:]`` views of a ``[B, 2]`` batch reads the pairs in place)."""
    _call("dice_lookup_compose_vec", rel, int(model), int(normalize), _ptr(idx_h), _ptr(idx_r), int(idx_stride),
          _ptr(dp_src),
          _ptr(ent_table), int(W), int(num_entities), int(num_relations), _ptr(rel), _ptr(coeff), _ptr(q_dst_table),
          int(n_dst), int(q_mc) or None, int(q_row_offset), _ptr(q_f32), _ptr(ids_dst_table), int(ids_stride), int(B),
          int(D), _ptr(status), others=(idx_h, idx_r, dp_src, ent_table, status, q_f32))


def compose_backward(model: int, normalize: bool, idx_h, idx_r, ent_table, W: int, rel, coeff, dq, g_ent_table,
                     g_rel, g_coeff, B: int, D: int, touched_table: Optional[torch.Tensor] = None,
                     dq_table: Optional[torch.Tensor] = None, n_dq: int = 0, dq_row_offset: int = 0) -> None:
    """Chain rule of the composition.  With ``dq_table`` the query gradient of batch item ``i`` is the sum over the
    ``n_dq`` buffers (one per rank) of their row ``dq_row_offset + i``: the reduce-scatter of the partial query
    gradients happens here, by peer loads."""
    _call("dice_compose_backward", rel, model, int(normalize), _ptr(idx_h), _ptr(idx_r), _ptr(ent_table), W,
          _ptr(rel), _ptr(coeff), _ptr(dq), _ptr(g_ent_table), _ptr(g_rel), _ptr(g_coeff), B, D, _ptr(touched_table),
          _ptr(dq_table), int(n_dq), int(dq_row_offset), others=(idx_h, idx_r, dq, g_rel))


def compose_backward_owner(model: int, normalize: bool, idx_h, idx_r, ent_local: torch.Tensor, W: int, rank: int,
                           num_entities: int, num_relations: int, rel: torch.Tensor, coeff, dq, dq_table, n_dq: int,
                           dq_mc: int, g_ent_local: torch.Tensor, g_rel: torch.Tensor, g_coeff, n: int, D: int,
                           status: torch.Tensor, idx_stride: int = 1) -> None:
    """Backward of the composition for the queries whose head row this rank owns.  The query gradient is read through
    the multicast address ``dq_mc`` (``multimem.ld_reduce``: the sum over all ranks is formed inside the switch), else
    as the sum of the ``n_dq`` buffers of ``dq_table`` (peer loads), else from ``dq``.  Row gradients stay local."""
    _req(ent_local, torch.float32, "ent_local")
    _req(g_ent_local, torch.float32, "g_ent_local")
    _req(g_rel, torch.float32, "g_rel")
    _call("dice_compose_backward_owner", rel, int(model), int(normalize), _ptr(idx_h), _ptr(idx_r), int(idx_stride),
          _ptr(ent_local),
          int(W), int(rank), int(num_entities), int(num_relations), _ptr(rel), _ptr(coeff), _ptr(dq), _ptr(dq_table),
          int(n_dq), int(dq_mc) or None, _ptr(g_ent_local), _ptr(g_rel), _ptr(g_coeff), int(n), int(D), _ptr(status),
          others=(idx_h, idx_r, ent_local, dq, g_ent_local, g_rel, status))


def owned_rows(idx_h, n: int, W: int, rank: int, num_entities: int, rows: torch.Tensor, count: torch.Tensor,
               status: torch.Tensor, idx_stride: int = 1) -> None:
    """Compact the batch rows whose head entity this rank owns (``h % W == rank``) into ``rows[0 .. count)``;
    ``count`` (int32 scalar) must be zero on entry."""
    _req(rows, torch.int32, "rows")
    _req(count, torch.int32, "count")
    _call("dice_owned_rows", rows, _ptr(idx_h), int(idx_stride), int(n), int(W), int(rank), int(num_entities),
          _ptr(rows), _ptr(count), _ptr(status), others=(idx_h, count, status))


def dq_pull_owner(rows: torch.Tensor, count: torch.Tensor, dq_table: torch.Tensor, n_dq: int, dq_local: torch.Tensor,
                  D: int, status: torch.Tensor) -> None:
    """Reduce-scatter of the partial query gradients on its own: for the listed batch rows (see :func:`owned_rows`),
    ``dq_local[i] = Σ_k dq_table[k][i]`` (peer loads), in place.  A persistent grid of light blocks (16 bytes per work
    item, ~30 registers) that fits beside a scoring launch, so the NVLink transfer hides under tensor-core work."""
    _req(dq_local, torch.float32, "dq_local")
    _call("dice_dq_pull_owner", dq_local, _ptr(rows), _ptr(count), _ptr(dq_table), int(n_dq), _ptr(dq_local), int(D),
          _ptr(status), others=(rows, count, dq_table, status))


def mask_stride(n_bits: int) -> int:
    """Words per mask row: one bit per column, padded to a multiple of 4 words (and of the 128-column tile)."""
    return ((n_bits + 127) // 128) * 4


def build_label_masks(dp_idx, offsets, values, n: int, W: int, rank: int, mask_q: torch.Tensor,
                      mask_e: torch.Tensor, first: Optional[torch.Tensor] = None,
                      num_data_points: int = 0, num_local_rows: int = 0,
                      status: Optional[torch.Tensor] = None, variant: str = "block") -> None:
    """Set the positive-label bits of a batch in both mask orientations (masks must be zeroed by the caller).

    ``variant``: ``"block"`` (default) is one launch in which every block scans the positive counts of 64 consecutive
    batch items in shared memory and deals their positives to its threads; ``"scan"`` (needs ``first``, int32
    ``[n + 1]`` scratch) counts, scans globally and spreads one thread per positive in three launches; ``"warp"`` walks
    one data point per warp.  ``num_data_points`` / ``num_local_rows`` (with ``status``) switch on range checks of the
    data-point ids and of the CSR values."""
    _req(mask_q, torch.int32, "mask_q")
    _req(mask_e, torch.int32, "mask_e")
    if variant == "scan":
        assert first is not None
    if variant in ("block", "scan"):
        use_first = first if variant == "scan" else None
        if use_first is not None:
            _req(use_first, torch.int32, "first")
            assert use_first.numel() >= n + 1
        _call("dice_build_label_masks_flat", mask_q, _ptr(dp_idx), _ptr(offsets), _ptr(values), _ptr(use_first), n, W,
              rank, _ptr(mask_q), mask_q.shape[1], _ptr(mask_e), mask_e.shape[1], int(num_data_points),
              int(num_local_rows), _ptr(status), others=(dp_idx, offsets, values, use_first, mask_e, status))
        return
    _call("dice_build_label_masks", mask_q, _ptr(dp_idx), _ptr(offsets), _ptr(values), n, W, rank, _ptr(mask_q),
          mask_q.shape[1], _ptr(mask_e), mask_e.shape[1], others=(dp_idx, offsets, values, mask_e))


def positive_scan(dp_idx, offsets, n: int, first) -> None:
    _call("dice_positive_scan", first, _ptr(dp_idx), _ptr(offsets), n, _ptr(first), others=(dp_idx, offsets))


def positive_correction(dp_idx, offsets, values, first, q, e, dq, de, loss_acc, weight: float, scale: float, n: int,
                        D: int, W: int = 1, rank: int = 0, dq_table: Optional[torch.Tensor] = None,
                        dq_block_rows: int = 0) -> None:
    _call("dice_positive_correction", q, _ptr(dp_idx), _ptr(offsets), _ptr(values), _ptr(first), _ptr(q), _ptr(e),
          _ptr(dq), _ptr(de), _ptr(loss_acc), float(weight), float(scale), n, D, W, rank, _ptr(dq_table),
          int(dq_block_rows), others=(dp_idx, offsets, values, first, e, dq, de, loss_acc))


def optimizer_step(kind: int, param, grad, m, v, shadow, step, lr, beta1, beta2, eps, weight_decay,
                   grad_table: Optional[torch.Tensor] = None, n_grad: int = 0, grad_mc: int = 0,
                   status: Optional[torch.Tensor] = None) -> None:
    """Fused Adam / AdamW / SGD / ADOPT sweep.  The gradient is ``grad``, or the sum of the ``n_grad`` buffers of
    ``grad_table`` (peer loads), or the sum over all ranks read through the multicast address ``grad_mc``
    (``multimem.ld_reduce``); with ``status`` the sweep is skipped once that word holds an error."""
    _call("dice_optimizer_step", param, kind, _ptr(param), _ptr(grad), _ptr(m), _ptr(v), _ptr(shadow), _ptr(step),
          param.numel(), float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), _ptr(grad_table),
          int(n_grad), int(grad_mc) or None, _ptr(status), others=(grad, m, v, shadow, step, status))


def bucket_reduce_update(kind: int, p_table: torch.Tensor, p_mc: int, p_local: torch.Tensor, g_table: torch.Tensor,
                         g_mc: int, m: torch.Tensor, v: torch.Tensor, step: torch.Tensor, lo: int, hi: int, W: int,
                         lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, grad_scale: float,
                         status: Optional[torch.Tensor] = None) -> None:
    """Two-shot all-reduce of the slice ``[lo, hi)`` of a flat gradient vector fused with its optimiser update and the
    broadcast of the updated parameters: the gradient slice is summed over the ``W`` ranks (``g_mc``:
    ``multimem.ld_reduce``; else peer loads through ``g_table``), the optimiser is applied to ``p_local[lo:hi]`` with
    the moments ``m`` / ``v``, and the result is stored into every rank's parameter buffer (``p_mc``: ``multimem.st``;
    else peer stores through ``p_table``)."""
    _req(p_local, torch.float32, "p_local")
    _call("dice_bucket_reduce_update", p_local, int(kind), _ptr(p_table), int(p_mc) or None, _ptr(p_local),
          _ptr(g_table), int(g_mc) or None, _ptr(m), _ptr(v), _ptr(step), int(lo), int(hi), int(W), float(lr),
          float(beta1), float(beta2), float(eps), float(weight_decay), float(grad_scale), _ptr(status),
          others=(p_table, g_table, m, v, step, status))


class StepTail:
    """End of a training step as ONE launch: optimiser sweeps over up to three parameter segments and, with
    ``finish=True``, the closing of the step (loss = accumulator / count, accumulator cleared, step counter advanced)
    by the block that finishes last.  The pointer arrays are built once; :meth:`launch` only passes scalars."""

    def __init__(self, kind: int, segments, step: torch.Tensor, status: Optional[torch.Tensor], finish: bool,
                 acc: Optional[torch.Tensor] = None, loss_out: Optional[torch.Tensor] = None,
                 acc_table: Optional[torch.Tensor] = None, n_acc: int = 0, n_grad: int = 0):
        """``segments``: list of dicts with ``param, grad, m, v`` and optional ``shadow`` (bf16), ``grad_table``
        (device pointer table of ``n_grad`` gradient buffers) and ``grad_mc`` (multicast address)."""
        import ctypes
        assert 1 <= len(segments) <= 3
        self.kind, self.n_seg, self.n_grad = int(kind), len(segments), int(n_grad)
        self.step, self.status, self.acc, self.loss_out = step, status, acc, loss_out
        self.acc_table, self.n_acc = acc_table, int(n_acc)
        self.anchor = segments[0]["param"]
        self._keep = segments
        P = ctypes.c_void_p * self.n_seg
        self.param = P(*[s["param"].data_ptr() for s in segments])
        self.grad = P(*[_ptr(s.get("grad")) for s in segments])
        self.m = P(*[_ptr(s.get("m")) for s in segments])
        self.v = P(*[_ptr(s.get("v")) for s in segments])
        self.shadow = P(*[_ptr(s.get("shadow")) for s in segments])
        self.n = (ctypes.c_longlong * self.n_seg)(*[s["param"].numel() for s in segments])
        self.grad_table = P(*[_ptr(s.get("grad_table")) for s in segments])
        self.grad_mc = P(*[(int(s.get("grad_mc") or 0) or None) for s in segments])
        self.done = torch.zeros(1, dtype=torch.int32, device=self.anchor.device) if finish else None

    def launch(self, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, inv_count: float = 1.0):
        _call("dice_step_tail", self.anchor, self.kind, self.n_seg, self.param, self.grad, self.m, self.v, self.shadow,
              self.n, self.grad_table, self.grad_mc, self.n_grad, _ptr(self.step), float(lr), float(beta1),
              float(beta2), float(eps), float(weight_decay), _ptr(self.acc), _ptr(self.loss_out), float(inv_count),
              _ptr(self.acc_table), self.n_acc, _ptr(self.done), _ptr(self.status))


def cast_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    _call("dice_cast_bf16", src, _ptr(src), _ptr(dst), src.numel(), others=(dst,))


def finish_step(acc, loss_out, inv_count: float, step, acc_table: Optional[torch.Tensor] = None, n_acc: int = 0,
                status: Optional[torch.Tensor] = None) -> None:
    _call("dice_finish_step", loss_out, _ptr(acc), _ptr(loss_out), float(inv_count), _ptr(step), _ptr(acc_table),
          int(n_acc), _ptr(status), others=(acc, step, status))


def p2p_barrier(sig_table: torch.Tensor, rank: int, world: int, count: torch.Tensor, status: torch.Tensor,
                spin_limit: int = 0) -> None:
    """Bounded device-side barrier over the ranks' signal arrays (see ``p2p_barrier_kernel``)."""
    _call("dice_p2p_barrier", count, _ptr(sig_table), rank, world, _ptr(count), _ptr(status), int(spin_limit),
          others=(sig_table, status))


def timestamp(slots: torch.Tensor, index: int) -> None:
    """Write the GPU nanosecond timer into ``slots[index]`` (int64) in stream order; capturable in a CUDA graph."""
    _req(slots, torch.int64, "slots")
    _call("dice_timestamp", slots, slots.data_ptr() + 8 * int(index))


def uniform_int(out: torch.Tensor, high: int, seed: int, offset: int = 0, step: Optional[torch.Tensor] = None) -> None:
    """Fill ``out`` (int64; a contiguous tensor or a column block ``m[:, a:b]`` of a contiguous matrix) with uniform
    integers in ``[0, high)`` from the counter-based generator.  ``step`` (device int64 scalar) is added to ``offset``
    on the device, so a captured launch draws fresh numbers at every replay."""
    if not out.is_cuda or out.dtype != torch.int64:
        raise KernelError("out: expected a CUDA int64 tensor")
    if out.is_contiguous():
        stride, row_len = 0, 0
    else:
        assert out.dim() == 2 and out.stride(1) == 1, "only column blocks of a row-major matrix are supported"
        stride, row_len = out.stride(0), out.shape[1]
    _call("dice_uniform_int", out, _ptr(out), out.numel(), int(high), int(seed) & (2 ** 64 - 1),
          int(offset) & (2 ** 64 - 1), _ptr(step), int(stride), int(row_len), others=(step,))


def neg_sample(pos: torch.Tensor, k: int, num_entities: int, seed: int, offset: int, y: torch.Tensor,
               x: Optional[torch.Tensor] = None, hrt: Optional[Sequence[torch.Tensor]] = None,
               label_pos: float = 1.0, label_neg: float = 0.0, per_negative_coin: bool = False,
               step: Optional[torch.Tensor] = None) -> None:
    """Row ``i < B`` of the output is ``pos[i]``; row ``B + j·B + i`` is the j-th corruption of ``pos[i]`` (head or
    tail replaced by a uniform entity).  Written as ``x [N, 3]`` and / or three column tensors ``hrt``; ``y`` gets
    the labels.  ``step`` (device int64 scalar) is added to ``offset`` on the device."""
    _req(pos, torch.int64, "pos")
    _req(y, torch.float32, "y")
    B = pos.shape[0]
    N = B * (1 + k)
    assert y.numel() >= N
    if x is not None:
        _req(x, torch.int64, "x")
        assert x.shape[0] >= N
    h = r = t = None
    if hrt is not None:
        h, r, t = hrt
        for c in (h, r, t):
            _req(c, torch.int64, "hrt")
            assert c.numel() >= N
    _call("dice_neg_sample", pos, _ptr(pos), B, int(k), int(num_entities), int(seed) & (2 ** 64 - 1),
          int(offset) & (2 ** 64 - 1), _ptr(step), int(per_negative_coin), float(label_pos), float(label_neg),
          _ptr(x), _ptr(h), _ptr(r), _ptr(t), _ptr(y), others=(y, x, h, r, t, step))


def candidate_bce(q: torch.Tensor, cand: torch.Tensor, cand_stride: int, cand_step: int, C: int,
                  labels: Optional[torch.Tensor], ent_table: torch.Tensor, W: int,
                  g_ent_table: Optional[torch.Tensor] = None, dq: Optional[torch.Tensor] = None,
                  scores: Optional[torch.Tensor] = None, loss_acc: Optional[torch.Tensor] = None,
                  scale: float = 1.0, kind: int = 0, margin: float = 0.0, eps: float = 0.0,
                  touched_table: Optional[torch.Tensor] = None, num_entities: int = 0,
                  status: Optional[torch.Tensor] = None) -> None:
    """Scores of every query against its own candidate list, BCE loss and gradients (see ``dice_candidate_bce``).
    With ``num_entities`` and ``status`` candidate ids outside ``[0, num_entities)`` are reported and skipped."""
    _req(q, torch.float32, "q")
    _req(cand, torch.int64, "cand")
    if labels is not None:
        _req(labels, torch.float32, "labels")
    if dq is not None:
        _req(dq, torch.float32, "dq")
    if loss_acc is not None:
        _req(loss_acc, torch.float64, "loss_acc")
    N, D = q.shape
    _call("dice_candidate_bce", q, _ptr(q), _ptr(cand), int(cand_stride), int(cand_step), int(C), _ptr(labels),
          _ptr(ent_table), _ptr(g_ent_table), _ptr(dq), _ptr(scores), _ptr(loss_acc), float(scale), int(kind),
          float(margin), float(eps), N, D, int(W), _ptr(touched_table), int(num_entities), _ptr(status),
          others=(cand, labels, ent_table, dq, scores, loss_acc, status))


def sparse_rows_optimizer(kind: int, param, grad, m, v, shadow, touched: torch.Tensor, step, lr, beta1, beta2, eps,
                          weight_decay) -> None:
    """Update only the rows of ``param [rows, D]`` whose ``touched`` flag (uint8) is set; clears flag and gradient."""
    _req(touched, torch.uint8, "touched")
    rows, D = param.shape
    _call("dice_sparse_rows_optimizer", param, int(kind), _ptr(param), _ptr(grad), _ptr(m), _ptr(v), _ptr(shadow),
          _ptr(touched), int(rows), int(D), _ptr(step), float(lr), float(beta1), float(beta2), float(eps),
          float(weight_decay), others=(grad, m, v, shadow, touched, step))


def eval_rank(x: torch.Tensor, y: torch.Tensor, target: Optional[torch.Tensor], target_idx: Optional[torch.Tensor],
              greater: Optional[torch.Tensor], status: torch.Tensor, col_bias: Optional[torch.Tensor] = None,
              y_offset: int = 0, y_stride: int = 1, k: int = 0, cand_score: Optional[torch.Tensor] = None,
              cand_idx: Optional[torch.Tensor] = None, cand_count: Optional[torch.Tensor] = None,
              num_ctas: int = 0, margin: Optional[torch.Tensor] = None, band_rows: Optional[torch.Tensor] = None,
              band_cols: Optional[torch.Tensor] = None, band_count: Optional[torch.Tensor] = None,
              row_floor: Optional[torch.Tensor] = None) -> None:
    """``greater[i] += #{c : (x_i · y_c + col_bias[c]) > target[i], c != column of target_idx[i]}`` on the tcgen05
    path, plus per-segment top-``k`` candidates appended to ``cand_*`` when ``k > 0``.  Nothing of the score matrix
    is written to memory.  With ``margin`` (band mode) only scores above ``target + margin`` are counted and the
    pairs within ``±margin`` of the target are appended to ``band_rows / band_cols`` (``band_count``: int64 scalar)
    for :func:`eval_band_exact`.  ``row_floor`` (top-k mode; fp32 ``[x_rows]`` filled with ``-inf``) lets finished
    segments publish their k-th best score so that later segments of the same row start with a tight threshold."""
    _req(x, torch.bfloat16, "x")
    if row_floor is not None:
        _req(row_floor, torch.float32, "row_floor")
    _req(y, torch.bfloat16, "y")
    assert x.shape[1] == y.shape[1]
    if target is not None:
        _req(target, torch.float32, "target")
    if target_idx is not None:
        _req(target_idx, torch.int32, "target_idx")
    if greater is not None:
        _req(greater, torch.int32, "greater")
    if col_bias is not None:
        _req(col_bias, torch.float32, "col_bias")
    cap = 0
    if k != 0:   # k > 0: running top-k per segment; k == -1: collect every score >= row_floor[row]
        _req(cand_score, torch.float32, "cand_score")
        _req(cand_idx, torch.int32, "cand_idx")
        _req(cand_count, torch.int32, "cand_count")
        cap = cand_score.shape[1]
    _call("dice_eval_rank", x, _ptr(x), x.shape[0], _ptr(y), y.shape[0], x.shape[1], _ptr(target), _ptr(target_idx),
          _ptr(col_bias), int(y_offset), int(y_stride), _ptr(greater), int(k), int(cap), _ptr(cand_score),
          _ptr(cand_idx), _ptr(cand_count), _ptr(status), int(num_ctas), _ptr(margin), _ptr(band_rows),
          _ptr(band_cols), _ptr(band_count), 0 if band_rows is None else band_rows.numel(), _ptr(row_floor),
          others=(y, target, target_idx, greater, status, col_bias, cand_score, cand_idx, cand_count, margin,
                  band_rows, band_cols, band_count, row_floor))


def eval_band_exact(q: torch.Tensor, y: torch.Tensor, band_rows: torch.Tensor, band_cols: torch.Tensor,
                    band_count: torch.Tensor, target: torch.Tensor, greater: torch.Tensor,
                    col_bias: Optional[torch.Tensor] = None, y_offset: int = 0, y_stride: int = 1) -> None:
    """Exact fp32 decision for the pairs the band mode of :func:`eval_rank` left open."""
    _req(q, torch.float32, "q")
    _req(y, torch.float32, "y")
    _req(band_rows, torch.int32, "band_rows")
    _req(band_cols, torch.int32, "band_cols")
    _req(band_count, torch.int64, "band_count")
    _req(greater, torch.int32, "greater")
    _call("dice_eval_band_exact", q, _ptr(q), _ptr(y), q.shape[1], y.shape[0], int(y_offset), int(y_stride),
          _ptr(col_bias), _ptr(band_rows), _ptr(band_cols), _ptr(band_count), band_rows.numel(), _ptr(target),
          _ptr(greater), others=(y, band_rows, band_cols, band_count, target, greater, col_bias))


def eval_rank_cand_cap(x_rows: int, y_rows: int, D: int, k: int, num_ctas: int = 0) -> int:
    """Capacity (entries per row) the candidate lists of ``eval_rank`` need for this problem shape."""
    return int(_lib.lib().dice_eval_rank_cand_cap(int(x_rows), int(y_rows), int(D), int(k), int(num_ctas)))


def eval_sparse(q: torch.Tensor, y: torch.Tensor, target_idx: torch.Tensor, target_score: Optional[torch.Tensor],
                filtered_greater: Optional[torch.Tensor], filt_ptr: Optional[torch.Tensor] = None,
                filt_cols: Optional[torch.Tensor] = None, col_bias: Optional[torch.Tensor] = None,
                target_in: Optional[torch.Tensor] = None, y_offset: int = 0, y_stride: int = 1) -> None:
    """Gather-dots of the ranking protocol: the target score of each query and the number of filtered entities (CSR
    ``filt_ptr`` int64 / ``filt_cols`` int32) that beat it."""
    fp32 = q.dtype == torch.float32
    _req(q, torch.float32 if fp32 else torch.bfloat16, "q")
    _req(y, q.dtype, "y")
    _req(target_idx, torch.int32, "target_idx")
    if filt_ptr is not None:
        _req(filt_ptr, torch.int64, "filt_ptr")
        _req(filt_cols, torch.int32, "filt_cols")
    _call("dice_eval_sparse", q, _ptr(q), _ptr(y), q.shape[0], q.shape[1], y.shape[0], int(y_offset), int(y_stride),
          _ptr(target_idx), _ptr(col_bias), _ptr(target_in), _ptr(filt_ptr), _ptr(filt_cols), _ptr(target_score),
          _ptr(filtered_greater), int(fp32),
          others=(y, target_idx, col_bias, target_in, filt_ptr, filt_cols, target_score, filtered_greater))


def peer_sum_f32(table: torch.Tensor, W: int, out: torch.Tensor, n: int, status: Optional[torch.Tensor] = None) -> None:
    """``out[i] = Σ_k table[k][i]`` over the ``W`` buffers (peer memory) whose base addresses ``table`` holds."""
    _req(out, torch.float32, "out")
    _call("dice_peer_sum_f32", out, _ptr(table), int(W), _ptr(out), int(n), _ptr(status), others=(table, status))


def merge_ranks(greater_table: torch.Tensor, filtered_table: torch.Tensor, W: int, ranks: torch.Tensor, n: int,
                status: Optional[torch.Tensor] = None) -> None:
    """``ranks[i] = 1 + Σ_k greater_k[i] − Σ_k filtered_k[i]`` from every rank's int32 count buffers (peer loads)."""
    _req(ranks, torch.int64, "ranks")
    _call("dice_merge_ranks", ranks, _ptr(greater_table), _ptr(filtered_table), int(W), _ptr(ranks), int(n),
          _ptr(status), others=(greater_table, filtered_table, status))


def merge_topk(score_table: torch.Tensor, idx_table: torch.Tensor, W: int, k: int, stride: int, out_s: torch.Tensor,
               out_i: torch.Tensor, n: int, status: Optional[torch.Tensor] = None) -> None:
    """Best ``k`` of the ``W · k`` candidates per query held in every rank's candidate buffers (peer loads)."""
    _req(out_s, torch.float32, "out_s")
    _req(out_i, torch.int64, "out_i")
    _call("dice_merge_topk", out_s, _ptr(score_table), _ptr(idx_table), int(W), int(k), int(stride), _ptr(out_s),
          _ptr(out_i), int(n), _ptr(status), others=(score_table, idx_table, out_i, status))


def check_status(status: torch.Tensor, where: str = "") -> None:
    """Read the device status word (synchronises) and raise if a kernel reported a failure."""
    code = int(status.item())
    if code != 0:
        status.zero_()
        raise KernelError(f"kernel status {code} ({STATUS_TEXT.get(code, '?')}) {where}")
