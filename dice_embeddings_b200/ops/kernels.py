"""Typed Python wrappers over the ``extern "C"`` kernel entry points.

Every wrapper takes CUDA tensors, checks dtype / contiguity / device, passes raw pointers plus the current stream
and raises on a non-zero return code.  There is no silent fallback: if the library is missing or the launch is
rejected the call fails.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib

MODEL_CODE = {"DistMult": 0, "ComplEx": 1, "QMult": 2, "OMult": 3, "Keci": 4, "CKeci": 4}
OPT_CODE = {"Adam": 0, "AdamW": 1, "SGD": 2, "Adopt": 3}

STATUS_TEXT = {0: "ok", 1: "producer wait timed out", 2: "mma wait timed out", 3: "epilogue wait timed out",
               4: "peer wait timed out", 5: "index out of range", 6: "inbox overflow", 7: "copy drain timed out"}


class KernelError(RuntimeError):
    pass


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str):
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def _req(t: torch.Tensor, dtype, name: str):
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise KernelError(f"{name}: expected contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}")


def pointer_table(tensors: Sequence[torch.Tensor], device) -> torch.Tensor:
    """Device int64 tensor holding the base addresses of ``tensors`` (an array of pointers for the kernels)."""
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=device)


def kvsall_fused(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor, loss_acc: Optional[torch.Tensor],
                 status: torch.Tensor, base: float, scale: float, with_loss: bool, num_ctas: int = 0) -> None:
    """``out[x_rows, D] += scale · (sigmoid(X Yᵀ) − base) · Y`` and optionally
    ``loss_acc += Σ softplus(X Yᵀ) − base · X Yᵀ`` on the tcgen05 path.  ``x``/``y`` bf16, ``out`` fp32."""
    _req(x, torch.bfloat16, "x")
    _req(y, torch.bfloat16, "y")
    _req(out, torch.float32, "out")
    D = x.shape[1]
    assert y.shape[1] == D and out.shape[0] >= x.shape[0] and out.shape[1] == D
    if with_loss:
        _req(loss_acc, torch.float64, "loss_acc")
    rc = _lib.lib().dice_kvsall_fused(_ptr(x), x.shape[0], _ptr(y), y.shape[0], D, _ptr(out), _ptr(loss_acc),
                                      float(base), float(scale), int(with_loss), _ptr(status), int(num_ctas),
                                      _stream())
    _check(rc, "dice_kvsall_fused")


def lookup_compose(model: int, normalize: bool, idx_h, idx_r, ent_table: torch.Tensor, W: int, num_entities: int,
                   rel: torch.Tensor, coeff: Optional[torch.Tensor], q_dst_table: torch.Tensor, n_dst: int,
                   q_row_offset: int, q_f32: Optional[torch.Tensor], B: int, D: int, status: torch.Tensor) -> None:
    rc = _lib.lib().dice_lookup_compose(model, int(normalize), _ptr(idx_h), _ptr(idx_r), _ptr(ent_table), W,
                                        int(num_entities), _ptr(rel), _ptr(coeff), _ptr(q_dst_table), n_dst,
                                        int(q_row_offset), _ptr(q_f32), B, D, _ptr(status), _stream())
    _check(rc, "dice_lookup_compose")


def compose_backward(model: int, normalize: bool, idx_h, idx_r, ent_table, W: int, rel, coeff, dq, g_ent_table,
                     g_rel, g_coeff, B: int, D: int) -> None:
    rc = _lib.lib().dice_compose_backward(model, int(normalize), _ptr(idx_h), _ptr(idx_r), _ptr(ent_table), W,
                                          _ptr(rel), _ptr(coeff), _ptr(dq), _ptr(g_ent_table), _ptr(g_rel),
                                          _ptr(g_coeff), B, D, _stream())
    _check(rc, "dice_compose_backward")


def positive_scan(dp_idx, offsets, n: int, first) -> None:
    _check(_lib.lib().dice_positive_scan(_ptr(dp_idx), _ptr(offsets), n, _ptr(first), _stream()), "dice_positive_scan")


def positive_correction(dp_idx, offsets, values, first, q, e, dq, de, loss_acc, weight: float, scale: float, n: int,
                        D: int, W: int = 1, rank: int = 0) -> None:
    rc = _lib.lib().dice_positive_correction(_ptr(dp_idx), _ptr(offsets), _ptr(values), _ptr(first), _ptr(q), _ptr(e),
                                             _ptr(dq), _ptr(de), _ptr(loss_acc), float(weight), float(scale), n, D, W,
                                             rank, _stream())
    _check(rc, "dice_positive_correction")


def optimizer_step(kind: int, param, grad, m, v, shadow, step, lr, beta1, beta2, eps, weight_decay) -> None:
    rc = _lib.lib().dice_optimizer_step(kind, _ptr(param), _ptr(grad), _ptr(m), _ptr(v), _ptr(shadow), _ptr(step),
                                        param.numel(), float(lr), float(beta1), float(beta2), float(eps),
                                        float(weight_decay), _stream())
    _check(rc, "dice_optimizer_step")


def cast_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    _check(_lib.lib().dice_cast_bf16(_ptr(src), _ptr(dst), src.numel(), _stream()), "dice_cast_bf16")


def finish_step(acc, loss_out, inv_count: float, step) -> None:
    _check(_lib.lib().dice_finish_step(_ptr(acc), _ptr(loss_out), float(inv_count), _ptr(step), _stream()),
           "dice_finish_step")


def check_status(status: torch.Tensor, where: str = "") -> None:
    """Read the device status word (synchronises) and raise if a kernel reported a failure."""
    code = int(status.item())
    if code != 0:
        status.zero_()
        raise KernelError(f"kernel status {code} ({STATUS_TEXT.get(code, '?')}) {where}")
