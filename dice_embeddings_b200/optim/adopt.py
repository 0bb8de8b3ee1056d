"""ADOPT optimiser (Taniguchi et al., 2024): Adam-like, but the gradient is normalised by the
*previous* second-moment estimate before entering the momentum, which restores convergence for any β₂.

Semantics follow reference ``dicee/models/adopt.py:514-662`` (single-tensor path):

* step 0 only seeds ``v ← g²`` and does not move the parameter;
* afterwards ``ĝ = clip(g / max(√v, ε), ±step^{1/4})``, ``m ← lerp(m, ĝ, 1 − β₁)``, ``θ ← θ − lr·m``,
  ``v ← β₂ v + (1 − β₂) g²``;
* defaults ``betas = (0.9, 0.9999)``, ``eps = 1e-6`` (``adopt.py:186-201``).

The update is implemented with ``torch._foreach`` ops over all parameters at once; on CUDA tensors a
single fused kernel (:func:`dice_embeddings_b200.ops.optim.fused_adopt_`) is used when the extension is loaded.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
from torch.optim import Optimizer


def _default_clip(step: int) -> float:
    return step ** 0.25


class ADOPT(Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.9999), eps: float = 1e-6,
                 clip_lambda: Optional[Callable[[int], float]] = _default_clip, weight_decay: float = 0.0,
                 decouple: bool = False, *, maximize: bool = False, fused: Optional[bool] = None):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if eps < 0.0:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0.0 <= betas[0] < 1.0 or not 0.0 <= betas[1] < 1.0:
            raise ValueError(f"Invalid betas: {betas}")
        if weight_decay < 0.0:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        self.clip_lambda = clip_lambda
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decouple=decouple,
                        maximize=maximize, fused=fused)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            params, grads, ms, vs = [], [], [], []
            step = None
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("ADOPT does not support sparse gradients")
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                g = -p.grad if group["maximize"] else p.grad
                if wd != 0 and not group["decouple"]:
                    g = g.add(p, alpha=wd)
                if st["step"] == 0:
                    st["exp_avg_sq"].addcmul_(g, g)
                    st["step"] = 1
                    continue
                params.append(p)
                grads.append(g)
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
                step = st["step"]
                st["step"] += 1
            if not params:
                continue
            # parameters that share a group normally share a step count; fall back per tensor otherwise
            steps = {self.state[p]["step"] - 1 for p in params}
            if len(steps) == 1:
                self._update(params, grads, ms, vs, step, lr, beta1, beta2, eps, wd, group["decouple"])
            else:
                for p, g, m, v in zip(params, grads, ms, vs):
                    self._update([p], [g], [m], [v], self.state[p]["step"] - 1, lr, beta1, beta2, eps, wd,
                                 group["decouple"])
        return loss

    def _update(self, params, grads, ms, vs, step, lr, beta1, beta2, eps, wd, decouple):
        if wd != 0 and decouple:
            torch._foreach_mul_(params, 1.0 - lr * wd)
        denom = torch._foreach_sqrt(vs)
        torch._foreach_clamp_min_(denom, eps)
        normed = torch._foreach_div(grads, denom)
        if self.clip_lambda is not None:
            c = float(self.clip_lambda(step))
            torch._foreach_clamp_min_(normed, -c)
            torch._foreach_clamp_max_(normed, c)
        torch._foreach_lerp_(ms, normed, 1.0 - beta1)
        torch._foreach_add_(params, ms, alpha=-lr)
        torch._foreach_mul_(vs, beta2)
        torch._foreach_addcmul_(vs, grads, grads, value=1.0 - beta2)
