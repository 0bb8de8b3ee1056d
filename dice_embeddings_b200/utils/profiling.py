"""Device-side timing and trace annotations.

The reference only has wall-clock decorators (``dicee/static_funcs.py:129-146``).  Here every phase of a step can be
bracketed by CUDA events on the launching stream (:class:`PhaseTimer`) and by NVTX ranges (:func:`nvtx_range`) that
show up in Nsight timelines; ``roofline_fraction`` relates an achieved rate to the peaks measured on this machine."""
from __future__ import annotations

import contextlib
import json
import os
from collections import OrderedDict
from typing import Dict, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """``mark(name)`` records an event; ``times()`` synchronises once and returns milliseconds per phase (time from
    the previous mark), summed over repeated marks of the same name."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._events = []

    def mark(self, name: str) -> None:
        if self.enabled:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._events.append((name, e))

    def times(self, reset: bool = True) -> Dict[str, float]:
        out: "OrderedDict[str, float]" = OrderedDict()
        if not self._events:
            return out
        torch.cuda.synchronize()
        for (_, a), (name, b) in zip(self._events[:-1], self._events[1:]):
            if name != "start":
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        if reset:
            self._events = []
        return out


def measured_peaks(root: Optional[str] = None) -> Dict[str, float]:
    """``{"hbm_gbs", "bf16_tflops", "bf16_tflops_sustained", "source"}`` from ``MEASURED_PEAKS.json`` at the
    repository root when present, else an earlier measurement of the same GPU model."""
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def roofline_fraction(flops: float = 0.0, bytes_moved: float = 0.0, seconds: float = 1.0,
                      peaks: Optional[Dict[str, float]] = None) -> Dict[str, float]:
    """Achieved TFLOP/s and GB/s of a kernel and their fractions of the peaks."""
    p = peaks or measured_peaks()
    tf, gb = flops / seconds / 1e12, bytes_moved / seconds / 1e9
    return {"tflops": tf, "gbs": gb, "frac_compute": tf / p["bf16_tflops"], "frac_memory": gb / p["hbm_gbs"],
            "peaks": p["source"]}
