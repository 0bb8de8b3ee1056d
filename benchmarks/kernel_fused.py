"""Stand-alone timing of the fused scoring kernel: ``python benchmarks/kernel_fused.py``.

Times both roles of ``kvsall_fused`` (entity-stationary with loss, query-stationary) with CUDA events after
warm-up, flushing L2 between launches, and reports the achieved tensor throughput (two GEMMs of
``2·nx·ny·D`` FLOP per launch) as a fraction of the cuBLAS bf16 figure in ``MEASURED_PEAKS.json`` when that file
is present (else of 1.59 PFLOP/s).  It is also the small, self-terminating program used for ``ncu`` captures.
"""
from __future__ import annotations

import argparse
import json
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout

from dice_embeddings_b200.ops import kernels as K


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--nx", type=int, default=14541)
    ap.add_argument("--ny", type=int, default=4096)
    ap.add_argument("--d", type=int, default=256)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--mask", action="store_true")
    ap.add_argument("--trace", action="store_true", help="print per-tile pipeline stamps of CTA 0 (cycles)")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    x = (torch.randn(a.nx, a.d, device=dev) * 0.1).to(torch.bfloat16)
    y = (torch.randn(a.ny, a.d, device=dev) * 0.1).to(torch.bfloat16)
    out_x, out_y = torch.zeros(a.nx, a.d, device=dev), torch.zeros(a.ny, a.d, device=dev)
    loss = torch.zeros(1, dtype=torch.float64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    mx = torch.zeros(a.nx, K.mask_stride(a.ny), dtype=torch.int32, device=dev) if a.mask else None
    my = torch.zeros(a.ny, K.mask_stride(a.nx), dtype=torch.int32, device=dev) if a.mask else None
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peak, tag = 1590.0, "of fallback"
    pk = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(pk):
        peak, tag = float(json.load(open(pk))["bf16_tflops"]), "of measured"
    tr = {"buf": None}
    roles = [("X=entities (loss)", lambda: K.kvsall_fused(x, y, out_x, loss, status, 0.0, 1.0, True, mask=mx, pos_delta=1.0,
                                                         trace=tr["buf"])),
             ("X=queries", lambda: K.kvsall_fused(y, x, out_y, None, status, 0.0, 1.0, False, mask=my, pos_delta=1.0,
                                                  trace=tr["buf"]))]
    flop = 2 * 2.0 * a.nx * a.ny * a.d
    for name, fn in roles:
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        ms = 0.0
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms += e0.elapsed_time(e1)
        ms /= a.iters
        tf = flop / (ms * 1e-3) / 1e12
        print(f"{name:20s} nx={a.nx} ny={a.ny} D={a.d} mask={a.mask}: {ms * 1e3:8.1f} us  {tf:7.1f} TFLOP/s  "
              f"{tf / peak:.2f} {tag} ({peak:.0f})")
        if a.trace:
            buf = torch.zeros(64, 8, dtype=torch.int64, device=dev)
            tr["buf"] = buf
            fn()
            torch.cuda.synchronize()
            tr["buf"] = None
            t = buf.cpu()
            t0 = int(t[0, 0])
            print("  tile | Y load issued | S gemm issued | 2nd gemm issued | epi sees S | epi wrote dS | out drained"
                  " | 2nd-half load issued")
            for g in range(64):
                if int(t[g, 0]) == 0:
                    break
                print("  %4d | %s" % (g, " | ".join("%8d" % (int(v) - t0) if int(v) else "       -" for v in t[g, :7])))
    K.check_status(status)


if __name__ == "__main__":
    main()
