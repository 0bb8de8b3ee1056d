"""Stand-alone timing of the ranking kernel: ``python benchmarks/kernel_eval.py``.

Times ``eval_rank`` (counting mode and top-k mode) with CUDA events after warm-up, flushing L2 between launches, and
reports the achieved tensor throughput (one GEMM of ``2·B·|E|·D`` FLOP per launch) as a fraction of the cuBLAS bf16
figure in ``MEASURED_PEAKS.json``.  With ``--compare`` it also times the PyTorch formulation of the same counts
(``torch.mm`` per 1024 queries + comparison + row sum).  It is the small, self-terminating program used for ``ncu``
captures of this kernel."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout

import torch

from dice_embeddings_b200.utils.profiling import measured_peaks
from dice_embeddings_b200.ops import kernels as K
from dice_embeddings_b200.ops.eval_rank import FusedRanker


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--queries", type=int, default=4096)
    ap.add_argument("--entities", type=int, default=262144)
    ap.add_argument("--d", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--topk", type=int, default=0, help="also time top-k mode with this k on the first 256 queries")
    ap.add_argument("--topk_queries", type=int, default=256)
    ap.add_argument("--compare", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    q = (torch.randn(a.queries, a.d, device=dev) * 0.3).to(torch.bfloat16)
    y = (torch.randn(a.entities, a.d, device=dev) * 0.3).to(torch.bfloat16)
    tgt = torch.randint(0, a.entities, (a.queries,), device=dev, dtype=torch.int32)
    ts = torch.zeros(a.queries, device=dev)
    greater = torch.zeros(a.queries, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    K.eval_sparse(q, y, tgt, ts, None)
    pk = measured_peaks()

    def timed(fn, iters):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        ms = 0.0
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms += e0.elapsed_time(e1)
        return ms / iters

    ms = timed(lambda: K.eval_rank(q, y, ts, tgt, greater, status), a.iters)
    tf = 2.0 * a.queries * a.entities * a.d / (ms * 1e-3) / 1e12
    print(f"eval_rank  B={a.queries} E={a.entities} D={a.d}: {ms * 1e3:9.1f} us  {tf:7.1f} TFLOP/s  "
          f"{tf / pk['bf16_tflops']:.2f} of {pk['source']} ({pk['bf16_tflops']:.0f})")
    if a.topk:
        r = FusedRanker(y)
        n = min(a.topk_queries, a.queries)
        ms = timed(lambda: r.topk(q[:n], a.topk), max(a.iters // 2, 1))
        print(f"top-{a.topk} of {n} queries over {a.entities} entities: {ms * 1e3:9.1f} us (with candidate merge)")
        cap = K.eval_rank_cand_cap(n, a.entities, a.d, a.topk)
        cs = torch.full((n, cap), float("-inf"), device=dev)
        ci = torch.full((n, cap), -1, dtype=torch.int32, device=dev)
        cc = torch.zeros(n, dtype=torch.int32, device=dev)
        qn = q[:n].contiguous()

        fl = torch.empty(n, device=dev)

        def kernel_only():
            cc.zero_()
            fl.fill_(float("-inf"))
            K.eval_rank(qn, y, None, None, None, status, k=a.topk, cand_score=cs, cand_idx=ci, cand_count=cc,
                        row_floor=fl)
        ms = timed(kernel_only, max(a.iters // 2, 1))
        tfk = 2.0 * n * a.entities * a.d / (ms * 1e-3) / 1e12
        print(f"   kernel alone: {ms * 1e3:9.1f} us  {tfk:7.1f} TFLOP/s  (candidate capacity {cap} per row)")
    if a.compare:
        def torch_counts():
            out = []
            for i in range(0, a.queries, 1024):
                s = q[i:i + 1024] @ y.t()
                out.append((s > ts[i:i + 1024, None].to(s.dtype)).sum(1))
            return torch.cat(out)
        ms = timed(torch_counts, max(a.iters // 3, 1))
        print(f"torch.mm + compare + sum (1024-query slices): {ms * 1e3:9.1f} us")
    K.check_status(status)


if __name__ == "__main__":
    main()
