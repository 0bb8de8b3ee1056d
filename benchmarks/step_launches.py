"""A few training steps of the headline configuration without graph replay: ``python benchmarks/step_launches.py``.

ComplEx, KvsAll, 14 541 entities, 237 relations, 272 115 triples, d = 256, 4096 queries, label smoothing 0.1, Adam: three
warm-up steps and ``--steps`` (default 2) more, every kernel launched separately, the L2 flushed before each step.  The
program is small and ends by itself, which makes it the one to put under a launch list::

    ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file launches.csv \\
        python benchmarks/step_launches.py

It prints the number of kernels of this library per step and the CUDA-event time of the last step.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a source checkout

from dice_embeddings_b200.data.datasets import KvsAll  # noqa: E402
from dice_embeddings_b200.data.synthetic import zipf_kg  # noqa: E402
from dice_embeddings_b200.models import MODEL_REGISTRY  # noqa: E402
from dice_embeddings_b200.ops.fused_step import FusedKvsAllEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--model", default="ComplEx")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    NE, NR, NT, D, B = 14541, 237, 272115, 256, 4096
    ds = KvsAll(zipf_kg(NE, NR, NT, 1.0, 1.0, seed=0), NE, NR, "EntityPrediction", label_smoothing_rate=0.1).to(dev)
    torch.manual_seed(0)
    with torch.device(dev):
        model = MODEL_REGISTRY[a.model][0](dict(model=a.model, embedding_dim=D, num_entities=NE, num_relations=NR,
                                                optim="Adam", learning_rate=0.1, scoring_technique="KvsAll", p=0, q=1))
    eng = FusedKvsAllEngine(model, ds, batch_size=B, lr=0.1, device=dev, use_graph=False)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator().manual_seed(1)
    ms = 0.0
    for i in range(3 + a.steps):
        idx = torch.randperm(len(ds), generator=g)[:B].to(dev)
        x = ds.train_data[idx]
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loss = eng.step((x, idx))
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    eng.sync_to_model()
    print(f"{a.model} KvsAll d={D} B={B}: {eng.launches_per_step()} library kernels per step, last step {ms * 1e3:.1f} us "
          f"without graph replay, loss {float(loss):.5f}")


if __name__ == "__main__":
    main()
