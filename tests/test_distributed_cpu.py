"""Multi-process paths on CPU ranks (Gloo): the data-parallel trainer launched through torchrun + the CLI, sharding
arithmetic, and host-side failure detection (a rank that never joins ends the collective with an error)."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(n, args, port, timeout=600, env_extra=None):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port)] + args
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def test_ddp_trainer_two_gloo_ranks(umls_like_dir, tmp_path):
    out = tmp_path / "ddp"
    res = _torchrun(2, ["-m", "dice_embeddings_b200", "--dataset_dir", umls_like_dir, "--path_to_store_single_run",
                        str(out), "--model", "ComplEx", "--scoring_technique", "KvsAll", "--trainer", "torchDDP",
                        "--num_epochs", "40", "--batch_size", "128", "--optim", "Adam", "--embedding_dim", "32",
                        "--lr", "0.1"], 29671)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    rep = json.load(open(out / "eval_report.json"))
    assert rep["Train"]["MRR"] > 0.6
    assert os.path.isfile(out / "model.pt") and os.path.isfile(out / "memory_map_details.json")


def test_cyclic_sharding_roundtrip():
    from dice_embeddings_b200.parallel.sharded_engine import (local_row, owner_of, scatter_shard_back, shard_rows,
                                                              take_shard)
    for n, w in [(10, 3), (7, 8), (1003, 4), (16, 4)]:
        full = torch.arange(n * 2, dtype=torch.float32).view(n, 2)
        rebuilt = torch.zeros_like(full)
        total = 0
        for r in range(w):
            sh = take_shard(full, r, w)
            assert sh.shape[0] == shard_rows(n, r, w)
            total += sh.shape[0]
            pad = torch.zeros((n + w - 1) // w, 2)
            pad[: sh.shape[0]] = sh
            scatter_shard_back(rebuilt, pad, r, w)
        assert total == n and torch.equal(rebuilt, full)
        e = torch.arange(n)
        assert torch.equal(owner_of(e, w) + w * local_row(e, w), e)


WORKER = r'''
import datetime, os, sys, torch, torch.distributed as dist
rank = int(os.environ["RANK"])
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
t = torch.ones(1)
dist.all_reduce(t)          # both ranks present: succeeds
if rank == 1:
    os._exit(0)             # leaves between steps, nothing in flight
try:
    dist.all_reduce(t)      # the survivor's next collective must fail fast, not hang
    print("NO_ERROR")
except Exception as e:
    print("DETECTED", type(e).__name__)
'''


def test_missing_rank_is_detected_by_timeout(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    res = _torchrun(2, [str(script)], 29672, timeout=120)
    assert "DETECTED" in res.stdout and "NO_ERROR" not in res.stdout, res.stdout[-1500:] + res.stderr[-1500:]
