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


def test_batch_loader_pads_the_tail_and_never_yields_zero_steps():
    """A fixed-batch engine gets full batches without losing items: the tail is filled by wrap-around, ``len`` agrees
    with what is yielded, and a batch size above the per-rank share still gives one step."""
    from dice_embeddings_b200.data.datasets import KvsAll
    from dice_embeddings_b200.data.synthetic import uniform_kg
    from dice_embeddings_b200.trainer.base import BatchLoader
    ds = KvsAll(uniform_kg(50, 5, 600, seed=1), 50, 5, label_smoothing_rate=0.0)
    n = len(ds)
    for world, bs in [(1, 64), (4, 64), (4, 10 ** 6), (3, 7)]:
        per = -(-n // world)
        b = min(bs, per)
        seen = []
        for rank in range(world):
            ld = BatchLoader(ds, b, shuffle=True, seed=3, rank=rank, world_size=world, pad_last=True)
            batches = list(ld)
            assert len(batches) == len(ld) >= 1
            assert all(x[0].shape[0] == b for x in batches)
            seen.append(torch.cat([x[0] for x in batches]))
        pairs = {tuple(r) for t in seen for r in t.tolist()}
        assert pairs == {tuple(r) for r in ds.train_data.tolist()}      # every data point was visited
        ld = BatchLoader(ds, b, rank=0, world_size=world, drop_last=True)
        assert len(list(ld)) == len(ld) == per // b


def test_prefetching_loader_keeps_order():
    from dice_embeddings_b200.data.datasets import KvsAll
    from dice_embeddings_b200.data.synthetic import uniform_kg
    from dice_embeddings_b200.trainer.base import BatchLoader
    ds = KvsAll(uniform_kg(40, 4, 400, seed=2), 40, 4, label_smoothing_rate=0.1)
    a = list(BatchLoader(ds, 32, shuffle=True, seed=5))
    b = list(BatchLoader(ds, 32, shuffle=True, seed=5, num_workers=3))
    assert len(a) == len(b) and all(torch.equal(x[0], y[0]) and torch.equal(x[1], y[1]) for x, y in zip(a, b))


def test_partition_csr_keeps_owned_values_as_local_rows():
    from dice_embeddings_b200.parallel.sharded_engine import partition_csr
    g = torch.Generator().manual_seed(0)
    counts = torch.randint(0, 6, (40,), generator=g)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)])
    values = torch.randint(0, 1000, (int(counts.sum()),), generator=g)
    W = 3
    for rank in range(W):
        off, val = partition_csr(offsets, values, W, rank)
        assert off.numel() == offsets.numel() and int(off[-1]) == val.numel()
        for i in range(40):
            want = [int(v) // W for v in values[offsets[i]:offsets[i + 1]].tolist() if v % W == rank]
            assert val[off[i]:off[i + 1]].tolist() == want


HB_WORKER = r'''
import datetime, os, sys, time, torch.distributed as dist
sys.path.insert(0, os.environ["DICE_ROOT"])
from torch.distributed.distributed_c10d import _get_default_store
from dice_embeddings_b200.parallel.watchdog import Heartbeat, RankFailure
rank = int(os.environ["RANK"])
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=30))
hb = Heartbeat(_get_default_store(), rank, 2, timeout=1.5, interval=0.2).start()
for step in range(100):
    try:
        hb.raise_if_failed()            # what the trainer does before every launch
    except RankFailure as e:
        print("RANK_FAILURE_SEEN", e.rank, "at step", step, flush=True)
        os._exit(0)
    if rank == 1 and step == 5:
        hb.stop()                       # rank 1 stops stepping between steps (its process stays, silent)
        time.sleep(8)
        os._exit(0)
    time.sleep(0.1)
print("NO_FAILURE", flush=True)
'''


def test_heartbeat_over_the_process_group_store_reports_a_silent_rank(tmp_path):
    script = tmp_path / "hb_worker.py"
    script.write_text(HB_WORKER)
    res = _torchrun(2, [str(script)], 29673, timeout=120, env_extra={"DICE_ROOT": ROOT})
    assert "RANK_FAILURE_SEEN 1" in res.stdout and "NO_FAILURE" not in res.stdout, res.stdout[-1500:] + res.stderr[-1500:]


def test_pl_trainer_under_torchrun_is_data_parallel(umls_like_dir, tmp_path):
    """The reference's default trainer name means "all devices, data parallel": started with two ranks it must train
    as the data-parallel trainer does (one run folder, rank 0 writes it)."""
    out = tmp_path / "pl"
    res = _torchrun(2, ["-m", "dice_embeddings_b200", "--dataset_dir", umls_like_dir, "--path_to_store_single_run",
                        str(out), "--model", "DistMult", "--scoring_technique", "KvsAll", "--trainer", "PL",
                        "--num_epochs", "30", "--batch_size", "128", "--optim", "Adam", "--embedding_dim", "32",
                        "--lr", "0.1"], 29674)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    rep = json.load(open(out / "eval_report.json"))
    assert rep["Train"]["MRR"] > 0.5 and os.path.isfile(out / "model.pt")
