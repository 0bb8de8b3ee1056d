"""Multi-GPU checks of the row-sharded engine (needs at least two GPUs; each rank is its own process)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
    pytest.skip("needs two CUDA devices", allow_module_level=True)

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("name,optim", [("ComplEx", "SGD"), ("Keci", "Adam"), ("QMult", "SGD")])
def test_sharded_engines_agree(name, optim):
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(HERE, "_sharded_worker.py"), name, optim]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and "SHARDED_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


def test_sharded_checkpoint_resume_and_sharded_ranking():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29613", os.path.join(HERE, "_sharded_eval_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and "SHARDED_EVAL_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


def test_sharded_sampled_engine_matches_autograd_and_learns():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29615", os.path.join(HERE, "_sharded_sampled_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and "SHARDED_SAMPLED_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.parametrize("st,extra", [("NegSample", ["--neg_ratio", "16"]), ("KvsAll", []),
                                      ("KvsAll", ["--trainer", "torchDDP", "--model", "ConEx", "--num_of_output_channels", "2",
                                                  "--embedding_dim", "32", "--lr", "0.02"])])
def test_sharded_trainer_through_the_command_line(tmp_path, st, extra):
    """``--trainer Sharded`` end to end on two ranks: training, gathering the shards, evaluation, stored run; the
    last case is a model outside the fused kernels on ``torchDDP`` (replicated model, gradient all-reduce)."""
    import json
    sys.path.insert(0, os.path.dirname(HERE))
    from dice_embeddings_b200.data.synthetic import make_planted_kg
    kg = make_planted_kg(str(tmp_path / "kg"), num_entities=300, num_relations=10, seed=1)
    out = tmp_path / "run"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=os.path.dirname(HERE))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29617", "-m", "dice_embeddings_b200", "--dataset_dir", kg, "--model", "ComplEx",
           "--scoring_technique", st, "--trainer", "Sharded", "--embedding_dim", "64", "--num_epochs", "150",
           "--batch_size", "256", "--lr", "0.1", "--optim", "Adam", "--eval_model", "train_val_test",
           "--path_to_store_single_run", str(out)] + extra
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    rep = json.load(open(out / "eval_report.json"))
    assert rep["Train"]["MRR"] > (0.3 if (st != "KvsAll" or "ConEx" in extra) else 0.5), rep
    assert os.path.isfile(out / "model.pt")


def test_peer_allreduce_optimizer_matches_single_process_training():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29619", os.path.join(HERE, "_peer_optimizer_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and "PEER_OPT_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
