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
