import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(autouse=True)
def _full_fp32_matmul():
    """The reference switches ``torch.set_float32_matmul_precision('high')`` on at import
    (``dicee/trainer/torch_trainer_ddp.py:8``), and the parity tests import it while this directory is collected.
    fp32 oracles of the GPU tests need real fp32 products, so every test starts from the default again."""
    import torch
    torch.set_float32_matmul_precision("highest")
    yield


@pytest.fixture(scope="session")
def umls_like_dir(tmp_path_factory):
    """Small learnable KG (planted structure) written as train/valid/test text files."""
    from dice_embeddings_b200.data.synthetic import make_planted_kg
    d = tmp_path_factory.mktemp("kg")
    return make_planted_kg(str(d), num_entities=120, num_relations=12, seed=3)
