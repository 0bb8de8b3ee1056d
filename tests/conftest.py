import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def umls_like_dir(tmp_path_factory):
    """Small learnable KG (planted structure) written as train/valid/test text files."""
    from dice_embeddings_b200.data.synthetic import make_planted_kg
    d = tmp_path_factory.mktemp("kg")
    return make_planted_kg(str(d), num_entities=120, num_relations=12, seed=3)
