import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the two tiny configurations, written once per session into a temporary folder."""
    import torch

    from helpers import CONFIG_A, CONFIG_B, CONFIG_C, CONFIG_D
    from inferrs_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("models")
    return {
        "A": write_random_model(str(base / "A"), CONFIG_A, seed=0, dtype=torch.bfloat16),
        "B": write_random_model(str(base / "B"), CONFIG_B, seed=2, dtype=torch.bfloat16),
        "C": write_random_model(str(base / "C"), CONFIG_C, seed=5, dtype=torch.bfloat16),
        "D": write_random_model(str(base / "D"), CONFIG_D, seed=6, dtype=torch.bfloat16),
    }
