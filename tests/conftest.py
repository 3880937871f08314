import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders with random bfloat16 weights for the tiny configurations, written
    once per session into a temporary folder."""
    import torch
    from kidi_b200 import write_random_model
    from tiny_configs import ALL, sharpen_logits

    root = tmp_path_factory.mktemp("models")
    folders = {}
    for seed, (name, config) in enumerate(ALL.items()):
        folders[name] = write_random_model(config, str(root / name), seed=seed, dtype=torch.bfloat16)
        sharpen_logits(folders[name])
    return folders
