"""Shared fixtures: the tiny configurations, model folders with random weights (made in a
temporary folder), and the ``gpu`` marker."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA B200 (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors for every tiny configuration."""
    from tiny import TINY, make_model_dir

    root = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(name, str(root / name)) for name in TINY}
