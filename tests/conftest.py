"""Shared pytest configuration: the ``gpu`` marker and a fixed seed per test."""
import random

import numpy as np
import pytest
import torch


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200); run with `-m gpu`")
    config.addinivalue_line("markers", "multigpu: test needs more than one CUDA device")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    random.seed(95051)
    np.random.seed(95051)
    torch.manual_seed(95051)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(95051)
    yield
