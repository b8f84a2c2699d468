"""pytest configuration: registers the `gpu` marker and puts the repository root on sys.path."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    import torch
    path = os.path.join(ROOT, "tests", "golden", "ref_outputs.pt")
    return torch.load(path, map_location="cpu", weights_only=False)
