"""Shared fixtures.  Tests that need a GPU carry ``@pytest.mark.gpu``; everything else runs
on the CPU.  Model folders are written to temporary folders and never committed."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Tiny random-weight model folders, one per tiny configuration."""
    import tiny

    out = {}
    for name in tiny.CONFIGS:
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        tiny.write_model(name, str(d))
        out[name] = str(d)
    return out
