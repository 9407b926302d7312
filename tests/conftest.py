import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(REPO, "tests", "golden", "reference_outputs.npz")
    return np.load(path)


@pytest.fixture(autouse=True)
def _isolated_dispatch_cache(tmp_path, monkeypatch):
    # every test gets its own on-disk dispatcher cache
    monkeypatch.setenv("TRITONIX_B200_CACHE_DIR", str(tmp_path / "dispatch_cache"))
