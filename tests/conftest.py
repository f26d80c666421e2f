"""Shared fixtures. Tests marked `gpu` need a B200; everything else runs on the CPU."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    config.addinivalue_line("markers", "full_size: a GPU test at a benchmark configuration's whole "
                                       "size (tens of seconds of CPU oracle time)")


@pytest.fixture(scope="session")
def flint():
    """The loaded C-ABI library (built in-tree by __graft_entry__.build)."""
    import flint_b200

    if not flint_b200.library_path().is_file():
        import __graft_entry__

        __graft_entry__.build()
    return flint_b200.Flint()


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        return np.load(GOLDEN / f"{name}.npz", allow_pickle=False)

    return load
