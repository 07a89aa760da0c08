"""pytest configuration: the ``gpu`` marker and the package import.

The package directory carries a hyphen (``llm-experiments_b200``), which Python
cannot import by name, so ``__graft_entry__.import_package`` registers it as
``llm_experiments_b200``.
"""
import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "reference_recipes.npz")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__

    return __graft_entry__.import_package()
