import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)

import __graft_entry__ as entry  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def syn(pkg):
    return pkg.synthetic


@pytest.fixture(scope="session")
def ops(pkg):
    """The drop-in operator module; importing it needs neither CUDA nor the built library."""
    import importlib

    return importlib.import_module("pcfg_nat_b200.custom_ops.pcfg_loss")


def golden_path(name):
    return os.path.join(GOLDEN, name)
