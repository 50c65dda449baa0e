import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device")


@pytest.fixture(scope="session")
def built():
    """Build the native parts once per session (a no-op when they are up to date)."""
    subprocess.check_call(["make", "-j", str(os.cpu_count() or 4)], cwd=REPO, stdout=subprocess.DEVNULL)
    return REPO


@pytest.fixture(scope="session")
def test_binary(built):
    return os.path.join(built, "build", "bin", "tpb_test")


def pytest_collection_modifyitems(config, items):
    # Keep the file that must run last at the end regardless of how pytest was invoked.
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)
