import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def reference_path():
    """Directory that makes ``import heavyball`` resolve to the unmodified reference, or None: the in-tree
    install under ``baseline/_ref``, else a checkout named by the ``HEAVYBALL_REFERENCE`` environment variable."""
    for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("HEAVYBALL_REFERENCE", "")):
        if cand and os.path.isdir(os.path.join(cand, "heavyball")):
            return cand
    return None


@pytest.fixture(scope="session")
def ref_path():
    path = reference_path()
    if path is None:
        pytest.skip("reference package not available")
    return path
