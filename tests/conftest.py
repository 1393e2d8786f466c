import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)
GOLDEN = os.path.join(REPO, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def load_reference_kernel():
    """The reference's compiled extension (built by oracle/build_ref.py), or None.  Checker only."""
    ref = os.path.join(REPO, "oracle", "_ref")
    if not os.path.exists(os.path.join(ref, "FastAttention2", "kernel.so")):
        return None
    import importlib.util
    import torch  # noqa: F401

    # the extension's init symbol is PyInit_kernel, so the module must be named "kernel"
    spec = importlib.util.spec_from_file_location("kernel", os.path.join(ref, "FastAttention2", "kernel.so"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
