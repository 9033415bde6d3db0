import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """Build the host libraries (and cross-compile the CUDA one) once per run if missing."""
    from onyxia_b200 import build
    build.ensure_built(cuda=os.path.isdir(os.path.join(ROOT, "onyxia_b200", "csrc", "backend")))
