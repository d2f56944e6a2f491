import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def vpq():
    """The shipped library. Where nvcc exists the (incremental) build runs first, so the tests never
    meet a library older than the sources; otherwise it must already be in the tree."""
    import shutil

    import vpipe_b200
    from vpipe_b200 import build as vbuild
    if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc") or not os.path.exists(vpipe_b200.lib_path()):
        vbuild.build()
    vpipe_b200.lib()
    return vpipe_b200


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
