import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Where the reference project is mounted, for the tests that pin counts and file bytes on its own data files; they
# are skipped where it is absent.  AGPT_REFERENCE_ROOT overrides the default mount point.
REFERENCE_ROOT = os.environ.get("AGPT_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Both shared libraries exist before any test runs: the product and the checker."""
    from agpt_b200 import build as product_build
    from oracle import pyoracle
    product_build.build()
    pyoracle.build()
    yield


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
