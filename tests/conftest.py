import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with `-m gpu`")
    # A fresh checkout has no built library (it is not kept in history): build it once so that the tests that
    # only load it and check its exports can run.  Where the compiler is absent the tests fail loudly instead.
    from rai_b200 import build as b
    if not b.LIB.exists():
        b.build()


@pytest.fixture(scope="session")
def cuda():
    """The library context of GPU 0 (fails loudly when the extension or the GPU is missing)."""
    from rai_b200.device import Cuda
    dev = Cuda(0)
    dev.use_torch_stream()
    return dev
