import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')


@pytest.fixture(scope='session', autouse=True)
def _built():
    """The CUDA library and the oracle are built once per session (nvcc cross-compiles without a GPU)."""
    from statequant_b200 import build
    build.build()
    from oracle import oracle
    oracle.build()
