import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Everything the tests load is built in-tree first (nvcc cross-compiles without a GPU)."""
    from decx_b200 import build as b
    b.build_all()
    from oracle import binding as ob
    if not os.path.exists(ob.ORACLE_SO):
        ob.build()
