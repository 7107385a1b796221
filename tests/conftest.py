import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run on the GPU box with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    from tests import _oracle
    return _oracle.load_oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU code (oracle/_ref/libref.so), when it has been built."""
    from tests import _oracle
    lib = _oracle.load_ref()
    if lib is None:
        pytest.skip("oracle/_ref/libref.so not built (reference tree absent)")
    return lib


@pytest.fixture(scope="session")
def ctx():
    from bonsai_vk_b200 import Context
    c = Context(0)
    yield c
    c.close()
