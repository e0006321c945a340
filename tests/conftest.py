import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on a GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle, build_oracle
    build_oracle()
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own compiled CPU code; absent where its tree is absent."""
    from oracle.binding import Reference, reference_available
    if not reference_available():
        pytest.skip("oracle/_ref was not built (reference tree absent)")
    return Reference()


@pytest.fixture(scope="session")
def library():
    from clori_b200 import _build, abi
    if not os.path.exists(abi.LIB_PATH):
        _build.build()
    return abi.load()


@pytest.fixture()
def backend(library):
    import clori_b200
    b = clori_b200.Backend(0)
    yield b
    b.close()
