import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "strix-halo-engine-lab_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.loader import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU code; present only where oracle/_ref was built (it needs the reference checkout)."""
    from oracle.loader import Ref
    if not Ref.available():
        pytest.skip("oracle/_ref/libstrixref.so not built (reference checkout absent)")
    return Ref()
