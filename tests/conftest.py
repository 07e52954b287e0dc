import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding as oracle_lib
    return oracle_lib.load_oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own host code compiled from its sources (oracle/_ref), or skip where it was never built."""
    from oracle import binding as oracle_lib
    lib = oracle_lib.load_reference()
    if lib is None:
        pytest.skip("oracle/_ref/libanemone_ref.so not built (reference tree absent)")
    return lib
