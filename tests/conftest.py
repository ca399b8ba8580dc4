"""Shared pytest configuration: the ``gpu`` marker and path setup."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.restatement()


@pytest.fixture(scope="session")
def ref():
    import oracle
    r = oracle.reference()
    if r is None:
        pytest.skip("compiled reference (oracle/_ref) not built on this machine")
    return r


@pytest.fixture(scope="session")
def ref_long():
    import oracle
    r = oracle.reference(long_context=True)
    if r is None:
        pytest.skip("compiled reference (oracle/_ref) not built on this machine")
    return r
