import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def refcpu():
    from oracle.oracle import RefCpu
    if not RefCpu.available():
        pytest.skip("oracle/_ref not built (reference checkout absent)")
    return RefCpu()


@pytest.fixture(scope="session")
def be():
    """The CUDA backend, initialised on device 0. GPU tests only."""
    from colibri_b200.backend import Backend
    b = Backend()
    assert b.init_devices((0,)) == 1, "coli_cuda_init failed"
    yield b
    b.shutdown()
