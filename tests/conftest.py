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
    from oracle.oracle import Oracle
    b = Backend()
    assert b.init_devices((0,)) == 1, "coli_cuda_init failed"
    # the engine hands over its FP8 E4M3 decode table once after init (c/colibri.c:9366-9368)
    lut = Oracle().e4m3_table()
    assert b.fp8_set_lut(lut.ctypes.data) == 1
    yield b
    b.shutdown()


def pytest_sessionfinish(session, exitstatus):
    """After a GPU session: the parity errors the tests noted (floored and plain figures side by
    side), as a table in the run's output folder."""
    from tests import util
    if not util.ERRORS:
        return
    out = os.path.join(ROOT, "gpurun_out")
    try:
        os.makedirs(out, exist_ok=True)
        with open(os.path.join(out, "parity_errors.txt"), "w") as f:
            f.write("label | max |err|/(|want|+0.01 rms) | max |err|/|want| | max|err|/max|want|\n")
            for label, e, elem, norm in util.ERRORS:
                f.write(f"{label} | {e:.3e} | {elem:.3e} | {norm:.3e}\n")
    except OSError:
        pass
