"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/coli_cuda_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "coli_cuda_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(coli_cuda_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from colibri_b200 import build
    return ctypes.CDLL(build.build())


def test_header_lists_the_reference_interface():
    syms = declared_symbols()
    assert len(syms) >= 51 + 10
    for must in ("coli_cuda_expert_group", "coli_cuda_expert_group_issue", "coli_cuda_expert_group_take",
                 "coli_cuda_tensor_upload_g", "coli_cuda_matmul_mxfp4", "coli_cuda_pipe_router",
                 "coli_cuda_expert_group_resident_issue", "coli_cuda_moe_layer"):
        assert must in syms


def test_every_declared_symbol_is_exported(lib):
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_binding_tables_cover_the_header():
    from colibri_b200.backend import REFERENCE_ABI, ADDITIVE_ABI
    bound = {n for n, _, _ in REFERENCE_ABI + ADDITIVE_ABI}
    assert bound == set(declared_symbols())


def test_uninitialised_calls_refuse_cleanly(lib):
    # without coli_cuda_init nothing is configured: queries answer, compute refuses
    lib.coli_cuda_device_count.restype = ctypes.c_int
    assert lib.coli_cuda_device_count() == 0
    lib.coli_cuda_tensor_device.restype = ctypes.c_int
    lib.coli_cuda_tensor_device.argtypes = [ctypes.c_void_p]
    assert lib.coli_cuda_tensor_device(None) == -1
    lib.coli_cuda_tensor_bytes.restype = ctypes.c_size_t
    lib.coli_cuda_tensor_bytes.argtypes = [ctypes.c_void_p]
    assert lib.coli_cuda_tensor_bytes(None) == 0
    lib.coli_cuda_expert_group_take.restype = ctypes.c_void_p
    assert lib.coli_cuda_expert_group_take(0) is None
