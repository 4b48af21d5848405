import ctypes
import importlib
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

cg = importlib.import_module("catgrad-rs_b200")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_oracle_lib():
    """The CPU checker (oracle/liboracle.so); built on demand where a compiler exists."""
    path = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(path):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")])
    return ctypes.CDLL(path)


class OracleBackend(cg.TraitBackend):
    """The reference semantics on the CPU, behind the same trait mirror as the product."""

    def __init__(self, threads=0):
        lib = load_oracle_lib()
        lib.cgo_ctx_create.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]
        ctx = ctypes.c_void_p()
        assert lib.cgo_ctx_create(threads, ctypes.byref(ctx)) == 0
        super().__init__(lib, "cgo_", ctx)


@pytest.fixture(scope="session")
def oracle():
    return OracleBackend()


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.fixture(scope="session")
def cuda():
    if not _have_gpu():
        pytest.skip("no CUDA device")
    return cg.CudaBackend(0, cg.PREC_F32)


@pytest.fixture(scope="session")
def cuda_bf16():
    if not _have_gpu():
        pytest.skip("no CUDA device")
    return cg.CudaBackend(0, cg.PREC_BF16)
