"""Shared fixtures. Tests that need a GPU carry the `gpu` marker; everything
else runs on a machine without one."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "libpsk_oracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libpresk_ref.so")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def build_oracle():
    src = os.path.join(ROOT, "oracle", "psk_oracle.c")
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src) or not os.path.exists(REF_SO):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-s"], check=True)
    return ORACLE_SO


@pytest.fixture(scope="session")
def ref():
    """The reference's own C runtime, compiled from its tree (oracle/_ref)."""
    build_oracle()
    lib = C.CDLL(REF_SO)
    for name in ("presk_expf", "presk_logf", "presk_tanhf", "presk_sinf", "presk_cosf", "presk_erff"):
        getattr(lib, name).restype = C.c_float
        getattr(lib, name).argtypes = [C.c_float]
    return lib


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (oracle/psk_oracle.c)."""
    import oracle_lib
    return oracle_lib.load()


@pytest.fixture(scope="session")
def cuda():
    """The CUDA executor on device 0; fails (does not skip) when it cannot be made."""
    import presk_b200
    presk_b200.build.build()
    return presk_b200.Executor(0)


@pytest.fixture
def rng():
    return np.random.default_rng(0)
