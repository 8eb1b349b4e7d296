"""The device library's transcendental functions (presk_b200/csrc/psk_libm.cuh),
compiled for the host, give the bits of the reference's C library
(crates/presk-export-c/c/presk_libm.c, built into oracle/_ref) on a few million
inputs a function: dense where the functions switch branch, and over every
exponent. The GPU suite repeats the comparison on the device."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "support", "libm_host.cpp")
OUT = os.path.join(ROOT, "tests", "support", "_libm_host.so")


@pytest.fixture(scope="module")
def host_libm():
    dep = os.path.join(ROOT, "presk_b200", "csrc", "psk_libm.cuh")
    if not os.path.exists(OUT) or os.path.getmtime(OUT) < max(os.path.getmtime(SRC), os.path.getmtime(dep)):
        subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fPIC", "-shared", SRC, "-o", OUT], check=True)
    return C.CDLL(OUT)


def inputs(rng, lo, hi, n):
    """Random bit patterns, a dense sweep of [lo, hi], and the neighbours of each branch point."""
    anyf = rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32).view(np.float32)
    dense = rng.uniform(lo, hi, size=n).astype(np.float32)
    log_mag = (10.0 ** rng.uniform(-40, 38, size=n // 4) * rng.choice([-1.0, 1.0], size=n // 4)).astype(np.float32)
    return np.concatenate([anyf, dense, log_mag, np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.0, -1.0], dtype=np.float32)])


CASES = [
    ("expf", -110.0, 95.0), ("logf", 0.0, 1e6), ("tanhf", -12.0, 12.0), ("erff", -7.0, 7.0),
    ("sinf", -20.0, 20.0), ("cosf", -20.0, 20.0),
]


@pytest.mark.parametrize("name,lo,hi", CASES)
def test_function_bits(host_libm, ref, name, lo, hi):
    rng = np.random.default_rng(hash(name) % 1000)
    x = inputs(rng, lo, hi, 1_000_000)
    if name in ("sinf", "cosf"):
        # beyond 2^28·π/2 the device library declines (no Payne-Hanek table): compare below it
        x = x[~(np.abs(x) >= np.float32(4.2e8)) | ~np.isfinite(x)]
        # and the angles a rotary table holds: position times frequency
        pos = np.arange(4096, dtype=np.float32)[:, None] * np.exp(-np.arange(64, dtype=np.float32) / 64 * np.log(np.float32(1e4)))[None, :]
        x = np.concatenate([x, pos.astype(np.float32).ravel()])
    x = np.ascontiguousarray(x)
    mine = np.empty_like(x)
    getattr(host_libm, "host_" + name)(x.ctypes.data_as(C.c_void_p), mine.ctypes.data_as(C.c_void_p), C.c_long(x.size))
    # the reference, through one vectorised shim call per chunk
    theirs = np.empty_like(x)
    fn = getattr(ref, "presk_" + name)
    # ctypes per element is slow; the reference has no array entry, so build one on the fly
    theirs[:] = ref_map(name, x)
    a, b = mine.view(np.uint32), theirs.view(np.uint32)
    nan = np.isnan(mine) & np.isnan(theirs)
    bad = np.nonzero((a != b) & ~nan)[0]
    assert bad.size == 0, f"{name}: {bad.size} of {x.size} differ, first x={x[bad[0]]!r} ({a[bad[0]]:#x} vs {b[bad[0]]:#x})"


_REF_MAP = {}


def ref_map(name, x):
    """The reference's function over an array: a two-line C loop compiled against oracle/_ref."""
    so = os.path.join(ROOT, "tests", "support", "_ref_map.so")
    src = os.path.join(ROOT, "tests", "support", "_ref_map.c")
    if "lib" not in _REF_MAP:
        if not os.path.exists(so):
            with open(src, "w") as f:
                f.write("float presk_expf(float);float presk_logf(float);float presk_tanhf(float);float presk_sinf(float);float presk_cosf(float);float presk_erff(float);\n")
                for n in ("expf", "logf", "tanhf", "sinf", "cosf", "erff"):
                    f.write(f"void map_{n}(const float*x,float*y,long n){{for(long i=0;i<n;++i)y[i]=presk_{n}(x[i]);}}\n")
            ref_dir = os.path.join(ROOT, "oracle", "_ref")
            subprocess.run(["gcc", "-std=c11", "-O2", "-ffp-contract=off", "-fPIC", "-shared", src, "-L" + ref_dir, "-lpresk_ref", "-Wl,-rpath," + ref_dir, "-o", so], check=True)
        _REF_MAP["lib"] = C.CDLL(so)
    y = np.empty_like(x)
    getattr(_REF_MAP["lib"], "map_" + name)(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), C.c_long(x.size))
    return y
