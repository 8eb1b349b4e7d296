"""Builds libpresk_cuda.so: the CUDA executor and the host program, for sm_100a.

The library is built in-tree (presk_b200/_lib/) with nvcc; nothing is compiled
at import time on a machine that already holds the built file and whose
sources are not newer.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_lib")
LIB = os.path.join(OUT_DIR, "libpresk_cuda.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # every product is rounded before it is added: the reference's kernels
    # never contract a*b+c (presk-export-c/c/presk_rt.h, "Build with")
    "--fmad=false",
    "-diag-suppress", "39",  # (x - x) / 0 makes the NaN the library's functions return
    "-Xcompiler", "-fPIC",
]


def _nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found: libpresk_cuda.so cannot be built")


def sources():
    return [os.path.join(CSRC, f) for f in ("psk_exec.cu", "psk_host.cpp", "psk_noalloc.cu", "psk_comm.cpp", "psk_describe.cpp", "psk_data.cu") if os.path.exists(os.path.join(CSRC, f))]


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "presk_cuda.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compiles the library if it is missing or older than its sources."""
    if not force and not stale():
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []
    for src in sources():
        obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu" if src.endswith(".cu") else "c++", "-c", src, "-o", obj]
        subprocess.run(cmd, check=True)
        objs.append(obj)
    subprocess.run([_nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart", "-ldl"], check=True)
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
