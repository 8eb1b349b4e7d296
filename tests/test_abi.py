"""The C-ABI library loads and exports every symbol include/presk_cuda.h declares."""
import ctypes as C
import os
import re

import pytest

from presk_b200 import abi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return abi.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "presk_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(psk_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_binds():
    names = declared_functions()
    assert names, "no function found in the header"
    assert set(names) == set(abi.PROTOTYPES), set(names) ^ set(abi.PROTOTYPES)


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared and not exported"


def test_struct_layouts_match_the_library(lib):
    for which, cls in enumerate([abi.Launch, abi.Operand, abi.Step, abi.Gemm, abi.Value, abi.ExecVtable]):
        assert lib.psk_abi_sizeof(which) == C.sizeof(cls), cls.__name__


def test_no_gpu_means_an_error_not_a_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert not lib.psk_exec_create(0)
    assert b"CUDA" in lib.psk_last_error(None)


def test_product_does_not_reach_into_the_oracle():
    for d, _, files in os.walk(os.path.join(ROOT, "presk_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(d, f), errors="ignore").read()
                assert "oracle/" not in text.replace("the CPU oracle's, loaded from oracle/", "") and "psk_oracle" not in text, f


def test_the_target_description_is_in_the_reference_schema():
    """presk_b200/targets/b200.json must parse under the reference's `Target` (deny_unknown_fields:
    presk-precision/src/target.rs): only its keys, an order of its vocabulary, modes of two operands."""
    import json
    import pathlib

    t = json.loads((pathlib.Path(__file__).resolve().parents[1] / "presk_b200" / "targets" / "b200.json").read_text())
    assert set(t) <= {"name", "about", "storage", "scaled", "params", "quant", "arith", "contractions", "order"}
    assert {"name", "storage", "arith"} <= set(t)
    assert t["order"]["kind"] in ("sequential", "blocked", "interleaved", "chunked")
    for m in t["contractions"]:
        assert set(m) <= {"name", "operands", "product", "accum"} and len(m["operands"]) == 2
    for s in t["scaled"]:
        assert set(s) == {"int", "scheme"} and s["scheme"] in ("absmax", "pow2", "minmax")
