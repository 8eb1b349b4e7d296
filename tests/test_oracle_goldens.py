"""Known answers of the reference pin the oracle and the host program:

  - the first four normal draws of the key seed 0 names and the FNV fold of the
    next 100 000 (crates/presk-interp/src/key.rs:86-93) pin the build of the
    reference's C runtime in oracle/_ref (ChaCha keys, musl log and cos);
  - the seed-0 outputs of `LayerNorm{8}.apply` and `RMSNorm{8}.apply` at
    batch 3 from the exact interpreter (tests/run/*.snap, 12 digits) pin the
    launch sequences of the host program and the oracle's kernels: an f32
    realization must agree with the exact reals to f32 accuracy.
"""
import ctypes as C
import json
import os

import numpy as np
import pytest

from presk_b200 import Host, abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = json.load(open(os.path.join(ROOT, "tests", "golden", "reference_vectors.json")))


def normals(ref, seed, split_of, index, n):
    out = np.empty(n, dtype=np.float64)
    ref.ref_normals.argtypes = [C.c_uint64, C.c_int, C.c_int, C.c_void_p, C.c_size_t]
    ref.ref_normals(seed, split_of, index, out.ctypes.data, n)
    return out


def test_key_draws_are_the_reference_s(ref):
    x = normals(ref, 0, 0, 0, 100_004)
    assert [int(b) for b in x[:4].view(np.uint64)] == GOLD["seed0_first_normals_bits"]
    h = 0xCBF29CE484222325
    for b in x[4:].view(np.uint64).tolist():
        h = ((h ^ b) * 0x00000100000001B3) & 0xFFFFFFFFFFFFFFFF
    assert h == GOLD["seed0_next_100000_fnv"]


@pytest.mark.parametrize("model,key", [("layernorm", "layernorm_apply"), ("rmsnorm", "rmsnorm_apply")])
def test_norm_goldens_on_the_oracle(oracle, ref, model, key):
    want = np.array(GOLD[key]["values"])
    b, d = GOLD[key]["shape"]
    # the entry's parameters are (θ, x, eps): x is drawn from the second of three keys
    x = normals(ref, 0, 3, 1, b * d).reshape(b, d)
    h = Host(oracle.vtable(), "f32").prepare(model)
    h.set_param("γ", np.ones(d))
    if model == "layernorm":
        h.set_param("β", np.zeros(d))
    h.set_logging(True)
    got = h.call("apply", [x], (b, d), np.float32)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-6)
    log = h.launch_log()
    if model == "layernorm":
        # crates/presk-core/tests/snapshots/lower__core_minigpt.snap + fusion.rs: five launches
        assert log == ["mean axis model", "fused 2 steps", "mean axis model", "fused 2 steps", "fused 4 steps"]
    else:
        assert log == ["pow 2", "mean axis model", "fused 2 steps", "fused 2 steps"]


def test_bf16_storage_rounds_every_site(oracle, ref):
    """Under `--realize bf16` each launch's output is a bf16 number (storage rounding at every site)."""
    b, d = 3, 8
    x = normals(ref, 0, 3, 1, b * d).reshape(b, d)
    h = Host(oracle.vtable(), "bf16").prepare("rmsnorm")
    h.set_param("γ", np.ones(d))
    got = h.call("apply", [x], (b, d), np.float32)
    bits = got.view(np.uint32)
    assert np.all(bits & 0xFFFF == 0)
    want = np.array(GOLD["rmsnorm_apply"]["values"])
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)
