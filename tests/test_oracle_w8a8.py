"""`product: i32, accum: i32` over scaled values on the oracle, against written-out integer
arithmetic: 300 random trials of the reference's own construction
(crates/presk-kernel/tests/scaled.rs:269-358), sums that wrap included."""
import numpy as np

import exact
import w8a8_cases
from presk_b200 import abi


def test_integer_sums_match_exact_arithmetic(oracle):
    rng = np.random.default_rng(0x180004)
    wrapped = 0
    for trial in range(300):
        l, ins, sw, out_bytes, view, want = w8a8_cases.make_case(rng, trial)
        out = np.zeros(out_bytes, np.uint8)
        oracle.run(l, ins + [out, sw])
        got = w8a8_cases.decode(out, view, *want.shape)
        assert np.array_equal(got, want), f"trial {trial}: {got} vs {want}"
        wrapped += trial % 7 == 0
    assert wrapped > 10


def test_affine_store_of_reals(oracle):
    """q = clamp(rne(x / s) + z) with the quotient exact: ties, both ends of the range, NaN."""
    rng = np.random.default_rng(5)
    oracle.lib.psk_o_affine_code.restype = __import__("ctypes").c_int64
    oracle.lib.psk_o_affine_code.argtypes = [__import__("ctypes").c_double, __import__("ctypes").c_int, __import__("ctypes").c_float, __import__("ctypes").c_int]
    for _ in range(3000):
        kind = int(rng.integers(1, 3))
        s = w8a8_cases.rand_scale(rng)
        z = int(rng.integers(0, 256)) if kind == 2 else int(rng.integers(-128, 128))
        k = int(rng.integers(-300, 300))
        x = float(np.float32((k + rng.choice([0.0, 0.5, 0.5, 0.25, rng.uniform(0, 1)])) * float(s)))
        want = exact.affine_code(exact.Fraction(x), kind, s, z)
        assert oracle.lib.psk_o_affine_code(x, kind, float(s), z) == want, (x, kind, s, z)
    assert oracle.lib.psk_o_affine_code(float("nan"), 1, 0.5, 7) == 7
    assert oracle.lib.psk_o_affine_code(float("inf"), 2, 0.5, 7) == 255
    assert oracle.lib.psk_o_affine_code(float("-inf"), 1, 0.5, 7) == -128


def test_float_sums_stored_into_a_scaled_site(oracle):
    """exec.rs:758-782 stores any kernel's value through its output's format: a contraction that sums in f32 and
    writes a `scaled` site stores clamp(rne(acc / s) + z) of its binary32 sum. The sum is taken from the same
    contraction with an f32 result; the code expected of it is exact arithmetic's (fractions), both saturated ends
    of both formats among them. Likewise a reduction into a scaled site."""
    from presk_b200 import launch_desc
    rng = np.random.default_rng(11)
    m, k, n = 9, 33, 14
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)

    def contract(out_dtype, affine=None):
        l = launch_desc(abi.OP_CONTRACT, abi.F32, [m, n], [k])
        l.n_inputs = 2
        l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = abi.F32, m * k, k, 1
        l.inputs[1].dtype, l.inputs[1].numel, l.inputs[1].stride[1], l.inputs[1].stride[2] = abi.F32, k * n, 1, n
        l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = out_dtype, m * n, n, 1
        if affine:
            l.out.affine, l.out.affine_zero, l.out.affine_scale = affine
        return l

    acc = np.zeros(m * n, np.float32)
    oracle.run(contract(abi.F32), [x, w, acc.view(np.uint8)])
    np.testing.assert_allclose(acc.reshape(m, n), x.astype(np.float64) @ w.astype(np.float64), rtol=0, atol=1e-4)
    seen = set()
    for kind, zero, scale in ((1, 0, 0.05), (2, 131, 0.05), (1, -7, 0.5), (2, 0, 0.02)):
        codes = np.full(m * n, 0xA5, np.uint8)
        oracle.run(contract(abi.U8 if kind == 2 else abi.I8, (kind, zero, scale)), [x, w, codes])
        got = codes.view(np.uint8 if kind == 2 else np.int8).astype(np.int64)
        want = np.array([exact.affine_code(exact.Fraction(float(a)), kind, np.float32(scale), zero) for a in acc])
        assert np.array_equal(got, want), (kind, zero, scale, np.nonzero(got != want)[0][:5])
        seen |= set(got.tolist())
    assert {-128, 127, 0, 255} <= seen  # both formats saturated at both ends
    # a reduction (sum over the last axis) into a scaled site
    r = launch_desc(abi.OP_REDUCE, abi.F32, [m], [k])
    r.n_inputs, r.kind = 1, abi.REDUCE_SUM
    r.inputs[0].dtype, r.inputs[0].numel, r.inputs[0].stride[0], r.inputs[0].stride[1] = abi.F32, m * k, k, 1
    r.out.dtype, r.out.numel, r.out.stride[0] = abi.F32, m, 1
    sums = np.zeros(m, np.float32)
    oracle.run(r, [x, sums.view(np.uint8)])
    r.out.dtype, r.out.affine, r.out.affine_zero, r.out.affine_scale = abi.I8, 1, 3, 0.25
    codes = np.zeros(m, np.uint8)
    oracle.run(r, [x, codes])
    assert np.array_equal(codes.view(np.int8).astype(np.int64), [exact.affine_code(exact.Fraction(float(a)), 1, np.float32(0.25), 3) for a in sums])


def w8a8_dense_case(seed=0, rows=4, k=16, n=8):
    """examples/tests/formats/w8a8.json on examples/tests/formats/w8a8.psk: relu stored u8/sat, the
    product's sums in i32, the result stored i8/sat, weights int8 over axis 0; with static scales."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.3).astype(np.float32)
    s_a, z_a = np.float32(np.abs(x).max() / 255.0), 3
    s_o, z_o = np.float32(0.05), -4
    rz = {"default": "f32", "order": {"kind": "sequential"},
          "scaled": {"Dense.apply/%2": {"int": "u8/sat", "scale": float(s_a), "zero": z_a}, "Dense.apply/%4": {"int": "i8/sat", "scale": float(s_o), "zero": z_o}},
          "product": {"Dense.apply/%4": "i32"}, "accum": {"Dense.apply/%4": "i32"}, "quant": {"w": {"bits": 8, "over": 0}}}
    # expected, in exact arithmetic
    sw = (np.abs(w.astype(np.float64)).max(axis=0) / 127.0).astype(np.float32)
    qw = np.clip(np.rint(w.astype(np.float64) / sw.astype(np.float64)), -127, 127).astype(np.int64)
    relu = np.where(x < 0, np.float32(0), x)
    qa = np.array([[exact.affine_code(exact.Fraction(float(v)), 2, s_a, z_a) for v in row] for row in relu])
    want = np.zeros((rows, n))
    for r in range(rows):
        for c in range(n):
            acc = 0
            for t in range(k):
                acc = exact.wrap32(acc + (int(qa[r, t]) - z_a) * int(qw[t, c]))
            v = exact.Fraction(acc) * exact.f32_fraction(s_a) * exact.f32_fraction(sw[c])
            want[r, c] = (exact.affine_code(v, 1, s_o, z_o) - z_o) * float(s_o)
    return rz, x, w, want


def test_w8a8_through_the_host_program(oracle):
    from presk_b200 import Host, PreskError
    rz, x, w, want = w8a8_dense_case()
    h = Host(oracle.vtable(), rz).prepare("dense")
    h.set_param("w", w)
    got = h.call("apply", [x], want.shape, np.float64)
    assert np.array_equal(got, want)
    import pytest
    with pytest.raises(PreskError, match="E7006"):
        Host(oracle.vtable(), {"default": "f32", "scaled": {"Dense.apply/%2": {"int": "u8/sat", "scheme": "minmax"}}})
    with pytest.raises(PreskError, match="E7005"):
        Host(oracle.vtable(), {"default": "f32", "accum": {"Dense.apply/%4": "i16/sat"}, "product": {"Dense.apply/%4": "i32"}})
