"""The oracle's storage formats against the reference's own C (oracle/_ref)
and against the known answers of the reference's format tests
(crates/presk-format/src/lib.rs:1780-2093; crates/presk-rt/tests/codes.rs)."""
import ctypes as C

import numpy as np
import pytest


def sample_f32_bits(rng, n):
    """Bit patterns that cover every exponent, ties, subnormals, infinities and NaNs."""
    a = rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    edge = []
    for e in range(0, 256):
        for m in (0, 1, 0x1000, 0x0fff, 0x1001, 0x2000, 0x3000, 0x7fffff, 0x400000, 0x7f, 0x80, 0x81, 0x100, 0x180, 0x7fff, 0x8000, 0x8001, 0x18000, 0xffff, 0x10000):
            edge.append((e << 23) | m)
            edge.append((1 << 31) | (e << 23) | m)
    return np.concatenate([a, np.array(edge, dtype=np.uint32)])


@pytest.fixture(scope="module")
def bits():
    return sample_f32_bits(np.random.default_rng(1), 120_000)


def each(fn, xs, argtype):
    return [fn(argtype(x)) for x in xs]


def test_f32_narrowings_match_the_reference(oracle, ref, bits):
    ref.ref_f32_to_bf16.restype = C.c_uint16; ref.ref_f32_to_bf16.argtypes = [C.c_float]
    ref.ref_f32_to_f16.restype = C.c_uint16; ref.ref_f32_to_f16.argtypes = [C.c_float]
    ref.ref_f32_to_e8m15.restype = C.c_uint32; ref.ref_f32_to_e8m15.argtypes = [C.c_float]
    ref.ref_overflows_f16.restype = C.c_uint32; ref.ref_overflows_f16.argtypes = [C.c_float]
    ref.ref_overflows_e8m15.restype = C.c_uint32; ref.ref_overflows_e8m15.argtypes = [C.c_float]
    o = oracle.lib
    bad = 0
    for b in bits.tolist():
        x = np.uint32(b).view(np.float32)
        xf = C.c_float(x)
        assert o.psk_o_f32_to_bf16(xf) == ref.ref_f32_to_bf16(xf), hex(b)
        assert o.psk_o_f32_to_f16(xf) == ref.ref_f32_to_f16(xf), hex(b)
        assert o.psk_o_f32_to_e8m15(xf) == ref.ref_f32_to_e8m15(xf), hex(b)
        assert o.psk_o_overflows(4, xf) == ref.ref_overflows_f16(xf), hex(b)
        assert o.psk_o_overflows(5, xf) == ref.ref_overflows_e8m15(xf), hex(b)
    assert bad == 0


def test_widenings_match_the_reference_on_every_code(oracle, ref):
    ref.ref_f16_to_f32.restype = C.c_float; ref.ref_f16_to_f32.argtypes = [C.c_uint16]
    ref.ref_bf16_to_f32.restype = C.c_float; ref.ref_bf16_to_f32.argtypes = [C.c_uint16]
    o = oracle.lib
    for c in range(65536):
        a, b = o.psk_o_f16_to_f32(c), ref.ref_f16_to_f32(c)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32), hex(c)
        a, b = o.psk_o_bf16_to_f32(c), ref.ref_bf16_to_f32(c)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32), hex(c)


def test_f64_narrowings_round_once_as_the_reference(oracle, ref):
    ref.ref_f64_to_f16.restype = C.c_uint16; ref.ref_f64_to_f16.argtypes = [C.c_double]
    ref.ref_f64_to_e8m15.restype = C.c_uint32; ref.ref_f64_to_e8m15.argtypes = [C.c_double]
    rng = np.random.default_rng(2)
    xs = np.concatenate([
        rng.standard_normal(100_000) * 10.0 ** rng.integers(-45, 40, 100_000),
        # double-rounding traps: just above a tie of the narrow format
        np.array([1.0 + 2.0**-11 + 2.0**-40, 1.0 + 2.0**-11, 1.0 + 2.0**-11 - 2.0**-40, 65519.999, 65520.0, 65504.0, 6e-8, 2.9802322387695312e-08, 2.98023223876953125e-08 * 1.0000001, 1e-50, 1e300, -1e300, np.inf, -np.inf]),
    ])
    o = oracle.lib
    for x in xs.tolist():
        assert o.psk_o_f64_to_f16(x) == ref.ref_f64_to_f16(x), x
        assert o.psk_o_f64_to_e8m15(x) == ref.ref_f64_to_e8m15(x), x


def test_known_answers_of_the_reference_format_tests(oracle):
    o = oracle.lib
    # binary16: 65519 rounds down to the largest finite number, 65520 up to the infinity (presk-format tests)
    assert o.psk_o_f32_to_f16(65519.0) == 0x7bff
    assert o.psk_o_f16_to_f32(0x7bff) == 65504.0
    assert o.psk_o_f32_to_f16(65520.0) == 0x7c00
    assert o.psk_o_overflows(4, 65520.0) == 1 and o.psk_o_overflows(4, 65519.0) == 0
    assert o.psk_o_overflows(4, float("inf")) == 0
    # e4m3fn: 464 rounds to 448 (a tie, to even), 465 has nowhere to go and is the NaN
    assert o.psk_o_e4m3_to_f32(o.psk_o_f32_to_e4m3(464.0)) == 448.0
    assert np.isnan(o.psk_o_e4m3_to_f32(o.psk_o_f32_to_e4m3(465.0)))
    assert o.psk_o_e4m3_to_f32(o.psk_o_f32_to_e4m3(448.0)) == 448.0
    assert o.psk_o_e4m3_to_f32(0x01) == 2.0**-9
    # every e4m3 code but the NaNs survives a round trip
    for c in range(256):
        if c & 0x7f == 0x7f:
            continue
        assert o.psk_o_f32_to_e4m3(o.psk_o_e4m3_to_f32(c)) == c, hex(c)
    # e8m15 is the top 24 bits of the f32, rounded at bit 8
    assert o.psk_o_f32_to_e8m15(1.0) == 0x3f8000
    assert o.psk_o_e8m15_to_f32(0x3f8000) == 1.0
    # bf16 ties to even
    assert o.psk_o_f32_to_bf16(np.uint32(0x3f808000).view(np.float32)) == 0x3f80
    assert o.psk_o_f32_to_bf16(np.uint32(0x3f818000).view(np.float32)) == 0x3f82
