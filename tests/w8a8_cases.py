"""Random cases of an integer contraction over affine activations and int8 weights, with the
exact expected result of each (tests/exact.py)."""
import numpy as np

import exact
from presk_b200 import abi, launch_desc

FORMATS = {abi.F32: (23, 8), abi.BF16: (7, 8), abi.F16: (10, 5), abi.E8M15: (15, 8)}


def rand_scale(rng):
    return np.float32(rng.uniform(1.0, 2.0) * 2.0 ** int(rng.integers(-14, 3)))


def make_case(rng, trial, m=3, k=48, n=5):
    kind = 2 if trial % 2 == 0 else 1  # u8/sat, i8/sat
    lo, hi = (0, 255) if kind == 2 else (-128, 127)
    s_a, z_a = rand_scale(rng), int(rng.integers(lo, hi + 1))
    codes = rng.integers(lo, hi + 1, size=(m, k))
    qw = rng.integers(-127, 128, size=(k, n))
    sw = np.array([rand_scale(rng) for _ in range(n)], np.float32)
    store = [abi.F16, "affine", abi.F32, abi.BF16, abi.E8M15, "affine"][trial % 6]
    out_scale = np.float32((int(rng.integers(0, 1 << 20)) + 1.0) * float(s_a) * float(sw[0]) * 64.0)
    out_zero = int(rng.integers(-20, 21))
    if trial % 7 == 0:  # make the sum large enough to wrap: a zero point at the far end and aligned signs
        z_a = lo
        codes[:] = hi
        qw[:] = 127
        k_big = True
    # expected
    want = np.zeros((m, n), dtype=np.int64)
    for r in range(m):
        for c in range(n):
            acc = 0
            for t in range(k):
                acc = exact.wrap32(acc + (int(codes[r, t]) - z_a) * int(qw[t, c]))
            v = exact.Fraction(acc) * exact.f32_fraction(s_a) * exact.f32_fraction(sw[c])
            if store == "affine":
                want[r, c] = exact.affine_code(v, 1, out_scale, out_zero)
            else:
                want[r, c] = exact.float_code(v, *FORMATS[store])
    # the launch
    l = launch_desc(abi.OP_CONTRACT, abi.F32, [m, n], [k], name=b"dot")
    l.n_inputs, l.int_accum = 2, 1
    a_arr = codes.astype(np.uint8 if kind == 2 else np.int8)
    l.inputs[0].dtype = abi.U8 if kind == 2 else abi.I8
    l.inputs[0].affine, l.inputs[0].affine_zero, l.inputs[0].affine_scale = kind, z_a, float(s_a)
    l.inputs[0].stride[0], l.inputs[0].stride[2], l.inputs[0].numel = k, 1, m * k
    l.inputs[1].dtype = abi.I8
    l.inputs[1].stride[1], l.inputs[1].stride[2], l.inputs[1].numel = 1, n, k * n
    l.inputs[1].scale_stride[1] = 1
    l.out.stride[0], l.out.stride[1], l.out.numel = n, 1, m * n
    if store == "affine":
        l.out.dtype, l.out.affine, l.out.affine_zero, l.out.affine_scale = abi.I8, 1, out_zero, float(out_scale)
        out_bytes, view = m * n, np.int8
    else:
        l.out.dtype = store
        out_bytes = m * n * abi.DTYPE_BYTES[store]
        view = {abi.F32: np.uint32, abi.BF16: np.uint16, abi.F16: np.uint16, abi.E8M15: None}[store]
    return l, [a_arr, qw.astype(np.int8)], sw, out_bytes, view, want


def decode(raw, view, m, n):
    if view is None:  # e8m15: three bytes little-endian
        b = raw.reshape(m * n, 3).astype(np.int64)
        return (b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)).reshape(m, n)
    return raw.view(view).astype(np.int64).reshape(m, n)
