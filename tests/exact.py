"""Exact arithmetic in Python integers and fractions: the independent statement the integer
contraction and the affine formats are held against (the recipe of the reference's
crates/presk-kernel/tests/scaled.rs:269-358, which uses GMP for the same purpose)."""
from fractions import Fraction

import numpy as np


def f32_fraction(x):
    return Fraction(float(np.float32(x)))


def round_half_even(q):
    """The integer nearest a Fraction, ties to even."""
    f = q.numerator // q.denominator
    r = q - f
    if r > Fraction(1, 2) or (r == Fraction(1, 2) and f % 2 == 1):
        f += 1
    return f


def float_code(v, t, w):
    """The code of the IEEE format with t fraction and w exponent bits nearest the Fraction v
    (ties to even, overflow to the infinity)."""
    sign = 1 if v < 0 else 0
    a = -v if v < 0 else v
    inf = ((1 << w) - 1) << t
    if a == 0:
        return sign << (t + w)
    bias = (1 << (w - 1)) - 1
    emin = 1 - bias
    # the exponent of the leading bit
    e = a.numerator.bit_length() - a.denominator.bit_length()
    if Fraction(2) ** e > a:
        e -= 1
    if Fraction(2) ** (e + 1) <= a:
        e += 1
    ulp_exp = max(e, emin) - t
    q = round_half_even(a / Fraction(2) ** ulp_exp)  # in units of the last place
    if e >= emin:
        code = ((e + bias - 1) << t) + q  # q has its leading one, which adds into the exponent
    else:
        code = q
    return (sign << (t + w)) | min(code, inf)


def wrap32(n):
    return ((n + (1 << 31)) % (1 << 32)) - (1 << 31)


def affine_code(v, kind, scale, zero):
    lo, hi = (0, 255) if kind == 2 else (-128, 127)
    q = round_half_even(v / f32_fraction(scale)) + zero
    return min(max(q, lo), hi)
