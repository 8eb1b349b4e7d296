// The transcendental functions a kernel calls, in f32, for the device.
//
// Every executor of the reference computes exp, log, tanh, sin, cos and erf
// with one library, musl's as it was before 1.1.23 (the Rust `libm` crate's
// port; presk-kernel/src/exec.rs:146-183, presk-export-c/c/presk_rt.h
// "The transcendental functions the kernels call"), so that a kernel's bits
// do not depend on the machine. These are the same published algorithms
// (Sun's fdlibm as FreeBSD's msun carries them in float: e_expf.c, e_logf.c,
// s_expm1f.c, s_tanhf.c, s_sinf.c, s_cosf.c, k_sinf.c, k_cosf.c,
// e_rem_pio2f.c, s_erff.c), written for CUDA. Compile with --fmad=false and
// without fast-math: each product is rounded before it is added, divisions
// and square roots are IEEE's, subnormals are kept.
//
// Arguments of sinf/cosf at or beyond 2^28·π/2 need the Payne-Hanek reduction
// with the 2/π table; below, the two-term Cody-Waite reduction in f64 is what
// musl uses, and it is what is written here. Beyond, these return a NaN and
// raise `*unsupported` where the caller passes one.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define PSK_LIBM_DEV __device__ __forceinline__
#else
// Compiled by a host compiler (with -ffp-contract=off) only so that a test can
// compare these functions with the reference's C on the CPU.
#include <math.h>
#include <string.h>
#define PSK_LIBM_DEV static inline
#endif

namespace psk {

#ifdef __CUDACC__
PSK_LIBM_DEV float lm_bits_f(uint32_t w) { return __uint_as_float(w); }
PSK_LIBM_DEV uint32_t lm_f_bits(float x) { return __float_as_uint(x); }
#else
PSK_LIBM_DEV float lm_bits_f(uint32_t w) { float x; memcpy(&x, &w, 4); return x; }
PSK_LIBM_DEV uint32_t lm_f_bits(float x) { uint32_t w; memcpy(&w, &x, 4); return w; }
#endif

// x·2^n with at most one rounding into the subnormals.
PSK_LIBM_DEV float lm_scalbnf(float x, int n)
{
    float y = x;
    if (n > 127) {
        y *= 0x1p127f;
        n -= 127;
        if (n > 127) {
            y *= 0x1p127f;
            n -= 127;
            if (n > 127) n = 127;
        }
    } else if (n < -126) {
        y *= 0x1p-126f * 0x1p24f;
        n += 126 - 24;
        if (n < -126) {
            y *= 0x1p-126f * 0x1p24f;
            n += 126 - 24;
            if (n < -126) n = -126;
        }
    }
    return y * lm_bits_f((uint32_t)(0x7f + n) << 23);
}

// exp, written with selections where the original branches on the argument's
// range, so that the lanes of a warp stay together: the three cases of the
// reduction (k = 0, k = -1 or 1, k computed) share one sequence of operations,
// because with k = 0 that sequence leaves x as it is (x - 0·ln2hi = x, lo = 0);
// y·2^0 = y stands for "no scaling"; |x| <= 2^-14 selects 1 + x at the end.
// Only the rare cases branch: NaN, overflow, the results below 2^-126.
PSK_LIBM_DEV float lm_expf(float x)
{
    const float ln2hi = 6.9314575195e-1f, ln2lo = 1.4286067653e-6f, invln2 = 1.4426950216e+0f;
    const float P1 = 1.6666625440e-1f, P2 = -2.7667332906e-3f;
    const uint32_t ux = lm_f_bits(x);
    const int sign = (int)(ux >> 31);
    const uint32_t hx = ux & 0x7fffffffu;
    if (hx >= 0x42aeac50u) { // |x| >= 87.33655 or NaN
        if (hx > 0x7f800000u) return x;
        if (hx >= 0x42b17218u && !sign) return x * 0x1p127f; // overflow
        if (sign && hx >= 0x42cff1b5u) return 0.0f;          // underflow
    }
    const float half = sign ? -0.5f : 0.5f;
    int k = (int)(invln2 * x + half);
    k = hx > 0x3f851592u ? k : 1 - sign - sign; // |x| <= 1.5 ln2
    k = hx > 0x3eb17218u ? k : 0;               // |x| <= 0.5 ln2
    const float fk = (float)k;
    const float hi = x - fk * ln2hi;
    const float lo = fk * ln2lo;
    const float xr = hi - lo;
    const float xx = xr * xr;
    const float c = xr - xx * (P1 + xx * P2);
    const float y = 1.0f + (xr * c / (2.0f - c) - lo + hi);
    float r;
    if (k >= -126 && k <= 127) r = y * lm_bits_f((uint32_t)(0x7f + k) << 23);
    else r = lm_scalbnf(y, k);
    return hx > 0x39000000u ? r : 1.0f + x; // |x| <= 2^-14
}

PSK_LIBM_DEV float lm_logf(float x)
{
    const float ln2_hi = 6.9313812256e-01f, ln2_lo = 9.0580006145e-06f;
    const float Lg1 = 0xaaaaaa.0p-24f, Lg2 = 0xccce13.0p-25f, Lg3 = 0x91e9ee.0p-25f, Lg4 = 0xf89e26.0p-26f;
    uint32_t ix = lm_f_bits(x);
    int k = 0;
    if (ix < 0x00800000u || (ix >> 31)) {
        if ((ix << 1) == 0) return -1.0f / (x * x);
        if (ix >> 31) return (x - x) / 0.0f;
        k -= 25;
        x *= 0x1p25f;
        ix = lm_f_bits(x);
    } else if (ix >= 0x7f800000u) {
        return x;
    } else if (ix == 0x3f800000u) {
        return 0.0f;
    }
    ix += 0x3f800000u - 0x3f3504f3u;
    k += (int)(ix >> 23) - 0x7f;
    ix = (ix & 0x007fffffu) + 0x3f3504f3u;
    x = lm_bits_f(ix);
    float f = x - 1.0f;
    float s = f / (2.0f + f);
    float z = s * s;
    float w = z * z;
    float t1 = w * (Lg2 + w * Lg4);
    float t2 = z * (Lg1 + w * Lg3);
    float R = t2 + t1;
    float hfsq = 0.5f * f * f;
    float dk = (float)k;
    return s * (hfsq + R) + dk * ln2_lo - hfsq + f + dk * ln2_hi;
}

PSK_LIBM_DEV float lm_expm1f(float x)
{
    const float ln2_hi = 6.9313812256e-01f, ln2_lo = 9.0580006145e-06f, invln2 = 1.4426950216e+00f;
    const float Q1 = -3.3333212137e-2f, Q2 = 1.5807170421e-3f;
    uint32_t ux = lm_f_bits(x), hx = ux & 0x7fffffffu;
    int sign = (int)(ux >> 31), k;
    float hi, lo, c = 0.0f, t;
    if (hx >= 0x4195b844u) { // |x| >= 27 ln2
        if (hx > 0x7f800000u) return x;
        if (sign) return -1.0f;
        if (hx > 0x42b17217u) return x * 0x1p127f;
    }
    if (hx > 0x3eb17218u) {
        if (hx < 0x3F851592u) {
            if (!sign) { hi = x - ln2_hi; lo = ln2_lo; k = 1; }
            else { hi = x + ln2_hi; lo = -ln2_lo; k = -1; }
        } else {
            k = (int)(invln2 * x + (sign ? -0.5f : 0.5f));
            t = (float)k;
            hi = x - t * ln2_hi;
            lo = t * ln2_lo;
        }
        x = hi - lo;
        c = (hi - x) - lo;
    } else if (hx < 0x33000000u) {
        return x;
    } else {
        k = 0;
    }
    float hfx = 0.5f * x;
    float hxs = x * hfx;
    float r1 = 1.0f + hxs * (Q1 + hxs * Q2);
    t = 3.0f - r1 * hfx;
    float e = hxs * ((r1 - t) / (6.0f - x * t));
    if (k == 0) return x - (x * e - hxs);
    e = x * (e - c) - c;
    e -= hxs;
    if (k == -1) return 0.5f * (x - e) - 0.5f;
    if (k == 1) {
        if (x < -0.25f) return -2.0f * (e - (x + 0.5f));
        return 1.0f + 2.0f * (x - e);
    }
    float twopk = lm_bits_f((uint32_t)(0x7f + k) << 23);
    float y;
    if (k < 0 || k > 56) {
        y = x - e + 1.0f;
        if (k == 128) y = y * 2.0f * 0x1p127f;
        else y = y * twopk;
        return y - 1.0f;
    }
    float twomk = lm_bits_f((uint32_t)(0x7f - k) << 23);
    if (k < 23) y = (x - e + (1.0f - twomk)) * twopk;
    else y = (x - (e + twomk) + 1.0f) * twopk;
    return y;
}

PSK_LIBM_DEV float lm_tanhf(float x)
{
    uint32_t u = lm_f_bits(x);
    int sign = (int)(u >> 31);
    uint32_t w = u & 0x7fffffffu;
    x = lm_bits_f(w);
    float t;
    if (w > 0x3f0c9f54u) { // |x| > log(3)/2
        if (w > 0x41200000u) { // |x| > 10
            t = 1.0f + 0.0f / x;
        } else {
            t = lm_expm1f(2.0f * x);
            t = 1.0f - 2.0f / (t + 2.0f);
        }
    } else if (w > 0x3e82c578u) { // |x| > log(5/3)/2
        t = lm_expm1f(2.0f * x);
        t = t / (t + 2.0f);
    } else if (w >= 0x00800000u) {
        t = lm_expm1f(-2.0f * x);
        t = -t / (t + 2.0f);
    } else {
        t = x;
    }
    return sign ? -t : t;
}

// sin and cos on [-π/4, π/4], evaluated in f64 and rounded once.
PSK_LIBM_DEV float lm_k_sindf(double x)
{
    const double S1 = -0x15555554cbac77.0p-55, S2 = 0x111110896efbb2.0p-59, S3 = -0x1a00f9e2cae774.0p-65, S4 = 0x16cd878c3b46a7.0p-71;
    double z = x * x;
    double w = z * z;
    double r = S3 + z * S4;
    double s = z * x;
    return (float)((x + s * (S1 + z * S2)) + s * w * r);
}

PSK_LIBM_DEV float lm_k_cosdf(double x)
{
    const double C0 = -0x1ffffffd0c5e81.0p-54, C1 = 0x155553e1053a42.0p-57, C2 = -0x16c087e80f1e27.0p-62, C3 = 0x199342e0ee5069.0p-68;
    double z = x * x;
    double w = z * z;
    double r = C2 + z * C3;
    return (float)(((1.0 + z * C0) + w * C1) + (w * z) * r);
}

// x = y + n·π/2 with |y| <= π/4, for |x| < 2^28·π/2. Returns n; -1 beyond.
PSK_LIBM_DEV int lm_rem_pio2f(float x, double *y, int *beyond)
{
    const double toint = 1.5 / 2.220446049250313e-16, invpio2 = 6.36619772367581382433e-01, pio2_1 = 1.57079631090164184570e+00, pio2_1t = 1.58932547735281966916e-08;
    uint32_t ix = lm_f_bits(x) & 0x7fffffffu;
    if (ix < 0x4dc90fdbu) {
        double fn = (double)x * invpio2 + toint - toint;
        int n = (int)fn;
        *y = x - fn * pio2_1 - fn * pio2_1t;
        return n;
    }
    *beyond = 1;
    *y = (double)(x - x) / 0.0; // NaN
    return 0;
}

PSK_LIBM_DEV float lm_sinf(float x, int *beyond)
{
    const double pio2 = 1.57079632679489661923;
    const double s1pio2 = 1 * pio2, s2pio2 = 2 * pio2, s3pio2 = 3 * pio2, s4pio2 = 4 * pio2;
    uint32_t ix = lm_f_bits(x);
    int sign = (int)(ix >> 31);
    ix &= 0x7fffffffu;
    if (ix <= 0x3f490fdau) { // |x| <= π/4
        if (ix < 0x39800000u) return x;
        return lm_k_sindf(x);
    }
    if (ix <= 0x407b53d1u) { // |x| <= 5π/4
        if (ix <= 0x4016cbe3u) { // |x| <= 3π/4
            if (sign) return -lm_k_cosdf(x + s1pio2);
            return lm_k_cosdf(x - s1pio2);
        }
        return lm_k_sindf(sign ? -(x + s2pio2) : -(x - s2pio2));
    }
    if (ix <= 0x40e231d5u) { // |x| <= 9π/4
        if (ix <= 0x40afeddfu) { // |x| <= 7π/4
            if (sign) return lm_k_cosdf(x + s3pio2);
            return -lm_k_cosdf(x - s3pio2);
        }
        return lm_k_sindf(sign ? x + s4pio2 : x - s4pio2);
    }
    if (ix >= 0x7f800000u) return x - x;
    double y;
    int n = lm_rem_pio2f(x, &y, beyond);
    switch (n & 3) {
    case 0: return lm_k_sindf(y);
    case 1: return lm_k_cosdf(y);
    case 2: return lm_k_sindf(-y);
    default: return -lm_k_cosdf(y);
    }
}

PSK_LIBM_DEV float lm_cosf(float x, int *beyond)
{
    const double pio2 = 1.57079632679489661923;
    const double c1pio2 = 1 * pio2, c2pio2 = 2 * pio2, c3pio2 = 3 * pio2, c4pio2 = 4 * pio2;
    uint32_t ix = lm_f_bits(x);
    int sign = (int)(ix >> 31);
    ix &= 0x7fffffffu;
    if (ix <= 0x3f490fdau) {
        if (ix < 0x39800000u) return 1.0f;
        return lm_k_cosdf(x);
    }
    if (ix <= 0x407b53d1u) {
        if (ix > 0x4016cbe3u) return -lm_k_cosdf(sign ? x + c2pio2 : x - c2pio2);
        if (sign) return lm_k_sindf(x + c1pio2);
        return lm_k_sindf(c1pio2 - x);
    }
    if (ix <= 0x40e231d5u) {
        if (ix > 0x40afeddfu) return lm_k_cosdf(sign ? x + c4pio2 : x - c4pio2);
        if (sign) return lm_k_sindf(-x - c3pio2);
        return lm_k_sindf(x - c3pio2);
    }
    if (ix >= 0x7f800000u) return x - x;
    double y;
    int n = lm_rem_pio2f(x, &y, beyond);
    switch (n & 3) {
    case 0: return lm_k_cosdf(y);
    case 1: return lm_k_sindf(-y);
    case 2: return -lm_k_cosdf(y);
    default: return lm_k_sindf(y);
    }
}

PSK_LIBM_DEV float lm_erfc1f(float x)
{
    const float erx = 8.4506291151e-01f;
    const float pa0 = -2.3621185683e-03f, pa1 = 4.1485610604e-01f, pa2 = -3.7220788002e-01f, pa3 = 3.1834661961e-01f, pa4 = -1.1089469492e-01f, pa5 = 3.5478305072e-02f, pa6 = -2.1663755178e-03f;
    const float qa1 = 1.0642088205e-01f, qa2 = 5.4039794207e-01f, qa3 = 7.1828655899e-02f, qa4 = 1.2617121637e-01f, qa5 = 1.3637083583e-02f, qa6 = 1.1984500103e-02f;
    float s = fabsf(x) - 1.0f;
    float P = pa0 + s * (pa1 + s * (pa2 + s * (pa3 + s * (pa4 + s * (pa5 + s * pa6)))));
    float Q = 1.0f + s * (qa1 + s * (qa2 + s * (qa3 + s * (qa4 + s * (qa5 + s * qa6)))));
    return 1.0f - erx - P / Q;
}

PSK_LIBM_DEV float lm_erfc2f(uint32_t ix, float x)
{
    const float ra0 = -9.8649440333e-03f, ra1 = -6.9385856390e-01f, ra2 = -1.0558626175e+01f, ra3 = -6.2375331879e+01f, ra4 = -1.6239666748e+02f, ra5 = -1.8460508728e+02f, ra6 = -8.1287437439e+01f, ra7 = -9.8143291473e+00f;
    const float sa1 = 1.9651271820e+01f, sa2 = 1.3765776062e+02f, sa3 = 4.3456588745e+02f, sa4 = 6.4538726807e+02f, sa5 = 4.2900814819e+02f, sa6 = 1.0863500214e+02f, sa7 = 6.5702495575e+00f, sa8 = -6.0424413532e-02f;
    const float rb0 = -9.8649431020e-03f, rb1 = -7.9928326607e-01f, rb2 = -1.7757955551e+01f, rb3 = -1.6063638306e+02f, rb4 = -6.3756646729e+02f, rb5 = -1.0250950928e+03f, rb6 = -4.8351919556e+02f;
    const float sb1 = 3.0338060379e+01f, sb2 = 3.2579251099e+02f, sb3 = 1.5367296143e+03f, sb4 = 3.1998581543e+03f, sb5 = 2.5530502930e+03f, sb6 = 4.7452853394e+02f, sb7 = -2.2440952301e+01f;
    if (ix < 0x3fa00000u) return lm_erfc1f(x); // |x| < 1.25
    x = fabsf(x);
    float s = 1.0f / (x * x), R, S;
    if (ix < 0x4036db6du) { // |x| < 1/0.35
        R = ra0 + s * (ra1 + s * (ra2 + s * (ra3 + s * (ra4 + s * (ra5 + s * (ra6 + s * ra7))))));
        S = 1.0f + s * (sa1 + s * (sa2 + s * (sa3 + s * (sa4 + s * (sa5 + s * (sa6 + s * (sa7 + s * sa8)))))));
    } else {
        R = rb0 + s * (rb1 + s * (rb2 + s * (rb3 + s * (rb4 + s * (rb5 + s * rb6)))));
        S = 1.0f + s * (sb1 + s * (sb2 + s * (sb3 + s * (sb4 + s * (sb5 + s * (sb6 + s * sb7))))));
    }
    float z = lm_bits_f(lm_f_bits(x) & 0xffffe000u);
    return lm_expf(-z * z - 0.5625f) * lm_expf((z - x) * (z + x) + R / S) / x;
}

PSK_LIBM_DEV float lm_erff(float x)
{
    const float efx8 = 1.0270333290e+00f;
    const float pp0 = 1.2837916613e-01f, pp1 = -3.2504209876e-01f, pp2 = -2.8481749818e-02f, pp3 = -5.7702702470e-03f, pp4 = -2.3763017452e-05f;
    const float qq1 = 3.9791721106e-01f, qq2 = 6.5022252500e-02f, qq3 = 5.0813062117e-03f, qq4 = 1.3249473704e-04f, qq5 = -3.9602282413e-06f;
    uint32_t ix = lm_f_bits(x);
    int sign = (int)(ix >> 31);
    ix &= 0x7fffffffu;
    if (ix >= 0x7f800000u) return (float)(1 - 2 * sign) + 1.0f / x;
    if (ix < 0x3f580000u) { // |x| < 0.84375
        if (ix < 0x31800000u) return 0.125f * (8.0f * x + efx8 * x);
        float z = x * x;
        float r = pp0 + z * (pp1 + z * (pp2 + z * (pp3 + z * pp4)));
        float s = 1.0f + z * (qq1 + z * (qq2 + z * (qq3 + z * (qq4 + z * qq5))));
        float y = r / s;
        return x + x * y;
    }
    float y;
    if (ix < 0x40c00000u) y = 1.0f - lm_erfc2f(ix, x);
    else y = 1.0f - 0x1p-120f;
    return sign ? -y : y;
}

} // namespace psk
