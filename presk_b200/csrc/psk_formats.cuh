// Storage formats of a realization, packed and unpacked in registers.
//
// A kernel computes in f32; only its loads and stores convert
// (presk-rt/src/lib.rs:147-152). A load widens exactly. A store rounds once,
// to nearest, ties to even; a NaN stays a NaN, quiet, with the top bits of its
// payload. The bit patterns are those of presk-rt/src/lib.rs:228-241 (bf16),
// presk-rt/src/codes.rs:29-184 (binary16, e8m15) and
// presk-format/src/lib.rs:136,328-361 (e4m3fn); the overflow guard's test is
// codes.rs `overflows` (thresholds 65520 and (2 - 2^-16)·2^127).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/presk_cuda.h"

#define PSK_DEV __device__ __forceinline__

namespace psk {

PSK_DEV float bits_f32(uint32_t w) { return __uint_as_float(w); }
PSK_DEV uint32_t f32_bits(float x) { return __float_as_uint(x); }

// ---- bf16: the top sixteen bits of an f32 --------------------------------
PSK_DEV float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

PSK_DEV uint16_t f32_to_bf16(float x)
{
    uint32_t b = f32_bits(x);
    if ((b & 0x7fffffffu) > 0x7f800000u)
        return (uint16_t)((b >> 16) | 0x0040u);
    return (uint16_t)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}

// Two f32 rounded to bf16 and packed, the first in the low half. The hardware's
// conversion is the same rounding for every number and infinity; it makes any
// NaN the canonical one, where the reference keeps sign and payload, so a pair
// that holds a NaN is redone by the integer form.
PSK_DEV uint32_t pack_bf16x2_hw(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

PSK_DEV uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t r = pack_bf16x2_hw(lo, hi);
    if (lo != lo || hi != hi) r = (uint32_t)f32_to_bf16(lo) | ((uint32_t)f32_to_bf16(hi) << 16);
    return r;
}

PSK_DEV uint32_t pack_f16x2_hw(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---- binary16 ------------------------------------------------------------
// The hardware conversions are IEEE's for every number; only NaNs need care,
// since cvt gives a canonical NaN where the reference keeps sign and payload.
PSK_DEV float f16_to_f32(uint16_t c)
{
    uint32_t mag = c & 0x7fffu;
    if (mag > 0x7c00u)
        return bits_f32(((uint32_t)(c & 0x8000u) << 16) | 0x7fc00000u | (mag << 13));
    return __half2float(__ushort_as_half(c));
}

PSK_DEV uint16_t f32_to_f16(float x)
{
    uint32_t b = f32_bits(x), a = b & 0x7fffffffu;
    if (a > 0x7f800000u)
        return (uint16_t)((b >> 16 & 0x8000u) | (((a >> 13) | 0x7e00u) & 0x7fffu));
    return __half_as_ushort(__float2half_rn(x));
}

// ---- e8m15: the top 24 bits of an f32, three bytes little-endian ---------
PSK_DEV float e8m15_to_f32(uint32_t code) { return bits_f32(code << 8); }

PSK_DEV uint32_t f32_to_e8m15(float x)
{
    uint32_t b = f32_bits(x);
    if ((b & 0x7fffffffu) > 0x7f800000u)
        return (b >> 8) | 0x4000u;
    return (b + 0x7fu + ((b >> 8) & 1u)) >> 8;
}

PSK_DEV uint32_t load_e8m15(const uint8_t *p, int64_t i)
{
    const uint8_t *q = p + 3 * i;
    return (uint32_t)q[0] | (uint32_t)q[1] << 8 | (uint32_t)q[2] << 16;
}

PSK_DEV void store_e8m15(uint8_t *p, int64_t i, uint32_t code)
{
    uint8_t *q = p + 3 * i;
    q[0] = (uint8_t)code;
    q[1] = (uint8_t)(code >> 8);
    q[2] = (uint8_t)(code >> 16);
}

// ---- e4m3fn: 1+4+3 bits, bias 7, no infinity, NaN = 0x7f; max 448 --------
PSK_DEV float e4m3_to_f32(uint8_t c)
{
    uint32_t sign = (uint32_t)(c & 0x80u) << 24, mag = c & 0x7fu;
    if (mag == 0x7fu)
        return bits_f32(sign | 0x7fc00000u);
    uint32_t e = mag >> 3, m = mag & 7u;
    float v = e == 0 ? (float)m * 0.001953125f /* 2^-9 */ : bits_f32(((e + 120u) << 23) | (m << 20));
    return bits_f32(f32_bits(v) | sign);
}

// Round to nearest even; a magnitude that rounds past 448 has no infinity to
// go to and becomes the NaN (presk-format/src/lib.rs tests: 464 -> 448,
// 465 -> NaN).
PSK_DEV uint8_t f32_to_e4m3(float x)
{
    uint32_t b = f32_bits(x), sign = (b >> 24) & 0x80u, a = b & 0x7fffffffu;
    if (a > 0x7f800000u)
        return (uint8_t)(sign | 0x7fu);
    float ax = bits_f32(a);
    if (ax < 0.015625f) { // below 2^-6: subnormal, a multiple of 2^-9
        float t = ax * 512.0f + 12582912.0f; // 1.5·2^23: the addition rounds to an integer, ties to even
        uint32_t q = f32_bits(t) - 0x4b400000u;
        return (uint8_t)(sign | q);
    }
    // normal: round the 23-bit fraction at bit 20
    uint32_t r = a + 0x7ffffu + ((a >> 20) & 1u);
    uint32_t e = (r >> 23), m = (r >> 20) & 7u;
    if (e > 135u || (e == 135u && m == 7u))
        return (uint8_t)(sign | 0x7fu);
    return (uint8_t)(sign | ((e - 120u) << 3) | m);
}

// ---- the overflow guard ---------------------------------------------------
// Whether storing x rounds a finite value to an infinity.
PSK_DEV uint32_t overflows(float x, uint32_t threshold)
{
    return ((f32_bits(x) & 0x7fffffffu) - threshold) < (0x7f800000u - threshold);
}
constexpr uint32_t kF16Overflow = 0x477ff000u;   // 65520
constexpr uint32_t kE8m15Overflow = 0x7f7fff80u; // (2 - 2^-16)·2^127

PSK_DEV uint32_t store_overflows(int dtype, float x)
{
    if (dtype == PSK_F16) return overflows(x, kF16Overflow);
    if (dtype == PSK_E8M15) return overflows(x, kE8m15Overflow);
    return 0u;
}

PSK_DEV size_t dtype_bytes(int dtype)
{
    switch (dtype) {
    case PSK_F64: case PSK_I64: return 8;
    case PSK_F32: return 4;
    case PSK_BF16: case PSK_F16: return 2;
    case PSK_E8M15: return 3;
    default: return 1;
    }
}

// ---- a saturating conversion of a real to an index ------------------------
// toward zero, 0 for a NaN (presk_rt.h `presk_f64_to_i64`, Cranelift's
// fcvt_to_sint_sat), which is what cvt.rzi.s64 does.
PSK_DEV int64_t f32_to_i64(float x) { return x != x ? 0 : __float2ll_rz(x); }

// ---- generic element access by runtime dtype ------------------------------
// A load in a kernel of arithmetic f32: the stored value widened exactly; an
// f64 is rounded to f32 (exec.rs:642-662, `from_f64(x) = x as f32`); an index
// is converted as `i as f64 as f32`.
PSK_DEV float load_real(const void *p, int dtype, int64_t i)
{
    switch (dtype) {
    case PSK_F32: return ((const float *)p)[i];
    case PSK_BF16: return bf16_to_f32(((const uint16_t *)p)[i]);
    case PSK_F16: return f16_to_f32(((const uint16_t *)p)[i]);
    case PSK_E8M15: return e8m15_to_f32(load_e8m15((const uint8_t *)p, i));
    case PSK_F64: return (float)((const double *)p)[i];
    case PSK_I64: return (float)(double)((const int64_t *)p)[i];
    case PSK_E4M3: return e4m3_to_f32(((const uint8_t *)p)[i]);
    case PSK_I8: return (float)((const int8_t *)p)[i];
    default: return 0.0f;
    }
}

// A store: rounded once to the buffer's type; returns the guard's test.
PSK_DEV uint32_t store_real(void *p, int dtype, int64_t i, float x)
{
    switch (dtype) {
    case PSK_F32: ((float *)p)[i] = x; return 0u;
    case PSK_BF16: ((uint16_t *)p)[i] = f32_to_bf16(x); return 0u;
    case PSK_F16: ((uint16_t *)p)[i] = f32_to_f16(x); return overflows(x, kF16Overflow);
    case PSK_E8M15: store_e8m15((uint8_t *)p, i, f32_to_e8m15(x)); return overflows(x, kE8m15Overflow);
    case PSK_F64: ((double *)p)[i] = (double)x; return 0u;
    case PSK_I64: ((int64_t *)p)[i] = f32_to_i64(x); return 0u;
    case PSK_E4M3: ((uint8_t *)p)[i] = f32_to_e4m3(x); return 0u;
    default: return 0u;
    }
}

// The value a kernel of type `kdtype` sees of an input stored as `dtype`:
// itself when the input is as wide or narrower (a widening at the kernel's
// edge or in its loads is exact), else rounded to the kernel's type first,
// as the host converts a buffer at a kernel's edge through f64
// (host.rs:809-829; to bf16 by way of f32, presk-rt/src/lib.rs:868-876).
PSK_DEV float edge_round(float x, int kdtype, int dtype, uint32_t *ovf)
{
    if (dtype == kdtype || dtype == PSK_I64 || dtype == PSK_I8)
        return x;
    switch (kdtype) {
    case PSK_BF16: return (dtype == PSK_F32 || dtype == PSK_F64 || dtype == PSK_F16 || dtype == PSK_E8M15) ? bf16_to_f32(f32_to_bf16(x)) : x;
    case PSK_F16:
        if (dtype == PSK_E4M3) return x;
        *ovf |= overflows(x, kF16Overflow);
        return f16_to_f32(f32_to_f16(x));
    case PSK_E8M15:
        if (dtype == PSK_BF16 || dtype == PSK_F16 || dtype == PSK_E4M3) return x;
        *ovf |= overflows(x, kE8m15Overflow);
        return e8m15_to_f32(f32_to_e8m15(x));
    default: return x;
    }
}

} // namespace psk
