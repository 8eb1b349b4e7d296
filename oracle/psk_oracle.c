/* psk_oracle.c: TEST INFRASTRUCTURE. A CPU restatement of the reference's
 * kernel semantics for the launches of include/presk_cuda.h, used only by
 * tests/, by __graft_entry__.smoke() and by bench.py's CPU legs as the checker
 * and the timed CPU baseline. The product (presk_b200/) never links, loads or
 * calls it.
 *
 * What it follows, in presk-lang/presk:
 *   - crates/presk-kernel/src/exec.rs:146-183 (`impl Elem for f32`): one IEEE
 *     operation in f32 per Bin/Un, musl's transcendental functions;
 *     :642-662 loads widen exactly; :758-782 stores round once; :847-859
 *     f32, bf16, binary16 and e8m15 kernels all compute in f32;
 *   - crates/presk-kernel/src/lower.rs, per primitive (cited at each function);
 *   - crates/presk-rt/src/lib.rs:228-241 (bf16), crates/presk-rt/src/codes.rs
 *     (binary16, e8m15, the overflow guard), presk-rt/src/quant.rs:128-167.
 *
 * The transcendental functions are the reference's own C
 * (crates/presk-export-c/c/presk_libm.c), compiled where it lies into
 * oracle/_ref/libpresk_ref.so by oracle/Makefile and linked here: the same
 * bits the reference's executors compute (its tests/libm.rs pins that C to
 * the `libm` crate on 10^6 inputs a function). Everything else in this file
 * is a restatement, pinned by tests/test_oracle_*.py against that library's
 * conversions and against the reference's golden vectors.
 *
 * Build: cc -std=c11 -O2 -ffp-contract=off (never -ffast-math), as the
 * reference builds its C (crates/presk-export-c/src/lib.rs:90). -fopenmp
 * divides the outermost loop of a launch among the host's cores, as the
 * native executor divides one parallel loop among its workers
 * (crates/presk-cranelift/src/lib.rs:1636-1691); the bits do not depend on it.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "../include/presk_cuda.h"

/* the reference's libm, from oracle/_ref/libpresk_ref.so */
float presk_expf(float);
float presk_logf(float);
float presk_tanhf(float);
float presk_sinf(float);
float presk_cosf(float);
float presk_erff(float);

static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* ---- storage formats -------------------------------------------------------- */
float psk_o_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* presk-rt/src/lib.rs:228-236: to nearest, ties to even; a NaN quiet */
uint16_t psk_o_f32_to_bf16(float x)
{
    uint32_t b = f2u(x);
    if (x != x) return (uint16_t)((b >> 16) | 0x40u);
    return (uint16_t)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}

/* binary16 widened exactly; a NaN keeps sign and payload, made quiet (codes.rs) */
float psk_o_f16_to_f32(uint16_t c)
{
    uint32_t sign = (uint32_t)(c & 0x8000u) << 16, e = (c >> 10) & 0x1fu, m = c & 0x3ffu;
    if (e == 0x1f) return u2f(sign | 0x7f800000u | (m ? 0x400000u | (m << 13) : 0u));
    if (e == 0) {
        float v = (float)m * 0x1p-24f; /* subnormal: m·2^-24, exact */
        return u2f(f2u(v) | sign);
    }
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

/* The code of the IEEE format with t fraction bits and w exponent bits
 * nearest a finite magnitude given as an integer significand `sig` (its top
 * bit set at position `top`) times 2^(exp - top): ties to even, overflow to
 * the infinity's code. The one rounding of codes.rs `narrow`. */
static uint32_t round_to_format(uint64_t sig, int top, int exp, unsigned t, unsigned w)
{
    const int bias = (1 << (w - 1)) - 1, emin = 1 - bias;
    const uint32_t inf = ((1u << w) - 1u) << t;
    /* the result keeps t+1 significant bits where normal, fewer below emin */
    int drop = top - (int)t;
    if (exp < emin) drop += emin - exp;
    uint64_t q, rem, half;
    if (drop <= 0) {
        q = sig << -drop;
        rem = 0;
        half = 1;
    } else if (drop > 63) {
        q = 0;
        rem = sig != 0;
        half = 2; /* below half of the least subnormal */
    } else {
        q = sig >> drop;
        rem = sig & (((uint64_t)1 << drop) - 1);
        half = (uint64_t)1 << (drop - 1);
    }
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    uint64_t code;
    if (exp >= emin) code = ((uint64_t)(exp + bias - 1) << t) + q; /* the leading one adds into the exponent */
    else code = q;
    return code < inf ? (uint32_t)code : inf;
}

uint16_t psk_o_f32_to_f16(float x)
{
    uint32_t b = f2u(x), sign = (b >> 16) & 0x8000u, a = b & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | (((a >> 13) | 0x7e00u) & 0x7fffu));
    if (a == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
    uint32_t e = a >> 23, m = a & 0x7fffffu;
    if (e == 0) return (uint16_t)sign; /* an f32 subnormal is far below half of binary16's least */
    return (uint16_t)(sign | round_to_format((uint64_t)m | 0x800000u, 23, (int)e - 127, 10, 5));
}

static uint32_t narrow_f64(double x, unsigned t, unsigned w)
{
    uint64_t b;
    memcpy(&b, &x, 8);
    uint32_t sign = (uint32_t)(b >> 63) << (t + w);
    uint64_t a = b & ~((uint64_t)1 << 63);
    const uint32_t inf = ((1u << w) - 1u) << t;
    if (a > (uint64_t)0x7ff << 52) return sign | inf | (1u << (t - 1)) | (uint32_t)((a >> (52 - t)) & ((1u << (t - 1)) - 1u));
    if (a == (uint64_t)0x7ff << 52) return sign | inf;
    int e = (int)(a >> 52);
    if (e == 0) return sign;
    return sign | round_to_format((a & (((uint64_t)1 << 52) - 1)) | ((uint64_t)1 << 52), 52, e - 1023, t, w);
}

uint16_t psk_o_f64_to_f16(double x) { return (uint16_t)narrow_f64(x, 10, 5); }
uint32_t psk_o_f64_to_e8m15(double x) { return narrow_f64(x, 15, 8); }

float psk_o_e8m15_to_f32(uint32_t code) { return u2f(code << 8); }

/* codes.rs:96-102 */
uint32_t psk_o_f32_to_e8m15(float x)
{
    uint32_t b = f2u(x);
    if (x != x) return (b >> 8) | 0x4000u;
    return (b + 0x7fu + ((b >> 8) & 1u)) >> 8;
}

/* presk-format/src/lib.rs:136: e4m3fn, bias 7, no infinity, one NaN, max 448 */
float psk_o_e4m3_to_f32(uint8_t c)
{
    uint32_t sign = (uint32_t)(c & 0x80u) << 24, e = (c >> 3) & 0xfu, m = c & 7u;
    if ((c & 0x7fu) == 0x7fu) return u2f(sign | 0x7fc00000u);
    float v = e == 0 ? (float)m * 0x1p-9f : ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
    return u2f(f2u(v) | sign);
}

uint8_t psk_o_f32_to_e4m3(float x)
{
    uint32_t b = f2u(x), sign = (b >> 24) & 0x80u, a = b & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7fu);
    if (a == 0x7f800000u) return (uint8_t)(sign | 0x7fu); /* no infinity: the NaN */
    uint32_t e = a >> 23, m = a & 0x7fffffu;
    if (e == 0) return (uint8_t)sign;
    /* as an IEEE format of 3 fraction and 4 exponent bits, then the top code is the NaN */
    const int bias = 7, emin = 1 - bias, t = 3;
    int exp = (int)e - 127, drop = 23 - t;
    if (exp < emin) drop += emin - exp;
    uint64_t sig = (uint64_t)m | 0x800000u, q, rem, half;
    if (drop > 63) { q = 0; rem = 1; half = 2; }
    else { q = sig >> drop; rem = sig & (((uint64_t)1 << drop) - 1); half = (uint64_t)1 << (drop - 1); }
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    uint64_t code = exp >= emin ? ((uint64_t)(exp + bias - 1) << t) + q : q;
    if (code >= 0x7f) return (uint8_t)(sign | 0x7fu);
    return (uint8_t)(sign | code);
}

/* codes.rs `overflows`: a finite value the store turns into an infinity */
uint32_t psk_o_overflows(int dtype, float x)
{
    uint32_t a = f2u(x) & 0x7fffffffu;
    if (dtype == PSK_F16) return a >= 0x477ff000u && a < 0x7f800000u;
    if (dtype == PSK_E8M15) return a >= 0x7f7fff80u && a < 0x7f800000u;
    return 0;
}

static size_t elem_bytes(int dtype)
{
    switch (dtype) {
    case PSK_F64: case PSK_I64: return 8;
    case PSK_F32: return 4;
    case PSK_BF16: case PSK_F16: return 2;
    case PSK_E8M15: return 3;
    default: return 1;
    }
}

/* exec.rs:642-662: a load in a kernel of arithmetic f32 */
static float load_real(const void *p, int dtype, int64_t i)
{
    switch (dtype) {
    case PSK_F32: return ((const float *)p)[i];
    case PSK_BF16: return psk_o_bf16_to_f32(((const uint16_t *)p)[i]);
    case PSK_F16: return psk_o_f16_to_f32(((const uint16_t *)p)[i]);
    case PSK_E8M15: {
        const uint8_t *q = (const uint8_t *)p + 3 * i;
        return psk_o_e8m15_to_f32((uint32_t)q[0] | (uint32_t)q[1] << 8 | (uint32_t)q[2] << 16);
    }
    case PSK_F64: return (float)((const double *)p)[i];
    case PSK_I64: return (float)(double)((const int64_t *)p)[i];
    case PSK_E4M3: return psk_o_e4m3_to_f32(((const uint8_t *)p)[i]);
    case PSK_I8: return (float)((const int8_t *)p)[i];
    default: return 0.0f;
    }
}

/* presk_rt.h `presk_f64_to_i64`: toward zero, saturating, 0 for a NaN */
static int64_t f32_to_i64(float x)
{
    if (x != x) return 0;
    if (x >= 9223372036854775808.0f) return INT64_MAX;
    if (x < -9223372036854775808.0f) return INT64_MIN;
    return (int64_t)x;
}

/* exec.rs:758-782: a store, rounded once; returns the guard's test */
static uint32_t store_real(void *p, int dtype, int64_t i, float x)
{
    switch (dtype) {
    case PSK_F32: ((float *)p)[i] = x; return 0;
    case PSK_BF16: ((uint16_t *)p)[i] = psk_o_f32_to_bf16(x); return 0;
    case PSK_F16: ((uint16_t *)p)[i] = psk_o_f32_to_f16(x); return psk_o_overflows(PSK_F16, x);
    case PSK_E8M15: {
        uint32_t c = psk_o_f32_to_e8m15(x);
        uint8_t *q = (uint8_t *)p + 3 * i;
        q[0] = (uint8_t)c; q[1] = (uint8_t)(c >> 8); q[2] = (uint8_t)(c >> 16);
        return psk_o_overflows(PSK_E8M15, x);
    }
    case PSK_F64: ((double *)p)[i] = (double)x; return 0;
    case PSK_I64: ((int64_t *)p)[i] = f32_to_i64(x); return 0;
    case PSK_E4M3: ((uint8_t *)p)[i] = psk_o_f32_to_e4m3(x); return 0;
    default: return 0;
    }
}

/* host.rs:809-829: an input of another type than the kernel's is converted at
 * its edge, Buf::of(kdtype, b.to_f64()); a widening is exact, so only a
 * narrowing changes a value. Done here element by element as it is loaded. */
static float edge_round(float x, int kdtype, int dtype, uint32_t *ovf)
{
    if (dtype == kdtype || dtype == PSK_I64 || dtype == PSK_I8) return x;
    switch (kdtype) {
    case PSK_BF16:
        return (dtype == PSK_F32 || dtype == PSK_F64 || dtype == PSK_F16 || dtype == PSK_E8M15) ? psk_o_bf16_to_f32(psk_o_f32_to_bf16(x)) : x;
    case PSK_F16:
        if (dtype == PSK_E4M3) return x;
        *ovf |= psk_o_overflows(PSK_F16, x);
        return psk_o_f16_to_f32(psk_o_f32_to_f16(x));
    case PSK_E8M15:
        if (dtype == PSK_BF16 || dtype == PSK_F16 || dtype == PSK_E4M3) return x;
        *ovf |= psk_o_overflows(PSK_E8M15, x);
        return psk_o_e8m15_to_f32(psk_o_f32_to_e8m15(x));
    default: return x;
    }
}

/* ---- affine formats and exact integer sums (presk-format/src/lib.rs:865-954, 1148-1193;
 *      presk-kernel/src/exec.rs:493-526, 601-616) ------------------------------------- */
typedef unsigned __int128 u128;

static int64_t affine_min(int kind) { return kind == 2 ? 0 : -128; }
static int64_t affine_max(int kind) { return kind == 2 ? 255 : 127; }

/* x = m·2^e with m an integer: a finite double taken apart. */
static void take_apart(double x, int64_t *m, int *e)
{
    uint64_t b;
    memcpy(&b, &x, 8);
    int field = (int)((b >> 52) & 0x7ff);
    uint64_t frac = b & (((uint64_t)1 << 52) - 1);
    int64_t mag = field ? (int64_t)(frac | ((uint64_t)1 << 52)) : (int64_t)frac;
    *e = (field ? field : 1) - 1075;
    *m = (b >> 63) ? -mag : mag;
}

/* The integer nearest (mag·2^e) / s with the sign given, ties to even, for mag < 2^90 and s a
 * positive normal f32: the exact quotient's rounding (presk-format `quotient_round`), saturated
 * at +-2^62. */
static int64_t quotient_round_exact(int neg, u128 mag, int e, float s)
{
    if (mag == 0) return 0;
    int64_t ms64;
    int es;
    take_apart((double)s, &ms64, &es);
    while ((ms64 & 1) == 0) { ms64 >>= 1; ++es; } /* s = ms·2^es with ms odd, below 2^24 */
    const u128 ms = (u128)ms64;
    int bits = 0;
    for (u128 t = mag; t; t >>= 1) ++bits;
    const int k = e - es; /* the quotient is mag·2^k / ms */
    u128 num = mag, den = ms;
    if (k >= 0) {
        if (bits + k > 120) return neg ? -((int64_t)1 << 62) : ((int64_t)1 << 62);
        num = mag << k;
    } else {
        if (-k > bits + 2) return 0; /* below a quarter */
        den = ms << -k;              /* below 2^(24 + 92) */
    }
    u128 q = num / den, r = num % den, twice = r << 1;
    if (twice > den || (twice == den && (q & 1))) q += 1;
    if (q > ((u128)1 << 62)) q = (u128)1 << 62;
    return neg ? -(int64_t)q : (int64_t)q;
}

/* A real stored in an affine format: q = clamp(rne(x / s) + z), the quotient exact
 * (Affine::round_scaled with quotient None, zero added after). A NaN is the zero point. */
int64_t psk_o_affine_code(double x, int kind, float scale, int zero)
{
    if (x != x) return zero;
    if (isinf(x)) return x > 0 ? affine_max(kind) : affine_min(kind);
    int64_t m;
    int e;
    take_apart(x, &m, &e);
    int64_t n = quotient_round_exact(m < 0, (u128)(m < 0 ? -m : m), e, scale);
    int64_t q = n + zero;
    return q < affine_min(kind) ? affine_min(kind) : (q > affine_max(kind) ? affine_max(kind) : q);
}

/* The exact value n·base (base the product of two f32 scales, exact in a double) rounded once
 * into the IEEE format of t fraction and w exponent bits: its code. */
static uint32_t round_count_to_float(int64_t n, double base, unsigned t, unsigned w)
{
    if (n == 0) return 0;
    int64_t mb;
    int eb;
    take_apart(base, &mb, &eb);
    u128 mag = (u128)(n < 0 ? -n : n) * (u128)mb;
    int bits = 0;
    for (u128 v = mag; v; v >>= 1) ++bits;
    /* keep 62 bits and a sticky one: the rounding position is far above */
    int drop = bits > 62 ? bits - 62 : 0;
    uint64_t sig = (uint64_t)(mag >> drop);
    if (drop && (mag & ((((u128)1) << drop) - 1))) sig |= 1;
    int top = bits - drop - 1;
    uint32_t code = round_to_format(sig, top, eb + drop + top, t, w);
    return (n < 0 ? (1u << (t + w)) : 0u) | code;
}

/* Whether a kernel of type kd reads an input stored as `dtype` without rounding it. */
static int edge_is_identity(int kd, int dtype)
{
    uint32_t ovf = 0;
    (void)ovf;
    if (dtype == kd || dtype == PSK_I8 || dtype == PSK_I64) return 1;
    if (kd == PSK_F32) return 1;
    if (kd == PSK_E8M15) return dtype == PSK_BF16 || dtype == PSK_F16 || dtype == PSK_E4M3;
    return 0;
}

/* ---- a launch's operands ------------------------------------------------------ */
typedef struct {
    const uint8_t *p;
    const float *scales;
    const psk_operand *o;
} operand;

static int64_t offset_of(const int64_t *stride, const int64_t *dims, int first, int n, int64_t lin)
{
    int64_t off = 0;
    for (int a = first + n - 1; a >= first; --a) {
        int64_t d = dims[a], i = lin % d;
        lin /= d;
        off += i * stride[a];
    }
    return off;
}

/* The integer a counted nest reads of an operand, and its unit (exec.rs `from_scaled`). */
static int32_t load_count(const operand *x, int64_t off, int64_t soff, double *unit)
{
    if (x->o->affine) {
        *unit = (double)x->o->affine_scale;
        int q = x->o->affine == 2 ? (int)((const uint8_t *)x->p)[off] : (int)((const int8_t *)x->p)[off];
        return q - x->o->affine_zero;
    }
    *unit = (double)x->scales[soff];
    return (int)((const int8_t *)x->p)[off];
}

static float load_operand(const operand *x, int64_t off, int64_t soff, int kdtype, uint32_t *ovf)
{
    if (x->o->affine) { /* (q - z)·s, exact in a double, read by an f32 nest: rounded to f32 */
        int q = x->o->affine == 2 ? (int)((const uint8_t *)x->p)[off] : (int)((const int8_t *)x->p)[off];
        return (float)((double)(q - x->o->affine_zero) * (double)x->o->affine_scale);
    }
    if (x->o->dtype == PSK_I8) return (float)((const int8_t *)x->p)[off] * x->scales[soff]; /* quant.rs:250-252 */
    return edge_round(load_real(x->p, x->o->dtype, off), kdtype, x->o->dtype, ovf);
}

/* lower.rs:184-226, exec.rs:146-183 */
static float prim_unary(int prim, float x, int imm)
{
    switch (prim) {
    case PSK_NEG: return -x;
    case PSK_EXP: return presk_expf(x);
    case PSK_LOG: return presk_logf(x);
    case PSK_TANH: return presk_tanhf(x);
    case PSK_SQRT: return sqrtf(x);
    case PSK_SIN: return presk_sinf(x);
    case PSK_COS: return presk_cosf(x);
    case PSK_ABS: return fabsf(x);
    case PSK_GELU: {
        float phi = (1.0f + presk_erff(x / (float)1.4142135623730951)) / 2.0f;
        return x * phi;
    }
    case PSK_GELU_DERIV: {
        float phi = (1.0f + presk_erff(x / (float)1.4142135623730951)) / 2.0f;
        float dens = presk_expf((-(x * x)) / 2.0f) / (float)2.5066282746310002;
        return phi + x * dens;
    }
    case PSK_RELU: return x < 0.0f ? 0.0f : x;
    case PSK_HEAVISIDE: return x > 0.0f ? 1.0f : 0.0f;
    case PSK_SIGN: return x < 0.0f ? -1.0f : (x > 0.0f ? 1.0f : 0.0f);
    case PSK_SIGMOID: return 1.0f / (1.0f + presk_expf(-x));
    case PSK_POW: {
        if (imm == 0) return 1.0f;
        float e = x;
        for (int i = 1; i < imm; ++i) e = e * x;
        return e;
    }
    case PSK_DIV_N: return x / (float)(double)imm; /* lower.rs:1266 `mean_vjp` */
    case PSK_ROUND: /* a site inside a merged group: rounded as its own launch would have stored it */
        return imm == PSK_BF16 ? psk_o_bf16_to_f32(psk_o_f32_to_bf16(x)) : imm == PSK_F16 ? psk_o_f16_to_f32(psk_o_f32_to_f16(x)) : imm == PSK_E8M15 ? psk_o_e8m15_to_f32(psk_o_f32_to_e8m15(x)) : x;
    default: return x;
    }
}

static float prim_binary(int prim, float x, float y)
{
    switch (prim) {
    case PSK_ADD: return x + y;
    case PSK_SUB: return x - y;
    case PSK_MUL: return x * y;
    case PSK_DIV: return x / y;
    case PSK_MAX: return x > y ? x : y;
    default: return x < y ? x : y;
    }
}

/* A store into the launch's output: its float type, or its affine format (exec.rs:758-782). */
static uint32_t store_out(const psk_launch *l, uint8_t *outp, int64_t off, float x)
{
    if (l->out.affine) {
        int64_t q = psk_o_affine_code((double)x, l->out.affine, l->out.affine_scale, l->out.affine_zero);
        if (l->out.affine == 2) ((uint8_t *)outp)[off] = (uint8_t)q;
        else ((int8_t *)outp)[off] = (int8_t)q;
        return 0;
    }
    return store_real(outp, l->out.dtype, off, x);
}

/* ---- the launches ------------------------------------------------------------- */
static int psk_oracle_run_merged(const psk_launch *l, void *const *table, uint32_t *overflow);

/* Summed axes that every operand walks as one (stride[a] = stride[a+1]·dims[a+1]) are one axis:
 * the terms come in the same lexicographic order either way, so a contraction over several
 * contiguous axes (the output projection's groups, per, hd) is the nest over their product. */
int psk_oracle_run(const psk_launch *l, void *const *table, uint32_t *overflow);

/* PSK_OP_ATTENTION is by definition its four launches one after the other (examples/coverage/llama.psk:100-102:
 * ein(q*k), / rt, softmax where mask, ein(a*v)), each of them the reference's own nest with its result stored in
 * its site's type. The space (.., seq, hd | seq2) is re-read as (.., seq, seq2 | hd) for the first three. */
static void attn_operand(psk_operand *d, const psk_operand *s, int no)
{
    *d = *s;
    d->stride[no - 1] = s->stride[no];     /* seq2 becomes the last outer axis */
    d->stride[no] = s->stride[no - 1];     /* hd the summed one */
    d->scale_stride[no - 1] = s->scale_stride[no];
    d->scale_stride[no] = s->scale_stride[no - 1];
}

static void attn_contiguous(psk_operand *d, int dtype, const int64_t *dims, int naxes, int skip)
{
    memset(d, 0, sizeof *d);
    d->dtype = dtype;
    int64_t acc = 1;
    for (int a = naxes - 1; a >= 0; --a) {
        if (a == skip) continue;
        d->stride[a] = acc;
        acc *= dims[a];
    }
    d->numel = acc;
}

static int attention_unfused(const psk_launch *l, void *const *table, uint32_t *overflow)
{
    const int no = l->n_outer;
    if (no < 2 || no > PSK_MAX_RANK || l->n_inner != 1 || (l->n_inputs != 4 && l->n_inputs != 5)) return PSK_E7001;
    const int64_t hd = l->dims[no - 1], t2 = l->dims[no];
    int64_t rows = 1;
    for (int a = 0; a < no - 1; ++a) rows *= l->dims[a];
    const int d_scores = (int)l->iparam[1], d_scaled = (int)l->iparam[2], d_soft = (int)l->iparam[3];
    const size_t n = (size_t)(rows * t2 ? rows * t2 : 1);
    void *se = malloc(n * elem_bytes(d_scores)), *sc = malloc(n * elem_bytes(d_scaled)), *sm = malloc(n * elem_bytes(d_soft));
    uint32_t ovf = 0, o1 = 0;
    int rc = PSK_OK;
    psk_launch m;
    int64_t dims[PSK_MAX_AXES];
    for (int a = 0; a < no - 1; ++a) dims[a] = l->dims[a];
    dims[no - 1] = t2;
    dims[no] = hd;
    /* scores */
    memset(&m, 0, sizeof m);
    m.name = "attention: scores"; m.op = PSK_OP_CONTRACT; m.dtype = d_scores; m.order = l->order; m.guarded = l->guarded;
    m.n_inputs = 2; m.n_outer = no; m.n_inner = 1;
    memcpy(m.dims, dims, sizeof dims);
    attn_operand(&m.in[0], &l->in[0], no);
    attn_operand(&m.in[1], &l->in[1], no);
    attn_contiguous(&m.out, d_scores, dims, no, -1);
    { void *t[3] = {table[0], table[1], se}; rc = psk_oracle_run(&m, t, &o1); ovf |= o1; }
    /* scores / rt */
    if (rc == PSK_OK) {
        memset(&m, 0, sizeof m);
        m.name = "attention: div"; m.op = PSK_OP_FUSED; m.dtype = d_scaled; m.order = l->order; m.guarded = l->guarded;
        m.n_inputs = 2; m.n_outer = no; m.n_inner = 0;
        memcpy(m.dims, dims, sizeof dims);
        attn_contiguous(&m.in[0], d_scores, dims, no, -1);
        m.in[1] = l->in[3];
        memset(m.in[1].stride, 0, sizeof m.in[1].stride);
        attn_contiguous(&m.out, d_scaled, dims, no, -1);
        m.n_steps = 1;
        m.steps[0].prim = PSK_DIV; m.steps[0].nargs = 2; m.steps[0].src[0] = 0; m.steps[0].src[1] = 1;
        void *t[3] = {se, table[3], sc};
        rc = psk_oracle_run(&m, t, &o1); ovf |= o1;
    }
    /* softmax over seq2 */
    if (rc == PSK_OK) {
        memset(&m, 0, sizeof m);
        m.name = "attention: softmax"; m.op = PSK_OP_SOFTMAX; m.dtype = d_soft; m.order = l->order; m.guarded = l->guarded;
        m.n_inputs = l->n_inputs == 5 ? 2 : 1; m.masked = l->n_inputs == 5; m.n_outer = no - 1; m.n_inner = 1;
        memcpy(m.dims, dims, sizeof dims);
        attn_contiguous(&m.in[0], d_scaled, dims, no, -1);
        attn_contiguous(&m.out, d_soft, dims, no, -1);
        if (m.masked) attn_operand(&m.in[1], &l->in[4], no);
        void *t[3] = {sc, m.masked ? table[4] : sm, sm};
        if (!m.masked) t[1] = sm;
        rc = psk_oracle_run(&m, t, &o1); ovf |= o1;
    }
    /* the weighted values */
    if (rc == PSK_OK) {
        m = *l;
        m.name = "attention: values"; m.op = PSK_OP_CONTRACT; m.n_inputs = 2;
        attn_contiguous(&m.in[0], d_soft, dims, no, -1);
        m.in[0].stride[no] = m.in[0].stride[no - 1]; /* seq2 is the summed axis again, */
        m.in[0].stride[no - 1] = 0;                  /* and hd is not an axis of the weights */
        m.in[1] = l->in[2];
        void *t[3] = {sm, table[2], table[l->n_inputs]};
        rc = psk_oracle_run(&m, t, &o1); ovf |= o1;
    }
    free(se); free(sc); free(sm);
    if (overflow) *overflow = ovf;
    return rc;
}

/* PSK_OP_RMSNORM is by definition RMSNorm.apply's four launches (examples/coverage/llama.psk:34-40): mul, mean over
 * the last axis, [add eps; sqrt], [div; mul gamma], each the reference's own nest with its result in its site's type. */
static int rmsnorm_unfused(const psk_launch *l, void *const *table, uint32_t *overflow)
{
    const int no = l->n_outer;
    if (no < 1 || l->n_inner != 0 || l->n_inputs != 3) return PSK_E7001;
    const int d2 = (int)l->iparam[1], d3 = (int)l->iparam[2], d7 = (int)l->iparam[3];
    int64_t rows = 1;
    for (int a = 0; a < no - 1; ++a) rows *= l->dims[a];
    const int64_t n = l->dims[no - 1];
    void *x2 = malloc((size_t)(rows * n ? rows * n : 1) * elem_bytes(d2)), *ms = malloc((size_t)(rows ? rows : 1) * elem_bytes(d3)), *rt = malloc((size_t)(rows ? rows : 1) * elem_bytes(d7));
    uint32_t ovf = 0, o1 = 0;
    int rc;
    psk_launch m;
    memset(&m, 0, sizeof m);
    m.name = "rmsnorm: mul"; m.op = PSK_OP_FUSED; m.dtype = d2; m.order = l->order; m.guarded = l->guarded;
    m.n_inputs = 2; m.n_outer = no;
    memcpy(m.dims, l->dims, sizeof m.dims);
    m.in[0] = l->in[0]; m.in[1] = l->in[0];
    attn_contiguous(&m.out, d2, l->dims, no, -1);
    m.n_steps = 1; m.steps[0].prim = PSK_MUL; m.steps[0].nargs = 2; m.steps[0].src[0] = 0; m.steps[0].src[1] = 1;
    { void *t[3] = {table[0], table[0], x2}; rc = psk_oracle_run(&m, t, &o1); ovf |= o1; }
    if (rc == PSK_OK) {
        memset(&m, 0, sizeof m);
        m.name = "rmsnorm: mean"; m.op = PSK_OP_REDUCE; m.kind = PSK_REDUCE_MEAN; m.dtype = d3; m.order = l->order; m.guarded = l->guarded;
        m.n_inputs = 1; m.n_outer = no - 1; m.n_inner = 1; m.iparam[0] = n;
        memcpy(m.dims, l->dims, sizeof m.dims);
        attn_contiguous(&m.in[0], d2, l->dims, no, -1);
        attn_contiguous(&m.out, d3, l->dims, no - 1, -1);
        void *t[2] = {x2, ms};
        rc = psk_oracle_run(&m, t, &o1); ovf |= o1;
    }
    if (rc == PSK_OK) {
        memset(&m, 0, sizeof m);
        m.name = "rmsnorm: root"; m.op = PSK_OP_FUSED; m.dtype = d7; m.order = l->order; m.guarded = l->guarded;
        m.n_inputs = 2; m.n_outer = no - 1;
        memcpy(m.dims, l->dims, sizeof m.dims);
        attn_contiguous(&m.in[0], d3, l->dims, no - 1, -1);
        m.in[1] = l->in[1];
        memset(m.in[1].stride, 0, sizeof m.in[1].stride);
        attn_contiguous(&m.out, d7, l->dims, no - 1, -1);
        m.n_steps = 2;
        m.steps[0].prim = PSK_ADD; m.steps[0].nargs = 2; m.steps[0].src[0] = 0; m.steps[0].src[1] = 1;
        m.steps[1].prim = PSK_SQRT; m.steps[1].nargs = 1; m.steps[1].src[0] = -1;
        void *t[3] = {ms, table[1], rt};
        rc = psk_oracle_run(&m, t, &o1); ovf |= o1;
    }
    if (rc == PSK_OK) {
        m = *l;
        m.name = "rmsnorm: scale"; m.op = PSK_OP_FUSED; m.n_inputs = 3;
        m.in[0] = l->in[0];
        attn_contiguous(&m.in[1], d7, l->dims, no - 1, -1); /* one root a row: no stride on the last axis */
        m.in[2] = l->in[2];
        m.n_steps = 2;
        m.steps[0].prim = PSK_DIV; m.steps[0].nargs = 2; m.steps[0].src[0] = 0; m.steps[0].src[1] = 1;
        m.steps[1].prim = PSK_MUL; m.steps[1].nargs = 2; m.steps[1].src[0] = -1; m.steps[1].src[1] = 2;
        void *t[4] = {table[0], rt, table[2], table[3]};
        rc = psk_oracle_run(&m, t, &o1); ovf |= o1;
    }
    free(x2); free(ms); free(rt);
    if (overflow) *overflow = ovf;
    return rc;
}

/* PSK_OP_ROPE: the two groups of three steps of `rope` (examples/coverage/llama.psk:69-70), each reading the two
 * halves of x through strides where the reference copies them out first, each writing its half of the result
 * where the reference concatenates afterwards. Copies do not change a value, so these are the reference's values. */
static int rope_unfused(const psk_launch *l, void *const *table, uint32_t *overflow)
{
    const int no = l->n_outer;
    if (no < 3 || l->n_inner != 0 || l->n_inputs != 3 || l->dims[no - 2] != 2) return PSK_E7001;
    uint32_t ovf = 0, o1 = 0;
    int rc = PSK_OK;
    for (int half = 0; half < 2 && rc == PSK_OK; ++half) {
        psk_launch m = *l;
        m.name = "rope: half"; m.op = PSK_OP_FUSED; m.n_inputs = 4;
        m.dims[no - 2] = 1;
        const int64_t xp = l->in[0].stride[no - 2];
        m.in[0] = l->in[0]; m.in[0].offset += half * xp;        /* this half */
        m.in[1] = l->in[1];
        m.in[2] = l->in[0]; m.in[2].offset += (1 - half) * xp;  /* the other */
        m.in[3] = l->in[2];
        m.out.offset += half * l->out.stride[no - 2];
        m.n_steps = 3;
        m.steps[0].prim = PSK_MUL; m.steps[0].nargs = 2; m.steps[0].src[0] = 0; m.steps[0].src[1] = 1;
        m.steps[1].prim = PSK_MUL; m.steps[1].nargs = 2; m.steps[1].src[0] = 2; m.steps[1].src[1] = 3;
        m.steps[2].prim = half ? PSK_ADD : PSK_SUB; m.steps[2].nargs = 2; m.steps[2].src[0] = -1; m.steps[2].src[1] = -2;
        void *t[5] = {table[0], table[1], table[0], table[2], table[3]};
        rc = psk_oracle_run(&m, t, &o1);
        ovf |= o1;
    }
    if (overflow) *overflow = ovf;
    return rc;
}

/* PSK_OP_CONTRACT_ADD: the contraction into a buffer of its own site's type, then the addition, two launches. */
static int contract_add_unfused(const psk_launch *l, void *const *table, uint32_t *overflow)
{
    if (l->n_inputs != 3) return PSK_E7001;
    const int no = l->n_outer, dc = (int)l->iparam[1];
    int64_t total = 1;
    for (int a = 0; a < no; ++a) total *= l->dims[a];
    void *tmp = malloc((size_t)(total ? total : 1) * elem_bytes(dc));
    uint32_t ovf = 0, o1 = 0;
    psk_launch m = *l;
    m.op = PSK_OP_CONTRACT; m.n_inputs = 2; m.dtype = dc;
    attn_contiguous(&m.out, dc, l->dims, no, -1);
    int scale_slot = 4;
    void *t1[5] = {table[0], table[1], tmp, NULL, NULL};
    int extra = 3;
    for (int i = 0; i < 2; ++i)
        if (l->in[i].dtype == PSK_I8 && !l->in[i].affine) t1[extra++] = table[scale_slot++];
    int rc = psk_oracle_run(&m, t1, &o1);
    ovf |= o1;
    if (rc == PSK_OK) {
        psk_launch a;
        memset(&a, 0, sizeof a);
        a.name = "contract_add: add"; a.op = PSK_OP_FUSED; a.dtype = l->dtype; a.order = l->order; a.guarded = l->guarded;
        a.n_inputs = 2; a.n_outer = no;
        memcpy(a.dims, l->dims, sizeof a.dims);
        a.in[0] = l->in[2];
        for (int k = no; k < PSK_MAX_AXES; ++k) a.in[0].stride[k] = 0;
        attn_contiguous(&a.in[1], dc, l->dims, no, -1);
        a.out = l->out;
        a.n_steps = 1;
        a.steps[0].prim = PSK_ADD; a.steps[0].nargs = 2; a.steps[0].src[0] = 0; a.steps[0].src[1] = 1;
        void *t2[3] = {table[2], tmp, table[3]};
        rc = psk_oracle_run(&a, t2, &o1);
        ovf |= o1;
    }
    free(tmp);
    if (overflow) *overflow = ovf;
    return rc;
}

int psk_oracle_run(const psk_launch *l, void *const *table, uint32_t *overflow)
{
    if (l->op == PSK_OP_CONTRACT_ADD) return contract_add_unfused(l, table, overflow);
    if (l->op == PSK_OP_ROPE) return rope_unfused(l, table, overflow);
    if (l->op == PSK_OP_ATTENTION) return attention_unfused(l, table, overflow);
    if (l->op == PSK_OP_RMSNORM) return rmsnorm_unfused(l, table, overflow);
    if (l->op == PSK_OP_CONTRACT && l->order == PSK_ORDER_CHUNKED && l->n_inner != 1) return PSK_E7005; /* lower.rs:429-431: a chunked order sums ONE summed axis */
    if (l->op == PSK_OP_CONTRACT && l->n_inner > 1) {
        psk_launch m = *l;
        int no = l->n_outer, w = 0;
        for (int c = 1; c < l->n_inner; ++c) {
            int a = no + w, b = no + c, ok = 1;
            for (int i = 0; i < l->n_inputs; ++i)
                ok = ok && m.in[i].stride[a] == l->in[i].stride[b] * l->dims[b] && m.in[i].scale_stride[a] == l->in[i].scale_stride[b] * l->dims[b];
            if (ok) {
                m.dims[a] *= l->dims[b];
                for (int i = 0; i < l->n_inputs; ++i) { m.in[i].stride[a] = l->in[i].stride[b]; m.in[i].scale_stride[a] = l->in[i].scale_stride[b]; }
            } else {
                ++w;
                m.dims[no + w] = l->dims[b];
                for (int i = 0; i < l->n_inputs; ++i) { m.in[i].stride[no + w] = l->in[i].stride[b]; m.in[i].scale_stride[no + w] = l->in[i].scale_stride[b]; }
            }
        }
        m.n_inner = w + 1;
        return psk_oracle_run_merged(&m, table, overflow);
    }
    return psk_oracle_run_merged(l, table, overflow);
}

/* A counted sum n in the unit `base` (exact: the product of two binary32 scales), stored: rounded once into the
 * output's float type, or into its affine format by the exact quotient (exec.rs:601-616). Returns the guard's test. */
static uint32_t store_count(const psk_launch *l, uint8_t *outp, int64_t ooff, int64_t n, double base)
{
    if (l->out.affine) {
        int64_t mb;
        int eb;
        take_apart(base, &mb, &eb);
        int64_t nq = quotient_round_exact(n < 0, (u128)(n < 0 ? -n : n) * (u128)mb, eb, l->out.affine_scale);
        int64_t q = nq + l->out.affine_zero;
        q = q < affine_min(l->out.affine) ? affine_min(l->out.affine) : (q > affine_max(l->out.affine) ? affine_max(l->out.affine) : q);
        if (l->out.affine == 2) ((uint8_t *)outp)[ooff] = (uint8_t)q;
        else ((int8_t *)outp)[ooff] = (int8_t)q;
        return 0;
    }
    switch (l->out.dtype) {
    case PSK_F32: ((uint32_t *)outp)[ooff] = round_count_to_float(n, base, 23, 8); return 0;
    case PSK_BF16: ((uint16_t *)outp)[ooff] = (uint16_t)round_count_to_float(n, base, 7, 8); return 0;
    case PSK_F16: {
        uint32_t c = round_count_to_float(n, base, 10, 5);
        ((uint16_t *)outp)[ooff] = (uint16_t)c;
        return (c & 0x7fffu) == 0x7c00u; /* a count is finite: an infinity here is an overflow */
    }
    default: { /* PSK_E8M15 */
        uint32_t c = round_count_to_float(n, base, 15, 8);
        uint8_t *q = outp + 3 * ooff;
        q[0] = (uint8_t)c; q[1] = (uint8_t)(c >> 8); q[2] = (uint8_t)(c >> 16);
        return (c & 0x7fffffu) == 0x7f8000u;
    }
    }
}

static int psk_oracle_run_merged(const psk_launch *l, void *const *table, uint32_t *overflow)
{
    const int no = l->n_outer, ni = l->n_inner, kd = l->dtype;
    operand in[PSK_MAX_INPUTS];
    int scale_slot = l->n_inputs + 1;
    for (int i = 0; i < l->n_inputs; ++i) {
        in[i].o = &l->in[i];
        in[i].p = (const uint8_t *)table[i] + l->in[i].offset * (int64_t)elem_bytes(l->in[i].dtype);
        in[i].scales = (l->in[i].dtype == PSK_I8 && !l->in[i].affine) ? (const float *)table[scale_slot++] : NULL;
    }
    uint8_t *outp = (uint8_t *)table[l->n_inputs] + l->out.offset * (int64_t)elem_bytes(l->out.dtype);
    int64_t total = 1, inner = 1;
    for (int a = 0; a < no; ++a) total *= l->dims[a];
    for (int c = 0; c < ni; ++c) inner *= l->dims[no + c];
    uint32_t ovf_all = 0;
    if (kd == PSK_F64 && l->op != PSK_OP_CONVERT) return PSK_E7005;

    switch (l->op) {
    case PSK_OP_FUSED: /* lower.rs:328-360 */
#pragma omp parallel for schedule(static) reduction(| : ovf_all)
        for (int64_t lin = 0; lin < total; ++lin) {
            uint32_t ovf = 0;
            float vals[PSK_MAX_STEPS];
            for (int s = 0; s < l->n_steps; ++s) {
                const psk_step *st = &l->steps[s];
                float a[2] = {0, 0};
                for (int j = 0; j < st->nargs; ++j) {
                    int src = st->src[j];
                    a[j] = src >= 0 ? load_operand(&in[src], offset_of(l->in[src].stride, l->dims, 0, no, lin), offset_of(l->in[src].scale_stride, l->dims, 0, no, lin), kd, &ovf) : vals[-1 - src];
                }
                vals[s] = st->nargs == 1 ? prim_unary(st->prim, a[0], st->imm) : prim_binary(st->prim, a[0], a[1]);
            }
            ovf |= store_out(l, outp, offset_of(l->out.stride, l->dims, 0, no, lin), vals[l->n_steps - 1]);
            ovf_all |= ovf;
        }
        break;
    case PSK_OP_CONTRACT:
        if (l->int_accum) { /* exec.rs:493-526: counts in the scales' unit, i32 that wraps; :601-616 the store */
            if (l->n_inputs != 2) return PSK_E7005;
            for (int i = 0; i < 2; ++i) if (!l->in[i].affine && l->in[i].dtype != PSK_I8) return PSK_E7005;
            if (!l->out.affine && l->out.dtype != PSK_F32 && l->out.dtype != PSK_BF16 && l->out.dtype != PSK_F16 && l->out.dtype != PSK_E8M15) return PSK_E7005;
            /* The same sums by blocks of JB neighbouring results of one row, when the last output axis is carried
             * by the integer weights alone, contiguously, with one scale a column (a projection's layout):
             * sums that wrap in 32 bits do not depend on the order, so this is the loop below, only faster (the
             * parity checks at a model's full width need it). */
            if (ni == 1 && no >= 1 && inner > 0 && l->in[0].affine && !l->in[1].affine && in[1].scales && l->in[0].stride[no - 1] == 0 && l->in[1].stride[no - 1] == 1
                && l->in[1].scale_stride[no] == 0) {
                enum { JB = 64 };
                const int64_t K = inner, N = l->dims[no - 1], rows = total / N;
                const int64_t s0 = l->in[0].stride[no], s1 = l->in[1].stride[no], sj = l->in[1].scale_stride[no - 1], os = l->out.stride[no - 1];
                const int zero0 = l->in[0].affine_zero, kind0 = l->in[0].affine;
                const double unit0 = (double)l->in[0].affine_scale;
#pragma omp parallel for schedule(dynamic, 1) reduction(| : ovf_all)
                for (int64_t row = 0; row < rows; ++row) {
                    const int64_t lin0 = row * N;
                    const int64_t b0 = offset_of(l->in[0].stride, l->dims, 0, no, lin0), b1 = offset_of(l->in[1].stride, l->dims, 0, no, lin0);
                    const int64_t q1 = offset_of(l->in[1].scale_stride, l->dims, 0, no, lin0), o0 = offset_of(l->out.stride, l->dims, 0, no, lin0);
                    for (int64_t j0 = 0; j0 < N; j0 += JB) {
                        const int nj = (int)(N - j0 < JB ? N - j0 : JB);
                        uint32_t acc[JB];
                        for (int j = 0; j < nj; ++j) acc[j] = 0;
                        for (int64_t c = 0; c < K; ++c) {
                            const int64_t off = b0 + c * s0;
                            const int32_t a = (kind0 == 2 ? (int)((const uint8_t *)in[0].p)[off] : (int)((const int8_t *)in[0].p)[off]) - zero0;
                            const int8_t *w = (const int8_t *)in[1].p + b1 + c * s1 + j0;
                            for (int j = 0; j < nj; ++j) acc[j] += (uint32_t)(a * (int32_t)w[j]); /* the product fits; the sum wraps */
                        }
                        for (int j = 0; j < nj; ++j)
                            ovf_all |= store_count(l, outp, o0 + (j0 + j) * os, (int64_t)(int32_t)acc[j], unit0 * (double)in[1].scales[q1 + (j0 + j) * sj]);
                    }
                }
                break;
            }
#pragma omp parallel for schedule(static) reduction(| : ovf_all)
            for (int64_t lin = 0; lin < total; ++lin) {
                int64_t b0 = offset_of(l->in[0].stride, l->dims, 0, no, lin), b1 = offset_of(l->in[1].stride, l->dims, 0, no, lin);
                int64_t q0 = offset_of(l->in[0].scale_stride, l->dims, 0, no, lin), q1 = offset_of(l->in[1].scale_stride, l->dims, 0, no, lin);
                uint32_t acc = 0;
                double u0 = 1.0, u1 = 1.0;
                for (int64_t c = 0; c < inner; ++c) {
                    int64_t o0 = offset_of(l->in[0].stride, l->dims, no, ni, c), o1 = offset_of(l->in[1].stride, l->dims, no, ni, c);
                    int64_t s0 = offset_of(l->in[0].scale_stride, l->dims, no, ni, c), s1 = offset_of(l->in[1].scale_stride, l->dims, no, ni, c);
                    int32_t a = load_count(&in[0], b0 + o0, q0 + s0, &u0), b = load_count(&in[1], b1 + o1, q1 + s1, &u1);
                    acc += (uint32_t)(a * b); /* the product fits; the sum wraps */
                }
                if (inner == 0) { load_count(&in[0], b0, q0, &u0); load_count(&in[1], b1, q1, &u1); }
                /* the base is exact: two 24-bit significands */
                ovf_all |= store_count(l, outp, offset_of(l->out.stride, l->dims, 0, no, lin), (int64_t)(int32_t)acc, u0 * u1);
            }
            break;
        } /* lower.rs:465-474, 586-636: acc = acc + (x·w), the terms in lexicographic order */
        /* The tiled form of a contraction nest (lower.rs:906-1139, tile (1, JB)): when the last output axis
         * is carried by operand 1 alone, contiguously, a block of JB results is summed at once, each still
         * adding its own terms in increasing k, so the bits are those of the loop below. It is the form the
         * reference's executors run, and what makes this restatement a fair CPU baseline. */
        if (l->order == PSK_ORDER_CHUNKED && (ni != 1 || l->n_inputs != 2 || l->order_size < 1)) return PSK_E7005; /* lower.rs:429-431: one summed axis, two operands */
        if (l->order != PSK_ORDER_CHUNKED && ni == 1 && l->n_inputs == 2 && no >= 1 && l->in[0].stride[no - 1] == 0 && l->in[1].stride[no - 1] == 1 && l->out.stride[no - 1] == 1
            && l->in[0].dtype != PSK_I8 && (l->in[1].dtype == PSK_BF16 || l->in[1].dtype == PSK_F32 || l->in[1].dtype == PSK_I8)
            && edge_is_identity(kd, l->in[1].dtype) && inner > 0) {
            enum { JB = 64, RB = 8 };
            const int64_t K = inner, N = l->dims[no - 1], rows = total / N;
            const int64_t s0 = l->in[0].stride[no], s1 = l->in[1].stride[no], q1 = l->in[1].scale_stride[no];
            const int64_t sj = l->in[1].scale_stride[no - 1];
            const int64_t row_blocks = (rows + RB - 1) / RB, col_blocks = (N + JB - 1) / JB;
            /* rows that share operand 1 (the same offsets into it) can share a pass over it */
#pragma omp parallel reduction(| : ovf_all)
            {
                float *arow = (float *)malloc((size_t)K * RB * sizeof(float));
                uint32_t ovf = 0;
#pragma omp for schedule(dynamic, 1)
                for (int64_t rb = 0; rb < row_blocks; ++rb) {
                    int nr = (int)(rows - rb * RB < RB ? rows - rb * RB : RB);
                    int64_t b1[RB], sb1[RB], ob[RB];
                    for (int r = 0; r < nr; ++r) {
                        const int64_t row = rb * RB + r;
                        const int64_t b0 = offset_of(l->in[0].stride, l->dims, 0, no - 1, row);
                        b1[r] = offset_of(l->in[1].stride, l->dims, 0, no - 1, row);
                        sb1[r] = offset_of(l->in[1].scale_stride, l->dims, 0, no - 1, row);
                        ob[r] = offset_of(l->out.stride, l->dims, 0, no - 1, row);
                        for (int64_t k = 0; k < K; ++k) arow[r * K + k] = load_operand(&in[0], b0 + k * s0, 0, kd, &ovf);
                    }
                    /* a block shares the pass only while its rows read the same part of operand 1 */
                    int shared = 1;
                    for (int r = 1; r < nr; ++r) shared = shared && b1[r] == b1[0] && sb1[r] == sb1[0];
                    for (int r0 = 0; r0 < nr; r0 += shared ? nr : 1) {
                        const int rn = shared ? nr : 1;
                        for (int64_t cb = 0; cb < col_blocks; ++cb) {
                            const int64_t j0 = cb * JB;
                            const int jb = (int)(N - j0 < JB ? N - j0 : JB);
                            float acc[RB][JB];
                            for (int r = 0; r < rn; ++r)
                                for (int jj = 0; jj < JB; ++jj) acc[r][jj] = 0.0f;
                            for (int64_t k = 0; k < K; ++k) {
                                float wv[JB];
                                if (l->in[1].dtype == PSK_BF16) {
                                    const uint16_t *wr = (const uint16_t *)in[1].p + b1[r0] + j0 + k * s1;
                                    for (int jj = 0; jj < jb; ++jj) wv[jj] = u2f((uint32_t)wr[jj] << 16);
                                } else if (l->in[1].dtype == PSK_F32) {
                                    const float *wr = (const float *)in[1].p + b1[r0] + j0 + k * s1;
                                    for (int jj = 0; jj < jb; ++jj) wv[jj] = wr[jj];
                                } else { /* integer weights: f32(q)·s, one multiplication, as the value is loaded */
                                    const int8_t *wr = (const int8_t *)in[1].p + b1[r0] + j0 + k * s1;
                                    const float *sk = in[1].scales + sb1[r0] + j0 * sj + k * q1;
                                    for (int jj = 0; jj < jb; ++jj) wv[jj] = (float)wr[jj] * sk[jj * sj];
                                }
                                for (int r = 0; r < rn; ++r) {
                                    const float a = arow[(r0 + r) * K + k];
                                    for (int jj = 0; jj < jb; ++jj) {
                                        const float prod = a * wv[jj];
                                        acc[r][jj] = acc[r][jj] + prod;
                                    }
                                }
                            }
                            for (int r = 0; r < rn; ++r)
                                for (int jj = 0; jj < jb; ++jj) ovf |= store_out(l, outp, ob[r0 + r] + j0 + jj, acc[r][jj]);
                        }
                    }
                }
                ovf_all |= ovf;
                free(arow);
            }
            break;
        }
#pragma omp parallel for schedule(static) reduction(| : ovf_all)
        for (int64_t lin = 0; lin < total; ++lin) {
            uint32_t ovf = 0;
            int64_t base[PSK_MAX_INPUTS], sbase[PSK_MAX_INPUTS];
            for (int i = 0; i < l->n_inputs; ++i) {
                base[i] = offset_of(l->in[i].stride, l->dims, 0, no, lin);
                sbase[i] = offset_of(l->in[i].scale_stride, l->dims, 0, no, lin);
            }
            float acc = 0.0f;
            if (ni == 1 && l->n_inputs == 2 && l->order == PSK_ORDER_CHUNKED) {
                /* lower.rs:424-457: part = 0; the chunk's terms in order; acc = acc + part; the last chunk shorter */
                const int64_t s0 = l->in[0].stride[no], s1 = l->in[1].stride[no], q0 = l->in[0].scale_stride[no], q1 = l->in[1].scale_stride[no];
                const int64_t size = l->order_size;
                for (int64_t c0 = 0; c0 < inner; c0 += size) {
                    float part = 0.0f;
                    for (int64_t c = c0; c < inner && c < c0 + size; ++c) {
                        float x = load_operand(&in[0], base[0] + c * s0, sbase[0] + c * q0, kd, &ovf);
                        float w = load_operand(&in[1], base[1] + c * s1, sbase[1] + c * q1, kd, &ovf);
                        float prod = x * w;
                        part = part + prod;
                    }
                    acc = acc + part;
                }
            } else if (ni == 1 && l->n_inputs == 2) {
                const int64_t s0 = l->in[0].stride[no], s1 = l->in[1].stride[no], q0 = l->in[0].scale_stride[no], q1 = l->in[1].scale_stride[no];
                for (int64_t c = 0; c < inner; ++c) {
                    float x = load_operand(&in[0], base[0] + c * s0, sbase[0] + c * q0, kd, &ovf);
                    float w = load_operand(&in[1], base[1] + c * s1, sbase[1] + c * q1, kd, &ovf);
                    float prod = x * w;
                    acc = acc + prod;
                }
            } else {
                for (int64_t c = 0; c < inner; ++c) {
                    float prod = 1.0f;
                    for (int i = 0; i < l->n_inputs; ++i)
                        prod = prod * load_operand(&in[i], base[i] + offset_of(l->in[i].stride, l->dims, no, ni, c), sbase[i] + offset_of(l->in[i].scale_stride, l->dims, no, ni, c), kd, &ovf);
                    acc = acc + prod;
                }
            }
            ovf |= store_out(l, outp, offset_of(l->out.stride, l->dims, 0, no, lin), acc);
            ovf_all |= ovf;
        }
        break;
    case PSK_OP_REDUCE: /* lower.rs:1221-1255, 1693 */
#pragma omp parallel for schedule(static) reduction(| : ovf_all)
        for (int64_t lin = 0; lin < total; ++lin) {
            uint32_t ovf = 0;
            int64_t base = offset_of(l->in[0].stride, l->dims, 0, no, lin);
            float acc = 0.0f;
            for (int64_t c = 0; c < inner; ++c) {
                float x = load_operand(&in[0], base + offset_of(l->in[0].stride, l->dims, no, ni, c), 0, kd, &ovf);
                acc = acc + (l->kind == PSK_REDUCE_SUMSQ ? x * x : x);
                if (l->kind == PSK_REDUCE_SUM_STORED) { /* lower.rs:1677 `sum_to`: the sum lives in the output buffer */
                    ovf |= psk_o_overflows(l->out.dtype, acc);
                    acc = prim_unary(PSK_ROUND, acc, l->out.dtype);
                }
            }
            if (l->kind == PSK_REDUCE_MEAN) acc = acc / (float)(double)l->iparam[0];
            ovf |= store_out(l, outp, offset_of(l->out.stride, l->dims, 0, no, lin), acc);
            ovf_all |= ovf;
        }
        break;
    case PSK_OP_SOFTMAX: { /* lower.rs:1274-1311 and 1368-1419 (three passes) */
        const int64_t n = inner, s = l->in[0].stride[no], os = l->out.stride[no];
        if (n == 0) break;
#pragma omp parallel for schedule(static) reduction(| : ovf_all)
        for (int64_t row = 0; row < total; ++row) {
            uint32_t ovf = 0;
            int64_t base = offset_of(l->in[0].stride, l->dims, 0, no, row), obase = offset_of(l->out.stride, l->dims, 0, no, row);
#define X(k) load_operand(&in[0], base + (k) * s, 0, kd, &ovf)
            if (!l->masked) {
                float m = X(0);
                for (int64_t k = 0; k < n; ++k) if (X(k) > m) m = X(k);
                float z = 0.0f;
                for (int64_t k = 0; k < n; ++k) z = z + presk_expf(X(k) - m);
                for (int64_t k = 0; k < n; ++k) ovf |= store_out(l, outp, obase + k * os, presk_expf(X(k) - m) / z);
            } else {
                int64_t mbase = offset_of(l->in[1].stride, l->dims, 0, no, row), ms = l->in[1].stride[no];
                const int64_t *mk = (const int64_t *)in[1].p;
#define ALLOWED(k) ((float)(double)mk[mbase + (k) * ms] > 0.5f)
                float mx = 0.0f, first = 1.0f;
                for (int64_t k = 0; k < n; ++k) {
                    mx = ALLOWED(k) ? (first > 0.5f ? X(k) : (X(k) > mx ? X(k) : mx)) : mx;
                    first = ALLOWED(k) ? 0.0f : first;
                }
                float z = 0.0f;
                for (int64_t k = 0; k < n; ++k) z = z + (ALLOWED(k) ? presk_expf(X(k) - mx) : 0.0f);
                for (int64_t k = 0; k < n; ++k) ovf |= store_out(l, outp, obase + k * os, ALLOWED(k) ? presk_expf(X(k) - mx) / z : 0.0f);
#undef ALLOWED
            }
#undef X
            ovf_all |= ovf;
        }
        break;
    }
    case PSK_OP_XENT: { /* lower.rs:1459-1470: ln z + m - x[y] */
        const int64_t n = inner, s = l->in[0].stride[no];
        int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : ovf_all, bad)
        for (int64_t row = 0; row < total; ++row) {
            uint32_t ovf = 0;
            int64_t base = offset_of(l->in[0].stride, l->dims, 0, no, row);
            float m = load_operand(&in[0], base, 0, kd, &ovf);
            for (int64_t k = 0; k < n; ++k) {
                float x = load_operand(&in[0], base + k * s, 0, kd, &ovf);
                if (x > m) m = x;
            }
            float z = 0.0f;
            for (int64_t k = 0; k < n; ++k) z = z + presk_expf(load_operand(&in[0], base + k * s, 0, kd, &ovf) - m);
            int64_t y = ((const int64_t *)in[1].p)[offset_of(l->in[1].stride, l->dims, 0, no, row)];
            float xy = 0.0f;
            if (y >= 0 && y < n) xy = load_operand(&in[0], base + y * s, 0, kd, &ovf);
            else bad |= 1;
            ovf |= store_out(l, outp, offset_of(l->out.stride, l->dims, 0, no, row), (presk_logf(z) + m) - xy);
            ovf_all |= ovf;
        }
        if (bad) return PSK_E7001;
        break;
    }
    case PSK_OP_XENT_VJP: { /* lower.rs:1472-1488: (softmax(x) - onehot(y)) * ct, row by row */
        const int64_t n = inner, s = l->in[0].stride[no], os = l->out.stride[no];
#pragma omp parallel for schedule(static) reduction(| : ovf_all)
        for (int64_t row = 0; row < total; ++row) {
            uint32_t ovf = 0;
            int64_t base = offset_of(l->in[0].stride, l->dims, 0, no, row);
            float m = load_operand(&in[0], base, 0, kd, &ovf);
            for (int64_t k = 0; k < n; ++k) {
                float x = load_operand(&in[0], base + k * s, 0, kd, &ovf);
                if (x > m) m = x;
            }
            float z = 0.0f;
            for (int64_t k = 0; k < n; ++k) z = z + presk_expf(load_operand(&in[0], base + k * s, 0, kd, &ovf) - m);
            int64_t y = ((const int64_t *)in[1].p)[offset_of(l->in[1].stride, l->dims, 0, no, row)];
            float ct = load_operand(&in[2], offset_of(l->in[2].stride, l->dims, 0, no, row), 0, kd, &ovf);
            int64_t obase = offset_of(l->out.stride, l->dims, 0, no, row);
            for (int64_t k = 0; k < n; ++k) {
                /* the reference compares the two integers as reals of the kernel's type */
                float hot = (float)k == (float)y ? 1.0f : 0.0f;
                float sm = presk_expf(load_operand(&in[0], base + k * s, 0, kd, &ovf) - m) / z;
                ovf |= store_out(l, outp, obase + k * os, (sm - hot) * ct);
            }
            ovf_all |= ovf;
        }
        break;
    }
    case PSK_OP_EMBED_VJP: { /* lower.rs:1444-1457: zero fill, then one row added per index, in index order */
        const int last = no - 1;
        const int64_t d = l->dims[last], rows = total / (d ? d : 1), vocab = l->iparam[0];
        uint32_t ovf = 0;
        int bad = 0;
        for (int64_t v = 0; v < vocab; ++v)
            for (int64_t j = 0; j < d; ++j) store_out(l, outp, v * l->out.stride[0] + j * l->out.stride[1], 0.0f);
        for (int64_t row = 0; row < rows; ++row) {
            int64_t id = ((const int64_t *)in[1].p)[offset_of(l->in[1].stride, l->dims, 0, last, row)];
            if (id < 0 || id >= vocab) { bad = 1; continue; }
            int64_t cbase = offset_of(l->in[2].stride, l->dims, 0, last, row);
            for (int64_t j = 0; j < d; ++j) {
                int64_t o = id * l->out.stride[0] + j * l->out.stride[1];
                float acc = load_real(outp, l->out.dtype, o) + load_operand(&in[2], cbase + j * l->in[2].stride[last], 0, kd, &ovf);
                ovf |= store_out(l, outp, o, acc);
            }
        }
        ovf_all |= ovf;
        if (bad) return PSK_E7001;
        break;
    }
    case PSK_OP_ARGMAX: { /* lower.rs:1490: the last of equal maxima */
        const int64_t n = inner, s = l->in[0].stride[no];
        for (int64_t row = 0; row < total; ++row) {
            uint32_t ovf = 0;
            int64_t base = offset_of(l->in[0].stride, l->dims, 0, no, row);
            float m = load_operand(&in[0], base, 0, kd, &ovf);
            int64_t best = 0;
            for (int64_t k = 0; k < n; ++k) {
                float x = load_operand(&in[0], base + k * s, 0, kd, &ovf);
                if (x >= m) { m = x; best = k; }
            }
            ((int64_t *)outp)[offset_of(l->out.stride, l->dims, 0, no, row)] = best;
        }
        break;
    }
    case PSK_OP_EMBED: { /* lower.rs:1421-1437 */
        const int last = no - 1;
        const int64_t d = l->dims[last], rows = total / (d ? d : 1);
        int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : ovf_all, bad)
        for (int64_t row = 0; row < rows; ++row) {
            uint32_t ovf = 0;
            int64_t id = ((const int64_t *)in[1].p)[offset_of(l->in[1].stride, l->dims, 0, last, row)];
            int64_t obase = offset_of(l->out.stride, l->dims, 0, last, row);
            if (id < 0 || id >= l->iparam[0]) { bad |= 1; id = 0; }
            for (int64_t j = 0; j < d; ++j)
                ovf |= store_out(l, outp, obase + j * l->out.stride[last], load_operand(&in[0], id * l->in[0].stride[0] + j * l->in[0].stride[1], 0, kd, &ovf));
            ovf_all |= ovf;
        }
        if (bad) return PSK_E7001;
        break;
    }
    case PSK_OP_COPY: /* lower.rs:1554-1667: Store(Load) through the index maps */
#pragma omp parallel for schedule(static) reduction(| : ovf_all)
        for (int64_t lin = 0; lin < total; ++lin) {
            uint32_t ovf = 0;
            int64_t off = offset_of(l->in[0].stride, l->dims, 0, no, lin), ooff = offset_of(l->out.stride, l->dims, 0, no, lin);
            if (l->in[0].is_index) ((int64_t *)outp)[ooff] = ((const int64_t *)in[0].p)[off];
            else ovf |= store_out(l, outp, ooff, load_operand(&in[0], off, 0, kd, &ovf));
            ovf_all |= ovf;
        }
        break;
    case PSK_OP_IOTA: /* lower.rs:1706-1750 */
        for (int64_t lin = 0; lin < total; ++lin) {
            switch (l->kind) {
            case PSK_IOTA_POSITIONS: ((int64_t *)outp)[lin] = lin; break;
            case PSK_IOTA_CAUSAL: {
                int64_t n = l->dims[1], i = lin / n, j = lin % n;
                ((int64_t *)outp)[lin] = (float)(double)j <= (float)(double)i ? 1 : 0;
                break;
            }
            case PSK_IOTA_ONE_HOT: {
                int64_t v = l->dims[no - 1], row = lin / v, j = lin % v;
                int64_t id = ((const int64_t *)in[0].p)[offset_of(l->in[0].stride, l->dims, 0, no - 1, row)];
                ovf_all |= store_out(l, outp, lin, (float)(double)id == (float)(double)j ? 1.0f : 0.0f);
                break;
            }
            default: ovf_all |= store_out(l, outp, lin, (float)l->fparam[0]); break;
            }
        }
        break;
    case PSK_OP_CONVERT: /* presk-rt/src/lib.rs:868-876, presk_rt.c `presk_convert` */
        for (int64_t i = 0; i < total; ++i) {
            if (l->in[0].affine) {
                int q = l->in[0].affine == 2 ? (int)((const uint8_t *)in[0].p)[i] : (int)((const int8_t *)in[0].p)[i];
                double x = (double)(q - l->in[0].affine_zero) * (double)l->in[0].affine_scale;
                if (l->out.dtype == PSK_F64) ((double *)outp)[i] = x;
                else ovf_all |= store_out(l, outp, i, (float)x);
            } else if (l->in[0].dtype == PSK_F64) {
                double x = ((const double *)in[0].p)[i];
                switch (l->out.dtype) {
                case PSK_F64: ((double *)outp)[i] = x; break;
                case PSK_F16: ((uint16_t *)outp)[i] = psk_o_f64_to_f16(x); ovf_all |= (fabs(x) >= 65520.0 && fabs(x) < INFINITY); break;
                case PSK_E8M15: {
                    uint32_t c = psk_o_f64_to_e8m15(x);
                    uint8_t *q = outp + 3 * i;
                    q[0] = (uint8_t)c; q[1] = (uint8_t)(c >> 8); q[2] = (uint8_t)(c >> 16);
                    ovf_all |= (fabs(x) >= 0x1.ffffp127 && fabs(x) < INFINITY);
                    break;
                }
                default: ovf_all |= store_out(l, outp, i, (float)x); break; /* to bf16 by way of f32 */
                }
            } else {
                ovf_all |= store_out(l, outp, i, load_real(in[0].p, l->in[0].dtype, i));
            }
        }
        break;
    case PSK_OP_MAGNITUDE: { /* presk-precision/src/envelope.rs: max |x|, least non-zero |x|, least and greatest x */
        uint32_t *o = (uint32_t *)outp;
        for (int64_t i = 0; i < l->in[0].numel; ++i) {
            float x = load_real(in[0].p, l->in[0].dtype, i);
            if (x != x) continue;
            uint32_t b = f2u(x), a = b & 0x7fffffffu, ord = b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
            if (a > o[0]) o[0] = a;
            if (a != 0 && a < o[1]) o[1] = a;
            if (ord < o[2]) o[2] = ord;
            if (ord > o[3]) o[3] = ord;
        }
        break;
    }
    default:
        return PSK_E7001;
    }
    int guarded = l->guarded && (l->out.dtype == PSK_F16 || l->out.dtype == PSK_E8M15 || kd == PSK_F16 || kd == PSK_E8M15);
    if (overflow) *overflow = guarded ? ovf_all : 0;
    return PSK_OK;
}

/* presk-rt/src/quant.rs:128-167 (absmax): per channel m = max|w| over k, s =
 * f32(m / qmax), q = clamp(rne(w / s), +-qmax), 0 when s is 0 or w / s a NaN. */
void psk_oracle_quantize(const void *w, int from, int8_t *q, float *s, int64_t outer, int64_t k, int64_t inner)
{
#define W(e) (from == PSK_F64 ? ((const double *)w)[e] : (double)((const float *)w)[e])
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t in = 0; in < inner; ++in) {
            double m = 0.0;
            for (int64_t kk = 0; kk < k; ++kk) {
                double a = fabs(W((o * k + kk) * inner + in));
                if (a > m) m = a;
            }
            float sc = (float)(m / 127.0);
            s[o * inner + in] = sc;
            for (int64_t kk = 0; kk < k; ++kk) {
                int64_t e = (o * k + kk) * inner + in;
                double r = W(e) / (double)sc;
                int v = 0;
                if (sc != 0.0f && r == r) {
                    double t = nearbyint(r);
                    t = t > 127.0 ? 127.0 : (t < -127.0 ? -127.0 : t);
                    v = (int)t;
                }
                q[e] = (int8_t)v;
            }
        }
#undef W
}

/* ---- the oracle as an executor, so that the host program can run over it -------- */
typedef struct {
    char error[256];
    int64_t launches;
    int64_t first_overflow; /* 1 + the launch */
} oracle_exec;

static const char *o_name(void *s) { (void)s; return "oracle"; }
static void *o_alloc(void *s, size_t b) { (void)s; return malloc(b ? b : 1); }
static void o_free(void *s, void *p) { (void)s; free(p); }
static int o_upload(void *s, void *d, const void *h, size_t b) { (void)s; memcpy(d, h, b); return PSK_OK; }
static int o_download(void *s, void *h, const void *d, size_t b) { (void)s; memcpy(h, d, b); return PSK_OK; }
static int o_run(void *s, const psk_launch *l, void *const *t)
{
    oracle_exec *e = (oracle_exec *)s;
    uint32_t ovf = 0;
    struct timespec t0, t1;
    const int trace = getenv("PSK_ORACLE_TRACE") != NULL;
    if (trace) clock_gettime(CLOCK_MONOTONIC, &t0);
    int rc = psk_oracle_run(l, t, &ovf);
    if (trace) {
        clock_gettime(CLOCK_MONOTONIC, &t1);
        fprintf(stderr, "oracle\t%s\t%.3f ms\n", l->name ? l->name : "?", (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6);
    }
    if (rc != PSK_OK) snprintf(e->error, sizeof e->error, "%s: the oracle does not run this launch (%d)", l->name ? l->name : "?", rc);
    if (ovf && !e->first_overflow) e->first_overflow = e->launches + 1;
    e->launches += 1;
    return rc;
}
static int64_t o_overflow(void *s)
{
    oracle_exec *e = (oracle_exec *)s;
    int64_t r = e->first_overflow;
    e->first_overflow = 0;
    return r;
}
static int o_sync(void *s)
{
    oracle_exec *e = (oracle_exec *)s;
    int64_t o = o_overflow(s);
    if (o) {
        snprintf(e->error, sizeof e->error, "launch %lld: a store rounded a finite value to an infinity", (long long)(o - 1));
        return PSK_E7007;
    }
    return PSK_OK;
}
static const char *o_error(void *s) { return ((oracle_exec *)s)->error; }
static int o_quantize(void *s, const void *w, int32_t from, int8_t *q, float *sc, int64_t outer, int64_t k, int64_t inner)
{
    (void)s;
    psk_oracle_quantize(w, from, q, sc, outer, k, inner);
    return PSK_OK;
}

void psk_oracle_vtable(psk_exec_vtable *out)
{
    oracle_exec *e = (oracle_exec *)calloc(1, sizeof *e);
    out->self = e;
    out->name = o_name;
    out->alloc = o_alloc;
    out->free = o_free;
    out->upload = o_upload;
    out->download = o_download;
    out->run = o_run;
    out->sync = o_sync;
    out->overflow = o_overflow;
    out->last_error = o_error;
    out->quantize = o_quantize;
    out->init_normal = NULL;
}
