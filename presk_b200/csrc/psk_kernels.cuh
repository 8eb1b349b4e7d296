// The generic kernels: one family per psk_op, every one a restatement for the
// GPU of a lowering of presk-kernel/src/lower.rs under the arithmetic of
// presk-kernel/src/exec.rs (`impl Elem for f32`): each operation rounded once
// in f32, products rounded before they are added, loads widened exactly,
// stores rounded once. Under PSK_ORDER_SEQUENTIAL every sum adds its terms in
// index order from +0 and the results are the kernel interpreter's bits.
// Under PSK_ORDER_DEVICE row sums are shuffle trees (a declared
// reassociation); everything that is not a sum keeps its bits.
#pragma once
#include "psk_dev.cuh"

namespace psk {

// ---------------------------------------------------------------------------
// elementary operations (lower.rs:184-226)
// ---------------------------------------------------------------------------
PSK_DEV float prim_unary(int prim, float x, int imm, uint32_t *status)
{
    switch (prim) {
    case PSK_NEG: return -x;
    case PSK_EXP: return lm_expf(x);
    case PSK_LOG: return lm_logf(x);
    case PSK_TANH: return lm_tanhf(x);
    case PSK_SQRT: return __fsqrt_rn(x);
    case PSK_SIN: { int b = 0; float r = lm_sinf(x, &b); if (b) atomicOr(status, 1u); return r; }
    case PSK_COS: { int b = 0; float r = lm_cosf(x, &b); if (b) atomicOr(status, 1u); return r; }
    case PSK_ABS: return fabsf(x);
    case PSK_GELU: {
        float phi = __fdiv_rn(__fadd_rn(1.0f, lm_erff(__fdiv_rn(x, 1.41421354f))), 2.0f);
        return __fmul_rn(x, phi);
    }
    case PSK_GELU_DERIV: {
        float phi = __fdiv_rn(__fadd_rn(1.0f, lm_erff(__fdiv_rn(x, 1.41421354f))), 2.0f);
        float dens = __fdiv_rn(lm_expf(__fdiv_rn(-__fmul_rn(x, x), 2.0f)), 2.50662827f);
        return __fadd_rn(phi, __fmul_rn(x, dens));
    }
    case PSK_RELU: return x < 0.0f ? 0.0f : x;
    case PSK_HEAVISIDE: return x > 0.0f ? 1.0f : 0.0f;
    case PSK_SIGN: return x < 0.0f ? -1.0f : (x > 0.0f ? 1.0f : 0.0f);
    case PSK_SIGMOID: return __frcp_rn(__fadd_rn(1.0f, lm_expf(-x)));
    case PSK_POW: {
        if (imm == 0) return 1.0f;
        float e = x;
        for (int i = 1; i < imm; ++i) e = __fmul_rn(e, x);
        return e;
    }
    case PSK_DIV_N: return __fdiv_rn(x, (float)(double)imm);
    case PSK_ROUND: return imm == PSK_BF16 ? bf16_to_f32(f32_to_bf16(x)) : imm == PSK_F16 ? f16_to_f32(f32_to_f16(x)) : imm == PSK_E8M15 ? e8m15_to_f32(f32_to_e8m15(x)) : x;
    default: return x; // PSK_REAL
    }
}

PSK_DEV float prim_binary(int prim, float x, float y)
{
    switch (prim) {
    case PSK_ADD: return __fadd_rn(x, y);
    case PSK_SUB: return __fsub_rn(x, y);
    case PSK_MUL: return __fmul_rn(x, y);
    case PSK_DIV: return __fdiv_rn(x, y);
    case PSK_MAX: return x > y ? x : y; // the second operand at a tie
    default: return x < y ? x : y;      // PSK_MIN
    }
}

// ---------------------------------------------------------------------------
// Exact integer sums over scaled values and affine stores
// (presk-kernel/src/exec.rs:493-526, 601-616; presk-format/src/lib.rs:865-954,
// 1148-1193). A value stored in an affine format is a code q denoting
// (q - z)·s. Under `product: i32, accum: i32` a contraction reads both operands
// as integers in their scales' unit, sums the exact products in 32 bits that
// wrap, and rounds the exact value sum·s0·s1 once into the output's format:
// a float's, or another affine format's by the exact quotient. 128-bit
// integers carry the exact values.
// ---------------------------------------------------------------------------
typedef unsigned __int128 u128_t;

PSK_DEV void take_apart(double x, int64_t &m, int &e)
{
    const uint64_t b = (uint64_t)__double_as_longlong(x);
    const int field = (int)((b >> 52) & 0x7ff);
    const uint64_t frac = b & ((1ull << 52) - 1);
    const int64_t mag = field ? (int64_t)(frac | (1ull << 52)) : (int64_t)frac;
    e = (field ? field : 1) - 1075;
    m = (b >> 63) ? -mag : mag;
}

PSK_DEV int bit_length(u128_t v)
{
    const uint64_t hi = (uint64_t)(v >> 64), lo = (uint64_t)v;
    return hi ? 128 - __clzll((long long)hi) : (lo ? 64 - __clzll((long long)lo) : 0);
}

// The integer nearest (mag·2^e) / s with the sign given, ties to even, saturated at +-2^62.
PSK_DEV int64_t quotient_round_exact(bool neg, u128_t mag, int e, float s)
{
    if (mag == 0) return 0;
    int64_t ms64;
    int es;
    take_apart((double)s, ms64, es);
    const int tz = __ffsll(ms64) - 1;
    ms64 >>= tz;
    es += tz;
    const u128_t ms = (u128_t)ms64;
    const int bits = bit_length(mag), k = e - es;
    u128_t num = mag, den = ms;
    if (k >= 0) {
        if (bits + k > 120) return neg ? -(1ll << 62) : (1ll << 62);
        num = mag << k;
    } else {
        if (-k > bits + 2) return 0;
        den = ms << -k;
    }
    u128_t q = num / den;
    const u128_t r = num % den, twice = r << 1;
    if (twice > den || (twice == den && (q & 1))) q += 1;
    if (q > ((u128_t)1 << 62)) q = (u128_t)1 << 62;
    return neg ? -(int64_t)q : (int64_t)q;
}

PSK_DEV int64_t affine_clamp(int64_t q, int kind)
{
    const int64_t lo = kind == 2 ? 0 : -128, hi = kind == 2 ? 255 : 127;
    return q < lo ? lo : (q > hi ? hi : q);
}

// A real stored in an affine format: clamp(rne(x / s) + z), the quotient exact; a NaN is the zero point.
PSK_DEV int64_t affine_code_of(double x, int kind, float scale, int zero)
{
    if (x != x) return zero;
    if (isinf(x)) return x > 0 ? (kind == 2 ? 255 : 127) : (kind == 2 ? 0 : -128);
    int64_t m;
    int e;
    take_apart(x, m, e);
    const int64_t n = quotient_round_exact(m < 0, (u128_t)(m < 0 ? -m : m), e, scale);
    return affine_clamp(n + zero, kind);
}

// The same for a binary32 value in the kernels that store whole rows of codes, the quick way. With r = RN(1/s),
// v = RN(x·r) is within 2^-23 of the quotient x/s relatively. Codes saturate, so v is first clamped to ±vmax, two
// past the furthest code from the zero point (a quotient beyond it saturates whatever its fraction); then
// v + 1.5·2^23 rounds v to the nearest integer, ties to even, and holds that integer in its low bits. Unless v lies
// within vmax·2^-22 of a tie, that is the quotient's own nearest integer; the few that do, and NaNs (whose code is
// the zero point), go the exact way, kept out of line.
static __device__ __noinline__ int affine_code_exact(float x, int kind, float scale, int zero)
{
    return (int)affine_code_of((double)x, kind, scale, zero);
}

struct AffineQuick {
    float scale, rscale, vmax, tol;
    int kind, zero, bias, lo, hi;
};

PSK_DEV AffineQuick affine_quick_of(float scale, int kind, int zero)
{
    AffineQuick q;
    q.scale = scale; q.rscale = __frcp_rn(scale); q.kind = kind; q.zero = zero;
    q.lo = kind == 2 ? 0 : -128; q.hi = kind == 2 ? 255 : 127;
    const int far = (q.hi - zero) > (zero - q.lo) ? (q.hi - zero) : (zero - q.lo);
    q.vmax = (float)(far + 2);
    q.tol = q.vmax * 2.384185791015625e-07f; // 2^-22
    q.bias = zero - 0x4B400000;
    return q;
}

// The quick code and whether it is certain, without a branch: a caller takes several elements this way, so that
// their chains overlap, and then sends the uncertain ones (rare) through affine_code_exact.
PSK_DEV int affine_code_try(float x, const AffineQuick &q, bool &unsure)
{
    const float v = __fmul_rn(x, q.rscale);
    const float vc = fminf(fmaxf(v, -q.vmax), q.vmax);
    const float t = __fadd_rn(vc, 12582912.0f);
    const float d = __fsub_rn(vc, __fsub_rn(t, 12582912.0f)); // exact
    unsure = x != x || fabsf(fabsf(d) - 0.5f) <= q.tol;
    const int n = __float_as_int(t) + q.bias;
    return n < q.lo ? q.lo : (n > q.hi ? q.hi : n);
}

PSK_DEV int affine_code_quick(float x, const AffineQuick &q)
{
    bool unsure;
    const int n = affine_code_try(x, q, unsure);
    return unsure ? affine_code_exact(x, q.kind, q.scale, q.zero) : n;
}

// The code of the IEEE format of t fraction and w exponent bits nearest sig·2^(exp - top), sig's leading
// bit at position top: ties to even, overflow to the infinity's code.
PSK_DEV uint32_t round_sig_to_format(uint64_t sig, int top, int exp, int t, int w)
{
    const int bias = (1 << (w - 1)) - 1, emin = 1 - bias;
    const uint32_t inf = ((1u << w) - 1u) << t;
    int drop = top - t;
    if (exp < emin) drop += emin - exp;
    uint64_t q, rem, half;
    if (drop <= 0) { q = sig << -drop; rem = 0; half = 1; }
    else if (drop > 63) { q = 0; rem = sig != 0; half = 2; }
    else { q = sig >> drop; rem = sig & ((1ull << drop) - 1); half = 1ull << (drop - 1); }
    if (rem > half || (rem == half && (q & 1ull))) q += 1;
    const uint64_t code = exp >= emin ? ((uint64_t)(exp + bias - 1) << t) + q : q;
    return code < inf ? (uint32_t)code : inf;
}

// n·base, exactly, rounded once into the float format (t, w): its code.
PSK_DEV uint32_t round_count_to_float(int64_t n, double base, int t, int w)
{
    if (n == 0) return 0u;
    int64_t mb;
    int eb;
    take_apart(base, mb, eb);
    const u128_t mag = (u128_t)(n < 0 ? -n : n) * (u128_t)mb;
    const int bits = bit_length(mag), drop = bits > 62 ? bits - 62 : 0;
    uint64_t sig = (uint64_t)(mag >> drop);
    if (drop && (mag & ((((u128_t)1) << drop) - 1))) sig |= 1ull;
    const int top = bits - drop - 1;
    return (n < 0 ? (1u << (t + w)) : 0u) | round_sig_to_format(sig, top, eb + drop + top, t, w);
}

PSK_DEV int32_t load_count(const DevOperand &o, int64_t off, int64_t soff, double &unit)
{
    if (o.affine) {
        unit = (double)o.affine_scale;
        return affine_code_at(o, off) - o.affine_zero;
    }
    unit = (double)o.scales[soff];
    return (int)((const int8_t *)o.p)[off];
}

// A store into the launch's output: its float type, or its affine format.
PSK_DEV uint32_t store_out(const DevOperand &o, int64_t off, float x)
{
    if (o.affine) {
        const int64_t q = affine_code_of((double)x, o.affine, o.affine_scale, o.affine_zero);
        if (o.affine == 2) ((uint8_t *)const_cast<void *>(o.p))[off] = (uint8_t)q;
        else ((int8_t *)const_cast<void *>(o.p))[off] = (int8_t)q;
        return 0u;
    }
    return store_real(const_cast<void *>(o.p), o.dtype, off, x);
}

__global__ void __launch_bounds__(128) k_contract_int(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < L.total; lin += step) {
        const int64_t b0 = operand_offset(L.in[0], L.dims, 0, L.n_outer, lin), b1 = operand_offset(L.in[1], L.dims, 0, L.n_outer, lin);
        const int64_t q0 = L.in[0].affine ? 0 : scale_offset(L.in[0], L.dims, 0, L.n_outer, lin), q1 = L.in[1].affine ? 0 : scale_offset(L.in[1], L.dims, 0, L.n_outer, lin);
        uint32_t acc = 0;
        double u0 = 1.0, u1 = 1.0;
        for (int64_t c = 0; c < L.inner; ++c) {
            const int64_t o0 = operand_offset(L.in[0], L.dims, L.n_outer, L.n_inner, c), o1 = operand_offset(L.in[1], L.dims, L.n_outer, L.n_inner, c);
            const int64_t s0 = L.in[0].affine ? 0 : scale_offset(L.in[0], L.dims, L.n_outer, L.n_inner, c), s1 = L.in[1].affine ? 0 : scale_offset(L.in[1], L.dims, L.n_outer, L.n_inner, c);
            const int32_t a = load_count(L.in[0], b0 + o0, q0 + s0, u0), b = load_count(L.in[1], b1 + o1, q1 + s1, u1);
            acc += (uint32_t)(a * b); // the product of two 9-bit integers fits; the sum wraps
        }
        if (L.inner == 0) { load_count(L.in[0], b0, q0, u0); load_count(L.in[1], b1, q1, u1); }
        const int64_t n = (int32_t)acc;
        const double base = u0 * u1; // exact: two 24-bit significands
        const int64_t ooff = operand_offset(L.out, L.dims, 0, L.n_outer, lin);
        void *outp = const_cast<void *>(L.out.p);
        if (L.out.affine) {
            int64_t mb;
            int eb;
            take_apart(base, mb, eb);
            const int64_t nq = quotient_round_exact(n < 0, (u128_t)(n < 0 ? -n : n) * (u128_t)mb, eb, L.out.affine_scale);
            const int64_t q = affine_clamp(nq + L.out.affine_zero, L.out.affine);
            if (L.out.affine == 2) ((uint8_t *)outp)[ooff] = (uint8_t)q;
            else ((int8_t *)outp)[ooff] = (int8_t)q;
        } else if (L.out.dtype == PSK_F32) {
            ((uint32_t *)outp)[ooff] = round_count_to_float(n, base, 23, 8);
        } else if (L.out.dtype == PSK_BF16) {
            ((uint16_t *)outp)[ooff] = (uint16_t)round_count_to_float(n, base, 7, 8);
        } else if (L.out.dtype == PSK_F16) {
            const uint32_t c = round_count_to_float(n, base, 10, 5);
            ((uint16_t *)outp)[ooff] = (uint16_t)c;
            if ((c & 0x7fffu) == 0x7c00u) ovf |= 1u; // a count is finite: an infinity here is the store's overflow
        } else if (L.out.dtype == PSK_E8M15) {
            const uint32_t c = round_count_to_float(n, base, 15, 8);
            store_e8m15((uint8_t *)outp, ooff, c);
            if ((c & 0x7fffffu) == 0x7f8000u) ovf |= 1u;
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_FUSED, generic: one thread per output element.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_fused(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < L.total; lin += step) {
        int64_t off[PSK_MAX_INPUTS], soff[PSK_MAX_INPUTS], ooff = 0;
        for (int i = 0; i < L.n_in; ++i) off[i] = soff[i] = 0;
        int64_t r = lin;
        for (int a = L.n_outer - 1; a >= 0; --a) {
            int64_t d = L.dims[a], ix = r % d;
            r /= d;
            ooff += ix * L.out.stride[a];
            for (int i = 0; i < L.n_in; ++i) {
                off[i] += ix * L.in[i].stride[a];
                soff[i] += ix * L.in[i].sstride[a];
            }
        }
        float vals[PSK_MAX_STEPS];
        for (int s = 0; s < L.n_steps; ++s) {
            const psk_step st = L.steps[s];
            float a[2];
            for (int j = 0; j < st.nargs; ++j) {
                int src = st.src[j];
                a[j] = src >= 0 ? load_operand(L.in[src], off[src], soff[src], L.kdtype, &ovf) : vals[-1 - src];
            }
            vals[s] = st.nargs == 1 ? prim_unary(st.prim, a[0], st.imm, L.status) : prim_binary(st.prim, a[0], a[1]);
        }
        ovf |= store_out(L.out, ooff, vals[L.n_steps - 1]);
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// Eight consecutive elements of the last axis in one 128-bit access.
template <int V>
PSK_DEV void load_vec(const DevOperand &o, int64_t off, int64_t soff, int last_stride, int64_t slast, int kdtype, float (&x)[V], uint32_t *ovf)
{
    if (last_stride == 0) {
        float v = load_operand(o, off, soff, kdtype, ovf);
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] = v;
        return;
    }
    if (o.dtype == PSK_BF16 && V == 8) {
        uint4 w = *reinterpret_cast<const uint4 *>((const uint16_t *)o.p + off);
        uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = bits_f32(u[i] << 16);
            x[2 * i + 1] = bits_f32(u[i] & 0xffff0000u);
        }
        if (kdtype != PSK_BF16) {
#pragma unroll
            for (int i = 0; i < V; ++i) x[i] = edge_round(x[i], kdtype, PSK_BF16, ovf);
        }
        return;
    }
    if (o.dtype == PSK_F32 && V == 8) {
        const float4 *q = reinterpret_cast<const float4 *>((const float *)o.p + off);
        float4 a = q[0], b = q[1];
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        if (kdtype != PSK_F32) {
#pragma unroll
            for (int i = 0; i < V; ++i) x[i] = edge_round(x[i], kdtype, PSK_F32, ovf);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) x[i] = load_operand(o, off + i, soff + i * slast, kdtype, ovf);
}

template <int V>
PSK_DEV uint32_t store_vec(const DevOperand &o, int64_t off, const float (&x)[V])
{
    if (o.dtype == PSK_BF16 && V == 8) {
        uint32_t u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = (uint32_t)f32_to_bf16(x[2 * i]) | ((uint32_t)f32_to_bf16(x[2 * i + 1]) << 16);
        *reinterpret_cast<uint4 *>((uint16_t *)const_cast<void *>(o.p) + off) = make_uint4(u[0], u[1], u[2], u[3]);
        return 0u;
    }
    if (o.dtype == PSK_F32 && V == 8) {
        float4 *q = reinterpret_cast<float4 *>((float *)const_cast<void *>(o.p) + off);
        q[0] = make_float4(x[0], x[1], x[2], x[3]);
        q[1] = make_float4(x[4], x[5], x[6], x[7]);
        return 0u;
    }
    uint32_t ovf = 0;
#pragma unroll
    for (int i = 0; i < V; ++i) ovf |= store_real(const_cast<void *>(o.p), o.dtype, off + i, x[i]);
    return ovf;
}

// PSK_OP_FUSED, vectorised: the last axis is contiguous (stride 1) or
// broadcast (stride 0) in every operand, a multiple of 8 long, and every
// base and outer stride is a multiple of 8 elements; at most 8 steps.
// MAXS: the most steps a group may have here (8 for the forward groups; 12 for the optimizer's 9-step update)
template <int MAXS = 8>
__global__ void __launch_bounds__(256) k_fused_vec8(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int last = L.n_outer - 1;
    const int64_t nvec = L.total / 8, lastv = L.dims[last] / 8;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < nvec; lin += step) {
        int64_t off[PSK_MAX_INPUTS], soff[PSK_MAX_INPUTS], ooff;
        int64_t r = lin / lastv, c = (lin % lastv) * 8;
        ooff = c * L.out.stride[last];
        for (int i = 0; i < L.n_in; ++i) {
            off[i] = c * L.in[i].stride[last];
            soff[i] = c * L.in[i].sstride[last];
        }
        for (int a = last - 1; a >= 0; --a) {
            int64_t d = L.dims[a], ix = r % d;
            r /= d;
            ooff += ix * L.out.stride[a];
            for (int i = 0; i < L.n_in; ++i) {
                off[i] += ix * L.in[i].stride[a];
                soff[i] += ix * L.in[i].sstride[a];
            }
        }
        float vals[MAXS][8];
#pragma unroll
        for (int s = 0; s < MAXS; ++s) {
            if (s < L.n_steps) {
                const psk_step st = L.steps[s];
                float a[2][8];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (j < st.nargs) {
                        int src = st.src[j];
                        if (src >= 0) {
                            load_vec<8>(L.in[src], off[src], soff[src], (int)L.in[src].stride[last], L.in[src].sstride[last], L.kdtype, a[j], &ovf);
                        } else {
#pragma unroll
                            for (int t = 0; t < 8; ++t) {
                                // a step reads an earlier one: s' < s <= MAXS - 1
                                float v = 0.0f;
#pragma unroll
                                for (int q = 0; q < MAXS - 1; ++q)
                                    if (q == -1 - src) v = vals[q][t];
                                a[j][t] = v;
                            }
                        }
                    }
                }
#pragma unroll
                for (int t = 0; t < 8; ++t)
                    vals[s][t] = st.nargs == 1 ? prim_unary(st.prim, a[0][t], st.imm, L.status) : prim_binary(st.prim, a[0][t], a[1][t]);
            }
        }
        float res[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            float v = 0.0f;
#pragma unroll
            for (int q = 0; q < MAXS; ++q)
                if (q == L.n_steps - 1) v = vals[q][t];
            res[t] = v;
        }
        ovf |= store_vec<8>(L.out, ooff, res);
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_CONTRACT, exact and generic: one thread per output element, the
// terms added in the lexicographic order of the summed axes, acc = acc + x·w
// with the product rounded first (lower.rs:465-474, 586-636).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_contract_generic(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < L.total; lin += step) {
        int64_t base[PSK_MAX_INPUTS], sbase[PSK_MAX_INPUTS];
        for (int i = 0; i < L.n_in; ++i) {
            base[i] = operand_offset(L.in[i], L.dims, 0, L.n_outer, lin);
            sbase[i] = scale_offset(L.in[i], L.dims, 0, L.n_outer, lin);
        }
        int64_t ooff = operand_offset(L.out, L.dims, 0, L.n_outer, lin);
        float acc = 0.0f, part = 0.0f;
        const int64_t chunk = L.chunk; // 0: every term in index order; else the reference's chunked(size)
        for (int64_t c = 0; c < L.inner; ++c) {
            float prod = 1.0f;
            for (int i = 0; i < L.n_in; ++i) {
                int64_t o = base[i] + operand_offset(L.in[i], L.dims, L.n_outer, L.n_inner, c);
                int64_t so = sbase[i] + scale_offset(L.in[i], L.dims, L.n_outer, L.n_inner, c);
                prod = __fmul_rn(prod, load_operand(L.in[i], o, so, L.kdtype, &ovf));
            }
            if (chunk) {
                part = __fadd_rn(part, prod);
                if ((c + 1) % chunk == 0 || c + 1 == L.inner) { acc = __fadd_rn(acc, part); part = 0.0f; }
            } else {
                acc = __fadd_rn(acc, prod);
            }
        }
        ovf |= store_out(L.out, ooff, acc); // (a `scaled` site's codes too: exec.rs:758-782 stores any kernel's value through its output's format)
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// PSK_OP_CONTRACT, exact, for a matrix product with strides: C[b][i][j] =
// sum_k A[b][i][k]·B[b][k][j], batch b = blockIdx.z, 64x64 tiles of C, 16 of
// k at a time through shared memory, 4x4 outputs a thread. Every output still
// adds its own terms in increasing k from +0, each product rounded first: the
// tiling moves data, never an addition (the reference's layout space has the
// same property, presk-rt/src/layout.rs:6-11).
struct DevGemmExact {
    const void *a, *b;
    void *c;
    int a_dtype, b_dtype, c_dtype, kdtype;
    int64_t m, n, k;
    int64_t a_i, a_k, b_k, b_j;           // element strides of the operands
    int64_t batch_lo;                     // batch = hi * batch_lo + lo
    int64_t a_lo, a_hi, b_lo, b_hi, c_lo, c_hi;
    // row i of C at (i / c_row_lo_count) * c_row_hi + (i % c_row_lo_count) * c_row_lo, columns alike
    int64_t c_row_lo_count, c_row_lo, c_row_hi;
    int64_t c_col_lo_count, c_col_lo, c_col_hi;
    const float *b_scales;                // integer weights: the scale of column j is b_scales[... + j * b_sj]
    int64_t b_sj, b_slo, b_shi;
    uint32_t *ovf;
    int guarded;
    int64_t chunk;                        // 0, or the reference's chunked(size): partial sums of `chunk` terms (k_gemm_exact)
};

__global__ void __launch_bounds__(256) k_gemm_exact(const __grid_constant__ DevGemmExact G)
{
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int64_t i0 = (int64_t)blockIdx.y * 64, j0 = (int64_t)blockIdx.x * 64;
    const int64_t bz = blockIdx.z, blo = bz % G.batch_lo, bhi = bz / G.batch_lo;
    const int64_t aoff = blo * G.a_lo + bhi * G.a_hi, boff = blo * G.b_lo + bhi * G.b_hi, coff = blo * G.c_lo + bhi * G.c_hi;
    const int64_t soff = blo * G.b_slo + bhi * G.b_shi;
    uint32_t ovf = 0;
    float acc[4][4], part[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = part[r][c] = 0.0f;
    for (int64_t k0 = 0; k0 < G.k; k0 += 16) {
        // A tile: 64 rows x 16 k; B tile: 16 k x 64 columns; 4 elements a thread each
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            int e = tid + t * 256;
            {
                int kk, ii;
                if (G.a_k == 1) { kk = e % 16; ii = e / 16; } else { ii = e % 64; kk = e / 64; }
                int64_t i = i0 + ii, k = k0 + kk;
                float v = 0.0f;
                if (i < G.m && k < G.k) v = edge_round(load_real(G.a, G.a_dtype, aoff + i * G.a_i + k * G.a_k), G.kdtype, G.a_dtype, &ovf);
                As[kk][ii] = v;
            }
            {
                int kk, jj;
                if (G.b_k == 1) { kk = e % 16; jj = e / 16; } else { jj = e % 64; kk = e / 64; }
                int64_t j = j0 + jj, k = k0 + kk;
                float v = 0.0f;
                if (j < G.n && k < G.k) {
                    int64_t o = boff + k * G.b_k + j * G.b_j;
                    if (G.b_dtype == PSK_I8) v = (float)((const int8_t *)G.b)[o] * G.b_scales[soff + j * G.b_sj];
                    else v = edge_round(load_real(G.b, G.b_dtype, o), G.kdtype, G.b_dtype, &ovf);
                }
                Bs[kk][jj] = v;
            }
        }
        __syncthreads();
        const int kmax = (int)((G.k - k0) < 16 ? (G.k - k0) : 16);
        for (int kk = 0; kk < kmax; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) a[r] = As[kk][ty * 4 + r];
#pragma unroll
            for (int c = 0; c < 4; ++c) b[c] = Bs[kk][tx * 4 + c];
            if (G.chunk) {
                // chunked(size): the term joins its chunk's sum; a full chunk (or the last term) joins the total
                const bool close = (k0 + kk + 1) % G.chunk == 0 || k0 + kk + 1 == G.k;
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        part[r][c] = __fadd_rn(part[r][c], __fmul_rn(a[r], b[c]));
                        if (close) { acc[r][c] = __fadd_rn(acc[r][c], part[r][c]); part[r][c] = 0.0f; }
                    }
            } else {
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[r][c] = __fadd_rn(acc[r][c], __fmul_rn(a[r], b[c]));
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            int64_t i = i0 + ty * 4 + r, j = j0 + tx * 4 + c;
            if (i < G.m && j < G.n) {
                int64_t o = coff + (i / G.c_row_lo_count) * G.c_row_hi + (i % G.c_row_lo_count) * G.c_row_lo + (j / G.c_col_lo_count) * G.c_col_hi + (j % G.c_col_lo_count) * G.c_col_lo;
                ovf |= store_real(G.c, G.c_dtype, o, acc[r][c]);
            }
        }
    if (G.guarded && ovf) atomicOr(G.ovf, 1u);
}

// The same contraction for large operands: 128 x 128 tiles, 16 k a step, 8 x 8 results a thread, the next tile
// fetched while the current one is multiplied. Every result still adds its products one by one in increasing k
// (a multiplication, then an addition: no fused operation), so the bits are k_gemm_exact's. f32 and bf16 operands.
template <int ADT, int BDT>
__global__ void __launch_bounds__(256, 2) k_gemm_exact_big(const __grid_constant__ DevGemmExact G)
{
    __shared__ float As[2][16][128 + 4];
    __shared__ float Bs[2][16][128 + 4];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int64_t i0 = (int64_t)blockIdx.y * 128, j0 = (int64_t)blockIdx.x * 128;
    const int64_t bz = blockIdx.z, blo = bz % G.batch_lo, bhi = bz / G.batch_lo;
    const int64_t aoff = blo * G.a_lo + bhi * G.a_hi, boff = blo * G.b_lo + bhi * G.b_hi, coff = blo * G.c_lo + bhi * G.c_hi;
    uint32_t ovf = 0;
    float acc[8][8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[r][c] = 0.0f;
    // which elements of a 128 x 16 tile this thread fetches, eight of each operand: element e = tid + 256 t of the
    // tile, walked along k when k is the operand's contiguous axis, else along the rows (or columns)
    const bool ak = G.a_k == 1, bk = G.b_k == 1;
    const int a_kk0 = ak ? tid % 16 : tid / 128, a_ii0 = ak ? tid / 16 : tid % 128, a_dkk = ak ? 0 : 2, a_dii = ak ? 16 : 0;
    const int b_kk0 = bk ? tid % 16 : tid / 128, b_jj0 = bk ? tid / 16 : tid % 128, b_dkk = bk ? 0 : 2, b_djj = bk ? 16 : 0;
    float ra[8], rb[8];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const int64_t i = i0 + a_ii0 + t * a_dii, ka = k0 + a_kk0 + t * a_dkk, j = j0 + b_jj0 + t * b_djj, kb = k0 + b_kk0 + t * b_dkk;
            ra[t] = (i < G.m && ka < G.k) ? edge_round(load_real(G.a, ADT, aoff + i * G.a_i + ka * G.a_k), G.kdtype, ADT, &ovf) : 0.0f;
            rb[t] = (j < G.n && kb < G.k) ? edge_round(load_real(G.b, BDT, boff + kb * G.b_k + j * G.b_j), G.kdtype, BDT, &ovf) : 0.0f;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int t = 0; t < 8; ++t) { As[buf][a_kk0 + t * a_dkk][a_ii0 + t * a_dii] = ra[t]; Bs[buf][b_kk0 + t * b_dkk][b_jj0 + t * b_djj] = rb[t]; }
    };
    fetch(0);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int64_t k0 = 0; k0 < G.k; k0 += 16) {
        const bool more = k0 + 16 < G.k;
        if (more) fetch(k0 + 16);
        const int kmax = (int)((G.k - k0) < 16 ? (G.k - k0) : 16);
#pragma unroll 4
        for (int kk = 0; kk < kmax; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4]), a1 = *reinterpret_cast<const float4 *>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4]), b1 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[r][c] = __fadd_rn(acc[r][c], __fmul_rn(a[r], b[c]));
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int64_t i = i0 + (r < 4 ? ty * 4 + r : 64 + ty * 4 + r - 4), j = j0 + (c < 4 ? tx * 4 + c : 64 + tx * 4 + c - 4);
            if (i < G.m && j < G.n) {
                const int64_t o = coff + (i / G.c_row_lo_count) * G.c_row_hi + (i % G.c_row_lo_count) * G.c_row_lo + (j / G.c_col_lo_count) * G.c_col_hi + (j % G.c_col_lo_count) * G.c_col_lo;
                ovf |= store_real(G.c, G.c_dtype, o, acc[r][c]);
            }
        }
    if (G.guarded && ovf) atomicOr(G.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_REDUCE (lower.rs:1221-1255, 1693): sum, mean (sum / n), sum of
// squares; exact: one thread per output, the terms in lexicographic order.
// ---------------------------------------------------------------------------
PSK_DEV float reduce_finish(const DevLaunch &L, float acc)
{
    return L.kind == PSK_REDUCE_MEAN ? __fdiv_rn(acc, (float)(double)L.iparam[0]) : acc;
}

__global__ void __launch_bounds__(128) k_reduce_seq(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < L.total; lin += step) {
        int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, lin);
        int64_t ooff = operand_offset(L.out, L.dims, 0, L.n_outer, lin);
        float acc = 0.0f;
        if (L.n_inner == 1) {
            const int64_t s = L.in[0].stride[L.n_outer];
            for (int64_t c = 0; c < L.inner; ++c) {
                float x = load_operand(L.in[0], base + c * s, 0, L.kdtype, &ovf);
                acc = __fadd_rn(acc, L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x, x) : x);
                if (L.kind == PSK_REDUCE_SUM_STORED) { ovf |= store_overflows(L.out.dtype, acc); acc = prim_unary(PSK_ROUND, acc, L.out.dtype, L.status); }
            }
        } else {
            for (int64_t c = 0; c < L.inner; ++c) {
                float x = load_operand(L.in[0], base + operand_offset(L.in[0], L.dims, L.n_outer, L.n_inner, c), 0, L.kdtype, &ovf);
                acc = __fadd_rn(acc, L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x, x) : x);
                if (L.kind == PSK_REDUCE_SUM_STORED) { ovf |= store_overflows(L.out.dtype, acc); acc = prim_unary(PSK_ROUND, acc, L.out.dtype, L.status); }
            }
        }
        ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, ooff, reduce_finish(L, acc));
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// The sequential order for a few long sums (the mean over every position of a loss): one thread adding its terms
// one after the other waits a memory latency a term. Here a block owns an output: its threads bring 2048 terms at a
// time into shared memory, converted as the kernel's loads convert them, and thread 0 adds those in index order.
// The same additions in the same order as k_reduce_seq; one summed axis, any stride.
__global__ void __launch_bounds__(256) k_reduce_seq_staged(const __grid_constant__ DevLaunch L)
{
    __shared__ float buf[2048];
    uint32_t ovf = 0;
    const int64_t s = L.in[0].stride[L.n_outer];
    for (int64_t lin = blockIdx.x; lin < L.total; lin += gridDim.x) {
        const int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, lin);
        float acc = 0.0f;
        for (int64_t c0 = 0; c0 < L.inner; c0 += 2048) {
            const int n = (int)(L.inner - c0 < 2048 ? L.inner - c0 : 2048);
            for (int i = threadIdx.x; i < n; i += blockDim.x) buf[i] = load_operand(L.in[0], base + (c0 + i) * s, 0, L.kdtype, &ovf);
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int i = 0; i < n; ++i) {
                    const float x = buf[i];
                    acc = __fadd_rn(acc, L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x, x) : x);
                    if (L.kind == PSK_REDUCE_SUM_STORED) { ovf |= store_overflows(L.out.dtype, acc); acc = prim_unary(PSK_ROUND, acc, L.out.dtype, L.status); }
                }
            }
            __syncthreads();
        }
        if (threadIdx.x == 0) ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, operand_offset(L.out, L.dims, 0, L.n_outer, lin), reduce_finish(L, acc));
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

PSK_DEV float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

PSK_DEV float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// A block's sum or maximum, every thread receiving it. `red` holds 32 floats.
template <bool MAX>
PSK_DEV float block_reduce(float v, float *red)
{
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = MAX ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : (MAX ? -INFINITY : 0.0f);
    r = MAX ? warp_max(r) : warp_sum(r);
    return r;
}

// PSK_OP_REDUCE under PSK_ORDER_DEVICE over one contiguous summed axis: a
// warp a row, eight elements a lane a step, a shuffle tree at the end. The
// grouping of the additions differs from index order (declared).
__global__ void __launch_bounds__(256) k_reduce_rows_tree(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t n = L.inner;
    const bool vec = (n % 8 == 0);
    for (int64_t row = warp; row < L.total; row += nwarps) {
        int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        float acc = 0.0f;
        if (vec) {
            for (int64_t c = (int64_t)lane * 8; c < n; c += 256) {
                float x[8];
                load_vec<8>(L.in[0], base + c, 0, 1, 0, L.kdtype, x, &ovf);
#pragma unroll
                for (int t = 0; t < 8; ++t) acc += L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x[t], x[t]) : x[t];
            }
        } else {
            for (int64_t c = lane; c < n; c += 32) {
                float x = load_operand(L.in[0], base + c, 0, L.kdtype, &ovf);
                acc += L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x, x) : x;
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            int64_t ooff = operand_offset(L.out, L.dims, 0, L.n_outer, row);
            ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, ooff, reduce_finish(L, acc));
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// Sums over leading rows for every element of a contiguous last outer axis (a bias's or a gain's gradient: `sum_to`
// of [rows, n] into [n]) under PSK_ORDER_DEVICE: a block of 32 x 32 threads takes 32 neighbouring outputs, its 32
// thread rows stride through the summed index, and their partial sums meet in shared memory.
__global__ void __launch_bounds__(1024) k_reduce_cols_tree(const __grid_constant__ DevLaunch L)
{
    __shared__ float part[32][33];
    uint32_t ovf = 0;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int64_t o0 = (int64_t)blockIdx.x * 32; o0 < L.total; o0 += (int64_t)gridDim.x * 32) {
        const int64_t o = o0 + tx;
        float acc = 0.0f;
        if (o < L.total) {
            const int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, o);
            for (int64_t c = ty; c < L.inner; c += 32) {
                float x = load_operand(L.in[0], base + operand_offset(L.in[0], L.dims, L.n_outer, L.n_inner, c), 0, L.kdtype, &ovf);
                acc += L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x, x) : x;
            }
        }
        part[ty][tx] = acc;
        __syncthreads();
        if (ty == 0 && o < L.total) {
            float sum = 0.0f;
#pragma unroll
            for (int r = 0; r < 32; ++r) sum += part[r][tx];
            ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, operand_offset(L.out, L.dims, 0, L.n_outer, o), reduce_finish(L, sum));
        }
        __syncthreads();
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// A whole tensor summed to one number under PSK_ORDER_DEVICE: one block.
__global__ void __launch_bounds__(1024) k_reduce_all_tree(const __grid_constant__ DevLaunch L)
{
    __shared__ float red[32];
    uint32_t ovf = 0;
    float acc = 0.0f;
    for (int64_t c = threadIdx.x; c < L.inner; c += blockDim.x) {
        float x = load_operand(L.in[0], operand_offset(L.in[0], L.dims, L.n_outer, L.n_inner, c), 0, L.kdtype, &ovf);
        acc += L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x, x) : x;
    }
    acc = block_reduce<false>(acc, red);
    if (threadIdx.x == 0) ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, 0, reduce_finish(L, acc));
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// A leaf's sum (or sum of squares) when the leaf is one contiguous run of bf16 or f32 numbers that the kernel
// reads unrounded: sixteen bytes a load. The grid is fixed, so the order of the sum is too (a declared order of
// PSK_ORDER_DEVICE: a thread's vectors in turn, then the block's tree, then k_reduce_all_finish).
template <bool BF16>
__global__ void __launch_bounds__(512) k_reduce_all_partials_lin(const void *p, int64_t nvec, int sumsq, float *partials)
{
    __shared__ float red[32];
    float acc = 0.0f;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < nvec; c += step) {
        float x[8];
        if (BF16) {
            const uint4 w = reinterpret_cast<const uint4 *>(p)[c];
            const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { x[2 * i] = bits_f32(u[i] << 16); x[2 * i + 1] = bits_f32(u[i] & 0xffff0000u); }
        } else {
            const float4 a = reinterpret_cast<const float4 *>(p)[2 * c], b = reinterpret_cast<const float4 *>(p)[2 * c + 1];
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, sumsq ? __fmul_rn(x[i], x[i]) : x[i]);
    }
    acc = block_reduce<false>(acc, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

// AdamW's parameter update as one compile-time program (optim.rs:156-219, the group the host issues as nine steps:
// m̂ = m'/bc1, v̂ = v'/bc2, √v̂, + ε, m̂ / that, θ·λ, their sum, × lr, θ − that): the same nine IEEE operations in
// the same order on every element, so the bits of the generic group, at the memory's rate instead of the
// interpreter's. m', v' and θ are bf16 or f32 runs of 8·nvec elements, the five scalars any real type.
struct AdamwUpdate {
    const void *m, *v, *theta, *sc[5]; // sc: bc1, bc2, eps, lambda, lr
    void *out;
    int32_t m_bf16, v_bf16, t_bf16, o_bf16, sdt[5];
    int64_t nvec;
};

PSK_DEV void load8_real(const void *p, bool bf16, int64_t c, float (&x)[8])
{
    if (bf16) {
        const uint4 w = reinterpret_cast<const uint4 *>(p)[c];
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { x[2 * i] = bits_f32(u[i] << 16); x[2 * i + 1] = bits_f32(u[i] & 0xffff0000u); }
    } else {
        const float4 a = reinterpret_cast<const float4 *>(p)[2 * c], b = reinterpret_cast<const float4 *>(p)[2 * c + 1];
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
}

__global__ void __launch_bounds__(256) k_adamw_update(const __grid_constant__ AdamwUpdate P)
{
    const float bc1 = load_real(P.sc[0], P.sdt[0], 0), bc2 = load_real(P.sc[1], P.sdt[1], 0), eps = load_real(P.sc[2], P.sdt[2], 0);
    const float lambda = load_real(P.sc[3], P.sdt[3], 0), lr = load_real(P.sc[4], P.sdt[4], 0);
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < P.nvec; c += step) {
        float m[8], v[8], t[8], r[8];
        load8_real(P.m, P.m_bf16, c, m);
        load8_real(P.v, P.v_bf16, c, v);
        load8_real(P.theta, P.t_bf16, c, t);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float mh = __fdiv_rn(m[i], bc1), vh = __fdiv_rn(v[i], bc2);
            const float upd = __fdiv_rn(mh, __fadd_rn(__fsqrt_rn(vh), eps));
            r[i] = __fsub_rn(t[i], __fmul_rn(__fadd_rn(upd, __fmul_rn(t[i], lambda)), lr));
        }
        if (P.o_bf16) {
            uint4 w;
            w.x = (uint32_t)f32_to_bf16(r[0]) | ((uint32_t)f32_to_bf16(r[1]) << 16); w.y = (uint32_t)f32_to_bf16(r[2]) | ((uint32_t)f32_to_bf16(r[3]) << 16);
            w.z = (uint32_t)f32_to_bf16(r[4]) | ((uint32_t)f32_to_bf16(r[5]) << 16); w.w = (uint32_t)f32_to_bf16(r[6]) | ((uint32_t)f32_to_bf16(r[7]) << 16);
            reinterpret_cast<uint4 *>(P.out)[c] = w;
        } else {
            reinterpret_cast<float4 *>(P.out)[2 * c] = make_float4(r[0], r[1], r[2], r[3]);
            reinterpret_cast<float4 *>(P.out)[2 * c + 1] = make_float4(r[4], r[5], r[6], r[7]);
        }
    }
}

// The same for a large tensor (a parameter tree's leaf under `sum_squares`): every block sums its share into
// `partials`, a second launch of one block sums those. The grid's size is fixed, so the sum's order is too.
__global__ void __launch_bounds__(1024) k_reduce_all_partials(const __grid_constant__ DevLaunch L, float *partials)
{
    __shared__ float red[32];
    uint32_t ovf = 0;
    float acc = 0.0f;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < L.inner; c += step) {
        float x = load_operand(L.in[0], operand_offset(L.in[0], L.dims, L.n_outer, L.n_inner, c), 0, L.kdtype, &ovf);
        acc += L.kind == PSK_REDUCE_SUMSQ ? __fmul_rn(x, x) : x;
    }
    acc = block_reduce<false>(acc, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = acc;
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}
__global__ void __launch_bounds__(1024) k_reduce_all_finish(const __grid_constant__ DevLaunch L, const float *partials, int n)
{
    __shared__ float red[32];
    float acc = 0.0f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) acc += partials[c];
    acc = block_reduce<false>(acc, red);
    uint32_t ovf = 0;
    if (threadIdx.x == 0) ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, 0, reduce_finish(L, acc));
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_SOFTMAX (lower.rs:1274-1419), three passes, exact: a thread a row.
// Input 1, when masked, is indices 0 or 1 broadcast into the scores; iparam[0]
// = 1 says it is the causal mask of lower.rs:1718 (allowed iff k <= i), whose
// row i is iparam[1]-strided: then it is computed, not read.
// ---------------------------------------------------------------------------
PSK_DEV bool mask_allows(const DevLaunch &L, int64_t mbase, int64_t k, int64_t ms)
{
    if (L.iparam[0] == 1) return k <= mbase; // mbase is the row's position
    return (float)(double)((const int64_t *)L.in[1].p)[mbase + k * ms] > 0.5f;
}

__global__ void __launch_bounds__(128) k_softmax_seq(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t n = L.inner, s = L.in[0].stride[L.n_outer], os = L.out.stride[L.n_outer];
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; row < L.total; row += step) {
        if (n == 0) continue;
        int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        int64_t obase = operand_offset(L.out, L.dims, 0, L.n_outer, row);
        if (!L.masked) {
            float m = load_operand(L.in[0], base, 0, L.kdtype, &ovf);
            for (int64_t k = 0; k < n; ++k) {
                float x = load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf);
                if (x > m) m = x;
            }
            float z = 0.0f;
            for (int64_t k = 0; k < n; ++k) z = __fadd_rn(z, lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), m)));
            for (int64_t k = 0; k < n; ++k)
                ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, obase + k * os, __fdiv_rn(lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), m)), z));
        } else {
            int64_t mbase = operand_offset(L.in[1], L.dims, 0, L.n_outer, row);
            const int64_t ms = L.in[1].stride[L.n_outer];
            if (L.iparam[0] == 1) mbase = mbase / L.iparam[1];
            float mx = 0.0f;
            bool first = true;
            for (int64_t k = 0; k < n; ++k) {
                if (mask_allows(L, mbase, k, ms)) {
                    float x = load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf);
                    mx = first ? x : (x > mx ? x : mx);
                    first = false;
                }
            }
            float z = 0.0f;
            for (int64_t k = 0; k < n; ++k) {
                float e = mask_allows(L, mbase, k, ms) ? lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), mx)) : 0.0f;
                z = __fadd_rn(z, e);
            }
            for (int64_t k = 0; k < n; ++k) {
                float v = mask_allows(L, mbase, k, ms) ? __fdiv_rn(lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), mx)), z) : 0.0f;
                ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, obase + k * os, v);
            }
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// PSK_OP_SOFTMAX under PSK_ORDER_DEVICE over a contiguous axis: a warp a row,
// the row's exponentials kept in registers between the sum and the division
// (the same bits as computing them twice), the sum a shuffle tree. CACHE
// floats a lane: rows of up to 32·CACHE elements.
template <int CACHE>
__global__ void __launch_bounds__(128) k_softmax_rows_tree(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t n = L.inner;
    for (int64_t row = warp; row < L.total; row += nwarps) {
        int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        int64_t obase = operand_offset(L.out, L.dims, 0, L.n_outer, row);
        int64_t mbase = 0, ms = 0;
        if (L.masked) {
            mbase = operand_offset(L.in[1], L.dims, 0, L.n_outer, row);
            ms = L.in[1].stride[L.n_outer];
            if (L.iparam[0] == 1) mbase = mbase / L.iparam[1];
        }
        // element (c, t) of this lane is column (c·32 + lane)·8 + t
        float x[CACHE];
        uint32_t allow[CACHE / 8];
        float m = -INFINITY;
        bool any = false;
#pragma unroll
        for (int c = 0; c < CACHE / 8; ++c) {
            int64_t col = ((int64_t)c * 32 + lane) * 8;
            allow[c] = 0;
            if (col < n) {
                bool live = !(L.masked && L.iparam[0] == 1 && col > mbase);
                float v[8];
                if (live) load_vec<8>(L.in[0], base + col, 0, 1, 0, L.kdtype, v, &ovf);
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    bool ok = live && (!L.masked || mask_allows(L, mbase, col + t, ms));
                    x[c * 8 + t] = ok ? v[t] : 0.0f;
                    if (ok) {
                        allow[c] |= 1u << t;
                        m = fmaxf(m, v[t]);
                        any = true;
                    }
                }
            }
        }
        m = warp_max(m);
        any = __any_sync(0xffffffffu, any);
        float z = 0.0f;
#pragma unroll
        for (int c = 0; c < CACHE / 8; ++c)
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                float e = (allow[c] >> t & 1u) ? lm_expf(__fsub_rn(x[c * 8 + t], m)) : 0.0f;
                x[c * 8 + t] = e;
                z += e;
            }
        z = warp_sum(z);
#pragma unroll
        for (int c = 0; c < CACHE / 8; ++c) {
            int64_t col = ((int64_t)c * 32 + lane) * 8;
            if (col < n) {
                float r[8];
#pragma unroll
                for (int t = 0; t < 8; ++t) r[t] = (allow[c] >> t & 1u) ? __fdiv_rn(x[c * 8 + t], z) : 0.0f;
                ovf |= store_vec<8>(L.out, obase + col, r);
            }
        }
        (void)any;
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_XENT (lower.rs:1459): ln z + m - x[y] over the last axis.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k_xent_seq(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t n = L.inner, s = L.in[0].stride[L.n_outer];
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; row < L.total; row += step) {
        int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        int64_t ybase = operand_offset(L.in[1], L.dims, 0, L.n_outer, row);
        int64_t obase = operand_offset(L.out, L.dims, 0, L.n_outer, row);
        float m = load_operand(L.in[0], base, 0, L.kdtype, &ovf);
        for (int64_t k = 0; k < n; ++k) {
            float x = load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf);
            if (x > m) m = x;
        }
        float z = 0.0f;
        for (int64_t k = 0; k < n; ++k) z = __fadd_rn(z, lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), m)));
        int64_t y = ((const int64_t *)L.in[1].p)[ybase];
        float xy = 0.0f;
        if (y >= 0 && y < n) xy = load_operand(L.in[0], base + y * s, 0, L.kdtype, &ovf);
        else atomicOr(L.status, 2u);
        ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, obase, __fsub_rn(__fadd_rn(lm_logf(z), m), xy));
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_XENT_VJP (lower.rs:1472): (exp(x - m) / z - [k == y]) * ct over the last axis. A warp a row: lane 0
// takes the maximum and z in index order (the sum's order is the value), every lane then writes its share
// of the row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k_xent_vjp_rows(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int lane = threadIdx.x & 31;
    const int64_t n = L.inner, s = L.in[0].stride[L.n_outer], os = L.out.stride[L.n_outer];
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < L.total; row += warps) {
        const int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        float m = 0.0f, z = 0.0f;
        if (lane == 0) {
            m = load_operand(L.in[0], base, 0, L.kdtype, &ovf);
            for (int64_t k = 0; k < n; ++k) {
                float x = load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf);
                if (x > m) m = x;
            }
            for (int64_t k = 0; k < n; ++k) z = __fadd_rn(z, lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), m)));
        }
        m = __shfl_sync(0xffffffffu, m, 0);
        z = __shfl_sync(0xffffffffu, z, 0);
        const int64_t y = ((const int64_t *)L.in[1].p)[operand_offset(L.in[1], L.dims, 0, L.n_outer, row)];
        const float ct = load_operand(L.in[2], operand_offset(L.in[2], L.dims, 0, L.n_outer, row), 0, L.kdtype, &ovf);
        const int64_t obase = operand_offset(L.out, L.dims, 0, L.n_outer, row);
        for (int64_t k = lane; k < n; k += 32) {
            const float hot = (float)k == (float)y ? 1.0f : 0.0f; // the reference compares them as reals of the kernel's type
            const float sm = __fdiv_rn(lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), m)), z);
            ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, obase + k * os, __fmul_rn(__fsub_rn(sm, hot), ct));
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_EMBED_VJP (lower.rs:1444): the table's gradient. The reference zero-fills the table and adds one row of
// the cotangent per index, in index order, the sum kept in the output's storage. Here a block owns a row of
// the table: it walks the indices in order, 256 at a time, keeps the positions that name its row (in order),
// and each thread adds those rows of the cotangent into its columns: the same additions in the same order.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_embed_vjp(const __grid_constant__ DevLaunch L)
{
    __shared__ int64_t hits[256];
    __shared__ int warp_hits[8];
    uint32_t ovf = 0;
    const int last = L.n_outer - 1;
    const int64_t d = L.dims[last], rows = d ? L.total / d : 0, vocab = L.iparam[0];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int64_t v = blockIdx.x; v < vocab; v += gridDim.x) {
        // this thread's columns: tid, tid + 256, ...; the running sums live in the output, as the reference's do
        for (int64_t j = tid; j < d; j += 256) store_real(const_cast<void *>(L.out.p), L.out.dtype, v * L.out.stride[0] + j * L.out.stride[1], 0.0f);
        for (int64_t r0 = 0; r0 < rows; r0 += 256) {
            const int64_t row = r0 + tid;
            bool hit = false;
            if (row < rows) {
                const int64_t id = ((const int64_t *)L.in[1].p)[operand_offset(L.in[1], L.dims, 0, last, row)];
                hit = id == v;
                if (v == 0 && (id < 0 || id >= vocab)) atomicOr(L.status, 2u);
            }
            const uint32_t ballot = __ballot_sync(0xffffffffu, hit);
            if (lane == 0) warp_hits[warp] = __popc(ballot);
            __syncthreads();
            int before = 0, all = 0;
            for (int w = 0; w < 8; ++w) { if (w < warp) before += warp_hits[w]; all += warp_hits[w]; }
            if (hit) hits[before + __popc(ballot & ((1u << lane) - 1u))] = row;
            __syncthreads();
            for (int h = 0; h < all; ++h) {
                const int64_t cbase = operand_offset(L.in[2], L.dims, 0, last, hits[h]);
                for (int64_t j = tid; j < d; j += 256) {
                    const int64_t o = v * L.out.stride[0] + j * L.out.stride[1];
                    const float acc = __fadd_rn(load_real(L.out.p, L.out.dtype, o), load_operand(L.in[2], cbase + j * L.in[2].stride[last], 0, L.kdtype, &ovf));
                    ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, o, acc);
                }
            }
            __syncthreads();
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// Under PSK_ORDER_DEVICE: a block a row, z a tree sum.
__global__ void __launch_bounds__(256) k_xent_rows_tree(const __grid_constant__ DevLaunch L)
{
    __shared__ float red[32];
    uint32_t ovf = 0;
    const int64_t n = L.inner;
    const bool vec = (n % 8 == 0) && L.in[0].stride[L.n_outer] == 1;
    for (int64_t row = blockIdx.x; row < L.total; row += gridDim.x) {
        int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        float m = -INFINITY;
        if (vec) {
            for (int64_t c = (int64_t)threadIdx.x * 8; c < n; c += (int64_t)blockDim.x * 8) {
                float x[8];
                load_vec<8>(L.in[0], base + c, 0, 1, 0, L.kdtype, x, &ovf);
#pragma unroll
                for (int t = 0; t < 8; ++t) m = fmaxf(m, x[t]);
            }
        } else {
            for (int64_t c = threadIdx.x; c < n; c += blockDim.x) m = fmaxf(m, load_operand(L.in[0], base + c * L.in[0].stride[L.n_outer], 0, L.kdtype, &ovf));
        }
        m = block_reduce<true>(m, red);
        float z = 0.0f;
        if (vec) {
            for (int64_t c = (int64_t)threadIdx.x * 8; c < n; c += (int64_t)blockDim.x * 8) {
                float x[8];
                load_vec<8>(L.in[0], base + c, 0, 1, 0, L.kdtype, x, &ovf);
#pragma unroll
                for (int t = 0; t < 8; ++t) z += lm_expf(__fsub_rn(x[t], m));
            }
        } else {
            for (int64_t c = threadIdx.x; c < n; c += blockDim.x) z += lm_expf(__fsub_rn(load_operand(L.in[0], base + c * L.in[0].stride[L.n_outer], 0, L.kdtype, &ovf), m));
        }
        z = block_reduce<false>(z, red);
        if (threadIdx.x == 0) {
            int64_t ybase = operand_offset(L.in[1], L.dims, 0, L.n_outer, row);
            int64_t obase = operand_offset(L.out, L.dims, 0, L.n_outer, row);
            int64_t y = ((const int64_t *)L.in[1].p)[ybase];
            float xy = 0.0f;
            if (y >= 0 && y < n) xy = load_operand(L.in[0], base + y * L.in[0].stride[L.n_outer], 0, L.kdtype, &ovf);
            else atomicOr(L.status, 2u);
            ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, obase, __fsub_rn(__fadd_rn(lm_logf(z), m), xy));
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// PSK_OP_XENT_VJP under PSK_ORDER_DEVICE: a block a row, the maximum and z as trees, then every thread its share.
__global__ void __launch_bounds__(256) k_xent_vjp_rows_tree(const __grid_constant__ DevLaunch L)
{
    __shared__ float red[32];
    uint32_t ovf = 0;
    const int64_t n = L.inner, s = L.in[0].stride[L.n_outer], os = L.out.stride[L.n_outer];
    for (int64_t row = blockIdx.x; row < L.total; row += gridDim.x) {
        const int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        float m = -INFINITY;
        for (int64_t c = threadIdx.x; c < n; c += blockDim.x) m = fmaxf(m, load_operand(L.in[0], base + c * s, 0, L.kdtype, &ovf));
        m = block_reduce<true>(m, red);
        float z = 0.0f;
        for (int64_t c = threadIdx.x; c < n; c += blockDim.x) z += lm_expf(__fsub_rn(load_operand(L.in[0], base + c * s, 0, L.kdtype, &ovf), m));
        z = block_reduce<false>(z, red);
        const int64_t y = ((const int64_t *)L.in[1].p)[operand_offset(L.in[1], L.dims, 0, L.n_outer, row)];
        const float ct = load_operand(L.in[2], operand_offset(L.in[2], L.dims, 0, L.n_outer, row), 0, L.kdtype, &ovf);
        const int64_t obase = operand_offset(L.out, L.dims, 0, L.n_outer, row);
        for (int64_t k = threadIdx.x; k < n; k += blockDim.x) {
            const float hot = (float)k == (float)y ? 1.0f : 0.0f;
            const float sm = __fdiv_rn(lm_expf(__fsub_rn(load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf), m)), z);
            ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, obase + k * os, __fmul_rn(__fsub_rn(sm, hot), ct));
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_ARGMAX (lower.rs:1490): the last of equal maxima.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k_argmax(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t n = L.inner, s = L.in[0].stride[L.n_outer];
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; row < L.total; row += step) {
        int64_t base = operand_offset(L.in[0], L.dims, 0, L.n_outer, row);
        int64_t obase = operand_offset(L.out, L.dims, 0, L.n_outer, row);
        float m = load_operand(L.in[0], base, 0, L.kdtype, &ovf);
        int64_t best = 0;
        for (int64_t k = 0; k < n; ++k) {
            float x = load_operand(L.in[0], base + k * s, 0, L.kdtype, &ovf);
            if (x >= m) { m = x; best = k; }
        }
        ((int64_t *)const_cast<void *>(L.out.p))[obase] = best;
    }
}

// ---------------------------------------------------------------------------
// PSK_OP_EMBED (lower.rs:1421): out[iv, j] = table[idx[iv], j]. dims =
// (idx dims..., d); input 0 the table (stride over its two axes in stride[0],
// stride[1]), input 1 the indices. iparam[0] = rows of the table.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_embed(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int last = L.n_outer - 1;
    const int64_t d = L.dims[last], rows = L.total / d;
    const bool vec = d % 8 == 0 && L.in[0].stride[1] == 1 && L.out.stride[last] == 1 && L.in[0].stride[0] % 8 == 0;
    const int64_t per = vec ? d / 8 : d;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < rows * per; lin += step) {
        int64_t row = lin / per, c = lin % per;
        int64_t ioff = operand_offset(L.in[1], L.dims, 0, last, row);
        int64_t obase = operand_offset(L.out, L.dims, 0, last, row);
        int64_t id = ((const int64_t *)L.in[1].p)[ioff];
        bool ok = id >= 0 && id < L.iparam[0];
        if (!ok) { atomicOr(L.status, 2u); id = 0; }
        if (vec) {
            float x[8];
            load_vec<8>(L.in[0], id * L.in[0].stride[0] + c * 8, 0, 1, 0, L.kdtype, x, &ovf);
            ovf |= store_vec<8>(L.out, obase + c * 8, x);
        } else {
            float x = load_operand(L.in[0], id * L.in[0].stride[0] + c * L.in[0].stride[1], 0, L.kdtype, &ovf);
            ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, obase + c * L.out.stride[last], x);
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_COPY: out[o] = in[o] through strides (slice, a part of a concat,
// split_heads, merge_heads, index, broadcast_like). Reals pass through the
// kernel's arithmetic as the reference's `Store(Load)` does; indices are
// copied as integers.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_copy(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < L.total; lin += step) {
        int64_t off = 0, ooff = 0, r = lin;
        for (int a = L.n_outer - 1; a >= 0; --a) {
            int64_t d = L.dims[a], ix = r % d;
            r /= d;
            off += ix * L.in[0].stride[a];
            ooff += ix * L.out.stride[a];
        }
        if (L.in[0].is_index) ((int64_t *)const_cast<void *>(L.out.p))[ooff] = ((const int64_t *)L.in[0].p)[off];
        else ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, ooff, load_operand(L.in[0], off, 0, L.kdtype, &ovf));
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// The same, eight elements of a contiguous last axis at a time.
__global__ void __launch_bounds__(256) k_copy_vec8(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int last = L.n_outer - 1;
    const int64_t nvec = L.total / 8, lastv = L.dims[last] / 8;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < nvec; lin += step) {
        int64_t r = lin / lastv, c = (lin % lastv) * 8;
        int64_t off = c, ooff = c;
        for (int a = last - 1; a >= 0; --a) {
            int64_t d = L.dims[a], ix = r % d;
            r /= d;
            off += ix * L.in[0].stride[a];
            ooff += ix * L.out.stride[a];
        }
        float x[8];
        load_vec<8>(L.in[0], off, 0, 1, 0, L.kdtype, x, &ovf);
        ovf |= store_vec<8>(L.out, ooff, x);
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_IOTA (lower.rs:1706-1750).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_iota(const __grid_constant__ DevLaunch L)
{
    uint32_t ovf = 0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; lin < L.total; lin += step) {
        switch (L.kind) {
        case PSK_IOTA_POSITIONS: ((int64_t *)const_cast<void *>(L.out.p))[lin] = lin; break;
        case PSK_IOTA_CAUSAL: {
            int64_t n = L.dims[1], i = lin / n, j = lin % n;
            ((int64_t *)const_cast<void *>(L.out.p))[lin] = (float)(double)j <= (float)(double)i ? 1 : 0;
            break;
        }
        case PSK_IOTA_ONE_HOT: {
            int64_t v = L.dims[L.n_outer - 1], row = lin / v, j = lin % v;
            int64_t ioff = operand_offset(L.in[0], L.dims, 0, L.n_outer - 1, row);
            float hit = (float)(double)((const int64_t *)L.in[0].p)[ioff] == (float)(double)j ? 1.0f : 0.0f;
            ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, lin, hit);
            break;
        }
        default: ovf |= store_real(const_cast<void *>(L.out.p), L.out.dtype, lin, L.fparam); break;
        }
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

// ---------------------------------------------------------------------------
// PSK_OP_CONVERT: n reals of one type stored as another, through f64 as the
// host converts a buffer at a kernel's edge (presk-rt/src/lib.rs:868-876;
// presk-export-c/c/presk_rt.c `presk_convert`): a widening is exact; to f32
// rounds once; to bf16 rounds to f32 and then to bf16; to binary16 or e8m15
// rounds once, also from an f64.
// ---------------------------------------------------------------------------
// An f64 rounded to f32 toward zero with the lost bits or-ed into the last
// place ("to odd"): rounding that to a narrower format gives the f64's own
// correctly rounded value, since f32 has more than two bits to spare.
PSK_DEV float f64_to_f32_odd(double x)
{
    float r = __double2float_rz(x);
    if (x == x && (double)r != x && fabsf(r) != INFINITY) r = bits_f32(f32_bits(r) | 1u);
    return r;
}

__global__ void __launch_bounds__(256) k_convert(const void *src, int from, void *dst, int to, int64_t n, int guarded, uint32_t *flag, int affine, int zero, float scale)
{
    uint32_t ovf = 0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        if (affine) { // the codes' values, (q - z)·s: exact in a double
            const int q = affine == 2 ? (int)((const uint8_t *)src)[i] : (int)((const int8_t *)src)[i];
            const double x = (double)(q - zero) * (double)scale;
            if (to == PSK_F64) ((double *)dst)[i] = x;
            else ovf |= store_real(dst, to, i, (float)x);
        } else if (from == PSK_F64) {
            double x = ((const double *)src)[i];
            if (to == PSK_F64) ((double *)dst)[i] = x;
            else if (to == PSK_F32 || to == PSK_BF16) ovf |= store_real(dst, to, i, (float)x);
            else ovf |= store_real(dst, to, i, f64_to_f32_odd(x));
        } else {
            float x = load_real(src, from, i);
            ovf |= store_real(dst, to, i, x);
        }
    }
    if (guarded && ovf) atomicOr(flag, 1u);
}

// ---------------------------------------------------------------------------
// Integer weights (presk-rt/src/quant.rs:128-167; presk_rt.c `presk_quantize`):
// a tensor read as outer x k x inner, one scale per (outer, inner) channel:
// m = max|w| over k (a NaN passed over), s = f32(m / 127) (absmax), q =
// clamp(rne(w / s), ±127), 0 when s is 0 or w / s is a NaN. The reference
// quantises f64 reals; this kernel takes f32 or f64 and computes in f64.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_quant_scales(const void *w, int from, float *s, int64_t outer, int64_t k, int64_t inner)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ch < outer * inner; ch += step) {
        int64_t o = ch / inner, in = ch % inner;
        double m = 0.0;
        for (int64_t kk = 0; kk < k; ++kk) {
            int64_t e = (o * k + kk) * inner + in;
            double x = from == PSK_F64 ? ((const double *)w)[e] : (double)((const float *)w)[e];
            double a = fabs(x);
            if (a > m) m = a;
        }
        s[ch] = (float)(m / 127.0);
    }
}

__global__ void __launch_bounds__(256) k_quant_codes(const void *w, int from, const float *s, int8_t *q, int64_t outer, int64_t k, int64_t inner)
{
    const int64_t n = outer * k * inner, step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += step) {
        int64_t ch = (e / (k * inner)) * inner + e % inner;
        double x = from == PSK_F64 ? ((const double *)w)[e] : (double)((const float *)w)[e];
        double sc = (double)s[ch];
        double r = x / sc;
        int v = 0;
        if (sc != 0.0 && r == r) {
            double t = rint(r); // to nearest, ties to even
            t = t > 127.0 ? 127.0 : (t < -127.0 ? -127.0 : t);
            v = (int)t;
        }
        q[e] = (int8_t)v;
    }
}

// PSK_OP_MAGNITUDE: a tensor's max |x|, least non-zero |x|, least and greatest x, merged into four
// words by atomic max and min on order-preserving integer views of the floats. Order-free, so exact.
PSK_DEV uint32_t ordered_bits(float x)
{
    const uint32_t b = f32_bits(x);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

__global__ void __launch_bounds__(256) k_magnitude(const void *src, int dtype, int64_t n, uint32_t *out)
{
    uint32_t mx = 0u, mn = 0x7f800000u, lo = 0xff800000u, hi = 0x007fffffu;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        const float x = load_real(src, dtype, i);
        if (x != x) continue;
        const uint32_t a = f32_bits(x) & 0x7fffffffu, o = ordered_bits(x);
        mx = max(mx, a);
        if (a != 0u) mn = min(mn, a);
        lo = min(lo, o);
        hi = max(hi, o);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, s));
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, s));
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, s));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(out + 0, mx);
        atomicMin(out + 1, mn);
        atomicMin(out + 2, lo);
        atomicMax(out + 3, hi);
    }
}

// The integers of int8 weights as bf16 numbers (every integer of [-127, 127] is one, exactly): what the
// tensor-core contraction reads in place of the codes.
__global__ void __launch_bounds__(256) k_int8_to_bf16(const int8_t *q, uint16_t *out, int64_t n)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) out[i] = (uint16_t)(f32_bits((float)q[i]) >> 16);
}

// e4m3fn weights as bf16 numbers (4 exponent and 3 fraction bits fit bf16's 8 and 7; the subnormals are
// normal bf16 numbers; the NaN stays a NaN).
__global__ void __launch_bounds__(256) k_e4m3_to_bf16(const uint8_t *q, uint16_t *out, int64_t n)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) out[i] = (uint16_t)(f32_bits(e4m3_to_f32(q[i])) >> 16);
}

// Normal draws for parameters made on the device: a counter-based hash
// (splitmix64) and Box-Muller in f32 with CUDA's own logf/cosf. These are not
// the reference's keys; they only have to be the same on every run.
PSK_DEV uint64_t mix64(uint64_t z)
{
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

__global__ void __launch_bounds__(256) k_init_normal(void *dst, int to, int64_t n, uint64_t seed, float std)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        float v;
        if (std < 0.0f) {
            v = 1.0f;
        } else {
            uint64_t h = mix64(seed * 0x2545f4914f6cdd1dull + (uint64_t)i);
            float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);
            float u2 = (float)(uint32_t)((h >> 8) & 0xffffffu) * (1.0f / 16777216.0f);
            v = std * sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
        }
        store_real(dst, to, i, v);
    }
}


// An f32 matrix as three bf16 planes, hi + mid + lo = x exactly (24 significant bits in three runs of eight; an
// infinity or a NaN goes to hi whole). Element (r, c) of plane p is written at p * plane_stride + r * row_stride + c.
__global__ void k_split_f32(const float *src, int64_t rows, int64_t cols, int64_t src_row, uint16_t *dst, int64_t row_stride, int64_t plane_stride)
{
    const int64_t total = rows * cols, step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t r = i / cols, c = i - r * cols;
        const float x = src[r * src_row + c];
        const uint32_t b = f32_bits(x);
        const uint32_t hi = b >> 16;
        uint32_t mid = 0, lo = 0;
        if ((b & 0x7f800000u) != 0x7f800000u) {
            const float r1 = __fsub_rn(x, bits_f32(hi << 16));
            mid = f32_bits(r1) >> 16;
            lo = f32_bits(__fsub_rn(r1, bits_f32(mid << 16))) >> 16;
        }
        uint16_t *d = dst + r * row_stride + c;
        d[0] = (uint16_t)hi;
        d[plane_stride] = (uint16_t)mid;
        d[2 * plane_stride] = (uint16_t)lo;
    }
}
} // namespace psk

namespace psk {
// An e8m15 matrix as two bf16 planes, x = hi + lo exactly: hi is x cut to bf16's eight significant bits, lo the
// eight that remain (an infinity or a NaN goes to hi whole, lo zero; a remainder below bf16's least subnormal,
// which only a value near 2^-126 has, is dropped). Element (r, c) of plane p is written at
// p * plane_stride + r * row_stride + c, so the planes lie side by side along whichever axis is summed.
__global__ void k_split_e8m15(const uint8_t *src, int64_t rows, int64_t cols, int64_t src_row, uint16_t *dst, int64_t row_stride, int64_t plane_stride)
{
    const int64_t total = rows * cols, step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t r = i / cols, c = i - r * cols;
        const uint32_t code = load_e8m15(src, r * src_row + c);
        const uint32_t hi = code >> 8;
        uint32_t lo = 0;
        if ((code & 0x7f8000u) != 0x7f8000u) lo = f32_bits(__fsub_rn(bits_f32(code << 8), bits_f32(hi << 16))) >> 16;
        uint16_t *d = dst + r * row_stride + c;
        d[0] = (uint16_t)hi;
        d[plane_stride] = (uint16_t)lo;
    }
}

// The parts of a contraction whose summed axis was cut into `parts` runs (a few rows against a large weight matrix:
// each run a tensor-core launch of its own batch entry, so that every SM streams a share of the weights): the f32
// partial sums added in the runs' order, scaled by the column's scale when the weights are integers, rounded to
// the contraction's own site's type, then, with an addend, added to it and rounded to the result's type
// (PSK_OP_CONTRACT_ADD's two roundings). Rows of the result at `row_stride` elements.
__global__ void __launch_bounds__(256) k_sum_parts(const float *parts_p, int parts, int64_t m, int64_t n, void *out, int out_dtype, int site_dtype, int64_t row_stride,
                                                   const void *addend, int64_t add_row_stride, const float *col_scale, int64_t col_scale_stride, int guarded, uint32_t *ovf_flag)
{
    uint32_t ovf = 0;
    const int64_t total = m * n, step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t r = i / n, c = i - r * n;
        float acc = parts_p[i];
        for (int p = 1; p < parts; ++p) acc = __fadd_rn(acc, parts_p[(int64_t)p * total + i]);
        if (col_scale) acc = __fmul_rn(acc, col_scale[c * col_scale_stride]);
        if (addend) {
            uint32_t o2 = 0;
            const float site = edge_round(acc, site_dtype, PSK_F32, &o2); // as the contraction's site would store it
            ovf |= o2;
            acc = __fadd_rn(load_real(addend, out_dtype, r * add_row_stride + c), site);
        }
        ovf |= store_real(out, out_dtype, r * row_stride + c, acc);
    }
    if (guarded && ovf) atomicOr(ovf_flag, 1u);
}

// The gap between two results (presk-driver/src/gap.rs:35-64): the largest |p - q| over their elements and the
// largest |p|, both taken in binary64 on the exactly widened values, an element that is not finite counting as
// +infinity. out[0] = bits of the gap, out[1] = bits of max |p|: non-negative doubles order as their bit
// patterns do, so the maximum over threads is an integer maximum and the result does not depend on any order.
__global__ void __launch_bounds__(256) k_gap(const void *a, int a_dtype, const void *b, int b_dtype, int64_t n, unsigned long long *out)
{
    const double inf = __longlong_as_double(0x7ff0000000000000ll);
    double gap = 0.0, mx = 0.0;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
        const double p = a_dtype == PSK_F64 ? ((const double *)a)[i] : (double)load_real(a, a_dtype, i);
        const double q = b_dtype == PSK_F64 ? ((const double *)b)[i] : (double)load_real(b, b_dtype, i);
        double d = fabs(p - q), m = fabs(p);
        if (!(d <= 1.7976931348623157e308)) d = inf; // a NaN or an infinity
        if (!(m <= 1.7976931348623157e308)) m = inf;
        gap = fmax(gap, d);
        mx = fmax(mx, m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        gap = fmax(gap, __shfl_xor_sync(0xffffffffu, gap, o));
        mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(out, (unsigned long long)__double_as_longlong(gap));
        atomicMax(out + 1, (unsigned long long)__double_as_longlong(mx));
    }
}
} // namespace psk
