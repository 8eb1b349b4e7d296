// The memory-bound launches of a transformer prefill, written for HBM
// bandwidth: 128-bit accesses, 32-bit index arithmetic, no local memory, many
// resident warps. They compute exactly what the generic kernels of
// psk_kernels.cuh compute (the same operations in the same order on each
// element; row sums as shuffle trees under PSK_ORDER_DEVICE only); the
// executor picks them when a launch's strides and sizes allow.
#pragma once
#include "psk_kernels.cuh"

namespace psk {

// ---------------------------------------------------------------------------
// Elementwise groups of up to four steps over up to four inputs, seen as a
// matrix of `rows` x `cols`: each operand walks a row contiguously or holds
// one value for it (stride 1 or 0 along the columns) and moves from row to row
// by its own stride (0 for an operand every row shares, such as a gain).
// ---------------------------------------------------------------------------
struct EwParams {
    const void *in[4];
    void *out;
    int32_t dt[4], odt, kdt;
    int32_t cs[4];      // stride along the columns: 0 or 1
    int64_t rs[4], ors; // stride from row to row, in elements
    uint32_t rows, colv; // colv = cols / 8
    // rows in two levels (k_ew_prog only): row r = r0 * rows1 + r1 lies at r0 * rs0 + r1 * rs; rows1 = 0: one level
    uint32_t rows1, pad_;
    int64_t rs0[4], ors0;
    int32_t n_in, guarded;
    psk_step steps[4];
    uint32_t *ovf, *status;
    int32_t aff_kind, aff_zero; // k_ew_lut<.., AFF>: the result's affine format
    float aff_scale;
};

// Eight consecutive stored elements widened to f32, or one broadcast to all eight.
PSK_DEV void ew_load8(const void *p, int dt, int64_t off, int cs, int kdt, float (&x)[8], uint32_t *ovf)
{
    if (cs == 0) {
        const float v = edge_round(load_real(p, dt, off), kdt, dt, ovf);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = v;
        return;
    }
    if (dt == PSK_BF16) {
        const uint4 w = *reinterpret_cast<const uint4 *>((const uint16_t *)p + off);
        x[0] = bits_f32(w.x << 16); x[1] = bits_f32(w.x & 0xffff0000u);
        x[2] = bits_f32(w.y << 16); x[3] = bits_f32(w.y & 0xffff0000u);
        x[4] = bits_f32(w.z << 16); x[5] = bits_f32(w.z & 0xffff0000u);
        x[6] = bits_f32(w.w << 16); x[7] = bits_f32(w.w & 0xffff0000u);
    } else if (dt == PSK_F32) {
        const float4 *q = reinterpret_cast<const float4 *>((const float *)p + off);
        const float4 a = q[0], b = q[1];
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = load_real(p, dt, off + i);
    }
    if (dt != kdt) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = edge_round(x[i], kdt, dt, ovf);
    }
}

PSK_DEV uint32_t ew_store8(void *p, int dt, int64_t off, const float (&x)[8])
{
    if (dt == PSK_BF16) {
        uint4 w;
        w.x = pack_bf16x2(x[0], x[1]);
        w.y = pack_bf16x2(x[2], x[3]);
        w.z = pack_bf16x2(x[4], x[5]);
        w.w = pack_bf16x2(x[6], x[7]);
        *reinterpret_cast<uint4 *>((uint16_t *)p + off) = w;
        return 0u;
    }
    if (dt == PSK_F32) {
        float4 *q = reinterpret_cast<float4 *>((float *)p + off);
        q[0] = make_float4(x[0], x[1], x[2], x[3]);
        q[1] = make_float4(x[4], x[5], x[6], x[7]);
        return 0u;
    }
    uint32_t ovf = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) ovf |= store_real(p, dt, off + i, x[i]);
    return ovf;
}

// The rarer unary operations, out of line so that the kernel's body stays small
// and its values stay in registers.
__device__ __noinline__ float prim_unary_call(int prim, float x, int imm, uint32_t *status) { return prim_unary(prim, x, imm, status); }

template <int NSTEPS>
__global__ void __launch_bounds__(256, 2) k_ew(const __grid_constant__ EwParams E)
{
    uint32_t ovf = 0;
    const uint32_t total = E.rows * E.colv;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const uint32_t r = idx / E.colv, c = (idx - r * E.colv) * 8u;
        float iv[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (i < E.n_in) ew_load8(E.in[i], E.dt[i], (int64_t)r * E.rs[i] + (int64_t)c * E.cs[i], E.cs[i], E.kdt, iv[i], &ovf);
        float sv[NSTEPS][8];
#pragma unroll
        for (int s = 0; s < NSTEPS; ++s) {
            const psk_step st = E.steps[s];
            float a[2][8];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int src = st.src[j];
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    float v = iv[0][t];
                    if (src == 1) v = iv[1][t];
                    if (src == 2) v = iv[2][t];
                    if (src == 3) v = iv[3][t];
#pragma unroll
                    for (int q = 0; q < s; ++q)
                        if (src == -1 - q) v = sv[q][t];
                    a[j][t] = v;
                }
            }
            if (st.nargs == 2) {
                switch (st.prim) {
                case PSK_ADD:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = __fadd_rn(a[0][t], a[1][t]);
                    break;
                case PSK_SUB:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = __fsub_rn(a[0][t], a[1][t]);
                    break;
                case PSK_MUL:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = __fmul_rn(a[0][t], a[1][t]);
                    break;
                case PSK_DIV:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = __fdiv_rn(a[0][t], a[1][t]);
                    break;
                default:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = prim_binary(st.prim, a[0][t], a[1][t]);
                }
            } else {
                switch (st.prim) {
                case PSK_SIGMOID:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = __frcp_rn(__fadd_rn(1.0f, lm_expf(-a[0][t])));
                    break;
                case PSK_SQRT:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = __fsqrt_rn(a[0][t]);
                    break;
                default:
#pragma unroll
                    for (int t = 0; t < 8; ++t) sv[s][t] = prim_unary_call(st.prim, a[0][t], st.imm, E.status);
                }
            }
        }
        ovf |= ew_store8(E.out, E.odt, (int64_t)r * E.ors + c, sv[NSTEPS - 1]);
    }
    if (E.guarded && ovf) atomicOr(E.ovf, 1u);
}

// The same for the case that matters in a bf16 realization: every operand and
// the result stored as bf16, the kernel's type bf16. Each thread takes UNR
// vectors of eight elements a round and issues all of their loads before it
// computes on any, so that enough bytes are in flight to fill the memory
// system at a modest number of resident warps.
template <int NSTEPS, int UNR>
__global__ void __launch_bounds__(128, 3) k_ew_bf16(const __grid_constant__ EwParams E)
{
    const uint32_t total = E.rows * E.colv;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t idx0 = blockIdx.x * blockDim.x + threadIdx.x; idx0 < total; idx0 += stride * UNR) {
        uint4 raw[UNR][4];
        uint32_t rr[UNR], cc[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const uint32_t idx = idx0 + u * stride;
            rr[u] = idx / E.colv;
            cc[u] = (idx - rr[u] * E.colv) * 8u;
            if (idx < total) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (i < E.n_in) {
                        const uint16_t *p = (const uint16_t *)E.in[i] + (int64_t)rr[u] * E.rs[i];
                        if (E.cs[i]) raw[u][i] = *reinterpret_cast<const uint4 *>(p + cc[u]);
                        else raw[u][i].x = *p;
                    }
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (idx0 + u * stride >= total) break;
            float iv[4][8];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < E.n_in) {
                    if (E.cs[i]) {
                        const uint4 w = raw[u][i];
                        iv[i][0] = bits_f32(w.x << 16); iv[i][1] = bits_f32(w.x & 0xffff0000u);
                        iv[i][2] = bits_f32(w.y << 16); iv[i][3] = bits_f32(w.y & 0xffff0000u);
                        iv[i][4] = bits_f32(w.z << 16); iv[i][5] = bits_f32(w.z & 0xffff0000u);
                        iv[i][6] = bits_f32(w.w << 16); iv[i][7] = bits_f32(w.w & 0xffff0000u);
                    } else {
                        const float v = bits_f32(raw[u][i].x << 16);
#pragma unroll
                        for (int t = 0; t < 8; ++t) iv[i][t] = v;
                    }
                }
            float sv[NSTEPS][8];
#pragma unroll
            for (int s = 0; s < NSTEPS; ++s) {
                const psk_step st = E.steps[s];
                float a[2][8];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int src = st.src[j];
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        float v = iv[0][t];
                        if (src == 1) v = iv[1][t];
                        if (src == 2) v = iv[2][t];
                        if (src == 3) v = iv[3][t];
#pragma unroll
                        for (int q = 0; q < s; ++q)
                            if (src == -1 - q) v = sv[q][t];
                        a[j][t] = v;
                    }
                }
                if (st.nargs == 2) {
                    switch (st.prim) {
                    case PSK_ADD:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = __fadd_rn(a[0][t], a[1][t]);
                        break;
                    case PSK_SUB:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = __fsub_rn(a[0][t], a[1][t]);
                        break;
                    case PSK_MUL:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = __fmul_rn(a[0][t], a[1][t]);
                        break;
                    case PSK_DIV:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = __fdiv_rn(a[0][t], a[1][t]);
                        break;
                    default:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = prim_binary(st.prim, a[0][t], a[1][t]);
                    }
                } else {
                    switch (st.prim) {
                    case PSK_SIGMOID:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = __frcp_rn(__fadd_rn(1.0f, lm_expf(-a[0][t])));
                        break;
                    case PSK_SQRT:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = __fsqrt_rn(a[0][t]);
                        break;
                    default:
#pragma unroll
                        for (int t = 0; t < 8; ++t) sv[s][t] = prim_unary_call(st.prim, a[0][t], st.imm, E.status);
                    }
                }
            }
            ew_store8(E.out, PSK_BF16, (int64_t)rr[u] * E.ors + cc[u], sv[NSTEPS - 1]);
        }
    }
}

// The groups a transformer's forward pass is made of, with their steps fixed at
// compile time: no routing of step arguments at run time, a handful of
// instructions an element. A launch whose steps are exactly one of these (the
// executor compares them) and whose operands are all bf16 takes this kernel.
enum EwProg { EW_ADD = 0, EW_SUB, EW_MUL, EW_DIV, EW_DIV_MUL, EW_SILU, EW_MUL_MUL_SUB, EW_MUL_MUL_ADD, EW_SILU_MUL, EW_NPROG };

// a / b given r = the correctly rounded 1 / b (Markstein's correction): the quotient to nearest by one
// multiplication and two fused operations. That is the division's own result whenever no intermediate leaves
// the normal range, which holds when both exponents lie in [2^-55, 2^55]: the quotient is then within 2^+-111,
// the remainder is exact and nothing overflows. Outside (zero, tiny, huge, infinite or NaN), the division.
PSK_DEV bool div_by_in_range(float x) { return ((f32_bits(x) >> 23) & 0xffu) - 72u <= 110u; }

PSK_DEV float div_by(float a, float b, float r)
{
    if (!div_by_in_range(a) || !div_by_in_range(b)) return __fdiv_rn(a, b);
    const float q = __fmul_rn(a, r);
    const float rem = __fmaf_rn(-b, q, a);
    return __fmaf_rn(rem, r, q);
}

// The same with the divisor's test made once by the caller (one divisor, many numerators).
PSK_DEV float div_by_checked(float a, float b, float r, bool b_in_range)
{
    if (!b_in_range || !div_by_in_range(a)) return __fdiv_rn(a, b);
    const float q = __fmul_rn(a, r);
    const float rem = __fmaf_rn(-b, q, a);
    return __fmaf_rn(rem, r, q);
}

template <int PROG>
PSK_DEV float ew_eval(float a, float b, float c, float d)
{
    if constexpr (PROG == EW_ADD) return __fadd_rn(a, b);
    else if constexpr (PROG == EW_SUB) return __fsub_rn(a, b);
    else if constexpr (PROG == EW_MUL) return __fmul_rn(a, b);
    else if constexpr (PROG == EW_DIV) return __fdiv_rn(a, b);
    else if constexpr (PROG == EW_DIV_MUL) return __fmul_rn(__fdiv_rn(a, b), c);                              // [div 0,1; mul s0,2]
    else if constexpr (PROG == EW_SILU) return __fmul_rn(a, __frcp_rn(__fadd_rn(1.0f, lm_expf(-a))));    // [sigmoid 0; mul 0,s0]
    else if constexpr (PROG == EW_SILU_MUL)                                                                   // [sigmoid 0; mul 0,s0; round s1 to bf16; mul s2,1]
        return __fmul_rn(bf16_to_f32(f32_to_bf16(__fmul_rn(a, __frcp_rn(__fadd_rn(1.0f, lm_expf(-a)))))), b);
    else if constexpr (PROG == EW_MUL_MUL_SUB) return __fsub_rn(__fmul_rn(a, b), __fmul_rn(c, d));            // [mul 0,1; mul 2,3; sub s0,s1]
    else return __fadd_rn(__fmul_rn(a, b), __fmul_rn(c, d));                                                  // [mul 0,1; mul 2,3; add s0,s1]
}

template <int PROG>
struct EwArity {
    static constexpr int value = (PROG == EW_SILU) ? 1 : (PROG == EW_DIV_MUL) ? 3 : (PROG == EW_MUL_MUL_SUB || PROG == EW_MUL_MUL_ADD) ? 4 : 2;
};

PSK_DEV int64_t ew_row_offset(const EwParams &E, uint32_t r, int64_t s1, int64_t s0)
{
    if (E.rows1 == 0) return (int64_t)r * s1;
    const uint32_t r0 = r / E.rows1;
    return (int64_t)r0 * s0 + (int64_t)(r - r0 * E.rows1) * s1;
}

template <int PROG, int UNR>
__global__ void __launch_bounds__(256, EwArity<PROG>::value >= 4 ? 2 : 3) k_ew_prog(const __grid_constant__ EwParams E)
{
    constexpr int NIN = EwArity<PROG>::value;
    const uint32_t total = E.rows * E.colv;
    const uint32_t stride = gridDim.x * blockDim.x;
    // an operand that is one value for the whole launch (a rank-0 divisor) is read once
    uint32_t whole[NIN];
#pragma unroll
    for (int i = 0; i < NIN; ++i) {
        whole[i] = 0;
        if (E.cs[i] == 0 && E.rs[i] == 0 && E.rs0[i] == 0) {
            uint32_t dummy = 0;
            const uint32_t h = f32_bits(edge_round(load_real(E.in[i], E.dt[i], 0), PSK_BF16, E.dt[i], &dummy)) >> 16;
            whole[i] = h | (h << 16);
        }
    }
    for (uint32_t idx0 = blockIdx.x * blockDim.x + threadIdx.x; idx0 < total; idx0 += stride * UNR) {
        uint4 raw[UNR][NIN];
        uint32_t rr[UNR], cc[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const uint32_t idx = idx0 + u * stride;
            if (E.rows == 1) { rr[u] = 0; cc[u] = idx * 8u; }
            else { rr[u] = idx / E.colv; cc[u] = (idx - rr[u] * E.colv) * 8u; }
            if (idx < total) {
#pragma unroll
                for (int i = 0; i < NIN; ++i) {
                    const int64_t ro = ew_row_offset(E, rr[u], E.rs[i], E.rs0[i]);
                    const uint16_t *p = (const uint16_t *)E.in[i] + ro;
                    if (E.cs[i]) raw[u][i] = *reinterpret_cast<const uint4 *>(p + cc[u]);
                    else if (E.rs[i] == 0 && E.rs0[i] == 0) raw[u][i] = make_uint4(whole[i], whole[i], whole[i], whole[i]);
                    else {
                        // one value for the whole row, of any real type: the kernel's type is bf16, so the
                        // value it sees is the stored one rounded to bf16 at the kernel's edge
                        uint32_t dummy = 0;
                        const float v = edge_round(load_real(E.in[i], E.dt[i], ro), PSK_BF16, E.dt[i], &dummy);
                        const uint32_t h = f32_bits(v) >> 16;
                        raw[u][i] = make_uint4(h | (h << 16), h | (h << 16), h | (h << 16), h | (h << 16));
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (idx0 + u * stride >= total) break;
            uint32_t out[4];
            // a divisor that is one value for the vector (a row's root): its reciprocal once, then a
            // multiplication and a correction an element instead of a division
            constexpr bool DIVIDES = PROG == EW_DIV || PROG == EW_DIV_MUL;
            const bool by_scalar = DIVIDES && E.cs[1] == 0;
            float sdiv = 0.0f, srcp = 0.0f;
            bool sdiv_ok = false;
            if (DIVIDES && by_scalar) { sdiv = bits_f32(raw[u][1].x << 16); srcp = __frcp_rn(sdiv); sdiv_ok = div_by_in_range(sdiv); }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float lo[4], hi[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (i < NIN) {
                        const uint32_t w = q == 0 ? raw[u][i].x : q == 1 ? raw[u][i].y : q == 2 ? raw[u][i].z : raw[u][i].w;
                        lo[i] = bits_f32(w << 16);
                        hi[i] = bits_f32(w & 0xffff0000u);
                    } else {
                        lo[i] = hi[i] = 0.0f;
                    }
                }
                if (DIVIDES && by_scalar) {
                    float ql = div_by_checked(lo[0], sdiv, srcp, sdiv_ok), qh = div_by_checked(hi[0], sdiv, srcp, sdiv_ok);
                    if (PROG == EW_DIV_MUL) { ql = __fmul_rn(ql, lo[2]); qh = __fmul_rn(qh, hi[2]); }
                    out[q] = pack_bf16x2_hw(ql, qh);
                } else {
                    // every program ends in an arithmetic operation, whose NaN is the device's canonical one:
                    // the hardware's conversion and the reference's formula make the same bf16 of it
                    out[q] = pack_bf16x2_hw(ew_eval<PROG>(lo[0], lo[1], lo[2], lo[3]), ew_eval<PROG>(hi[0], hi[1], hi[2], hi[3]));
                }
            }
            *reinterpret_cast<uint4 *>((uint16_t *)E.out + ew_row_offset(E, rr[u], E.ors, E.ors0) + cc[u]) = make_uint4(out[0], out[1], out[2], out[3]);
        }
    }
}

// ---------------------------------------------------------------------------
// A group of one bf16 input and a bf16 result is a function of 65 536 codes.
// silu costs about fifty instructions an element when computed to the
// reference's bits (its expf with a division inside, a reciprocal), which
// makes a launch over [tokens, ff] instruction-bound at a quarter of the
// memory rate. So the executor evaluates the very same device function once
// over every code (k_table_silu), and launches read the result from a copy of
// that table in shared memory: the same bits by construction, NaN payloads
// included, at the memory's rate.
// ---------------------------------------------------------------------------
__global__ void k_table_silu(uint16_t *table)
{
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < 65536u) table[c] = f32_to_bf16(ew_eval<EW_SILU>(bf16_to_f32((uint16_t)c), 0.0f, 0.0f, 0.0f));
}

// out = T[in0] (MUL = false), or bf16(T[in0] * in1) (MUL = true: the group [.., round to bf16, mul s2,1]);
// AFF: the product stored as one-byte codes of an affine format (E.aff_*), as the generic group's store does.
template <bool MUL, bool AFF = false>
__global__ void __launch_bounds__(1024, 1) k_ew_lut(const __grid_constant__ EwParams E, const uint16_t *__restrict__ table)
{
    extern __shared__ uint16_t s_table[];
    for (uint32_t i = threadIdx.x; i < 65536u / 8u; i += blockDim.x)
        reinterpret_cast<uint4 *>(s_table)[i] = reinterpret_cast<const uint4 *>(table)[i];
    __syncthreads();
    const uint32_t total = E.rows * E.colv;
    const uint32_t stride = gridDim.x * blockDim.x;
    const AffineQuick aq = affine_quick_of(AFF ? E.aff_scale : 1.0f, E.aff_kind, E.aff_zero);
    constexpr int UNR = AFF ? 1 : 2; // (1024 threads a block: 64 registers each, which the codes' arithmetic fills)
    for (uint32_t idx0 = blockIdx.x * blockDim.x + threadIdx.x; idx0 < total; idx0 += stride * UNR) {
        uint4 a[UNR], b[UNR];
        int64_t oo[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const uint32_t idx = idx0 + u * stride;
            b[u] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < total) {
                uint32_t r = 0, c = idx * 8u;
                if (E.rows != 1) { r = idx / E.colv; c = (idx - r * E.colv) * 8u; }
                a[u] = *reinterpret_cast<const uint4 *>((const uint16_t *)E.in[0] + (int64_t)r * E.rs[0] + c);
                if (MUL) b[u] = *reinterpret_cast<const uint4 *>((const uint16_t *)E.in[1] + (int64_t)r * E.rs[1] + c);
                oo[u] = (int64_t)r * E.ors + c;
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (idx0 + u * stride >= total) break;
            const uint32_t w[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
            const uint32_t v[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
            uint32_t o[4];
            float val[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t lo = s_table[w[q] & 0xffffu], hi = s_table[w[q] >> 16];
                if (MUL && AFF) {
                    val[2 * q] = __fmul_rn(bits_f32(lo << 16), bits_f32(v[q] << 16));
                    val[2 * q + 1] = __fmul_rn(bits_f32(hi << 16), bits_f32(v[q] & 0xffff0000u));
                }
                else if (MUL) o[q] = pack_bf16x2(__fmul_rn(bits_f32(lo << 16), bits_f32(v[q] << 16)), __fmul_rn(bits_f32(hi << 16), bits_f32(v[q] & 0xffff0000u)));
                else o[q] = lo | (hi << 16);
            }
            if (MUL && AFF) {
                int code[8];
                uint32_t unsure = 0;
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    bool un;
                    code[t] = affine_code_try(val[t], aq, un);
                    unsure |= un ? (1u << t) : 0u;
                }
                if (unsure) {
#pragma unroll
                    for (int t = 0; t < 8; ++t)
                        if ((unsure >> t) & 1u) code[t] = affine_code_exact(val[t], aq.kind, aq.scale, aq.zero);
                }
                uint32_t lo4 = 0, hi4 = 0;
#pragma unroll
                for (int t = 0; t < 4; ++t) { lo4 |= ((uint32_t)code[t] & 0xffu) << (8 * t); hi4 |= ((uint32_t)code[4 + t] & 0xffu) << (8 * t); }
                *reinterpret_cast<uint2 *>((uint8_t *)E.out + oo[u]) = make_uint2(lo4, hi4);
            } else {
                *reinterpret_cast<uint4 *>((uint16_t *)E.out + oo[u]) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// PSK_OP_ROPE for bf16: a thread takes eight rotary positions of one row and
// writes both halves, so x is read once and the result written once, both as
// whole contiguous rows. Products are rounded to f32 before they are added
// (no fused multiply-add), the sums rounded once to bf16.
// ---------------------------------------------------------------------------
struct RopeParams {
    const uint16_t *x, *c, *s;
    uint16_t *out;
    int64_t rows;      // every leading axis and seq
    int32_t seq, rotv; // rotv = rot / 8
};

__global__ void __launch_bounds__(256, 4) k_rope_bf16(const __grid_constant__ RopeParams P)
{
    const int64_t total = P.rows * P.rotv;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int rot = P.rotv * 8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / P.rotv;
        const int cv = (int)(idx - row * P.rotv) * 8;
        const int t = (int)(row % P.seq);
        const uint16_t *xr = P.x + row * 2 * rot + cv;
        const uint4 a = *reinterpret_cast<const uint4 *>(xr), b = *reinterpret_cast<const uint4 *>(xr + rot);
        const uint4 c = *reinterpret_cast<const uint4 *>(P.c + (int64_t)t * rot + cv), s = *reinterpret_cast<const uint4 *>(P.s + (int64_t)t * rot + cv);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w}, cw[4] = {c.x, c.y, c.z, c.w}, sw[4] = {s.x, s.y, s.z, s.w};
        uint32_t o0[4], o1[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float a0 = bits_f32(aw[q] << 16), a1 = bits_f32(aw[q] & 0xffff0000u), b0 = bits_f32(bw[q] << 16), b1 = bits_f32(bw[q] & 0xffff0000u);
            const float c0 = bits_f32(cw[q] << 16), c1 = bits_f32(cw[q] & 0xffff0000u), s0 = bits_f32(sw[q] << 16), s1 = bits_f32(sw[q] & 0xffff0000u);
            o0[q] = pack_bf16x2_hw(__fsub_rn(__fmul_rn(a0, c0), __fmul_rn(b0, s0)), __fsub_rn(__fmul_rn(a1, c1), __fmul_rn(b1, s1)));
            o1[q] = pack_bf16x2_hw(__fadd_rn(__fmul_rn(b0, c0), __fmul_rn(a0, s0)), __fadd_rn(__fmul_rn(b1, c1), __fmul_rn(a1, s1)));
        }
        uint16_t *orow = P.out + row * 2 * rot + cv;
        *reinterpret_cast<uint4 *>(orow) = make_uint4(o0[0], o0[1], o0[2], o0[3]);
        *reinterpret_cast<uint4 *>(orow + rot) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    }
}

// ---------------------------------------------------------------------------
// PSK_OP_RMSNORM under PSK_ORDER_DEVICE, bf16 rows: a warp a row, the row read
// once into registers. The bits are those of the four launches it stands for,
// as this executor runs them under the same order:
//   x*x rounded to bf16 (the square's site);
//   their f32 sum in k_reduce_rows_tree's grouping (lane l adds the elements of
//   vectors l, l+32, .. in index order, then the xor tree), divided by n;
//   sqrt(mean + eps) in f32, rounded to bf16 at the last group's edge;
//   x / root * gamma, the division by the root's correctly rounded reciprocal
//   with one correction (k_ew_prog's), rounded to bf16.
// NV = vectors of eight a lane = n / 256.
// ---------------------------------------------------------------------------
struct RmsParams {
    const uint16_t *x, *gamma;
    const void *eps;
    uint16_t *out;          // bf16 numbers, or (AFF) one-byte codes of an affine format
    int64_t x_row, out_row; // element strides from row to row
    int64_t rows;
    int32_t n, eps_dtype;
    int32_t aff_kind, aff_zero; // AFF: 1 i8, 2 u8; the zero point
    float aff_scale;
};

// AFF: the result's site is stored in an affine format (a `scaled` site feeding an integer-sum contraction): the
// f32 value the last group computes goes straight into its code, as the generic group's store does.
template <int NV, bool AFF = false>
__global__ void __launch_bounds__(256, AFF ? 3 : 4) k_rmsnorm_rows(const __grid_constant__ RmsParams P)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const float eps = load_real(P.eps, P.eps_dtype, 0); // widened exactly: the root's group computes in f32
    const float nf = (float)(double)P.n;
    // vectors loaded before any is used: in the second pass the codes' arithmetic needs the registers (one vector at a
    // time there keeps the kernel free of spills); the first pass, which is the one that waits for memory, has room for eight
    constexpr int G = AFF ? 1 : (NV < 4 ? NV : 4);
    constexpr int G1 = AFF ? (NV < 8 ? NV : 8) : G;
    for (int64_t row = warp; row < P.rows; row += nwarps) {
        const uint16_t *xr = P.x + row * P.x_row + lane * 8;
        // pass 1: the sum of the rounded squares, vector by vector in index order. The row is not kept in
        // registers (that would leave one block an SM); the second pass finds it in the L1 or the L2.
        float acc = 0.0f;
#pragma unroll 1
        for (int j0 = 0; j0 < NV; j0 += G1) {
            uint4 v[G1];
#pragma unroll
            for (int j = 0; j < G1; ++j) v[j] = *reinterpret_cast<const uint4 *>(xr + (j0 + j) * 256);
#pragma unroll
            for (int j = 0; j < G1; ++j) {
                const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float lo = bits_f32(w[q] << 16), hi = bits_f32(w[q] & 0xffff0000u);
                    const uint32_t sq = pack_bf16x2_hw(__fmul_rn(lo, lo), __fmul_rn(hi, hi));
                    acc = __fadd_rn(acc, bits_f32(sq << 16));
                    acc = __fadd_rn(acc, bits_f32(sq & 0xffff0000u));
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
        const float ms = __fdiv_rn(acc, nf);
        const float root = bits_f32(pack_bf16x2_hw(__fsqrt_rn(__fadd_rn(ms, eps)), 0.0f) << 16);
        const float rr = __frcp_rn(root);
        const bool ok = div_by_in_range(root);
        uint16_t *orow = P.out + row * P.out_row + lane * 8;
        uint8_t *crow = reinterpret_cast<uint8_t *>(P.out) + row * P.out_row + lane * 8;
        const AffineQuick aq = affine_quick_of(AFF ? P.aff_scale : 1.0f, P.aff_kind, P.aff_zero);
        const uint16_t *gr = P.gamma + lane * 8;
#pragma unroll 1
        for (int j0 = 0; j0 < NV; j0 += G) {
            uint4 v[G], g[G];
#pragma unroll
            for (int j = 0; j < G; ++j) {
                v[j] = *reinterpret_cast<const uint4 *>(xr + (j0 + j) * 256);
                g[j] = *reinterpret_cast<const uint4 *>(gr + (j0 + j) * 256);
            }
#pragma unroll
            for (int j = 0; j < G; ++j) {
                const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
                const uint32_t gw[4] = {g[j].x, g[j].y, g[j].z, g[j].w};
                uint32_t o[4];
                float val[8];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float lo = div_by_checked(bits_f32(w[q] << 16), root, rr, ok), hi = div_by_checked(bits_f32(w[q] & 0xffff0000u), root, rr, ok);
                    val[2 * q] = __fmul_rn(lo, bits_f32(gw[q] << 16));
                    val[2 * q + 1] = __fmul_rn(hi, bits_f32(gw[q] & 0xffff0000u));
                    if (!AFF) o[q] = pack_bf16x2_hw(val[2 * q], val[2 * q + 1]);
                }
                if (AFF) {
                    // the eight codes without a branch, then the uncertain ones (rare) the exact way
                    int code[8];
                    uint32_t unsure = 0;
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        bool u;
                        code[t] = affine_code_try(val[t], aq, u);
                        unsure |= u ? (1u << t) : 0u;
                    }
                    if (unsure) {
#pragma unroll
                        for (int t = 0; t < 8; ++t)
                            if ((unsure >> t) & 1u) code[t] = affine_code_exact(val[t], aq.kind, aq.scale, aq.zero);
                    }
                    uint32_t lo4 = 0, hi4 = 0;
#pragma unroll
                    for (int t = 0; t < 4; ++t) { lo4 |= ((uint32_t)code[t] & 0xffu) << (8 * t); hi4 |= ((uint32_t)code[4 + t] & 0xffu) << (8 * t); }
                    *reinterpret_cast<uint2 *>(crow + (j0 + j) * 256) = make_uint2(lo4, hi4);
                } else {
                    *reinterpret_cast<uint4 *>(orow + (j0 + j) * 256) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Softmax over a contiguous axis under PSK_ORDER_DEVICE: a warp a row, the
// row held in shared memory between the passes, the exponentials computed
// once (the bits of computing them twice), the maximum and the sum shuffle
// trees. With the causal mask only the allowed prefix of a row is read or
// exponentiated; the refused tail is written as zeros, which is what the
// reference's selections give it (lower.rs:1368-1419).
// ---------------------------------------------------------------------------
// The division by the row's sum is `div_by` above.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 6) k_softmax_rows_smem(const __grid_constant__ DevLaunch L)
{
    extern __shared__ float s_rows[];
    uint32_t ovf = 0;
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int64_t n = L.inner;
    float *row = s_rows + (int64_t)wib * n;
    const int64_t nwarps = (int64_t)gridDim.x * WARPS;
    const uint32_t nv = (uint32_t)(n / 8);
    const bool causal = L.masked && L.iparam[0] == 1;
    const bool general_mask = L.masked && !causal;
    const bool bf16_io = L.in[0].dtype == PSK_BF16 && L.kdtype == PSK_BF16 && L.out.dtype == PSK_BF16;
    // iparam[2] = 1: the rows lie one after the other in the input and in the output, and under the
    // causal mask row r is position r mod iparam[3] of its sequence: no index arithmetic a row
    const bool flat = L.iparam[2] == 1;
    for (int64_t r = (int64_t)blockIdx.x * WARPS + wib; r < L.total; r += nwarps) {
        int64_t base, obase, mbase = 0, ms = 0;
        if (flat) {
            base = obase = r * n;
            if (causal) mbase = (int64_t)((uint32_t)r % (uint32_t)L.iparam[3]);
        } else {
            base = operand_offset(L.in[0], L.dims, 0, L.n_outer, r);
            obase = operand_offset(L.out, L.dims, 0, L.n_outer, r);
            if (L.masked) {
                mbase = operand_offset(L.in[1], L.dims, 0, L.n_outer, r);
                ms = L.in[1].stride[L.n_outer];
                if (causal) mbase = mbase / L.iparam[1];
            }
        }
        // under the causal mask the allowed elements are 0 .. count-1
        const uint32_t count = causal ? (uint32_t)min(n, mbase + 1) : (uint32_t)n;
        const uint32_t live = (count + 7u) / 8u;
        // pass 1: the row into shared memory as f32 (a refused element as -inf), and its maximum
        float m = -INFINITY;
        if (bf16_io && nv <= 256) {
            uint4 raw[8];
            const uint16_t *src = (const uint16_t *)L.in[0].p + base;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t v = lane + 32u * j;
                if (v < live) raw[j] = *reinterpret_cast<const uint4 *>(src + (size_t)v * 8);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t v = lane + 32u * j;
                if (v < live) {
                    const uint4 w = raw[j];
                    float x[8] = {bits_f32(w.x << 16), bits_f32(w.x & 0xffff0000u), bits_f32(w.y << 16), bits_f32(w.y & 0xffff0000u),
                                  bits_f32(w.z << 16), bits_f32(w.z & 0xffff0000u), bits_f32(w.w << 16), bits_f32(w.w & 0xffff0000u)};
                    if (v * 8u + 8u > count || general_mask) {
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const bool ok = v * 8u + t < count && (!general_mask || mask_allows(L, mbase, (int64_t)v * 8 + t, ms));
                            if (!ok) x[t] = -INFINITY;
                        }
                    }
#pragma unroll
                    for (int t = 0; t < 8; ++t) m = fmaxf(m, x[t]);
                    float4 *dst = reinterpret_cast<float4 *>(row + v * 8);
                    dst[0] = make_float4(x[0], x[1], x[2], x[3]);
                    dst[1] = make_float4(x[4], x[5], x[6], x[7]);
                }
            }
        } else {
            for (uint32_t v = lane; v < live; v += 32) {
                float x[8];
                ew_load8(L.in[0].p, L.in[0].dtype, base + (int64_t)v * 8, 1, L.kdtype, x, &ovf);
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const bool ok = v * 8u + t < count && (!general_mask || mask_allows(L, mbase, (int64_t)v * 8 + t, ms));
                    if (!ok) x[t] = -INFINITY;
                    m = fmaxf(m, x[t]);
                }
                float4 *dst = reinterpret_cast<float4 *>(row + v * 8);
                dst[0] = make_float4(x[0], x[1], x[2], x[3]);
                dst[1] = make_float4(x[4], x[5], x[6], x[7]);
            }
        }
        m = warp_max(m);
        __syncwarp();
        // pass 2: one element a lane a turn, consecutive lanes on consecutive words. A refused element
        // holds -inf: it adds 0 and gives 0, as the reference's selections do.
        float z = 0.0f;
        const uint32_t padded = live * 8u;
#pragma unroll 4
        for (uint32_t k = lane; k < padded; k += 32) {
            const float x = row[k];
            float e = 0.0f;
            if (x != -INFINITY) e = lm_expf(__fsub_rn(x, m));
            row[k] = e;
            z += e;
        }
        z = warp_sum(z);
        __syncwarp();
        // pass 3: e / z, eight a lane, stored as whole vectors; zeros past the allowed prefix
        const float rz = __frcp_rn(z);
        for (uint32_t v = lane; v < nv; v += 32) {
            float y[8];
            if (v < live) {
                const float4 *p = reinterpret_cast<const float4 *>(row + v * 8);
                const float4 a = p[0], b = p[1];
                const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int t = 0; t < 8; ++t) y[t] = x[t] == 0.0f ? 0.0f : div_by(x[t], z, rz);
            } else {
#pragma unroll
                for (int t = 0; t < 8; ++t) y[t] = 0.0f;
            }
            ovf |= ew_store8(const_cast<void *>(L.out.p), L.out.dtype, obase + (int64_t)v * 8, y);
        }
        __syncwarp();
    }
    if (L.guarded && ovf) atomicOr(L.ovf, 1u);
}

} // namespace psk
