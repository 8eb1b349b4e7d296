// PSK_OP_ATTENTION for one query position against a cache of keys and values (the decode step after a prefill):
// q [batch, groups, per, 1, 128], k [batch, groups, seq2, 128], v [batch, seq2, groups, 128], no mask, bf16
// everywhere. The four launches it stands for (scores, their division by the root, the softmax over seq2, the
// weighted sum of the values) keep their roundings: every score, scaled score and normalised weight is rounded to
// bf16 where the separate launches would have stored it, the exponential is the executor's own, and the sums run in
// binary32. Only the ORDER of the three sums differs from index order (the declared device order): a score is summed
// four elements a lane and then across the warp, the denominator and the values' sum a warp a stride of positions.
//
// The work is a stream of the cache: 2 · seq2 · 256 bytes a head, nothing reused, so the kernel is bound by HBM and
// needs no tensor core: one CTA a (batch entry, query head), a warp a key position, eight bytes a lane. The scores
// of a head stay in shared memory (4 bytes a position).
#pragma once
#include "psk_attn.cuh"
#include "psk_kernels.cuh"

namespace psk {
namespace attn_step {

constexpr int THREADS = 256, WARPS = THREADS / 32, HD = 128;

struct Params {
    const uint16_t *q, *k, *v;
    uint16_t *out;
    int64_t q_b, q_g, q_p;  // element strides of q over batch, group and query-of-the-group
    int64_t k_b, k_g, k_t;  // of k over batch, group and position
    int64_t v_b, v_g, v_t;
    int64_t o_b, o_g, o_p;
    int32_t G, Pn, len;
    const void *rt;
    int32_t rt_dtype;
    int32_t aff_kind, aff_zero; // the result as one-byte codes of an affine format (kind 1 i8, 2 u8; 0: bf16)
    float aff_scale;
};

PSK_DEV void unpack4(uint2 w, float *f)
{
    f[0] = bits_f32(w.x << 16);
    f[1] = bits_f32(w.x & 0xffff0000u);
    f[2] = bits_f32(w.y << 16);
    f[3] = bits_f32(w.y & 0xffff0000u);
}

__global__ void __launch_bounds__(THREADS) k_attn_step(const __grid_constant__ Params P)
{
    extern __shared__ float sc[]; // the head's scores, then its exponentials
    __shared__ float red[32];
    __shared__ float part[WARPS][HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t head = blockIdx.x;
    const int64_t p = head % P.Pn, g = (head / P.Pn) % P.G, b = head / ((int64_t)P.Pn * P.G);
    const float rtv = attn::bf16_round(load_real(P.rt, P.rt_dtype, 0)); // the division's kernel is bf16: it reads the root rounded at its edge

    float qv[4];
    unpack4(*reinterpret_cast<const uint2 *>(P.q + b * P.q_b + g * P.q_g + p * P.q_p + 4 * lane), qv);
    const uint16_t *kb = P.k + b * P.k_b + g * P.k_g + 4 * lane;
    const uint16_t *vb = P.v + b * P.v_b + g * P.v_g + 4 * lane;

    // scores: a warp a position, eight positions in flight a warp
    for (int t0 = warp * 8; t0 < P.len; t0 += WARPS * 8) {
        uint2 kw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) kw[j] = t0 + j < P.len ? *reinterpret_cast<const uint2 *>(kb + (int64_t)(t0 + j) * P.k_t) : make_uint2(0u, 0u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float kf[4];
            unpack4(kw[j], kf);
            float s = __fadd_rn(__fadd_rn(__fmul_rn(qv[0], kf[0]), __fmul_rn(qv[1], kf[1])), __fadd_rn(__fmul_rn(qv[2], kf[2]), __fmul_rn(qv[3], kf[3])));
            s = warp_sum(s);
            if (lane == 0 && t0 + j < P.len) sc[t0 + j] = attn::bf16_round(__fdiv_rn(attn::bf16_round(s), rtv));
        }
    }
    __syncthreads();

    // the softmax over the positions: maximum, exponentials, their sum
    float m = -INFINITY;
    for (int t = threadIdx.x; t < P.len; t += THREADS) m = fmaxf(m, sc[t]);
    m = block_reduce<true>(m, red);
    float z = 0.0f;
    for (int t = threadIdx.x; t < P.len; t += THREADS) {
        const float e = lm_expf(__fsub_rn(sc[t], m));
        sc[t] = e;
        z = __fadd_rn(z, e);
    }
    z = block_reduce<false>(z, red);
    __syncthreads();
    // the weights, rounded to bf16 as the softmax's site stores them: one division a position (not one a lane)
    for (int t = threadIdx.x; t < P.len; t += THREADS) sc[t] = attn::bf16_round(__fdiv_rn(sc[t], z));
    __syncthreads();

    // the values: a warp a position again, eight positions in flight a warp
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int t0 = warp * 8; t0 < P.len; t0 += WARPS * 8) {
        uint2 vw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) vw[j] = t0 + j < P.len ? *reinterpret_cast<const uint2 *>(vb + (int64_t)(t0 + j) * P.v_t) : make_uint2(0u, 0u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (t0 + j >= P.len) break;
            const float w = sc[t0 + j];
            float vf[4];
            unpack4(vw[j], vf);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(w, vf[i]));
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) part[warp][4 * lane + i] = acc[i];
    __syncthreads();
    if (threadIdx.x < HD) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s = __fadd_rn(s, part[w][threadIdx.x]);
        const int64_t o = b * P.o_b + g * P.o_g + p * P.o_p + threadIdx.x;
        if (P.aff_kind) ((uint8_t *)P.out)[o] = (uint8_t)affine_code_quick(s, affine_quick_of(P.aff_scale, P.aff_kind, P.aff_zero)); // the binary32 sum's code, as the separate launch stores it
        else P.out[o] = f32_to_bf16(s);
    }
}

} // namespace attn_step
} // namespace psk
