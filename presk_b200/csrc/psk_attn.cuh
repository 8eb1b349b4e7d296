// Blockwise causal attention for sm_100a: scores, scaling, masked softmax and
// the product with the values in one kernel, the scores never in memory.
//
// What it replaces: the launches `ein[.., seq, seq2](q*k)`, `div` by sqrt(hd),
// `softmax axis seq2 where mask`, `ein[.., seq, .., hd](a*v)` of an attention
// function (examples/coverage/llama.psk:100-102), each of which the reference
// runs as its own nest with its result stored in memory. It is used only under
// the declared order "device" with `"attention": "blockwise"`, since it is a
// different realization and not only a reordering of sums:
//   - a score is rounded to bf16, divided by the root and rounded to bf16
//     again, exactly as the two stored sites would hold it (the quotient of
//     two bf16 numbers rounds to the same bf16 number whether it is computed by
//     a division or by the correctly rounded reciprocal; see the kernel);
//   - the row's maximum is taken over those values in a first pass over the
//     key blocks, so the exponentials have the reference's arguments;
//   - exp is the hardware's ex2 (relative error about 2^-22), the row's sum is
//     accumulated block by block in f32, the unnormalised exponentials are
//     rounded to bf16 for the second product and the quotient by the sum is
//     taken once at the end, where the reference rounds exp/sum to bf16 first.
// The result agrees with the unfused sequence to about a bf16 unit in the last
// place of the output (tests state the tolerance).
//
// One CTA per (batch, head, block of 128 queries), 576 threads: warp 0 loads Q
// once and K, V blocks through rings with TMA; warp 1 issues tcgen05.mma for
// S = Q·K^T (into one of two 128-column accumulators) and O += P·V; warps 2-17
// do the softmax, four warps to a quadrant of tensor memory: a thread holds one
// query row (its TMEM lane) and 32 of a block's 128 keys, so a row's maximum
// and sum are exchanged between four threads once a pass, through shared
// memory. P is double-buffered, so the exponentials of block i+1 are computed
// while the tensor core multiplies block i. Head dimension 128, bf16 in and
// out, sequence a multiple of 128. Every wait on an mbarrier is bounded as in
// psk_gemm_tc.cuh; the two named barriers among the softmax warps are reached
// by every one of them whether or not a wait has run out.
#pragma once
#include "psk_gemm_tc.cuh"
#include "psk_hot.cuh"

namespace psk {
namespace attn {

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int SOFTMAX_WARPS = 16;     // four to a quadrant of tensor memory, each 32 of a block's 128 keys
constexpr int THREADS = (2 + SOFTMAX_WARPS) * 32;
constexpr int TILE = 128 * 128 * 2;   // a 128 x 128 bf16 tile: two 16 KB halves of 64 columns
constexpr int HALF = 128 * 64 * 2;
constexpr int SMEM_TILES = 7 * TILE;  // Q, K x2, V x2, P x2
constexpr int SMEM_TOTAL = SMEM_TILES + 256 + 1024;

struct Params {
    int64_t T;
    int32_t causal;
    int32_t per; // query heads to a key/value head
    void *out;
    int64_t o_b, o_g, o_t; // element strides of the output over batch, head, query (hd is contiguous)
    const void *rt;        // the divisor, a rank-0 tensor
    int32_t rt_dtype;
    uint32_t *status;
    int32_t aff_kind, aff_zero; // k_attn_fwd3 only: the result as one-byte codes of an affine format (kind 1 i8, 2 u8; 0: bf16)
    float aff_scale;
};

PSK_DEV float bf16_round(float x) { return bits_f32(pack_bf16x2_hw(x, 0.0f) << 16); }

PSK_DEV float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

PSK_DEV void softmax_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1) k_attn_fwd(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __grid_constant__ Params P)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sK = smem + TILE, *sV = smem + 3 * TILE, *sP = smem + 5 * TILE;
    uint64_t *bars = (uint64_t *)(smem + SMEM_TILES);
    // 0 q_full; 1,2 k_full; 3,4 k_empty; 5,6 v_full; 7,8 v_empty; 9,10 s_full; 11,12 s_free;
    // 13,14 p_full; 15,16 p_free; 17 o_full
    uint32_t *tmem_slot = (uint32_t *)(bars + 18);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    const uint32_t bar0 = tc::smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nqb = (int)(P.T / BM);
    const int qb = nqb - 1 - (int)blockIdx.x; // the longest rows first
    const int g = blockIdx.y, b = blockIdx.z;
    const int gk = g / P.per; // the key/value head this query head reads
    const int nkb = P.causal ? qb + 1 : nqb;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 18; ++i) {
            uint32_t count = 1;
            if (i >= 11 && i <= 14) count = SOFTMAX_WARPS; // s_free, p_full: one arrival a softmax warp
            tc::mbar_init(bar(i), count);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS0 = tmem, tO = tmem + 256;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            tc::mbar_expect_tx(bar(0), TILE);
            tc::tma_load_4d(tc::smem_u32(sQ), &map_q, bar(0), 0, qb * BM, g, b);
            tc::tma_load_4d(tc::smem_u32(sQ + HALF), &map_q, bar(0), 64, qb * BM, g, b);
            uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
            for (int pass = 0; pass < 2 && ok; ++pass)
                for (int kb = 0; kb < nkb && ok; ++kb) {
                    ok = tc::mbar_wait(bar(3 + ks), kph ^ 1u, abort_flag, P.status, 0x11u);
                    if (!ok) break;
                    tc::mbar_expect_tx(bar(1 + ks), TILE);
                    tc::tma_load_4d(tc::smem_u32(sK + ks * TILE), &map_k, bar(1 + ks), 0, kb * BN, gk, b);
                    tc::tma_load_4d(tc::smem_u32(sK + ks * TILE + HALF), &map_k, bar(1 + ks), 64, kb * BN, gk, b);
                    if (++ks == 2) { ks = 0; kph ^= 1u; }
                    if (pass == 1) {
                        ok = tc::mbar_wait(bar(7 + vs), vph ^ 1u, abort_flag, P.status, 0x12u);
                        if (!ok) break;
                        tc::mbar_expect_tx(bar(5 + vs), TILE);
                        tc::tma_load_4d(tc::smem_u32(sV + vs * TILE), &map_v, bar(5 + vs), 0, kb * BN, gk, b);
                        tc::tma_load_4d(tc::smem_u32(sV + vs * TILE + HALF), &map_v, bar(5 + vs), 64, kb * BN, gk, b);
                        if (++vs == 2) { vs = 0; vph ^= 1u; }
                    }
                }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = tc::instr_desc(0, 0, BN), idesc_pv = tc::instr_desc(0, 1, HD);
            bool ok = tc::mbar_wait(bar(0), 0u, abort_flag, P.status, 0x21u);
            uint32_t ks = 0, kph = 0, vs = 0, vph = 0, qk_count = 0;
            auto issue_qk = [&]() -> bool {
                const uint32_t sb = qk_count & 1u, sph = (qk_count >> 1) & 1u;
                if (!tc::mbar_wait(bar(1 + ks), kph, abort_flag, P.status, 0x22u)) return false;
                if (!tc::mbar_wait(bar(11 + sb), sph ^ 1u, abort_flag, P.status, 0x23u)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t qa = tc::smem_u32(sQ), ka = tc::smem_u32(sK + ks * TILE);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t off = (uint32_t)(kk >> 2) * HALF + (uint32_t)(kk & 3) * 32u;
                    tc::umma(tS0 + sb * 128u, tc::smem_desc(qa + off, 16, 1024), tc::smem_desc(ka + off, 16, 1024), idesc_qk, kk != 0 ? 1u : 0u);
                }
                tc::umma_commit(bar(3 + ks));  // the K block is free once these have read it
                tc::umma_commit(bar(9 + sb));  // S is there
                if (++ks == 2) { ks = 0; kph ^= 1u; }
                ++qk_count;
                return true;
            };
            // pass 1: the scores only, for the rows' maxima
            for (int kb = 0; kb < nkb && ok; ++kb) ok = issue_qk();
            // pass 2: scores of block kb+1 are issued before the product of block kb waits for P
            if (ok) ok = issue_qk();
            for (int kb = 0; kb < nkb && ok; ++kb) {
                if (kb + 1 < nkb) ok = issue_qk();
                if (!ok) break;
                const uint32_t pb = (uint32_t)kb & 1u, pph = ((uint32_t)kb >> 1) & 1u;
                ok = tc::mbar_wait(bar(13 + pb), pph, abort_flag, P.status, 0x24u);
                if (!ok) break;
                ok = tc::mbar_wait(bar(5 + vs), vph, abort_flag, P.status, 0x25u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t pa = tc::smem_u32(sP + pb * TILE), va = tc::smem_u32(sV + vs * TILE);
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint32_t aoff = (uint32_t)(kk >> 2) * HALF + (uint32_t)(kk & 3) * 32u;
                    tc::umma(tO, tc::smem_desc(pa + aoff, 16, 1024), tc::smem_desc(va + (uint32_t)kk * 2048u, HALF, 1024), idesc_pv, (kb | kk) != 0 ? 1u : 0u);
                }
                tc::umma_commit(bar(7 + vs));  // the V block is free
                tc::umma_commit(bar(15 + pb)); // and this P may be overwritten
                if (++vs == 2) { vs = 0; vph ^= 1u; }
            }
            if (ok) tc::umma_commit(bar(17));
        }
    } else {
        const int quad = warp & 3;            // the tensor-memory lanes this warp may read: 32·quad ..
        const int cq = (warp - 2) >> 2;       // its quarter of a block's keys, and of the output's columns
        const int row = quad * 32 + lane;     // this thread's query within the block
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float rtv = bf16_round(load_real(P.rt, P.rt_dtype, 0)); // the division's kernel is bf16: it reads rt rounded to bf16 at its edge
        const float rr = __frcp_rn(rtv);
        float *xch = reinterpret_cast<float *>(sP); // the P tiles are idle whenever the warps exchange a row's parts
        bool ok = true;
        uint32_t qk_count = 0;
        // ---- pass 1: the greatest and the least raw score of the row ------------------
        // bf16(bf16(S) / rt) is monotone in S, so the row's maximum of the stored scaled scores is that
        // function of the greatest raw score (of the least, if rt is negative).
        // rt > 0 (a root): only the greatest raw score matters; otherwise only the least. One comparison an element.
        const bool want_max = !(rtv < 0.0f);
        float ext = want_max ? -INFINITY : INFINITY;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const uint32_t sb = qk_count & 1u, sph = (qk_count >> 1) & 1u;
            ok = tc::mbar_wait(bar(9 + sb), sph, abort_flag, P.status, 0x31u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t v[32];
            tc::tmem_ld32(tS0 + lane_base + sb * 128u + (uint32_t)(cq * 32), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(11 + sb)); // the scores are in registers
            ++qk_count;
            const int allowed = (P.causal && kb == qb) ? row - cq * 32 : 31; // the last allowed key of these 32
            if (want_max) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i <= allowed) ext = fmaxf(ext, __uint_as_float(v[i]));
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i <= allowed) ext = fminf(ext, __uint_as_float(v[i]));
            }
        }
        xch[cq * 128 + row] = ext;
        softmax_sync();
#pragma unroll
        for (int c = 0; c < 4; ++c) ext = want_max ? fmaxf(ext, xch[c * 128 + row]) : fminf(ext, xch[c * 128 + row]);
        softmax_sync(); // before the first P is written over the exchange
        const float m = bf16_round(__fdiv_rn(bf16_round(ext), rtv));
        // ---- pass 2: exponentials, the row's sum, P for the second product --------------
        const float LOG2E = 1.44269504f;
        const float m2 = __fmul_rn(m, LOG2E);
        float z = 0.0f;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const uint32_t sb = qk_count & 1u, sph = (qk_count >> 1) & 1u;
            ok = tc::mbar_wait(bar(9 + sb), sph, abort_flag, P.status, 0x32u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t v[32];
            tc::tmem_ld32(tS0 + lane_base + sb * 128u + (uint32_t)(cq * 32), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(11 + sb));
            ++qk_count;
            const bool diag = P.causal && kb == qb;
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                // the two stored sites: bf16(S), then bf16(bf16(S) / rt). With a and rt both bf16 numbers the
                // quotient is never within 2^-17 (relative) of the midpoint of two bf16 numbers without being one of
                // them, and it cannot be such a midpoint (an odd 9-bit significand times rt's has more than a's 8
                // bits), so a·RN(1/rt), which is within 2^-23 of a/rt, rounds to the same bf16 number as a/rt.
                const uint32_t s1 = pack_bf16x2_hw(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                const float d0 = __fmul_rn(bits_f32(s1 << 16), rr), d1 = __fmul_rn(bits_f32(s1 & 0xffff0000u), rr);
                const uint32_t s2 = pack_bf16x2_hw(d0, d1);
                float e0 = fast_exp2(__fmaf_rn(bits_f32(s2 << 16), LOG2E, -m2));
                float e1 = fast_exp2(__fmaf_rn(bits_f32(s2 & 0xffff0000u), LOG2E, -m2));
                if (diag) {
                    if (cq * 32 + 2 * i > row) e0 = 0.0f;
                    if (cq * 32 + 2 * i + 1 > row) e1 = 0.0f;
                }
                z += e0;
                z += e1;
                packed[i] = pack_bf16x2_hw(e0, e1);
            }
            // P of two blocks before must have been read by its product
            const uint32_t pb = (uint32_t)kb & 1u, pph = ((uint32_t)kb >> 1) & 1u;
            ok = tc::mbar_wait(bar(15 + pb), pph ^ 1u, abort_flag, P.status, 0x33u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            // keys cq*32 .. +31 of this row: half (cq / 2), 16-byte units (cq % 2) * 4 .. +3, swizzled by the row
            uint8_t *dst = sP + pb * TILE + (cq >> 1) * HALF + row * 128;
            const int u0 = (cq & 1) * 4;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                *reinterpret_cast<uint4 *>(dst + (((u0 + u) ^ (row & 7)) << 4)) = make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the tensor core reads P through the async proxy
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(13 + pb));
        }
        if (ok) {
            ok = tc::mbar_wait(bar(17), 0u, abort_flag, P.status, 0x34u); // every product is done: P is idle again
            ok = __all_sync(0xffffffffu, ok);
        }
        xch[cq * 128 + row] = z;
        softmax_sync();
        z = __fadd_rn(__fadd_rn(xch[row], xch[128 + row]), __fadd_rn(xch[256 + row], xch[384 + row]));
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t t = (int64_t)qb * BM + row;
            uint16_t *orow = (uint16_t *)P.out + (int64_t)b * P.o_b + (int64_t)g * P.o_g + t * P.o_t + cq * 32;
            uint32_t v[32];
            tc::tmem_ld32(tO + lane_base + (uint32_t)(cq * 32), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const float rz = __frcp_rn(z);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    w[i] = pack_bf16x2_hw(div_by(__uint_as_float(v[u * 8 + 2 * i]), z, rz), div_by(__uint_as_float(v[u * 8 + 2 * i + 1]), z, rz));
                *reinterpret_cast<uint4 *>(orow + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}


// ---------------------------------------------------------------------------
// The same computation with key blocks of 64 and half the threads, sized so that two CTAs share an SM (96 KB of
// shared memory, 256 tensor-memory columns, 320 threads each): while one CTA waits (for its first tiles, for a
// product, at its end), the other computes. K and V blocks travel through one ring of three 16 KB stages in the
// order the products use them; P is single-buffered; a row is held by two threads (32 of a block's 64 keys each).
// ---------------------------------------------------------------------------
namespace v2 {
constexpr int BN2 = 64;
constexpr int SOFTMAX_WARPS2 = 8;
constexpr int THREADS2 = (2 + SOFTMAX_WARPS2) * 32;
constexpr int KV_STAGE = BN2 * HD * 2;        // 16 KB: two halves of [64 keys x 64 hd]
constexpr int KV_HALF = BN2 * 64 * 2;         // 8 KB
constexpr int RING = 3;
constexpr int P_BYTES = BM * BN2 * 2;         // 16 KB: [128 rows x 64 keys]
constexpr int SMEM_TILES2 = TILE + RING * KV_STAGE + P_BYTES;
constexpr int SMEM_TOTAL2 = SMEM_TILES2 + 256 + 1024;

PSK_DEV void softmax_sync2()
{
    asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS2 * 32) : "memory");
}

__global__ void __launch_bounds__(THREADS2, 2) k_attn_fwd2(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __grid_constant__ Params P)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sR = smem + TILE, *sP = smem + TILE + RING * KV_STAGE;
    uint64_t *bars = (uint64_t *)(smem + SMEM_TILES2);
    // 0 q_full; 1..3 ring full; 4..6 ring empty; 7,8 s_full; 9,10 s_free; 11 p_full; 12 p_free; 13 o_full
    uint32_t *tmem_slot = (uint32_t *)(bars + 14);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    const uint32_t bar0 = tc::smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nqb = (int)(P.T / BM);
    const int qb = nqb - 1 - (int)blockIdx.x; // the longest rows first
    const int g = blockIdx.y, b = blockIdx.z;
    const int gk = g / P.per;
    const int nkb = P.causal ? 2 * (qb + 1) : (int)(P.T / BN2);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 14; ++i) tc::mbar_init(bar(i), (i == 9 || i == 10 || i == 11) ? SOFTMAX_WARPS2 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS0 = tmem, tO = tmem + 128;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            tc::mbar_expect_tx(bar(0), TILE);
            tc::tma_load_4d(tc::smem_u32(sQ), &map_q, bar(0), 0, qb * BM, g, b);
            tc::tma_load_4d(tc::smem_u32(sQ + HALF), &map_q, bar(0), 64, qb * BM, g, b);
            uint32_t ps = 0, pph = 0;
            auto load = [&](const CUtensorMap *map, int kb) -> bool {
                if (!tc::mbar_wait(bar(4 + ps), pph ^ 1u, abort_flag, P.status, 0x41u)) return false;
                tc::mbar_expect_tx(bar(1 + ps), KV_STAGE);
                tc::tma_load_4d(tc::smem_u32(sR + ps * KV_STAGE), map, bar(1 + ps), 0, kb * BN2, gk, b);
                tc::tma_load_4d(tc::smem_u32(sR + ps * KV_STAGE + KV_HALF), map, bar(1 + ps), 64, kb * BN2, gk, b);
                if (++ps == RING) { ps = 0; pph ^= 1u; }
                return true;
            };
            for (int kb = 0; kb < nkb && ok; ++kb) ok = load(&map_k, kb);
            if (ok) ok = load(&map_k, 0);
            for (int kb = 0; kb < nkb && ok; ++kb) {
                if (kb + 1 < nkb) ok = load(&map_k, kb + 1);
                if (ok) ok = load(&map_v, kb);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = tc::instr_desc(0, 0, BN2), idesc_pv = tc::instr_desc(0, 1, HD);
            bool ok = tc::mbar_wait(bar(0), 0u, abort_flag, P.status, 0x51u);
            uint32_t rs = 0, rph = 0, qk_count = 0;
            auto issue_qk = [&]() -> bool {
                const uint32_t sb = qk_count & 1u, sph = (qk_count >> 1) & 1u;
                if (!tc::mbar_wait(bar(1 + rs), rph, abort_flag, P.status, 0x52u)) return false;
                if (!tc::mbar_wait(bar(9 + sb), sph ^ 1u, abort_flag, P.status, 0x53u)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t qa = tc::smem_u32(sQ), ka = tc::smem_u32(sR + rs * KV_STAGE);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t qoff = (uint32_t)(kk >> 2) * HALF + (uint32_t)(kk & 3) * 32u;
                    const uint32_t koff = (uint32_t)(kk >> 2) * KV_HALF + (uint32_t)(kk & 3) * 32u;
                    tc::umma(tS0 + sb * 64u, tc::smem_desc(qa + qoff, 16, 1024), tc::smem_desc(ka + koff, 16, 1024), idesc_qk, kk != 0 ? 1u : 0u);
                }
                tc::umma_commit(bar(4 + rs));
                tc::umma_commit(bar(7 + sb));
                if (++rs == RING) { rs = 0; rph ^= 1u; }
                ++qk_count;
                return true;
            };
            for (int kb = 0; kb < nkb && ok; ++kb) ok = issue_qk();
            if (ok) ok = issue_qk();
            for (int kb = 0; kb < nkb && ok; ++kb) {
                if (kb + 1 < nkb) ok = issue_qk();
                if (!ok) break;
                ok = tc::mbar_wait(bar(11), (uint32_t)(kb & 1), abort_flag, P.status, 0x54u);
                if (!ok) break;
                ok = tc::mbar_wait(bar(1 + rs), rph, abort_flag, P.status, 0x55u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t pa = tc::smem_u32(sP), va = tc::smem_u32(sR + rs * KV_STAGE);
#pragma unroll
                for (int kk = 0; kk < BN2 / 16; ++kk)
                    tc::umma(tO, tc::smem_desc(pa + (uint32_t)kk * 32u, 16, 1024), tc::smem_desc(va + (uint32_t)kk * 2048u, KV_HALF, 1024), idesc_pv, (kb | kk) != 0 ? 1u : 0u);
                tc::umma_commit(bar(4 + rs)); // the V block is free
                tc::umma_commit(bar(12));     // and P may be overwritten
                if (++rs == RING) { rs = 0; rph ^= 1u; }
            }
            if (ok) tc::umma_commit(bar(13));
        }
    } else {
        const int quad = warp & 3;
        const int ch = (warp - 2) >> 2;      // which 32 of a block's 64 keys, and which half of the output's columns
        const int row = quad * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float rtv = bf16_round(load_real(P.rt, P.rt_dtype, 0));
        const float rr = __frcp_rn(rtv);
        float *xch = reinterpret_cast<float *>(sP);
        bool ok = true;
        uint32_t qk_count = 0;
        const bool want_max = !(rtv < 0.0f);
        float ext = want_max ? -INFINITY : INFINITY;
        // the last allowed key among this thread's 32 of block kb (31 or more: all of them; negative: none)
        auto limit = [&](int kb) { return P.causal ? (qb * BM + row) - (kb * BN2 + ch * 32) : 31; };
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const uint32_t sb = qk_count & 1u, sph = (qk_count >> 1) & 1u;
            ok = tc::mbar_wait(bar(7 + sb), sph, abort_flag, P.status, 0x61u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t v[32];
            tc::tmem_ld32(tS0 + lane_base + sb * 64u + (uint32_t)(ch * 32), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(9 + sb));
            ++qk_count;
            const int lim = limit(kb);
            if (want_max) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i <= lim) ext = fmaxf(ext, __uint_as_float(v[i]));
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i <= lim) ext = fminf(ext, __uint_as_float(v[i]));
            }
        }
        xch[ch * 128 + row] = ext;
        softmax_sync2();
        ext = want_max ? fmaxf(xch[row], xch[128 + row]) : fminf(xch[row], xch[128 + row]);
        softmax_sync2();
        const float m = bf16_round(__fdiv_rn(bf16_round(ext), rtv));
        const float LOG2E = 1.44269504f;
        const float m2 = __fmul_rn(m, LOG2E);
        float z = 0.0f;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const uint32_t sb = qk_count & 1u, sph = (qk_count >> 1) & 1u;
            ok = tc::mbar_wait(bar(7 + sb), sph, abort_flag, P.status, 0x62u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t v[32];
            tc::tmem_ld32(tS0 + lane_base + sb * 64u + (uint32_t)(ch * 32), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(9 + sb));
            ++qk_count;
            const int lim = limit(kb);
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                // bf16(S), then bf16(bf16(S) / rt) by the reciprocal (exact for bf16 operands: see k_attn_fwd)
                const uint32_t s1 = pack_bf16x2_hw(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                const float d0 = __fmul_rn(bits_f32(s1 << 16), rr), d1 = __fmul_rn(bits_f32(s1 & 0xffff0000u), rr);
                const uint32_t s2 = pack_bf16x2_hw(d0, d1);
                float e0 = fast_exp2(__fmaf_rn(bits_f32(s2 << 16), LOG2E, -m2));
                float e1 = fast_exp2(__fmaf_rn(bits_f32(s2 & 0xffff0000u), LOG2E, -m2));
                if (lim < 31) {
                    if (2 * i > lim) e0 = 0.0f;
                    if (2 * i + 1 > lim) e1 = 0.0f;
                }
                z += e0;
                z += e1;
                packed[i] = pack_bf16x2_hw(e0, e1);
            }
            ok = tc::mbar_wait(bar(12), (uint32_t)(kb & 1) ^ 1u, abort_flag, P.status, 0x63u); // P of the block before was read
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            uint8_t *dst = sP + row * 128;
            const int u0 = ch * 4;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                *reinterpret_cast<uint4 *>(dst + (((u0 + u) ^ (row & 7)) << 4)) = make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(11));
        }
        if (ok) {
            ok = tc::mbar_wait(bar(13), 0u, abort_flag, P.status, 0x64u);
            ok = __all_sync(0xffffffffu, ok);
        }
        xch[ch * 128 + row] = z;
        softmax_sync2();
        z = __fadd_rn(xch[row], xch[128 + row]);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t t = (int64_t)qb * BM + row;
            uint16_t *orow = (uint16_t *)P.out + (int64_t)b * P.o_b + (int64_t)g * P.o_g + t * P.o_t + ch * 64;
            const float rz = __frcp_rn(z);
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t v[32];
                tc::tmem_ld32(tO + lane_base + (uint32_t)(ch * 64 + c0), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        w[i] = pack_bf16x2_hw(div_by(__uint_as_float(v[u * 8 + 2 * i]), z, rz), div_by(__uint_as_float(v[u * 8 + 2 * i + 1]), z, rz));
                    *reinterpret_cast<uint4 *>(orow + c0 + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}
} // namespace v2


// ---------------------------------------------------------------------------
// One pass over the key blocks (the declared order `attention: online`): the exponentials are taken against a
// running reference maximum instead of the row's final one, so the scores are multiplied once, not twice.
//
//   * A thread owns a query row (its tensor-memory lane) and all 64 keys of a block: no exchange between threads,
//     ever. Four softmax warps a CTA, two CTAs an SM.
//   * The reference m of a row (in units of log2: score · log2(e) / rt) starts as the first block's maximum. A later
//     block whose maximum exceeds m by more than RESCALE_AT moves it: the row's sum and its accumulator in tensor
//     memory are multiplied by 2^(m_old - m_new) (tcgen05.ld, multiply, tcgen05.st), between the product that last
//     added to the accumulator and the next one. Until then exponentials may reach 2^RESCALE_AT, which bf16 and the
//     f32 accumulator hold exactly as well as numbers below one. Rows whose maximum settles early never pay.
//   * Unlike the two-pass kernels, the raw and the scaled scores are not rounded to bf16 in between (no memory ever
//     holds them here): exp2(s · c - m) straight from the f32 score, c = log2(e) / rt. The result is nearer the exact
//     attention than the four launches' and differs from theirs by their own roundings; the tests state by how much.
// K and V blocks travel through one ring of three stages in the order the products use them, P is single-buffered,
// every mbarrier wait is bounded, as in k_attn_fwd2.
// ---------------------------------------------------------------------------
namespace v3 {
constexpr int BN3 = 64;
constexpr int SOFTMAX_WARPS3 = 4;
constexpr int THREADS3 = (2 + SOFTMAX_WARPS3) * 32;
constexpr int KV_STAGE3 = BN3 * HD * 2;       // 16 KB: two halves of [64 keys x 64 hd]
constexpr int KV_HALF3 = BN3 * 64 * 2;
constexpr int RING3 = 3;
constexpr int P_BYTES3 = BM * BN3 * 2;        // 16 KB: [128 rows x 64 keys]
constexpr int SMEM_TILES3 = TILE + RING3 * KV_STAGE3 + P_BYTES3;
constexpr int SMEM_TOTAL3 = SMEM_TILES3 + 256 + 1024;
constexpr float RESCALE_AT = 8.0f;

PSK_DEV void tmem_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__global__ void __launch_bounds__(THREADS3, 2) k_attn_fwd3(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __grid_constant__ Params P)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sR = smem + TILE, *sP = smem + TILE + RING3 * KV_STAGE3;
    uint64_t *bars = (uint64_t *)(smem + SMEM_TILES3);
    // 0 q_full; 1..3 ring full; 4..6 ring empty; 7,8 s_full; 9,10 s_free; 11 p_full; 12 p_free; 13 o_full
    uint32_t *tmem_slot = (uint32_t *)(bars + 14);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    const uint32_t bar0 = tc::smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nqb = (int)(P.T / BM);
    const int qb = nqb - 1 - (int)blockIdx.x; // the longest rows first
    const int g = blockIdx.y, b = blockIdx.z;
    const int gk = g / P.per;
    const int nkb = P.causal ? 2 * (qb + 1) : (int)(P.T / BN3);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 14; ++i) tc::mbar_init(bar(i), (i == 9 || i == 10 || i == 11) ? SOFTMAX_WARPS3 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS0 = tmem, tO = tmem + 128;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            tc::mbar_expect_tx(bar(0), TILE);
            tc::tma_load_4d(tc::smem_u32(sQ), &map_q, bar(0), 0, qb * BM, g, b);
            tc::tma_load_4d(tc::smem_u32(sQ + HALF), &map_q, bar(0), 64, qb * BM, g, b);
            uint32_t ps = 0, pph = 0;
            auto load = [&](const CUtensorMap *map, int kb) -> bool {
                if (!tc::mbar_wait(bar(4 + ps), pph ^ 1u, abort_flag, P.status, 0x81u)) return false;
                tc::mbar_expect_tx(bar(1 + ps), KV_STAGE3);
                tc::tma_load_4d(tc::smem_u32(sR + ps * KV_STAGE3), map, bar(1 + ps), 0, kb * BN3, gk, b);
                tc::tma_load_4d(tc::smem_u32(sR + ps * KV_STAGE3 + KV_HALF3), map, bar(1 + ps), 64, kb * BN3, gk, b);
                if (++ps == RING3) { ps = 0; pph ^= 1u; }
                return true;
            };
            // in the order the products read them: K0, then (K of the next block, V of this one) a block
            ok = load(&map_k, 0);
            for (int kb = 0; kb < nkb && ok; ++kb) {
                if (kb + 1 < nkb) ok = load(&map_k, kb + 1);
                if (ok) ok = load(&map_v, kb);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = tc::instr_desc(0, 0, BN3), idesc_pv = tc::instr_desc(0, 1, HD);
            bool ok = tc::mbar_wait(bar(0), 0u, abort_flag, P.status, 0x91u);
            uint32_t rs = 0, rph = 0, qk_count = 0;
            auto issue_qk = [&]() -> bool {
                const uint32_t sb = qk_count & 1u, sph = (qk_count >> 1) & 1u;
                if (!tc::mbar_wait(bar(1 + rs), rph, abort_flag, P.status, 0x92u)) return false;
                if (!tc::mbar_wait(bar(9 + sb), sph ^ 1u, abort_flag, P.status, 0x93u)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t qa = tc::smem_u32(sQ), ka = tc::smem_u32(sR + rs * KV_STAGE3);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t qoff = (uint32_t)(kk >> 2) * HALF + (uint32_t)(kk & 3) * 32u;
                    const uint32_t koff = (uint32_t)(kk >> 2) * KV_HALF3 + (uint32_t)(kk & 3) * 32u;
                    tc::umma(tS0 + sb * 64u, tc::smem_desc(qa + qoff, 16, 1024), tc::smem_desc(ka + koff, 16, 1024), idesc_qk, kk != 0 ? 1u : 0u);
                }
                tc::umma_commit(bar(4 + rs));
                tc::umma_commit(bar(7 + sb));
                if (++rs == RING3) { rs = 0; rph ^= 1u; }
                ++qk_count;
                return true;
            };
            if (ok) ok = issue_qk();
            for (int kb = 0; kb < nkb && ok; ++kb) {
                if (kb + 1 < nkb) ok = issue_qk();
                if (!ok) break;
                ok = tc::mbar_wait(bar(11), (uint32_t)(kb & 1), abort_flag, P.status, 0x94u);
                if (!ok) break;
                ok = tc::mbar_wait(bar(1 + rs), rph, abort_flag, P.status, 0x95u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t pa = tc::smem_u32(sP), va = tc::smem_u32(sR + rs * KV_STAGE3);
#pragma unroll
                for (int kk = 0; kk < BN3 / 16; ++kk)
                    tc::umma(tO, tc::smem_desc(pa + (uint32_t)kk * 32u, 16, 1024), tc::smem_desc(va + (uint32_t)kk * 2048u, KV_HALF3, 1024), idesc_pv, (kb | kk) != 0 ? 1u : 0u);
                tc::umma_commit(bar(4 + rs)); // the V block is free
                tc::umma_commit(bar(12));     // and P may be overwritten, the accumulator rescaled
                if (++rs == RING3) { rs = 0; rph ^= 1u; }
            }
            if (ok) tc::umma_commit(bar(13));
        }
    } else {
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float rtv = bf16_round(load_real(P.rt, P.rt_dtype, 0)); // the division's kernel is bf16: it reads rt rounded to bf16 at its edge
        const float c = __fdiv_rn(1.44269504f, rtv);                  // log2(e) / rt
        const bool want_max = !(c < 0.0f);
        bool ok = true;
        float m = 0.0f, z = 0.0f;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const uint32_t sb = (uint32_t)kb & 1u, sph = ((uint32_t)kb >> 1) & 1u;
            ok = tc::mbar_wait(bar(7 + sb), sph, abort_flag, P.status, 0xa1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t va[32], vb[32];
            tc::tmem_ld32(tS0 + lane_base + sb * 64u, va);
            tc::tmem_ld32(tS0 + lane_base + sb * 64u + 32u, vb);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(9 + sb)); // the scores are in registers
            // the last allowed key of this row in this block (63 or more: all; negative: none)
            const int lim = P.causal ? (qb * BM + row) - kb * BN3 : 63;
            // the block's greatest scaled score over the allowed keys: c times the greatest raw score (the least, if c < 0)
            float blk = want_max ? -INFINITY : INFINITY;
            if (want_max) {
                if (lim >= 63) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) blk = fmaxf(blk, fmaxf(__uint_as_float(va[i]), __uint_as_float(vb[i])));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (i <= lim) blk = fmaxf(blk, __uint_as_float(va[i]));
                        if (i + 32 <= lim) blk = fmaxf(blk, __uint_as_float(vb[i]));
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (i <= lim) blk = fminf(blk, __uint_as_float(va[i]));
                    if (i + 32 <= lim) blk = fminf(blk, __uint_as_float(vb[i]));
                }
            }
            const float blk2 = __fmul_rn(blk, c); // -inf when the row sees nothing of this block
            float factor = 1.0f;
            if (kb == 0) {
                m = blk2; // every row sees the first key of the first block
            } else if (blk2 > m + RESCALE_AT) {
                factor = fast_exp2(m - blk2);
                z *= factor;
                m = blk2;
            }
            uint32_t packed[32];
            if (lim >= 63) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float e0 = fast_exp2(__fmaf_rn(__uint_as_float(va[2 * i]), c, -m)), e1 = fast_exp2(__fmaf_rn(__uint_as_float(va[2 * i + 1]), c, -m));
                    const float f0 = fast_exp2(__fmaf_rn(__uint_as_float(vb[2 * i]), c, -m)), f1 = fast_exp2(__fmaf_rn(__uint_as_float(vb[2 * i + 1]), c, -m));
                    z += e0 + e1;
                    z += f0 + f1;
                    packed[i] = pack_bf16x2_hw(e0, e1);
                    packed[16 + i] = pack_bf16x2_hw(f0, f1);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float e0 = fast_exp2(__fmaf_rn(__uint_as_float(va[2 * i]), c, -m)), e1 = fast_exp2(__fmaf_rn(__uint_as_float(va[2 * i + 1]), c, -m));
                    float f0 = fast_exp2(__fmaf_rn(__uint_as_float(vb[2 * i]), c, -m)), f1 = fast_exp2(__fmaf_rn(__uint_as_float(vb[2 * i + 1]), c, -m));
                    if (2 * i > lim) e0 = 0.0f;
                    if (2 * i + 1 > lim) e1 = 0.0f;
                    if (32 + 2 * i > lim) f0 = 0.0f;
                    if (33 + 2 * i > lim) f1 = 0.0f;
                    z += e0 + e1;
                    z += f0 + f1;
                    packed[i] = pack_bf16x2_hw(e0, e1);
                    packed[16 + i] = pack_bf16x2_hw(f0, f1);
                }
            }
            // the product of the block before has read P and added to the accumulator
            ok = tc::mbar_wait(bar(12), (uint32_t)(kb & 1) ^ 1u, abort_flag, P.status, 0xa2u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (__any_sync(0xffffffffu, factor != 1.0f)) {
                // this warp's 32 rows of the accumulator times their factors (1 for the rows that did not move)
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t o[32];
                    tc::tmem_ld32(tO + lane_base + (uint32_t)c0, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tmem_st32(tO + lane_base + (uint32_t)c0, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            uint8_t *dst = sP + row * 128;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                *reinterpret_cast<uint4 *>(dst + ((u ^ (row & 7)) << 4)) = make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the tensor core reads P through the async proxy
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(11));
        }
        if (ok) {
            ok = tc::mbar_wait(bar(13), 0u, abort_flag, P.status, 0xa3u);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t t = (int64_t)qb * BM + row;
            uint16_t *orow = (uint16_t *)P.out + (int64_t)b * P.o_b + (int64_t)g * P.o_g + t * P.o_t;
            const float rz = __frcp_rn(z);
            if (P.aff_kind) {
                // The row as codes of the site's affine format, 32 bytes a group: clamp(rne(acc / (z s)) + zero), the
                // quotient taken as acc times RN(RN(1/z) RN(1/s)) (a few units of binary32 from the quotient: this kernel
                // agrees with the separate launches within a tolerance anyway, and a code differs from theirs only
                // where the value lies that near a tie), clamped to the codes' range before 1.5 * 2^23 is added to
                // round it to an integer, ties to even, held in the sum's low bits. A NaN is the zero point.
                const int lo = P.aff_kind == 2 ? 0 : -128, hi = P.aff_kind == 2 ? 255 : 127;
                const float vlo = (float)(lo - P.aff_zero), vhi = (float)(hi - P.aff_zero);
                const float kq = __fmul_rn(rz, __frcp_rn(P.aff_scale));
                const int bias = P.aff_zero - 0x4B400000;
                uint8_t *crow = (uint8_t *)P.out + (int64_t)b * P.o_b + (int64_t)g * P.o_g + t * P.o_t;
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld32(tO + lane_base + (uint32_t)c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float q = __fmul_rn(__uint_as_float(v[i]), kq);
                        q = q == q ? q : 0.0f;
                        q = fminf(fmaxf(q, vlo), vhi);
                        v[i] = (uint32_t)(__float_as_int(__fadd_rn(q, 12582912.0f)) + bias);
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        w[u] = __byte_perm(__byte_perm(v[4 * u], v[4 * u + 1], 0x0040), __byte_perm(v[4 * u + 2], v[4 * u + 3], 0x0040), 0x5410);
                    *reinterpret_cast<uint4 *>(crow + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4 *>(crow + c0 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld32(tO + lane_base + (uint32_t)c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            w[i] = pack_bf16x2_hw(__fmul_rn(__uint_as_float(v[u * 8 + 2 * i]), rz), __fmul_rn(__uint_as_float(v[u * 8 + 2 * i + 1]), rz)); // (by the reciprocal: a unit or two of binary32 from the quotient, far inside this kernel's tolerance)
                        *reinterpret_cast<uint4 *>(orow + c0 + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}
} // namespace v3

} // namespace attn
} // namespace psk
