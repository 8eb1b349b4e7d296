// The tensor-core contraction on pairs of CTAs (tcgen05 cta_group::2), for sm_100a.
//
// Same arithmetic, same result bits and same epilogue as k_gemm_tc (psk_gemm_tc.cuh); another division of the
// work. Two CTAs of a cluster, each on its own SM, compute one 256 x 256 tile: CTA r holds rows 128·r .. of A and
// columns 128·r .. of B in its shared memory, the leader (rank 0) issues tcgen05.mma.cta_group::2 (M 256, N 256,
// K 16), and the unit reads either half of B from either SM. Each CTA then moves 32 KB from the L2 for a
// 128 x 256 x 64 block of products where the one-CTA form moves 48 KB (its 256-row variant 32 KB a 128 rows, but
// with both accumulators in use and the epilogue exposed): here each CTA's tensor memory holds two accumulators of
// 128 lanes x 256 columns, so a tile's epilogue runs under the next tile's products.
//
// Who signals whom (every wait is on a barrier of the waiting CTA's own shared memory, and bounded):
//   full[s]   in the leader; the leader's loader announces both CTAs' bytes (arrive.expect_tx), each CTA's TMA
//             loads complete on it (cp.async.bulk.tensor .cta_group::2 lets a load signal the peer's barrier);
//   empty[s]  in both; the leader's tcgen05.commit multicasts to the pair when the products have read stage s;
//   tfull[a]  in both; the same multicast commit when accumulator a is complete;
//   tempty[a] in the leader; the eight epilogue warps of each CTA arrive (the peer's through the cluster window).
// No load is multicast: each CTA fetches its own tiles.
#pragma once
#include "psk_gemm_tc.cuh"

namespace psk {
namespace tc2 {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2; // per CTA: its rows of A, its half of B
constexpr int TILE_BYTES = STAGES * (A_BYTES + B_BYTES);
constexpr int BAR_BYTES = 256;
constexpr int STAGE_OUT = 8 * 32 * 128;
constexpr int SMEM_TOTAL = TILE_BYTES + BAR_BYTES + STAGE_OUT + 1024;
constexpr int THREADS = 320;

PSK_DEV uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// The address, in the cluster's shared-memory window, of the same offset in CTA `rank`.
PSK_DEV uint32_t map_to_rank(uint32_t local, uint32_t rank)
{
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local), "r"(rank));
    return a;
}

PSK_DEV void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

PSK_DEV void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// A load of one CTA of the pair, its completion counted on a barrier given by its cluster address (the leader's).
PSK_DEV void tma_load_4d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

PSK_DEV void umma_pair(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives, once the products issued so far are complete, on the barrier at this offset in both CTAs of the pair.
PSK_DEV void umma_commit_pair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask) : "memory");
}

PSK_DEV uint32_t instr_desc_pair(int in_f16, int b_n_major)
{
    uint32_t d = 0;
    d |= 1u << 4;
    d |= (in_f16 ? 0u : 1u) << 7;
    d |= (in_f16 ? 0u : 1u) << 10;
    d |= (b_n_major ? 1u : 0u) << 16;
    d |= (uint32_t)(BN >> 3) << 17;
    d |= (uint32_t)(256 >> 4) << 24; // M of the pair
    return d;
}

// Takes psk_gemm_tc's parameters; the host sends it only shapes whose epilogue is one of the staged plain forms
// (bf16 result with or without a residual addend, f32 result; no scale, no planes, A and the result row-major).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1) k_gemm_tc2(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ tc::Params P)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * A_BYTES;
    uint64_t *bars = (uint64_t *)(smem + TILE_BYTES);
    // bars: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 4);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const uint32_t full0 = tc::smem_u32(bars), empty0 = tc::smem_u32(bars + STAGES);
    const uint32_t tfull0 = tc::smem_u32(bars + 2 * STAGES), tempty0 = tc::smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(full0 + 8 * s, 1);
            tc::mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(tfull0 + 8 * s, 1);
            tc::mbar_init(tempty0 + 8 * s, 16); // eight epilogue warps of each CTA of the pair
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // each CTA takes the whole of its own SM's tensor memory (all 512 columns, so both get the same base);
        // the pair's products then write the same columns of both
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync(); // the peer's barriers are initialised before anything arrives on them from here
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // tiles of 256 rows a pair
    const int64_t tiles_per_batch = P.tiles_m * P.tiles_n;
    const int64_t total_tiles = tiles_per_batch * P.batch;
    const int num_kb = (int)((P.k + BK - 1) / BK);
    const int64_t first = blockIdx.x >> 1, stride = gridDim.x >> 1;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t t = first; t < total_tiles && ok; t += stride) {
                const int64_t b = t / tiles_per_batch, r = t % tiles_per_batch;
                int64_t mt, nt;
                tc::tile_of(r, P.tiles_m, P.tiles_n, P.panel, mt, nt);
                const int m0 = (int)mt * 256 + (int)rank * BM, n0 = (int)nt * BN + (int)rank * (BN / 2);
                const int blo = (int)(b % P.batch_lo), bhi = (int)(b / P.batch_lo);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = tc::mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag, P.status, 0xb1u);
                    if (!ok) break;
                    const uint32_t fb = map_to_rank(full0 + 8 * stage, 0); // the leader's barrier
                    if (leader) tc::mbar_expect_tx(full0 + 8 * stage, 2 * (A_BYTES + B_BYTES));
                    const int k0 = kb * BK;
                    tma_load_4d_pair(tc::smem_u32(smem_a + stage * A_BYTES), &map_a, fb, k0, m0, blo, bhi);
                    if (!P.b_n_major) {
                        tma_load_4d_pair(tc::smem_u32(smem_b + stage * B_BYTES), &map_b, fb, k0, n0, blo, bhi);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 2 / 64; ++c)
                            tma_load_4d_pair(tc::smem_u32(smem_b + stage * B_BYTES + c * 8192), &map_b, fb, n0 + c * 64, k0, blo, bhi);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            const uint32_t idesc = instr_desc_pair(P.in_f16, P.b_n_major);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t t = first; t < total_tiles && ok; t += stride) {
                ok = tc::mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag, P.status, 0xb2u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tacc = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = tc::mbar_wait(full0 + 8 * stage, phase, abort_flag, P.status, 0xb3u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = tc::smem_u32(smem_a + stage * A_BYTES);
                    const uint32_t b_addr = tc::smem_u32(smem_b + stage * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / tc::UMMA_K; ++k) {
                        const uint64_t ad = tc::smem_desc(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = P.b_n_major ? tc::smem_desc(b_addr + k * 2048, 8192, 1024) : tc::smem_desc(b_addr + k * 32, 16, 1024);
                        umma_pair(tacc, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(empty0 + 8 * stage); // both CTAs' stage s is free once these have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(tfull0 + 8 * acc);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        const int quad = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        const int half_id = (warp - 2) >> 2;
        uint4 *stage_out = reinterpret_cast<uint4 *>(smem + TILE_BYTES + BAR_BYTES) + (warp - 2) * 32 * 8;
        const int group_cols = P.out_dtype == PSK_F32 ? 32 : 64;
        const bool with_add = P.addend != nullptr;
        const uint32_t tempty_leader0 = map_to_rank(tempty0, 0);
        for (int64_t t = first; t < total_tiles && ok; t += stride) {
            const int64_t b = t / tiles_per_batch, r = t % tiles_per_batch;
            int64_t mt, nt;
            tc::tile_of(r, P.tiles_m, P.tiles_n, P.panel, mt, nt);
            const int64_t m0 = mt * 256 + (int64_t)rank * BM, n0 = nt * BN;
            const int64_t blo = b % P.batch_lo, bhi = b / P.batch_lo;
            ok = tc::mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, P.status, 0xb4u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t row0 = m0 + quad * 32;
            const int64_t boff = blo * P.c_lo + bhi * P.c_hi;
            const int64_t row = row0 + lane;
            const uint32_t rcnt = (uint32_t)(P.c_row_lo_count < 0x7fffffffll ? P.c_row_lo_count : 0x7fffffffll);
            const uint32_t ccnt = (uint32_t)(P.c_col_lo_count < 0x7fffffffll ? P.c_col_lo_count : 0x7fffffffll);
            int64_t row_off;
            {
                const uint32_t rq = (uint32_t)row / rcnt;
                row_off = boff + (int64_t)rq * P.c_row_hi + (int64_t)((uint32_t)row - rq * rcnt) * P.c_row_lo;
            }
            int64_t row_offs[8];
            bool rows_ok[8];
            {
                const uint32_t q0 = (uint32_t)row0 / rcnt, r0 = (uint32_t)row0 - q0 * rcnt;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const uint32_t rr = (uint32_t)(it * 4 + (lane >> 3));
                    uint32_t rq = q0, rm = r0 + rr;
                    if (rm >= rcnt) {
                        if (rcnt >= 32u) { rm -= rcnt; rq += 1u; }
                        else { rq += rm / rcnt; rm = rm % rcnt; }
                    }
                    row_offs[it] = boff + (int64_t)rq * P.c_row_hi + (int64_t)rm * P.c_row_lo;
                    rows_ok[it] = row0 + rr < P.m;
                }
            }
            const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c0 = half_id * group_cols; c0 < BN; c0 += 2 * group_cols) {
                const int64_t col = n0 + c0;
                const uint32_t cq = (uint32_t)col / ccnt;
                const int64_t col_off = (int64_t)cq * P.c_col_hi + (int64_t)((uint32_t)col - cq * ccnt);
                if (P.out_dtype == PSK_F32) {
                    uint32_t v[32];
                    tc::tmem_ld32(tbase + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int q = 0; q < 8; ++q) stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                } else {
                    uint32_t va[32], vb[32];
                    tc::tmem_ld32(tbase + c0, va);
                    tc::tmem_ld32(tbase + c0 + 32, vb);
                    if (with_add) {
                        // the residual of this lane's row, 128 bytes, fetched while tensor memory is being read
                        uint4 ad[8];
                        const bool live = row < P.m;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            ad[j] = (live && col + j * 8 < P.n) ? *reinterpret_cast<const uint4 *>((const uint16_t *)P.addend + row_off + col_off + j * 8) : make_uint4(0u, 0u, 0u, 0u);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t aw[4] = {ad[j].x, ad[j].y, ad[j].z, ad[j].w};
                            uint32_t u[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int e = (j & 3) * 8 + 2 * i;
                                const uint32_t p = j < 4 ? pack_bf16x2_hw(__uint_as_float(va[e]), __uint_as_float(va[e + 1])) : pack_bf16x2_hw(__uint_as_float(vb[e]), __uint_as_float(vb[e + 1]));
                                u[i] = pack_bf16x2_hw(__fadd_rn(bits_f32(aw[i] << 16), bits_f32(p << 16)), __fadd_rn(bits_f32(aw[i] & 0xffff0000u), bits_f32(p & 0xffff0000u)));
                            }
                            stage_out[lane * 8 + (j ^ (lane & 7))] = make_uint4(u[0], u[1], u[2], u[3]);
                        }
                    } else {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(
                                pack_bf16x2_hw(__uint_as_float(va[q * 8]), __uint_as_float(va[q * 8 + 1])), pack_bf16x2_hw(__uint_as_float(va[q * 8 + 2]), __uint_as_float(va[q * 8 + 3])),
                                pack_bf16x2_hw(__uint_as_float(va[q * 8 + 4]), __uint_as_float(va[q * 8 + 5])), pack_bf16x2_hw(__uint_as_float(va[q * 8 + 6]), __uint_as_float(va[q * 8 + 7])));
                            stage_out[lane * 8 + ((4 + q) ^ (lane & 7))] = make_uint4(
                                pack_bf16x2_hw(__uint_as_float(vb[q * 8]), __uint_as_float(vb[q * 8 + 1])), pack_bf16x2_hw(__uint_as_float(vb[q * 8 + 2]), __uint_as_float(vb[q * 8 + 3])),
                                pack_bf16x2_hw(__uint_as_float(vb[q * 8 + 4]), __uint_as_float(vb[q * 8 + 5])), pack_bf16x2_hw(__uint_as_float(vb[q * 8 + 6]), __uint_as_float(vb[q * 8 + 7])));
                        }
                    }
                }
                __syncwarp();
                if (col < P.n) {
                    const int unit = lane & 7;
                    const int units_live = (int)((P.n - col) >= group_cols ? 8 : ((P.n - col) * (P.out_dtype == PSK_F32 ? 4 : 2)) / 16);
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3);
                        if (rows_ok[it] && unit < units_live) {
                            const int64_t off = row_offs[it] + col_off;
                            const uint4 w = stage_out[rr * 8 + (unit ^ (rr & 7))];
                            *reinterpret_cast<uint4 *>((uint8_t *)P.c + off * (P.out_dtype == PSK_F32 ? 4 : 2) + unit * 16) = w;
                        }
                    }
                }
                __syncwarp();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * acc); // the leader issues the products into it
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    // nobody leaves (or frees tensor memory the pair's products write) while the other CTA still works
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

} // namespace tc2
} // namespace psk
