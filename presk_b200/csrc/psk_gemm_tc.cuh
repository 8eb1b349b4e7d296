// The tensor-core contraction: C[b] = A[b]·B[b], bf16 or binary16 operands,
// f32 sums in tensor memory, for sm_100a.
//
// This is what a contraction nest of the reference (presk-kernel/src/lower.rs
// `emit_contraction_with`, :906-1139, and the generic `ein`, :586-636) becomes
// under the declared order PSK_ORDER_DEVICE. The products of two bf16 or two
// binary16 numbers are exact in f32; the sums are the tensor core's, grouped
// by its tiles and not in index order, so a result agrees with the kernel
// interpreter's within a tolerance and not bit for bit. The store rounds once
// to the site's storage type with the bits of psk_formats.cuh, and tests the
// overflow guard where the type is binary16 or e8m15.
//
// Shape of the kernel: one persistent CTA per SM, 320 threads.
//   warp 0      one lane issues the TMA loads of A and B tiles (128 x 64 and
//               BN x 64 elements, 128-byte swizzle) into a ring of STAGES
//               shared-memory stages;
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma
//               (cta_group::1, kind::f16, M = 128, N = BN, K = 16) four times
//               per stage into one of two accumulators of BN columns;
//   warps 2-9   the epilogue: tcgen05.ld of 32 columns a time, rounding, a
//               transposition through shared memory and 128-bit global stores
//               of whole 128-byte lines, of one accumulator while the other is
//               being computed; two warps a quadrant of tensor memory.
// No multicast, no cluster: every CTA loads its own tiles, and reuse between
// CTAs comes from the L2 through the order tiles are handed out in.
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records
// where in `status`, raises a flag in shared memory that ends every other
// loop, frees its tensor memory and returns.
#pragma once
#include <type_traits>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "psk_formats.cuh"

namespace psk {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 64; // elements: one 128-byte swizzle row of 16-bit elements
constexpr int UMMA_K = 16;
constexpr int THREADS = 320; // a TMA warp, an MMA warp, eight epilogue warps
constexpr long long WAIT_CYCLES = 4000000000ll; // about two seconds

struct Params {
    int64_t m, n, k;
    int64_t batch, batch_lo;
    int64_t tiles_m, tiles_n;
    int64_t panel; // tile-columns handed out together (tile_of)
    // Wider operands as `planes` bf16 planes each (an e8m15 number is the exact sum of two bf16 numbers, an f32
    // of three): the operands hold their planes side by side along the summed axis, planes·split_k long, and the
    // kernel's k runs over planes²·split_k: part t reads A's plane t / planes and B's plane t % planes, so all
    // the exact partial products add up in one accumulator. split_k = 0: the operands are what they are.
    int64_t split_k;
    int32_t planes, a_m_major; // a_m_major: A[batch][k][m], m contiguous (a transposed operand: dot_vjp_r's first)
    // PSK_OP_CONTRACT_ADD: bf16 values laid out exactly as C, added to the result after it has been rounded to
    // bf16 as its own site would store it; the sum is rounded to bf16 again. Staged bf16 epilogue only.
    const void *addend;
    int64_t c_row_lo_count, c_row_lo, c_row_hi;
    int64_t c_col_lo_count, c_col_hi;
    int64_t c_lo, c_hi;
    void *c;
    int out_dtype;
    int in_f16; // 1: binary16 operands; 0: bf16
    int b_n_major;
    int guarded;
    int vec_ok; // 128-bit stores are aligned
    float scale;
    int scale_on;
    // integer weights: operand 1 holds the weights' integers as bf16 numbers (exact), and the
    // accumulator of column c is multiplied once by the channel's scale col_scale[c * col_scale_stride
    // + batch terms] before it is rounded: (sum_k x·q)·s where the reference has sum_k x·(q·s)
    const float *col_scale;
    int64_t col_scale_stride, col_scale_lo, col_scale_hi;
    uint32_t *ovf;
    uint32_t *status;
};

PSK_DEV uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

PSK_DEV void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

PSK_DEV void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

PSK_DEV void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// A bounded wait: false when it gave up or another role already had.
PSK_DEV bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t *status, uint32_t where, long long limit = WAIT_CYCLES)
{
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if ((it & 255u) == 255u && clock64() - t0 > limit) {
            *abort_flag = 1;
            atomicOr(status, 0x100u | where);
            return false;
        }
    }
}

PSK_DEV void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// A shared-memory matrix descriptor for 128-byte-swizzled tiles: start
// address, leading and stride byte offsets in units of 16 bytes, version 1
// (sm_100), layout type 2 (128-byte swizzle).
PSK_DEV uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// The instruction descriptor of kind::f16: f32 accumulator, both operands
// bf16 or both binary16, A K-major, B K-major or N-major, M = 128, N = bn.
PSK_DEV uint32_t instr_desc(int in_f16, int b_n_major, int bn, int a_m_major = 0)
{
    uint32_t d = 0;
    d |= 1u << 4;                        // accumulator f32
    d |= (in_f16 ? 0u : 1u) << 7;        // A: 0 binary16, 1 bf16
    d |= (in_f16 ? 0u : 1u) << 10;       // B
    d |= (a_m_major ? 1u : 0u) << 15;    // A major: 0 K, 1 MN
    d |= (b_n_major ? 1u : 0u) << 16;    // B major: 0 K, 1 MN
    d |= (uint32_t)(bn >> 3) << 17;
    d |= (uint32_t)(BM >> 4) << 24;
    return d;
}

PSK_DEV void umma(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

PSK_DEV void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

PSK_DEV void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// Sixteen columns of this thread's row of an accumulator.
PSK_DEV void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Where tile `r` of a batch lies. Tiles are handed out in panels of PANEL
// tile-columns, down every tile-row of a panel before the next panel: the
// CTAs running at one time then share a few columns of B and a band of rows of
// A that together fit the L2, instead of sweeping all of B for a few rows of A.
// The panel's width is the host's choice (Params::panel): wide enough that A is not streamed from memory once a
// panel more often than needed, narrow enough that the panel's columns of B stay in the L2.
PSK_DEV void tile_of(int64_t r, int64_t tiles_m, int64_t tiles_n, int64_t PANEL, int64_t &mt, int64_t &nt)
{
    const int64_t per_panel = PANEL * tiles_m;
    const int64_t panel = r / per_panel, in_panel = r - panel * per_panel;
    const int64_t width = tiles_n - panel * PANEL < PANEL ? tiles_n - panel * PANEL : PANEL;
    mt = in_panel / width;
    nt = panel * PANEL + (in_panel - mt * width);
}

// The bounded wait by itself, for a test of the host's reporting: one thread waits on a barrier that nothing
// arrives at, gives up after `limit` cycles, records where (role 0x7f) and returns. Nothing else happens.
static __global__ void k_wait_runs_out(uint32_t *status, long long limit, int *gave_up)
{
    __shared__ uint64_t bar_word;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(smem_u32(&bar_word), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool ok = mbar_wait(smem_u32(&bar_word), 0u, &abort_word, status, 0x7fu, limit);
        *gave_up = ok ? 0 : 1;
    }
}

// MT: 128-row halves of a CTA's tile. With MT = 2 a CTA computes 256 x BN, both halves multiplying the same tile of B:
// a third fewer bytes from the L2 into shared memory a product, which is what the kernel's sustained rate under the
// power cap depends on (measured: with B's loads left out it holds cuBLAS's rate, 14 % above its own). The two
// accumulators then fill tensor memory, so the epilogue of a tile is overlapped with the next tile's loads only.
template <int BN, int MT = 1>
struct Smem {
    static constexpr int A_BYTES = MT * BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGES = MT == 2 ? 3 : (BN == 256) ? 4 : 6;
    static constexpr int TILE_BYTES = STAGES * (A_BYTES + B_BYTES);
    static constexpr int BAR_BYTES = 256;
    static constexpr int STAGE_OUT = 8 * 32 * 128; // the epilogue's staging: 32 rows of 128 bytes a warp
    static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + STAGE_OUT + 1024; // slack to align the base to 1024
};

// One element of the accumulator on its way to memory: the optional fused
// scaling as the reference's separate nest would compute it (round to the
// site's type, then one IEEE division... the caller passes the reciprocal
// only when that is exact), then the store's rounding.
// PER_BATCH: the guard's flag is one word a batch entry (P.ovf[b]) instead of
// one word a launch, for a caller that wants to know which entry overflowed.
// CS: the instantiation launched when columns carry a scale (integer weights); it alone holds the epilogue's
// vector paths for scales, so that the plain instantiation keeps its registers.
// PLAIN: the instantiations for a plain bf16 result (whole 16-byte runs, no scale, no column scales, no guard: what
// the host checks before it launches them), 1 without and 2 with a residual addend: their epilogue takes the accumulators out of tensor memory
// sixteen columns at a time into two buffers in turn, the next sixteen (the next group's, the other half-tile's) on
// their way while these are rounded and staged, so that the load's latency is not waited for once a group.
template <int BN, bool PER_BATCH = false, int MT = 1, bool CS = false, int PLAIN = 0>
__global__ void __launch_bounds__(THREADS, 1) k_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ Params P)
{
    static_assert(MT == 1 || (MT == 2 && BN == 256), "two halves fill tensor memory with 256 columns each");
    using S = Smem<BN, MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + S::STAGES * S::A_BYTES;
    uint64_t *bars = (uint64_t *)(smem + S::TILE_BYTES);
    // bars: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * S::STAGES + 4);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + S::STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * S::STAGES), tempty0 = smem_u32(bars + 2 * S::STAGES + 2);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull0 + 8 * s, 1);
            mbar_init(tempty0 + 8 * s, 8); // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int64_t tiles_per_batch = P.tiles_m * P.tiles_n;
    const int64_t total_tiles = tiles_per_batch * P.batch;
    const int num_kb = (int)((P.k + BK - 1) / BK);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int64_t b = t / tiles_per_batch, r = t % tiles_per_batch;
                int64_t mt, nt;
                tile_of(r, P.tiles_m, P.tiles_n, P.panel, mt, nt);
                const int m0 = (int)mt * BM * MT, n0 = (int)nt * BN; // the map of A has a box of BM * MT rows
                const int blo = (int)(b % P.batch_lo), bhi = (int)(b / P.batch_lo);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag, P.status, 1u);
                    if (!ok) break;
                    const uint32_t fb = full0 + 8 * stage;
                    mbar_expect_tx(fb, S::A_BYTES + S::B_BYTES);
                    int ka = kb * BK, kbb = kb * BK;
                    if (P.split_k) {
                        const int q = (int)(ka / P.split_k), r = (int)(ka - q * P.split_k);
                        ka = (q / P.planes) * (int)P.split_k + r;
                        kbb = (q % P.planes) * (int)P.split_k + r;
                    }
                    if (!P.a_m_major) {
                        tma_load_4d(smem_u32(smem_a + stage * S::A_BYTES), &map_a, fb, ka, m0, blo, bhi);
                    } else {
                        // 64 rows of the summed axis by 64 contiguous m a box, as B's N-major form below
#pragma unroll
                        for (int c = 0; c < BM * MT / 64; ++c)
                            tma_load_4d(smem_u32(smem_a + stage * S::A_BYTES + c * 8192), &map_a, fb, m0 + c * 64, ka, blo, bhi);
                    }
                    if (!P.b_n_major) {
                        tma_load_4d(smem_u32(smem_b + stage * S::B_BYTES), &map_b, fb, kbb, n0, blo, bhi);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tma_load_4d(smem_u32(smem_b + stage * S::B_BYTES + c * 8192), &map_b, fb, n0 + c * 64, kbb, blo, bhi);
                    }
                    if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(P.in_f16, P.b_n_major, BN, P.a_m_major);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                if constexpr (MT == 1) {
                    ok = mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag, P.status, 2u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                const uint32_t tacc = MT == 1 ? tmem_base + acc * BN : tmem_base;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, P.status, 3u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem_a + stage * S::A_BYTES);
                    const uint32_t b_addr = smem_u32(smem_b + stage * S::B_BYTES);
#pragma unroll
                    for (int h = 0; h < MT; ++h) {
                        if (MT == 2 && kb == 0) {
                            // this half's accumulator must have been drained by the epilogue of the tile before
                            ok = mbar_wait(tempty0 + 8 * h, acc_phase ^ 1u, abort_flag, P.status, 2u);
                            if (!ok) break;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t ad = P.a_m_major ? smem_desc(a_addr + h * (BM * BK * 2) + k * 2048, 8192, 1024) : smem_desc(a_addr + h * (BM * BK * 2) + k * 32, 16, 1024);
                            const uint64_t bd = P.b_n_major ? smem_desc(b_addr + k * 2048, 8192, 1024) : smem_desc(b_addr + k * 32, 16, 1024);
                            umma(tacc + h * BN, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    if (!ok) break;
                    umma_commit(empty0 + 8 * stage); // the stage is free once these have read it
                    if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if constexpr (MT == 1) {
                    umma_commit(tfull0 + 8 * acc);
                    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                } else {
                    umma_commit(tfull0);
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        const int quad = warp & 3; // the tensor-memory lanes this warp may read: 32·quad ..
        uint32_t acc = 0, acc_phase = 0, ovf = 0;
        bool ok = true;
        // this warp's staging tile: 32 rows of 128 bytes, 16-byte units swizzled by the row
        // two warps share a quadrant of tensor memory and take alternate column groups
        const int half_id = (warp - 2) >> 2;
        uint4 *stage_out = reinterpret_cast<uint4 *>(smem + S::TILE_BYTES + S::BAR_BYTES) + (warp - 2) * 32 * 8;
        const bool staged = P.vec_ok && (P.out_dtype == PSK_BF16 || P.out_dtype == PSK_F16 || P.out_dtype == PSK_F32);
        const int group_cols = P.out_dtype == PSK_F32 ? 32 : 64; // columns in 128 bytes
        const bool plain_bf16 = P.out_dtype == PSK_BF16 && !P.scale_on && !P.col_scale && !P.addend;
        const bool plain_add = P.out_dtype == PSK_BF16 && !P.scale_on && !P.col_scale && P.addend;
        const bool plain_f32 = P.out_dtype == PSK_F32 && !P.scale_on && !P.col_scale;
        const bool plain_cs = CS && P.out_dtype == PSK_BF16 && !P.scale_on && P.col_scale && P.col_scale_stride == 1 && !P.addend;
        const bool plain_cs_add = CS && P.out_dtype == PSK_BF16 && !P.scale_on && P.col_scale && P.col_scale_stride == 1 && P.addend;
        for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            const int64_t b = t / tiles_per_batch, r = t % tiles_per_batch;
            int64_t mt, nt;
            tile_of(r, P.tiles_m, P.tiles_n, P.panel, mt, nt);
            const int64_t m0 = mt * BM * MT, n0 = nt * BN;
            const int64_t blo = b % P.batch_lo, bhi = b / P.batch_lo;
            // A residual addend: this lane's 128 bytes of the group (row half mh, columns c0 ..) it will add next. The
            // first group's are asked for here, while the tile's products still run, and each later group's while the
            // one before it is rounded, so that no group waits for its addend.
            uint4 ad_next[PLAIN == 1 ? 1 : 8];
            auto fetch_addend = [&](int mh_, int c0_) {
                if constexpr (PLAIN == 1) return;
                const int64_t arow = m0 + mh_ * BM + quad * 32 + lane, acol = n0 + c0_;
                const uint32_t rcnt_ = (uint32_t)(P.c_row_lo_count < 0x7fffffffll ? P.c_row_lo_count : 0x7fffffffll);
                const uint32_t ccnt_ = (uint32_t)(P.c_col_lo_count < 0x7fffffffll ? P.c_col_lo_count : 0x7fffffffll);
                const uint32_t rq_ = (uint32_t)arow / rcnt_, cq_ = (uint32_t)acol / ccnt_;
                const int64_t off = blo * P.c_lo + bhi * P.c_hi + (int64_t)rq_ * P.c_row_hi + (int64_t)((uint32_t)arow - rq_ * rcnt_) * P.c_row_lo
                    + (int64_t)cq_ * P.c_col_hi + (int64_t)((uint32_t)acol - cq_ * ccnt_);
                const bool live = arow < P.m;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    ad_next[j] = (live && acol + j * 8 < P.n) ? *reinterpret_cast<const uint4 *>((const uint16_t *)P.addend + off + j * 8) : make_uint4(0u, 0u, 0u, 0u);
            };
            if (staged && plain_add) fetch_addend(0, half_id * group_cols);
            ok = mbar_wait(MT == 1 ? tfull0 + 8 * acc : tfull0, acc_phase, abort_flag, P.status, 4u);
            ok = __all_sync(0xffffffffu, ok); // the loads below want the whole warp
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t ca[16], cb[16]; // PLAIN: the two buffers; `primed`: the group about to start has its first sixteen on their way
            bool primed = false;
#pragma unroll 1
            for (int mh = 0; mh < MT; ++mh) { // the tile's 128-row halves, each with its own accumulator
            const int64_t row0 = m0 + mh * BM + quad * 32;
            const int64_t boff = blo * P.c_lo + bhi * P.c_hi;
            const float *cs_base = P.col_scale ? P.col_scale + blo * P.col_scale_lo + bhi * P.col_scale_hi : nullptr;
            const int64_t row = row0 + lane;
            int64_t row_off;
            {
                const uint32_t cnt = (uint32_t)(P.c_row_lo_count < 0x7fffffffll ? P.c_row_lo_count : 0x7fffffffll);
                const uint32_t rq = (uint32_t)row / cnt;
                row_off = boff + (int64_t)rq * P.c_row_hi + (int64_t)((uint32_t)row - rq * cnt) * P.c_row_lo;
            }
            const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + (MT == 1 ? acc : (uint32_t)mh) * BN;
            // Where the rows this lane stores lie (rows 4·it + lane / 8 of the warp's 32), once a half-tile and in 32-bit
            // arithmetic: a 64-bit division for every store was most of this epilogue's instructions.
            int64_t row_offs[8];
            bool rows_ok[8];
            {
                const uint32_t cnt = (uint32_t)(P.c_row_lo_count < 0x7fffffffll ? P.c_row_lo_count : 0x7fffffffll);
                const uint32_t first = (uint32_t)row0;
                const uint32_t q0 = first / cnt, r0 = first - q0 * cnt;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const uint32_t rr = (uint32_t)(it * 4 + (lane >> 3));
                    uint32_t rq = q0, rm = r0 + rr;
                    if (rm >= cnt) {
                        if (cnt >= 32u) { rm -= cnt; rq += 1u; }
                        else { rq += rm / cnt; rm = rm % cnt; }
                    }
                    row_offs[it] = boff + (int64_t)rq * P.c_row_hi + (int64_t)rm * P.c_row_lo;
                    rows_ok[it] = row0 + rr < P.m;
                }
            }
            if (staged) {
                // 128 bytes of every row at a time: through shared memory, so that a store
                // instruction writes whole 128-byte lines (8 lanes a row, 4 rows an instruction)
#pragma unroll 1
                for (int c0 = half_id * group_cols; c0 < BN; c0 += 2 * group_cols) {
                    const int64_t col = n0 + c0;
                    if (P.out_dtype == PSK_F32) {
                        uint32_t v[32];
                        tmem_ld32(tbase + c0, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (plain_f32) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            float x0 = __uint_as_float(v[4 * q]), x1 = __uint_as_float(v[4 * q + 1]), x2 = __uint_as_float(v[4 * q + 2]), x3 = __uint_as_float(v[4 * q + 3]);
                            if (P.scale_on) { x0 = __fmul_rn(x0, P.scale); x1 = __fmul_rn(x1, P.scale); x2 = __fmul_rn(x2, P.scale); x3 = __fmul_rn(x3, P.scale); }
                            if (P.col_scale) {
                                const int64_t cc = col + 4 * q;
                                if (cc + 3 < P.n) {
                                    x0 = __fmul_rn(x0, cs_base[cc * P.col_scale_stride]); x1 = __fmul_rn(x1, cs_base[(cc + 1) * P.col_scale_stride]);
                                    x2 = __fmul_rn(x2, cs_base[(cc + 2) * P.col_scale_stride]); x3 = __fmul_rn(x3, cs_base[(cc + 3) * P.col_scale_stride]);
                                }
                            }
                            stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(__float_as_uint(x0), __float_as_uint(x1), __float_as_uint(x2), __float_as_uint(x3));
                        }
                    } else {
                        int64_t add_col_off = 0;
                        if (P.addend) {
                            const uint32_t ccnt = (uint32_t)(P.c_col_lo_count < 0x7fffffffll ? P.c_col_lo_count : 0x7fffffffll);
                            const uint32_t cq = (uint32_t)col / ccnt;
                            add_col_off = (int64_t)cq * P.c_col_hi + (int64_t)((uint32_t)col - cq * ccnt);
                        }
                        if constexpr (PLAIN != 0) {
                            // columns 16k .. 16k + 15 of the group: two 16-byte units of the staged row (PLAIN 2: the
                            // product rounded to bf16, the residual added, the sum rounded again)
                            auto emit = [&](const uint32_t (&ch)[16], int k) {
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    uint32_t u[4];
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        u[i] = pack_bf16x2_hw(__uint_as_float(ch[8 * h + 2 * i]), __uint_as_float(ch[8 * h + 2 * i + 1]));
                                        if constexpr (PLAIN == 2) {
                                            const uint4 a4 = ad_next[(2 * k + h) & 7];
                                            const uint32_t aw = i == 0 ? a4.x : i == 1 ? a4.y : i == 2 ? a4.z : a4.w;
                                            u[i] = pack_bf16x2_hw(__fadd_rn(bits_f32(aw << 16), bits_f32(u[i] << 16)), __fadd_rn(bits_f32(aw & 0xffff0000u), bits_f32(u[i] & 0xffff0000u)));
                                        }
                                    }
                                    stage_out[lane * 8 + ((2 * k + h) ^ (lane & 7))] = make_uint4(u[0], u[1], u[2], u[3]);
                                }
                            };
                            if (!primed) tmem_ld16(tbase + c0, ca);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            tmem_ld16(tbase + c0 + 16, cb);
                            emit(ca, 0);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            tmem_ld16(tbase + c0 + 32, ca);
                            emit(cb, 1);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            tmem_ld16(tbase + c0 + 48, cb);
                            emit(ca, 2);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            if (c0 + 2 * group_cols < BN) { tmem_ld16(tbase + c0 + 2 * group_cols, ca); primed = true; }
                            else if (MT == 2 && mh + 1 < MT) { tmem_ld16(tbase + BN + half_id * group_cols, ca); primed = true; } // the other half-tile's accumulator lies BN columns on
                            else primed = false;
                            emit(cb, 3);
                            if constexpr (PLAIN == 2) { // the next group's residual, on its way during this group's stores
                                if (c0 + 2 * group_cols < BN) fetch_addend(mh, c0 + 2 * group_cols);
                                else if (mh + 1 < MT) fetch_addend(mh + 1, half_id * group_cols);
                            }
                        } else {
                        uint32_t va[32], vb[32];
                        tmem_ld32(tbase + c0, va);
                        tmem_ld32(tbase + c0 + 32, vb);
                        const bool cs_add = plain_cs_add && col + 64 <= P.n && (reinterpret_cast<uintptr_t>(cs_base + col) & 15) == 0;
                        if (plain_add) {
                            // the residual of this lane's row, 128 bytes, asked for a group ahead (taking it through the
                            // staging tile in whole lines was tried and is slower: 0.58 ms against 0.48 ms)
                            uint4 ad[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) ad[j] = ad_next[j];
                            if (c0 + 2 * group_cols < BN) fetch_addend(mh, c0 + 2 * group_cols);
                            else if (mh + 1 < MT) fetch_addend(mh + 1, half_id * group_cols);
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
                        } else if (cs_add) {
                            // integer weights and a residual: each column's sum times its channel's scale, rounded, then the
                            // addition, rounded; eight columns at a time (their scales and this row's addend fetched together)
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            const float4 *sc = reinterpret_cast<const float4 *>(cs_base + col);
                            const uint4 *ap = reinterpret_cast<const uint4 *>((const uint16_t *)P.addend + row_off + add_col_off);
                            const bool live = row < P.m;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const uint4 ad = live ? ap[j] : make_uint4(0u, 0u, 0u, 0u);
                                const float4 s0 = __ldg(sc + 2 * j), s1 = __ldg(sc + 2 * j + 1);
                                const uint32_t aw[4] = {ad.x, ad.y, ad.z, ad.w};
                                const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                                uint32_t u[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int e = (j & 3) * 8 + 2 * i;
                                    const float x0 = __fmul_rn(__uint_as_float(j < 4 ? va[e] : vb[e]), sv[2 * i]), x1 = __fmul_rn(__uint_as_float(j < 4 ? va[e + 1] : vb[e + 1]), sv[2 * i + 1]);
                                    const uint32_t p = pack_bf16x2_hw(x0, x1);
                                    u[i] = pack_bf16x2_hw(__fadd_rn(bits_f32(aw[i] << 16), bits_f32(p << 16)), __fadd_rn(bits_f32(aw[i] & 0xffff0000u), bits_f32(p & 0xffff0000u)));
                                }
                                stage_out[lane * 8 + (j ^ (lane & 7))] = make_uint4(u[0], u[1], u[2], u[3]);
                            }
                        } else {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (plain_bf16) {
                            // nothing but the rounding: the common case, kept free of the tests below
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(
                                    pack_bf16x2_hw(__uint_as_float(va[q * 8]), __uint_as_float(va[q * 8 + 1])), pack_bf16x2_hw(__uint_as_float(va[q * 8 + 2]), __uint_as_float(va[q * 8 + 3])),
                                    pack_bf16x2_hw(__uint_as_float(va[q * 8 + 4]), __uint_as_float(va[q * 8 + 5])), pack_bf16x2_hw(__uint_as_float(va[q * 8 + 6]), __uint_as_float(va[q * 8 + 7])));
                                stage_out[lane * 8 + ((4 + q) ^ (lane & 7))] = make_uint4(
                                    pack_bf16x2_hw(__uint_as_float(vb[q * 8]), __uint_as_float(vb[q * 8 + 1])), pack_bf16x2_hw(__uint_as_float(vb[q * 8 + 2]), __uint_as_float(vb[q * 8 + 3])),
                                    pack_bf16x2_hw(__uint_as_float(vb[q * 8 + 4]), __uint_as_float(vb[q * 8 + 5])), pack_bf16x2_hw(__uint_as_float(vb[q * 8 + 6]), __uint_as_float(vb[q * 8 + 7])));
                            }
                        } else if (plain_cs && col + 64 <= P.n && (reinterpret_cast<uintptr_t>(cs_base + col) & 15) == 0) {
                            // integer weights: each column's sum times its channel's scale (one f32 multiplication), then the
                            // rounding; the 64 scales of the group are the same for every lane (one line of the L1 a load)
                            const float4 *sc = reinterpret_cast<const float4 *>(cs_base + col);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float4 s0 = __ldg(sc + 2 * q), s1 = __ldg(sc + 2 * q + 1), s2 = __ldg(sc + 8 + 2 * q), s3 = __ldg(sc + 8 + 2 * q + 1);
                                stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(va[q * 8]), s0.x), __fmul_rn(__uint_as_float(va[q * 8 + 1]), s0.y)),
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(va[q * 8 + 2]), s0.z), __fmul_rn(__uint_as_float(va[q * 8 + 3]), s0.w)),
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(va[q * 8 + 4]), s1.x), __fmul_rn(__uint_as_float(va[q * 8 + 5]), s1.y)),
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(va[q * 8 + 6]), s1.z), __fmul_rn(__uint_as_float(va[q * 8 + 7]), s1.w)));
                                stage_out[lane * 8 + ((4 + q) ^ (lane & 7))] = make_uint4(
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(vb[q * 8]), s2.x), __fmul_rn(__uint_as_float(vb[q * 8 + 1]), s2.y)),
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(vb[q * 8 + 2]), s2.z), __fmul_rn(__uint_as_float(vb[q * 8 + 3]), s2.w)),
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(vb[q * 8 + 4]), s3.x), __fmul_rn(__uint_as_float(vb[q * 8 + 5]), s3.y)),
                                    pack_bf16x2_hw(__fmul_rn(__uint_as_float(vb[q * 8 + 6]), s3.z), __fmul_rn(__uint_as_float(vb[q * 8 + 7]), s3.w)));
                            }
                        } else
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t u[4];
                                uint4 add8 = make_uint4(0u, 0u, 0u, 0u);
                                if (P.addend && row < P.m && col + half * 32 + q * 8 < P.n) // the group's 64 columns lie in one column level (vec_ok)
                                    add8 = *reinterpret_cast<const uint4 *>((const uint16_t *)P.addend + row_off + add_col_off + half * 32 + q * 8);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    float x0 = __uint_as_float(half ? vb[q * 8 + 2 * i] : va[q * 8 + 2 * i]);
                                    float x1 = __uint_as_float(half ? vb[q * 8 + 2 * i + 1] : va[q * 8 + 2 * i + 1]);
                                    if (P.scale_on) { x0 = __fmul_rn(x0, P.scale); x1 = __fmul_rn(x1, P.scale); }
                                    if (P.col_scale) {
                                        const int64_t cc = col + half * 32 + q * 8 + 2 * i;
                                        if (cc + 1 < P.n) {
                                            x0 = __fmul_rn(x0, cs_base[cc * P.col_scale_stride]);
                                            x1 = __fmul_rn(x1, cs_base[(cc + 1) * P.col_scale_stride]);
                                        } else if (cc < P.n) {
                                            x0 = __fmul_rn(x0, cs_base[cc * P.col_scale_stride]);
                                        }
                                    }
                                    // the hardware's rounding: the reference's for every number; a NaN
                                    // comes out canonical (its sign and payload are not kept on this path)
                                    if (P.out_dtype == PSK_BF16) {
                                        u[i] = pack_bf16x2_hw(x0, x1);
                                        if (P.addend) {
                                            // this thread's row, the eight columns of (half, q): 16 bytes of the addend
                                            const uint32_t aw = i == 0 ? add8.x : i == 1 ? add8.y : i == 2 ? add8.z : add8.w;
                                            u[i] = pack_bf16x2_hw(__fadd_rn(bits_f32(aw << 16), bits_f32(u[i] << 16)), __fadd_rn(bits_f32(aw & 0xffff0000u), bits_f32(u[i] & 0xffff0000u)));
                                        }
                                    } else {
                                        ovf |= overflows(x0, kF16Overflow) | overflows(x1, kF16Overflow);
                                        u[i] = pack_f16x2_hw(x0, x1);
                                    }
                                }
                                stage_out[lane * 8 + ((half * 4 + q) ^ (lane & 7))] = make_uint4(u[0], u[1], u[2], u[3]);
                            }
                        }
                        } // not plain_add
                        } // not PLAIN
                    }
                    __syncwarp();
                    if (col < P.n) {
                        const uint32_t ccnt = (uint32_t)(P.c_col_lo_count < 0x7fffffffll ? P.c_col_lo_count : 0x7fffffffll);
                        const uint32_t cq = (uint32_t)col / ccnt;
                        const int64_t col_off = (int64_t)cq * P.c_col_hi + (int64_t)((uint32_t)col - cq * ccnt);
                        const int unit = lane & 7;
                        const int units_live = (int)((P.n - col) >= group_cols ? 8 : ((P.n - col) * (P.out_dtype == PSK_F32 ? 4 : 2)) / 16);
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const int rr = it * 4 + (lane >> 3);
                            if (rows_ok[it] && unit < units_live) {
                                const int64_t off = row_offs[it] + col_off;
                                const uint4 w = stage_out[rr * 8 + (unit ^ (rr & 7))];
                                uint8_t *dst = (uint8_t *)P.c + off * (P.out_dtype == PSK_F32 ? 4 : 2) + unit * 16;
                                *reinterpret_cast<uint4 *>(dst) = w;
                            }
                        }
                    }
                    __syncwarp();
                }
            } else {
#pragma unroll 1
                for (int c0 = half_id * 32; c0 < BN; c0 += 64) {
                    uint32_t v[32];
                    tmem_ld32(tbase + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int64_t col = n0 + c0;
                    if (row < P.m && col < P.n) {
                        for (int i = 0; i < 32; ++i)
                            if (col + i < P.n) {
                                const int64_t cc = col + i;
                                const int64_t o = row_off + (cc / P.c_col_lo_count) * P.c_col_hi + (cc % P.c_col_lo_count);
                                float x = __uint_as_float(v[i]);
                                if (P.scale_on) x = __fmul_rn(x, P.scale);
                                if (P.col_scale) x = __fmul_rn(x, cs_base[cc * P.col_scale_stride]);
                                ovf |= store_real(P.c, P.out_dtype, o, x);
                            }
                    }
                }
            }
            if constexpr (PER_BATCH) {
                if (P.guarded && ovf) atomicOr(P.ovf + b, 1u);
                ovf = 0;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * (MT == 1 ? acc : (uint32_t)mh));
            } // mh
            if (MT == 2) acc_phase ^= 1u;
            else if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (P.guarded && ovf) atomicOr(P.ovf, 1u);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

} // namespace tc
} // namespace psk
