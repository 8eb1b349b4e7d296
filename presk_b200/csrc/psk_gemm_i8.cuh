// The integer-sum contraction on the tensor cores: C[b] = rescale(A[b]·B[b]) with 8-bit integer operands and
// 32-bit integer sums in tensor memory (tcgen05.mma kind::i8), for sm_100a.
//
// What it computes is the reference's contraction under `product: i32, accum: i32`
// (crates/presk-kernel/src/exec.rs:493-526, `MixedCtx::counted`): both operands are read as integer counts in
// their scales' unit (an affine activation's code minus its zero point, an integer weight's code), the products
// and the sum are exact integers wrapped to 32 bits, and the store rounds the exact value sum·s_a·s_w ONCE into
// the output's format (exec.rs:601-616; presk-format/src/lib.rs:1148-1193). Addition modulo 2^32 is associative,
// so the tensor core's order of additions gives the reference's integer, bit for bit; this is the one contraction
// that is on the tensor cores and exact under every order.
//
//   * The tensor core sums the raw codes, sum_k a_k·w_k. The zero point is taken out afterwards:
//     sum_k (a_k - z)·w_k = sum_k a_k·w_k - z·sum_k w_k (mod 2^32), with the weights' column sums from a small
//     kernel before (k_colsum_i8), only when z != 0.
//   * The raw sum must not leave 32 bits for the identity above to hold whatever the unit does at an overflow
//     (it may saturate): |a| <= 255, |w| <= 128, so k <= 65536 keeps |sum| < 2^31. The host refuses longer sums
//     to this kernel; they run on k_contract_int.
//   * The rescale: n·(s_a·s_w) with s_a·s_w exact in binary64 (two 24-bit significands). For bf16 and f32 results
//     the product is formed in binary64 and rounded to the target unless it lies within one unit of that
//     intermediate of a rounding boundary of the target, in which case (a few elements in 10^5) the exact
//     128-bit routine of k_contract_int decides; so every stored code is the exact routine's. Affine codes likewise
//     (the quotient by the result's scale in binary64, the exact routine near a tie); binary16 and e8m15 results
//     always take the exact routine.
//   * A residual (PSK_OP_CONTRACT_ADD with integer sums, the ADD instance): the bf16 result as above, then
//     addend + result in binary32 rounded to bf16, element by element as the separate addition does, so the two
//     launches' bits under every order.
//
// Shape of the kernel: psk_gemm_tc.cuh's 256 x 256 form. One persistent CTA an SM, 320 threads: warp 0 issues TMA
// loads (A 256 rows x 128 bytes, B 256 columns x 128 bytes a stage, 128-byte swizzle, three stages, no multicast),
// warp 1 issues tcgen05.mma (M 128, N 256, K 32) into two accumulators of 256 columns, warps 2-9 drain them.
// Every mbarrier wait is bounded as there.
#pragma once
#include "psk_gemm_tc.cuh"
#include "psk_kernels.cuh"

namespace psk {
namespace tci8 {

constexpr int BM = 128, BN = 256, BKB = 128; // BKB: bytes = elements of the summed axis a stage
constexpr int B_BYTES = BN * BKB;
constexpr int BAR_BYTES = 256;
constexpr int STAGE_OUT = 8 * 32 * 128;
constexpr int SCALE_BYTES = 8 * 32 * 4; // a warp's 32 column scales, read back by every lane
constexpr int THREADS = 320;
// Two forms, as for the bf16 kernel. MT = 2: tiles of 256 rows, two accumulators sharing B's tile (a third less
// traffic from the L2 a product, three stages of 64 KB), the accumulators fill tensor memory and the rescale runs
// after the tile's products. MT = 1: tiles of 128 rows, the two accumulators used in turn, so that a tile's rescale
// runs under the next tile's products (four stages of 48 KB).
template <int MT>
struct Cfg {
    static constexpr int STAGES = MT == 2 ? 3 : 4;
    static constexpr int A_BYTES = MT * BM * BKB;
    static constexpr int TILE_BYTES = STAGES * (A_BYTES + B_BYTES);
    static constexpr int SMEM_TOTAL = TILE_BYTES + BAR_BYTES + STAGE_OUT + SCALE_BYTES + 1024;
};

struct Params {
    int64_t m, n, k;
    int64_t batch, batch_lo;
    int64_t tiles_m, tiles_n, panel;
    int64_t c_row_lo_count, c_row_lo, c_row_hi;
    int64_t c_col_lo_count, c_col_hi;
    int64_t c_lo, c_hi;
    void *c;
    int out_dtype;
    int out_affine, out_zero; // the result stored as affine codes: kind (1 i8, 2 u8) and zero point
    float out_scale;
    int a_unsigned;           // operand 0's codes are u8 (else i8)
    int a_zero;               // its zero point
    float a_scale;
    int b_n_major;
    const float *col_scale;   // the weights' scales: one a column (and batch entry)
    int64_t col_scale_stride, col_scale_lo, col_scale_hi;
    const int32_t *colsum;    // sum_k w[k, col] per (batch entry, column), when a_zero != 0
    const void *addend;       // a bf16 tensor laid out as the result, added to the rounded bf16 product (staged stores only)
    int guarded;
    int vec_ok;
    uint32_t *ovf;
    uint32_t *status;
};

PSK_DEV uint32_t instr_desc_i8(int a_unsigned, int b_n_major)
{
    uint32_t d = 0;
    d |= 2u << 4;                         // accumulator: 32-bit signed integers
    d |= (a_unsigned ? 0u : 1u) << 7;     // A: 0 unsigned 8-bit, 1 signed 8-bit
    d |= 1u << 10;                        // B: signed 8-bit
    d |= (b_n_major ? 1u : 0u) << 16;     // B major: 0 K, 1 MN
    d |= (uint32_t)(BN >> 3) << 17;
    d |= (uint32_t)(BM >> 4) << 24;
    return d;
}

// Two bf16 sums of a 32-bit word's halves, each rounded to nearest even.
PSK_DEV uint32_t add_bf16x2(uint32_t a, uint32_t b)
{
    return pack_bf16x2_hw(__fadd_rn(bits_f32(a << 16), bits_f32(b << 16)), __fadd_rn(bits_f32(a & 0xffff0000u), bits_f32(b & 0xffff0000u)));
}

PSK_DEV void umma_i8(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// sum_k w[k, col] for every (batch entry, column), wrapped to 32 bits: `out` starts at zero and every block adds
// its run of the summed axis (integer additions that wrap are associative, so the order the atomics land in does
// not matter). blockIdx.y: the run. N-major weights (s_n = 1): a thread a column, neighbouring threads neighbouring
// columns. K-major (s_k = 1): a warp a column, its lanes neighbouring k.
constexpr int COLSUM_RUN = 512;
static __global__ void __launch_bounds__(256) k_colsum_i8(const int8_t *w, int64_t n, int64_t k, int64_t batch, int64_t batch_lo, int64_t s_n, int64_t s_k, int64_t s_lo, int64_t s_hi, int32_t *out)
{
    const int64_t k0 = (int64_t)blockIdx.y * COLSUM_RUN, k1 = k0 + COLSUM_RUN < k ? k0 + COLSUM_RUN : k;
    const int64_t total = n * batch;
    if (s_k != 1) {
        const int64_t step = (int64_t)gridDim.x * blockDim.x;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
            const int64_t b = i / n, c = i - b * n;
            const int8_t *p = w + (b % batch_lo) * s_lo + (b / batch_lo) * s_hi + c * s_n;
            uint32_t acc = 0;
#pragma unroll 8
            for (int64_t t = k0; t < k1; ++t) acc += (uint32_t)(int32_t)p[t * s_k];
            atomicAdd(reinterpret_cast<unsigned int *>(out) + i, acc);
        }
    } else {
        const int lane = threadIdx.x & 31;
        const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
        for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < total; i += warps) {
            const int64_t b = i / n, c = i - b * n;
            const int8_t *p = w + (b % batch_lo) * s_lo + (b / batch_lo) * s_hi + c * s_n;
            uint32_t acc = 0;
            for (int64_t t = k0 + lane; t < k1; t += 32) acc += (uint32_t)(int32_t)p[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) atomicAdd(reinterpret_cast<unsigned int *>(out) + i, acc);
        }
    }
}

// n·base rounded once to bf16: the fast way when that is certain to be the exact routine's code.
PSK_DEV uint32_t count_to_bf16(int32_t n, double base)
{
    const float f = __double2float_rn((double)n * base);
    const uint32_t fb = __float_as_uint(f);
    // f is within half a unit of binary32 of n·base (plus 2^-53): the bf16 rounding of f is that of n·base
    // unless f sits within a unit of a midpoint between two bf16 numbers
    if (((fb & 0xffffu) - 0x7fffu) <= 2u) return round_count_to_float((int64_t)n, base, 7, 8);
    return (fb + 0x7fffu + ((fb >> 16) & 1u)) >> 16;
}

// The same in binary32 arithmetic only, for the staged bf16 epilogue. `basef` is the column's base rounded to
// binary32; n, basef and their product each carry at most 2^-24 of relative error, so f is within three of its own
// units of n·base, and the two round to the same bf16 number unless f lies within three units of a midpoint (low
// half 0x8000) or is subnormal. Those few go the exact way, with the base taken again from its two factors.
// (The exact routine is kept out of line: inlined into each of the 32 unrolled elements of the epilogue it made the
// loop some thousands of instructions long, and the warps waited on the instruction cache more than on anything.)
static __device__ __noinline__ uint32_t count_to_bf16_exact(int32_t n, double sa, const float *scale_of_col)
{
    return round_count_to_float((int64_t)n, sa * (double)*scale_of_col, 7, 8);
}

PSK_DEV uint32_t count_to_bf16_quick(int32_t n, float basef, double sa, const float *scale_of_col)
{
    const float f = (float)n * basef;
    const uint32_t fb = __float_as_uint(f);
    // (a zero sum has a zero exponent field and goes the exact way, which answers +0)
    if ((((fb & 0xffffu) - 0x7ffcu) <= 8u) || !(fb & 0x7f800000u)) return count_to_bf16_exact(n, sa, scale_of_col);
    return (fb + 0x7fffu + ((fb >> 16) & 1u)) >> 16;
}

static __device__ __noinline__ uint32_t count_to_f32_exact(int32_t n, double base)
{
    return round_count_to_float((int64_t)n, base, 23, 8);
}

PSK_DEV uint32_t count_to_f32(int32_t n, double base)
{
    const double d = (double)n * base;
    const uint64_t db = (uint64_t)__double_as_longlong(d);
    const uint32_t low = (uint32_t)(db & 0x1fffffffu); // the 29 bits binary32 drops from a normal number
    const double mag = fabs(d);
    if (!(mag >= 1.1754943508222875e-38) || ((low - 0x0fffffffu) <= 2u)) return count_to_f32_exact(n, base);
    return __float_as_uint(__double2float_rn(d));
}

// n·base / s rounded to the nearest integer, ties to even: fast when the quotient in binary64 is clear of a tie.
PSK_DEV int64_t count_to_affine(int32_t n, double base, float s)
{
    const double v = (double)n * base / (double)s; // within 2^-51 of the exact quotient, relatively
    if (fabs(v) >= 1e6) return v > 0 ? (1ll << 40) : -(1ll << 40); // far outside every code range: the caller's clamp decides
    const double r = rint(v);
    if (fabs(fabs(v - r) - 0.5) > 1e-3) return (int64_t)r;
    int64_t mb;
    int eb;
    take_apart(base, mb, eb);
    return quotient_round_exact(n < 0, (u128_t)(n < 0 ? -(int64_t)n : (int64_t)n) * (u128_t)mb, eb, s);
}

// ADD: the instance that adds P.addend to a bf16 result (its own instance so that the plain one keeps its registers).
template <int MT, bool ADD = false>
__global__ void __launch_bounds__(THREADS, 1) k_gemm_i8(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ Params P)
{
    constexpr int STAGES = Cfg<MT>::STAGES, A_BYTES = Cfg<MT>::A_BYTES, TILE_BYTES = Cfg<MT>::TILE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * A_BYTES;
    uint64_t *bars = (uint64_t *)(smem + TILE_BYTES);
    // bars: full[STAGES], empty[STAGES], tmem_full[2] (MT = 2 uses the first), tmem_empty[2]
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 4);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = tc::smem_u32(bars), empty0 = tc::smem_u32(bars + STAGES);
    const uint32_t tfull0 = tc::smem_u32(bars + 2 * STAGES), tempty0 = tc::smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(full0 + 8 * s, 1);
            tc::mbar_init(empty0 + 8 * s, 1);
        }
        tc::mbar_init(tfull0, 1);
        tc::mbar_init(tfull0 + 8, 1);
        for (int s = 0; s < 2; ++s) tc::mbar_init(tempty0 + 8 * s, 8); // one arrival per epilogue warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int64_t tiles_per_batch = P.tiles_m * P.tiles_n;
    const int64_t total_tiles = tiles_per_batch * P.batch;
    const int num_kb = (int)((P.k + BKB - 1) / BKB);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int64_t b = t / tiles_per_batch, r = t % tiles_per_batch;
                int64_t mt, nt;
                tc::tile_of(r, P.tiles_m, P.tiles_n, P.panel, mt, nt);
                const int m0 = (int)mt * BM * MT, n0 = (int)nt * BN;
                const int blo = (int)(b % P.batch_lo), bhi = (int)(b / P.batch_lo);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = tc::mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag, P.status, 0x71u);
                    if (!ok) break;
                    const uint32_t fb = full0 + 8 * stage;
                    tc::mbar_expect_tx(fb, A_BYTES + B_BYTES);
                    const int k0 = kb * BKB;
                    tc::tma_load_4d(tc::smem_u32(smem_a + stage * A_BYTES), &map_a, fb, k0, m0, blo, bhi);
                    if (!P.b_n_major) {
                        tc::tma_load_4d(tc::smem_u32(smem_b + stage * B_BYTES), &map_b, fb, k0, n0, blo, bhi);
                    } else {
                        // 128 rows of the summed axis by 128 contiguous columns a box
#pragma unroll
                        for (int c = 0; c < BN / 128; ++c)
                            tc::tma_load_4d(tc::smem_u32(smem_b + stage * B_BYTES + c * 16384), &map_b, fb, n0 + c * 128, k0, blo, bhi);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc_i8(P.a_unsigned, P.b_n_major);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = tc::mbar_wait(full0 + 8 * stage, phase, abort_flag, P.status, 0x73u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = tc::smem_u32(smem_a + stage * A_BYTES);
                    const uint32_t b_addr = tc::smem_u32(smem_b + stage * B_BYTES);
#pragma unroll
                    for (int h = 0; h < MT; ++h) {
                        const uint32_t slot = MT == 2 ? (uint32_t)h : acc; // the accumulator these products add into
                        if (kb == 0) {
                            // it must have been drained by the epilogue of the tile that used it before
                            ok = tc::mbar_wait(tempty0 + 8 * slot, acc_phase ^ 1u, abort_flag, P.status, 0x72u);
                            if (!ok) break;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
#pragma unroll
                        for (int k = 0; k < BKB / 32; ++k) {
                            // 32 elements of the summed axis a product: 32 bytes along a K-major row, 32 rows of
                            // 128 bytes of an N-major tile
                            const uint64_t ad = tc::smem_desc(a_addr + h * (BM * BKB) + k * 32, 16, 1024);
                            const uint64_t bd = P.b_n_major ? tc::smem_desc(b_addr + k * 4096, 16384, 1024) : tc::smem_desc(b_addr + k * 32, 16, 1024);
                            umma_i8(tmem_base + slot * BN, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    if (!ok) break;
                    tc::umma_commit(empty0 + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc::umma_commit(tfull0 + 8 * (MT == 2 ? 0u : acc));
                if (MT == 2) acc_phase ^= 1u;
                else if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        const int quad = warp & 3;
        uint32_t acc = 0, acc_phase = 0, ovf = 0;
        bool ok = true;
        const int half_id = (warp - 2) >> 2;
        uint4 *stage_out = reinterpret_cast<uint4 *>(smem + TILE_BYTES + BAR_BYTES) + (warp - 2) * 32 * 8;
        float *scale_area = reinterpret_cast<float *>(smem + TILE_BYTES + BAR_BYTES + STAGE_OUT);
        const bool staged = P.vec_ok && !P.out_affine && (P.out_dtype == PSK_BF16 || P.out_dtype == PSK_F32);
        const double sa = (double)P.a_scale;
        // A tile's part of the addend, asked into the L2 a tile ahead: this lane's row, the 64 bytes of each of this
        // warp's column groups. The loads that add it (below) then find it there.
        auto prefetch_addend = [&](int64_t t) {
            if (t >= total_tiles) return;
            const int64_t b = t / tiles_per_batch, r = t % tiles_per_batch;
            int64_t mt, nt;
            tc::tile_of(r, P.tiles_m, P.tiles_n, P.panel, mt, nt);
            const int64_t prow = mt * BM * MT + quad * 32 + lane, n0 = nt * BN;
            if (prow >= P.m) return;
            const uint32_t rcnt = (uint32_t)(P.c_row_lo_count < 0x7fffffffll ? P.c_row_lo_count : 0x7fffffffll);
            const uint32_t ccnt = (uint32_t)(P.c_col_lo_count < 0x7fffffffll ? P.c_col_lo_count : 0x7fffffffll);
            const uint32_t rq = (uint32_t)prow / rcnt;
            const int64_t roff = (b % P.batch_lo) * P.c_lo + (b / P.batch_lo) * P.c_hi + (int64_t)rq * P.c_row_hi + (int64_t)((uint32_t)prow - rq * rcnt) * P.c_row_lo;
#pragma unroll
            for (int c0 = half_id * 32; c0 < BN; c0 += 64) {
                const int64_t pcol = n0 + c0;
                if (pcol < P.n) {
                    const uint32_t cq = (uint32_t)pcol / ccnt;
                    const uint16_t *pa = (const uint16_t *)P.addend + roff + (int64_t)cq * P.c_col_hi + (int64_t)((uint32_t)pcol - cq * ccnt);
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(pa));
                }
            }
        };
        if constexpr (ADD) prefetch_addend(blockIdx.x);
        for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            const int64_t b = t / tiles_per_batch, r = t % tiles_per_batch;
            int64_t mt, nt;
            tc::tile_of(r, P.tiles_m, P.tiles_n, P.panel, mt, nt);
            const int64_t m0 = mt * BM * MT, n0 = nt * BN;
            const int64_t blo = b % P.batch_lo, bhi = b / P.batch_lo;
            if constexpr (ADD) prefetch_addend(t + gridDim.x); // the next tile's, while this one is rescaled and stored
            ok = tc::mbar_wait(tfull0 + 8 * (MT == 2 ? 0u : acc), acc_phase, abort_flag, P.status, 0x74u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float *cs_base = P.col_scale + blo * P.col_scale_lo + bhi * P.col_scale_hi;
            const int32_t *sum_base = P.colsum ? P.colsum + b * P.n : nullptr;
#pragma unroll 1
            for (int mh = 0; mh < MT; ++mh) {
                const int64_t row0 = m0 + mh * BM + quad * 32;
                const int64_t boff = blo * P.c_lo + bhi * P.c_hi;
                const int64_t row = row0 + lane;
                const uint32_t rcnt = (uint32_t)(P.c_row_lo_count < 0x7fffffffll ? P.c_row_lo_count : 0x7fffffffll);
                const uint32_t ccnt = (uint32_t)(P.c_col_lo_count < 0x7fffffffll ? P.c_col_lo_count : 0x7fffffffll);
                int64_t row_off;
                {
                    const uint32_t rq = (uint32_t)row / rcnt;
                    row_off = boff + (int64_t)rq * P.c_row_hi + (int64_t)((uint32_t)row - rq * rcnt) * P.c_row_lo;
                }
                const uint32_t slot = MT == 2 ? (uint32_t)mh : acc;
                const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + slot * BN;
                if (staged) {
                    // Groups of 32 columns of this lane's row, each rescaled, packed and sent through shared memory so
                    // that a store instruction writes whole runs of a row (bf16: 64 bytes; f32: 128 bytes). The
                    // accumulators come out of tensor memory sixteen columns at a time into two buffers in turn, the
                    // next sixteen on their way while these are rescaled.
                    uint32_t va[16], vb[16];
                    tc::tmem_ld16(tbase + half_id * 32, va);
#pragma unroll 1
                    for (int c0 = half_id * 32; c0 < BN; c0 += 64) {
                        const int64_t col = n0 + c0;
                        const bool any = col < P.n;
                        // this lane fetches the scale (and the zero-point correction) of column col + lane
                        const bool col_live = col + lane < P.n;
                        const float *my_scale = cs_base + (col_live ? (col + lane) * P.col_scale_stride : 0);
                        const float scale_l = col_live ? *my_scale : 0.0f;
                        const uint32_t corr_l = (sum_base && col_live) ? (uint32_t)P.a_zero * (uint32_t)sum_base[col + lane] : 0u;
                        uint32_t packed[32];
                        const double base_l = sa * (double)scale_l;
                        const bool whole = col + 32 <= P.n; // the group's 32 columns all exist
                        const float basef_l = __double2float_rn(base_l);
                        float *wscale = scale_area + (warp - 2) * 32; // this warp's 32 columns: bases (bf16 result) or scales (f32)
                        __syncwarp();
                        wscale[lane] = P.out_dtype == PSK_BF16 ? basef_l : scale_l;
                        __syncwarp();
                        const uint32_t live_mask = !any ? 0u : whole ? 0xffffffffu : ((1u << (uint32_t)(P.n - col)) - 1u);
                        // The rescale of sixteen sums in two phases: every element's quick result and whether it is
                        // certain, with no branch in between, so that the independent chains overlap (with a test and
                        // a call after each element the warps ran them one after the other, and the rescale cost more
                        // than the tile's products); then, for the few that are not certain, the exact routine.
                        auto rescale16 = [&](uint32_t (&vh)[16], int off) {
                            if (sum_base) { // the zero point's correction first (a shuffle a column)
#pragma unroll
                                for (int j = 0; j < 16; ++j) vh[j] -= __shfl_sync(0xffffffffu, corr_l, off + j);
                            }
                            uint32_t unsure = 0;
                            if (P.out_dtype == PSK_BF16) {
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    const uint32_t fb = __float_as_uint((float)(int32_t)vh[j] * wscale[off + j]);
                                    // within three binary32 units of a midpoint between bf16 numbers, or subnormal or zero
                                    // (a sum of zero is +0 whatever the scale: rows past the operand's end are all zeros)
                                    unsure |= ((((fb & 0xffffu) - 0x7ffcu) <= 8u || !(fb & 0x7f800000u)) && vh[j] != 0u) ? (1u << j) : 0u;
                                    packed[off + j] = vh[j] != 0u ? (fb + 0x7fffu + ((fb >> 16) & 1u)) >> 16 : 0u;
                                }
                                unsure &= live_mask >> off;
                                if (unsure) {
#pragma unroll
                                    for (int j = 0; j < 16; ++j)
                                        if ((unsure >> j) & 1u) packed[off + j] = count_to_bf16_exact((int32_t)vh[j], sa, cs_base + (col + off + j) * P.col_scale_stride);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    const double d = (double)(int32_t)vh[j] * (sa * (double)wscale[off + j]);
                                    const uint32_t low = (uint32_t)((uint64_t)__double_as_longlong(d) & 0x1fffffffu); // the 29 bits binary32 drops from a normal number
                                    unsure |= ((!(fabs(d) >= 1.1754943508222875e-38) || (low - 0x0fffffffu) <= 2u) && vh[j] != 0u) ? (1u << j) : 0u;
                                    packed[off + j] = vh[j] != 0u ? __float_as_uint(__double2float_rn(d)) : 0u;
                                }
                                unsure &= live_mask >> off;
                                if (unsure) {
#pragma unroll
                                    for (int j = 0; j < 16; ++j)
                                        if ((unsure >> j) & 1u) packed[off + j] = count_to_f32_exact((int32_t)vh[j], sa * (double)wscale[off + j]);
                                }
                            }
                        };
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); // va: columns c0 .. c0 + 15
                        tc::tmem_ld16(tbase + c0 + 16, vb);
                        rescale16(va, 0);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); // vb: columns c0 + 16 .. c0 + 31
                        if (c0 + 64 < BN) tc::tmem_ld16(tbase + c0 + 64, va);             // the next group's first half
                        rescale16(vb, 16);
                        if (!any) continue;
                        if (!whole) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) packed[i] = ((live_mask >> i) & 1u) ? packed[i] : 0u;
                        }
                        if (P.out_dtype == PSK_F32) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                stage_out[lane * 8 + (q ^ (lane & 7))] = make_uint4(packed[8 * q] | (packed[8 * q + 1] << 16), packed[8 * q + 2] | (packed[8 * q + 3] << 16), packed[8 * q + 4] | (packed[8 * q + 5] << 16), packed[8 * q + 6] | (packed[8 * q + 7] << 16));
                        }
                        __syncwarp();
                        const uint32_t cq = (uint32_t)col / ccnt;
                        const int64_t col_off = (int64_t)cq * P.c_col_hi + (int64_t)((uint32_t)col - cq * ccnt);
                        const int units = P.out_dtype == PSK_F32 ? 8 : 4;      // 16-byte units of a row's 32 columns
                        const int eb = P.out_dtype == PSK_F32 ? 4 : 2;
                        const int live = (int)(((P.n - col) >= 32 ? 32 : (P.n - col)) * eb / 16);
                        const int rows_a_pass = 32 / units;                      // rows one store instruction covers
                        const int unit = lane % units;
                        if constexpr (ADD) {
                            // bf16 (units = 4): the addend plus the rounded product, rounded again. The addend's lines were
                            // asked into the L2 a tile ahead; the four passes' loads go out together. (Loading them
                            // earlier, at the group's start or before its second half, made the compiler spill around
                            // them and was slower.)
                            int64_t offs[4];
                            uint4 ad[4];
#pragma unroll
                            for (int it = 0; it < 4; ++it) {
                                const int rr = it * 8 + lane / 4;
                                const int64_t rrow = row0 + rr;
                                offs[it] = -1;
                                ad[it] = make_uint4(0u, 0u, 0u, 0u);
                                if (rrow < P.m && unit < live) {
                                    const uint32_t rq = (uint32_t)rrow / rcnt;
                                    offs[it] = boff + (int64_t)rq * P.c_row_hi + (int64_t)((uint32_t)rrow - rq * rcnt) * P.c_row_lo + col_off + unit * 8;
                                    ad[it] = *reinterpret_cast<const uint4 *>((const uint16_t *)P.addend + offs[it]);
                                }
                            }
#pragma unroll
                            for (int it = 0; it < 4; ++it) {
                                const int rr = it * 8 + lane / 4;
                                if (offs[it] >= 0) {
                                    uint4 w = stage_out[rr * 8 + (unit ^ (rr & 7))];
                                    w.x = add_bf16x2(ad[it].x, w.x); w.y = add_bf16x2(ad[it].y, w.y); w.z = add_bf16x2(ad[it].z, w.z); w.w = add_bf16x2(ad[it].w, w.w);
                                    *reinterpret_cast<uint4 *>((uint16_t *)P.c + offs[it]) = w;
                                }
                            }
                        } else {
                            for (int it = 0; it < units; ++it) {
                                const int rr = it * rows_a_pass + lane / units;
                                const int64_t rrow = row0 + rr;
                                if (rrow < P.m && unit < live) {
                                    const uint32_t rq = (uint32_t)rrow / rcnt;
                                    const int64_t off = boff + (int64_t)rq * P.c_row_hi + (int64_t)((uint32_t)rrow - rq * rcnt) * P.c_row_lo + col_off;
                                    const uint4 w = stage_out[rr * 8 + (unit ^ (rr & 7))];
                                    *reinterpret_cast<uint4 *>((uint8_t *)P.c + off * eb + unit * 16) = w;
                                }
                            }
                        }
                        __syncwarp();
                    }
                } else {
#pragma unroll 1
                for (int c0 = half_id * 32; c0 < BN; c0 += 64) {
                    uint32_t v[32];
                    const int64_t col = n0 + c0;
                    // this lane fetches the scale (and the zero-point correction) of column col + lane while the
                    // accumulators come out of tensor memory; the row's loop below takes them by shuffle
                    const bool col_live = col + lane < P.n;
                    const float *my_scale = cs_base + (col_live ? (col + lane) * P.col_scale_stride : 0);
                    const float scale_l = col_live ? *my_scale : 0.0f;
                    const uint32_t corr_l = (sum_base && col_live) ? (uint32_t)P.a_zero * (uint32_t)sum_base[col + lane] : 0u;
                    tc::tmem_ld32(tbase + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (col >= P.n) continue;
                    if (row < P.m) {
                        for (int i = 0; i < 32; ++i) {
                            const int64_t cc = col + i;
                            if (cc >= P.n) break;
                            int32_t nsum = (int32_t)v[i];
                            if (sum_base) nsum = (int32_t)((uint32_t)nsum - (uint32_t)P.a_zero * (uint32_t)sum_base[cc]);
                            const double base = sa * (double)cs_base[cc * P.col_scale_stride];
                            const int64_t o = row_off + (int64_t)((uint32_t)cc / ccnt) * P.c_col_hi + (int64_t)((uint32_t)cc % ccnt);
                            if (P.out_affine) {
                                const int64_t q = affine_clamp(count_to_affine(nsum, base, P.out_scale) + P.out_zero, P.out_affine);
                                if (P.out_affine == 2) ((uint8_t *)P.c)[o] = (uint8_t)q;
                                else ((int8_t *)P.c)[o] = (int8_t)q;
                            } else if (P.out_dtype == PSK_F32) {
                                ((uint32_t *)P.c)[o] = count_to_f32(nsum, base);
                            } else if (P.out_dtype == PSK_BF16) {
                                ((uint16_t *)P.c)[o] = (uint16_t)count_to_bf16(nsum, base);
                            } else if (P.out_dtype == PSK_F16) {
                                const uint32_t c = round_count_to_float((int64_t)nsum, base, 10, 5);
                                ((uint16_t *)P.c)[o] = (uint16_t)c;
                                if ((c & 0x7fffu) == 0x7c00u) ovf |= 1u;
                            } else { // e8m15
                                const uint32_t c = round_count_to_float((int64_t)nsum, base, 15, 8);
                                store_e8m15((uint8_t *)P.c, o, c);
                                if ((c & 0x7fffffu) == 0x7f8000u) ovf |= 1u;
                            }
                        }
                    }
                }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(tempty0 + 8 * slot);
            }
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

} // namespace tci8
} // namespace psk
