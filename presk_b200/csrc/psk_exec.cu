// The CUDA executor behind include/presk_cuda.h: device buffers, the dispatch
// of a launch to a kernel of this library, the overflow guard's flags.
//
// It stands where the reference's `NativeExec` stands
// (crates/presk-cranelift/src/lib.rs:1544-1693): given a kernel and its
// buffers it runs the loop nest. Where the native executor compiles the nest
// it is given, this one recognises which of its ahead-of-time kernels the
// launch is (by operation, strides and types) and refuses what it has none
// for; it never computes on the host.
#include <cuda.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/presk_cuda.h"
#include "psk_gemm_tc.cuh"
#include "psk_kernels.cuh"
#include "psk_hot.cuh"
#include "psk_attn.cuh"
#include "psk_attn_step.cuh"
#include "psk_gemm_i8.cuh"
#include "psk_gemm_tc2.cuh"

using namespace psk;

namespace {

constexpr int kFlagSlots = 4096;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::string g_create_error;

} // namespace

struct psk_exec {
    int device = 0;
    int sms = 148;
    cudaStream_t stream = nullptr;
    std::string error;
    size_t live = 0, peak = 0;
    std::unordered_map<void *, size_t> sizes;          // every live buffer and its bytes
    std::map<size_t, std::vector<void *>> pool;        // freed buffers by exact size
    std::unordered_map<void *, int64_t> causal;        // buffers a causal_mask launch wrote: its n
    // int8 weights read by the tensor-core contraction: their integers as bf16, made once per buffer
    // (weights are never written after they are stored), keyed by the codes' address and count
    std::map<std::pair<const void *, int64_t>, void *> widened;
    size_t widened_bytes = 0;                 // what the kept copies hold
    size_t widened_budget = (size_t)4 << 30;  // beyond it a copy lives for one contraction only (PSK_WIDENED_MB)
    uint32_t *flags = nullptr;                         // kFlagSlots words of the overflow guard
    uint32_t *status = nullptr;                        // one word: kernel-side trouble
    std::vector<int64_t> flag_serial;                  // the launch each slot was last given to
    int64_t guarded_since = 0;
    int64_t latched_overflow = 0;                      // 1 + serial of an overflow found when the slots were recycled
    int64_t launches = 0, kernels = 0;
    std::string overflow_name;
    bool profiling = false;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    double last_ms = -1.0;
    // per-launch records while profiling: two pooled events, what ran, its algorithmic work
    struct ProfRec { std::string name; const char *kernel; double flops, bytes; cudaEvent_t a, b; };
    std::vector<ProfRec> prof;
    std::vector<cudaEvent_t> event_pool;
    std::string prof_text;
    const char *last_kernel = "";
    double last_flops = 0;
    EncodeTiledFn encode = nullptr;
    bool tc_attr_set = false;
    bool softmax_attr_set = false;
    bool attn_attr_set = false;
    bool attn_step_attr_set = false;
    bool lut_aff_attr_set = false;
    bool i8_attr_set = false;
    uint16_t *silu_table = nullptr; // silu of every bf16 code, computed once by the device's own exact function
};

namespace {

int fail(psk_exec *e, int code, const std::string &msg)
{
    if (e) e->error = msg;
    else g_create_error = msg;
    return code;
}

#define CUDA_TRY(e, call)                                                                   \
    do {                                                                                    \
        cudaError_t err__ = (call);                                                         \
        if (err__ != cudaSuccess)                                                           \
            return fail(e, PSK_E10001, std::string(#call) + ": " + cudaGetErrorString(err__)); \
    } while (0)

size_t elem_bytes(int dtype)
{
    switch (dtype) {
    case PSK_F64: case PSK_I64: return 8;
    case PSK_F32: return 4;
    case PSK_BF16: case PSK_F16: return 2;
    case PSK_E8M15: return 3;
    default: return 1;
    }
}

int grid_for(const psk_exec *e, int64_t work, int block, int per_sm)
{
    int64_t blocks = (work + block - 1) / block;
    int64_t cap = (int64_t)e->sms * per_sm;
    return (int)std::max<int64_t>(1, std::min(blocks, cap));
}

// ---- the device form of a launch ------------------------------------------
void fill_operand(DevOperand &d, const psk_operand &o, void *base, const float *scales, int naxes)
{
    d.p = (const uint8_t *)base + o.offset * (int64_t)elem_bytes(o.dtype);
    d.scales = scales;
    d.dtype = o.dtype;
    d.is_index = o.is_index;
    d.affine = o.affine;
    d.affine_zero = o.affine_zero;
    d.affine_scale = o.affine_scale;
    for (int a = 0; a < PSK_MAX_AXES; ++a) {
        d.stride[a] = a < naxes ? o.stride[a] : 0;
        d.sstride[a] = a < naxes ? o.scale_stride[a] : 0;
    }
}

// Merges adjacent outer axes every operand walks as one, and drops axes of
// length one: fewer divisions a thread, longer contiguous runs.
void coalesce_outer(DevLaunch &L)
{
    const int n = L.n_outer, ni = L.n_inner;
    auto move_axis = [&](int to, int from) {
        if (to == from) return;
        L.dims[to] = L.dims[from];
        L.out.stride[to] = L.out.stride[from];
        for (int i = 0; i < L.n_in; ++i) {
            L.in[i].stride[to] = L.in[i].stride[from];
            L.in[i].sstride[to] = L.in[i].sstride[from];
        }
    };
    // drop axes of length one (keeping one axis when there is nothing else)
    int kept = 0;
    for (int a = 0; a < n; ++a)
        if (L.dims[a] != 1) move_axis(kept++, a);
    if (kept == 0 && n > 0) {
        move_axis(0, n - 1);
        kept = 1;
    }
    // merge axis a into the one before when everyone walks them as one
    int r = 0;
    for (int a = 1; a < kept; ++a) {
        bool ok = L.out.stride[r] == L.out.stride[a] * L.dims[a];
        for (int i = 0; ok && i < L.n_in; ++i)
            ok = L.in[i].stride[r] == L.in[i].stride[a] * L.dims[a] && L.in[i].sstride[r] == L.in[i].sstride[a] * L.dims[a];
        if (ok) {
            int64_t d = L.dims[r] * L.dims[a];
            move_axis(r, a);
            L.dims[r] = d;
        } else {
            move_axis(++r, a);
        }
    }
    const int new_outer = kept == 0 ? 0 : r + 1;
    for (int c = 0; c < ni; ++c) move_axis(new_outer + c, n + c);
    L.n_outer = new_outer;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

// Which compile-time program a group's steps are, or -1 (psk_hot.cuh `EwProg`).
int match_program(const psk_launch *l)
{
    auto is = [&](int k, int prim, int nargs, int a, int b) {
        const psk_step &s = l->steps[k];
        return s.prim == prim && s.nargs == nargs && s.src[0] == a && (nargs == 1 || s.src[1] == b);
    };
    if (l->n_steps == 1 && l->n_inputs == 2) {
        if (is(0, PSK_ADD, 2, 0, 1)) return EW_ADD;
        if (is(0, PSK_SUB, 2, 0, 1)) return EW_SUB;
        if (is(0, PSK_MUL, 2, 0, 1)) return EW_MUL;
        if (is(0, PSK_DIV, 2, 0, 1)) return EW_DIV;
    }
    if (l->n_steps == 2 && l->n_inputs == 3 && is(0, PSK_DIV, 2, 0, 1) && is(1, PSK_MUL, 2, -1, 2)) return EW_DIV_MUL;
    if (l->n_steps == 2 && l->n_inputs == 1 && is(0, PSK_SIGMOID, 1, 0, 0) && is(1, PSK_MUL, 2, 0, -1)) return EW_SILU;
    if (l->n_steps == 4 && l->n_inputs == 2 && is(0, PSK_SIGMOID, 1, 0, 0) && is(1, PSK_MUL, 2, 0, -1) && is(2, PSK_ROUND, 1, -2, 0) && l->steps[2].imm == PSK_BF16 && is(3, PSK_MUL, 2, -3, 1)) return EW_SILU_MUL;
    if (l->n_steps == 3 && l->n_inputs == 4 && is(0, PSK_MUL, 2, 0, 1) && is(1, PSK_MUL, 2, 2, 3)) {
        if (is(2, PSK_SUB, 2, -1, -2)) return EW_MUL_MUL_SUB;
        if (is(2, PSK_ADD, 2, -1, -2)) return EW_MUL_MUL_ADD;
    }
    return -1;
}

template <int PROG>
void launch_prog(psk_exec *e, const EwParams &E)
{
    const int64_t work = (int64_t)E.rows * E.colv;
    const int g = grid_for(e, (work + 3) / 4, 256, 8);
    k_ew_prog<PROG, 4><<<g, 256, 0, e->stream>>>(E);
}

// Whether the operand can be read eight last-axis elements at a time.
bool vec8_operand(const DevOperand &o, const int64_t *dims, int n_outer, bool is_out)
{
    const int last = n_outer - 1;
    if (o.dtype == PSK_E8M15 || o.dtype == PSK_E4M3 || o.dtype == PSK_I8 || o.dtype == PSK_F64 || o.dtype == PSK_I64) {
        // read element by element inside the vector path: any alignment will do,
        // but an integer weight's scales must walk with it
        if (is_out) return o.stride[last] == 1;
        return o.stride[last] == 0 || o.stride[last] == 1;
    }
    if (o.stride[last] == 0 && !is_out) return true;
    if (o.stride[last] != 1) return false;
    const size_t eb = elem_bytes(o.dtype);
    if (((uintptr_t)o.p % (8 * eb > 16 ? 16 : 8 * eb)) != 0) return false;
    for (int a = 0; a < last; ++a)
        if (o.stride[a] % 8 != 0) return false;
    (void)dims;
    return true;
}

// ---- a contraction seen as a batched matrix product ------------------------
struct GemmMap {
    int64_t m = 1, n = 1, k = 1, batch = 1, batch_lo = 1;
    int64_t a_row = 0, a_k = 0, a_lo = 0, a_hi = 0;
    int64_t b_k = 0, b_n = 0, b_lo = 0, b_hi = 0;
    int64_t bs_n = 0, bs_lo = 0, bs_hi = 0;
    int64_t c_row_lo_count = 1, c_row_lo = 0, c_row_hi = 0;
    int64_t c_col_lo_count = 1, c_col_lo = 0, c_col_hi = 0;
    int64_t c_lo = 0, c_hi = 0;
};

struct Level {
    int64_t count, stride;
};

// The axes `ax` (in iteration order, outermost first) as at most `max_levels`
// strided levels of one operand, outermost first.
bool levels_of(const int64_t *dims, const int64_t *stride, const std::vector<int> &ax, size_t max_levels, std::vector<Level> &out)
{
    out.clear();
    for (int a : ax) {
        if (dims[a] == 1) continue;
        if (!out.empty() && out.back().stride == stride[a] * dims[a]) {
            out.back().count *= dims[a];
            out.back().stride = stride[a];
        } else {
            out.push_back({dims[a], stride[a]});
        }
    }
    return out.size() <= max_levels;
}

bool map_gemm(const DevLaunch &L, GemmMap &g)
{
    if (L.n_in != 2) return false;
    const DevOperand &A = L.in[0], &B = L.in[1];
    std::vector<int> ax_b, ax_m, ax_n, ax_k;
    for (int a = 0; a < L.n_outer; ++a) {
        if (L.dims[a] == 1) continue;
        bool ina = A.stride[a] != 0, inb = B.stride[a] != 0;
        if (ina && inb) ax_b.push_back(a);
        else if (ina) ax_m.push_back(a);
        else if (inb) ax_n.push_back(a);
        else return false; // an output axis no operand carries
    }
    for (int c = 0; c < L.n_inner; ++c) {
        int a = L.n_outer + c;
        if (L.dims[a] == 1) continue;
        if (A.stride[a] == 0 || B.stride[a] == 0) return false;
        ax_k.push_back(a);
    }
    std::vector<Level> lv;
    auto prod = [&](const std::vector<int> &ax) { int64_t p = 1; for (int a : ax) p *= L.dims[a]; return p; };
    g.m = prod(ax_m); g.n = prod(ax_n); g.k = prod(ax_k); g.batch = prod(ax_b);
    // K: one level in both operands
    if (!levels_of(L.dims, A.stride, ax_k, 1, lv)) return false;
    g.a_k = lv.empty() ? 1 : lv[0].stride;
    if (!levels_of(L.dims, B.stride, ax_k, 1, lv)) return false;
    g.b_k = lv.empty() ? 1 : lv[0].stride;
    // M: one level in A, two in C
    if (!levels_of(L.dims, A.stride, ax_m, 1, lv)) return false;
    g.a_row = lv.empty() ? 0 : lv[0].stride;
    if (!levels_of(L.dims, L.out.stride, ax_m, 2, lv)) return false;
    if (lv.size() == 2) { g.c_row_hi = lv[0].stride; g.c_row_lo_count = lv[1].count; g.c_row_lo = lv[1].stride; }
    else if (lv.size() == 1) { g.c_row_hi = 0; g.c_row_lo_count = lv[0].count; g.c_row_lo = lv[0].stride; }
    // N: one level in B (and its scales), two in C
    if (!levels_of(L.dims, B.stride, ax_n, 1, lv)) return false;
    g.b_n = lv.empty() ? 0 : lv[0].stride;
    if (B.dtype == PSK_I8) {
        if (!levels_of(L.dims, B.sstride, ax_n, 1, lv)) return false;
        g.bs_n = lv.empty() ? 0 : lv[0].stride;
        for (int a : ax_k) if (B.sstride[a] != 0) return false;
    }
    if (!levels_of(L.dims, L.out.stride, ax_n, 2, lv)) return false;
    if (lv.size() == 2) { g.c_col_hi = lv[0].stride; g.c_col_lo_count = lv[1].count; g.c_col_lo = lv[1].stride; }
    else if (lv.size() == 1) { g.c_col_hi = 0; g.c_col_lo_count = lv[0].count; g.c_col_lo = lv[0].stride; }
    // batch: two levels everywhere, split at the same place
    std::vector<Level> la, lb, lc, ls;
    if (!levels_of(L.dims, A.stride, ax_b, 2, la) || !levels_of(L.dims, B.stride, ax_b, 2, lb) || !levels_of(L.dims, L.out.stride, ax_b, 2, lc)) return false;
    // choose the split: the lowest level count any operand needs
    int64_t lo = g.batch;
    for (auto *v : {&la, &lb, &lc}) if (v->size() == 2) lo = std::min(lo, (*v)[1].count);
    auto split = [&](const std::vector<Level> &v, int64_t &s_lo, int64_t &s_hi) {
        if (v.empty()) { s_lo = s_hi = 0; return true; }
        if (v.size() == 1) { s_lo = v[0].stride; s_hi = v[0].stride * lo; return true; }
        if (v[1].count != lo) return false;
        s_lo = v[1].stride; s_hi = v[0].stride;
        return true;
    };
    g.batch_lo = lo;
    if (!split(la, g.a_lo, g.a_hi) || !split(lb, g.b_lo, g.b_hi) || !split(lc, g.c_lo, g.c_hi)) return false;
    if (B.dtype == PSK_I8) {
        if (!levels_of(L.dims, B.sstride, ax_b, 2, ls) || !split(ls, g.bs_lo, g.bs_hi)) return false;
    }
    return true;
}

// ---- tensor maps ------------------------------------------------------------
bool make_map(psk_exec *e, CUtensorMap *map, const void *base, int f16, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t box0, uint32_t box1)
{
    // strides in elements on entry; the driver wants bytes, multiples of 16
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {s1 * 2, s2 * 2, s3 * 2};
    for (int i = 0; i < 3; ++i) {
        if (dims[i + 1] == 1 && strides[i] == 0) strides[i] = (i == 0 ? d0 * 2 : strides[i - 1] * dims[i]);
        if (strides[i] % 16 != 0 || strides[i] == 0) return false;
    }
    cuuint32_t box[4] = {box0, box1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    // (the L2 promotion size makes no measurable difference to the sustained rate: 1 186 to 1 191 TFLOP/s for none, 128 B, 256 B)
    CUresult r = e->encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

int launch_tc(psk_exec *e, const psk_gemm &g, const void *a, const void *b, void *c, uint32_t *flag, const float *col_scale = nullptr, int64_t cs_stride = 0, int64_t cs_lo = 0, int64_t cs_hi = 0, int64_t split_k = 0, int planes = 2, const void *addend = nullptr)
{
    if (!e->encode) return fail(e, PSK_E10001, "cuTensorMapEncodeTiled is not available from this driver");
    const bool f16 = g.in_dtype == PSK_F16;
    const int bn = g.n >= 256 || g.n % 128 != 0 ? 256 : 128;
    const int64_t batch_hi = g.batch / g.batch_lo;
    // tiles of 256 rows (two accumulators sharing B's tile): a third less traffic a product, but the accumulators
    // fill tensor memory and a tile's epilogue is no longer hidden behind the next tile's products. Sustained, on
    // one box, against 128-row tiles: +12 % at K = 11008, +3 % at K = 4096 (N = 4096, 11008), +2 % for the f32 head.
    static const bool m256_on = getenv("PSK_GEMM_M256") ? atoi(getenv("PSK_GEMM_M256")) != 0 : true;
    const int mt_rows = (m256_on && bn == 256 && g.m >= 512) ? 2 : 1;
    CUtensorMap ma, mb;
    const uint64_t kphys = split_k ? (uint64_t)(planes * split_k) : (uint64_t)g.k; // what the operands hold along the summed axis
    const bool a_m_major = (g.b_n_major & 2) != 0, b_n_major = (g.b_n_major & 1) != 0;
    if (a_m_major && split_k) return fail(e, PSK_E7001, "tensor-core contraction: planes of a transposed operand");
    const bool oka = a_m_major
        ? make_map(e, &ma, a, f16, (uint64_t)g.m, kphys, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.a_row, (uint64_t)g.a_lo, (uint64_t)g.a_hi, 64, tc::BK)
        : make_map(e, &ma, a, f16, kphys, (uint64_t)g.m, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.a_row, (uint64_t)g.a_lo, (uint64_t)g.a_hi, tc::BK, (uint32_t)(tc::BM * mt_rows));
    if (!oka) return fail(e, PSK_E7001, "tensor-core contraction: operand 0's strides do not make a tensor map");
    bool okb = b_n_major
        ? make_map(e, &mb, b, f16, (uint64_t)g.n, kphys, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.b_row, (uint64_t)g.b_lo, (uint64_t)g.b_hi, 64, tc::BK)
        : make_map(e, &mb, b, f16, kphys, (uint64_t)g.n, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.b_row, (uint64_t)g.b_lo, (uint64_t)g.b_hi, tc::BK, (uint32_t)bn);
    if (!okb) return fail(e, PSK_E7001, "tensor-core contraction: operand 1's strides do not make a tensor map");
    tc::Params P;
    P.m = g.m; P.n = g.n; P.k = g.k; P.batch = g.batch; P.batch_lo = g.batch_lo;
    P.tiles_m = (g.m + tc::BM * mt_rows - 1) / (tc::BM * mt_rows);
    P.tiles_n = (g.n + bn - 1) / bn;
    P.split_k = split_k; P.planes = planes; P.a_m_major = a_m_major ? 1 : 0;
    P.addend = addend;
    {
        // a panel's columns of B (bn·k elements each) should stay in the L2 while A streams past them: a
        // quarter of the L2 for them; at least 8 columns, all of them when that fits
        static const long forced = getenv("PSK_GEMM_PANEL") ? atol(getenv("PSK_GEMM_PANEL")) : 0;
        const int64_t col_bytes = (int64_t)bn * g.k * 2;
        int64_t panel = std::max<int64_t>(8, (32ll << 20) / std::max<int64_t>(col_bytes, 1));
        if (forced > 0) panel = forced;
        P.panel = std::min<int64_t>(panel, P.tiles_n);
    }
    P.c_row_lo_count = g.c_row_lo_count; P.c_row_lo = g.c_row_lo; P.c_row_hi = g.c_row_hi;
    P.c_col_lo_count = g.c_col_lo_count; P.c_col_hi = g.c_col_hi;
    P.c_lo = g.c_lo; P.c_hi = g.c_hi;
    P.c = c; P.out_dtype = g.out_dtype; P.in_f16 = f16; P.b_n_major = b_n_major ? 1 : 0; P.guarded = g.guarded;
    const int64_t va = g.out_dtype == PSK_F32 ? 4 : 8; // elements in 16 bytes
    P.vec_ok = aligned16(c) && g.c_row_lo % va == 0 && g.c_row_hi % va == 0 && g.c_col_hi % va == 0 && g.c_lo % va == 0 && g.c_hi % va == 0 && g.c_col_lo_count % (g.out_dtype == PSK_F32 ? 32 : 64) == 0 && g.n % va == 0 && g.out_dtype != PSK_E8M15;
    P.scale = g.scale; P.scale_on = g.scale_on;
    P.col_scale = col_scale; P.col_scale_stride = cs_stride; P.col_scale_lo = cs_lo; P.col_scale_hi = cs_hi;
    P.ovf = flag; P.status = e->status;
    if (addend && !(P.vec_ok && g.out_dtype == PSK_BF16)) return fail(e, PSK_E7001, "tensor-core contraction: an addend needs the staged bf16 epilogue");
    if (!e->tc_attr_set) {
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<128>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256, 2>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256, false, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256, 2>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256, false, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256, false, 2, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256, 2>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256, false, 1, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256, false, 2, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256, 2>::TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tc::k_gemm_tc<256, false, 1, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256>::TOTAL));
        e->tc_attr_set = true;
    }
    const int64_t tiles = P.tiles_m * P.tiles_n * g.batch;
    const int grid = (int)std::min<int64_t>(tiles, e->sms);
    {
        // The same tiles on pairs of CTAs (psk_gemm_tc2.cuh), for the plain staged epilogues of large row counts.
        static const bool pair_on = getenv("PSK_GEMM_PAIR") ? atoi(getenv("PSK_GEMM_PAIR")) != 0 : false;
        const bool plain = P.vec_ok && !g.scale_on && !col_scale && !g.guarded && (g.out_dtype == PSK_BF16 || (g.out_dtype == PSK_F32 && !addend));
        if (pair_on && mt_rows == 2 && !split_k && !a_m_major && plain && e->sms >= 2) {
            CUtensorMap pa, pb;
            bool okp = make_map(e, &pa, a, f16, kphys, (uint64_t)g.m, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.a_row, (uint64_t)g.a_lo, (uint64_t)g.a_hi, tc::BK, 128);
            if (b_n_major) pb = mb;
            else okp = okp && make_map(e, &pb, b, f16, kphys, (uint64_t)g.n, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.b_row, (uint64_t)g.b_lo, (uint64_t)g.b_hi, tc::BK, 128);
            if (okp) {
                static bool attr_set = false;
                if (!attr_set) {
                    CUDA_TRY(e, cudaFuncSetAttribute(tc2::k_gemm_tc2, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2::SMEM_TOTAL));
                    attr_set = true;
                }
                const int pairs = (int)std::min<int64_t>(tiles, e->sms / 2);
                tc2::k_gemm_tc2<<<2 * pairs, tc2::THREADS, tc2::SMEM_TOTAL, e->stream>>>(pa, pb, P);
                CUDA_TRY(e, cudaGetLastError());
                e->kernels += 1;
                return PSK_OK;
            }
        }
    }
    // a plain bf16 result in whole 16-byte runs: the instantiation whose epilogue keeps tensor memory's loads ahead
    static const int plain_mode = getenv("PSK_GEMM_PLAIN") ? atoi(getenv("PSK_GEMM_PLAIN")) : 3; // bit 0: results without an addend, bit 1: with one
    const bool plain_any = P.vec_ok && g.out_dtype == PSK_BF16 && !g.scale_on && !col_scale && !split_k && !a_m_major && bn == 256;
    const bool plain_bf16 = plain_any && !addend && (plain_mode & 1), plain_add = plain_any && addend && (plain_mode & 2);
    if (plain_bf16 && mt_rows == 2) tc::k_gemm_tc<256, false, 2, false, 1><<<grid, tc::THREADS, tc::Smem<256, 2>::TOTAL, e->stream>>>(ma, mb, P);
    else if (plain_bf16) tc::k_gemm_tc<256, false, 1, false, 1><<<grid, tc::THREADS, tc::Smem<256>::TOTAL, e->stream>>>(ma, mb, P);
    else if (plain_add && mt_rows == 2) tc::k_gemm_tc<256, false, 2, false, 2><<<grid, tc::THREADS, tc::Smem<256, 2>::TOTAL, e->stream>>>(ma, mb, P);
    else if (plain_add) tc::k_gemm_tc<256, false, 1, false, 2><<<grid, tc::THREADS, tc::Smem<256>::TOTAL, e->stream>>>(ma, mb, P);
    else if (mt_rows == 2 && col_scale) tc::k_gemm_tc<256, false, 2, true><<<grid, tc::THREADS, tc::Smem<256, 2>::TOTAL, e->stream>>>(ma, mb, P);
    else if (bn == 256 && col_scale) tc::k_gemm_tc<256, false, 1, true><<<grid, tc::THREADS, tc::Smem<256>::TOTAL, e->stream>>>(ma, mb, P);
    else if (mt_rows == 2) tc::k_gemm_tc<256, false, 2><<<grid, tc::THREADS, tc::Smem<256, 2>::TOTAL, e->stream>>>(ma, mb, P);
    else if (bn == 256) tc::k_gemm_tc<256><<<grid, tc::THREADS, tc::Smem<256>::TOTAL, e->stream>>>(ma, mb, P);
    else tc::k_gemm_tc<128><<<grid, tc::THREADS, tc::Smem<128>::TOTAL, e->stream>>>(ma, mb, P);
    CUDA_TRY(e, cudaGetLastError());
    e->kernels += 1;
    return PSK_OK;
}

// A contraction of a few rows against a large second operand (one new position a sequence against a weight
// matrix): the tensor-core kernel's tiles are 128 rows by 256 columns, so n / 256 CTAs would stream the whole
// matrix while the other SMs idle. Here the summed axis is cut into `parts` runs, each a batch entry of one launch
// (tiles = parts · n / 256), whose f32 partial sums k_sum_parts adds in the runs' order: a declared order of the
// sum like any other of PSK_ORDER_DEVICE, fixed by the shape alone. Returns PSK_E7001 when the shape does not
// take it (the caller then launches the contraction whole).
int launch_tc_few_rows(psk_exec *e, const psk_gemm &g, const void *a, const void *b, void *c, uint32_t *flag, const float *col_scale, int64_t cs_stride, const void *addend, int site_dtype)
{
    static const bool on = getenv("PSK_GEMM_SPLITK") ? atoi(getenv("PSK_GEMM_SPLITK")) != 0 : true;
    const bool a_m_major = (g.b_n_major & 2) != 0;
    if (!on || g.batch != 1 || g.m > 32 || a_m_major || g.k < 1024 || g.n < 256) return PSK_E7001;
    if (g.c_row_lo_count < g.m || g.c_col_lo_count < g.n) return PSK_E7001; // a result laid out in levels: not here
    const int64_t tiles_n = (g.n + 255) / 256;
    int64_t parts = 1;
    while (parts * 2 * tiles_n <= (int64_t)e->sms + e->sms / 4 && g.k % (parts * 2) == 0 && (g.k / (parts * 2)) % 64 == 0 && g.k / (parts * 2) >= 256) parts *= 2;
    if (parts < 2) return PSK_E7001;
    const int64_t kc = g.k / parts;
    float *partial = (float *)psk_exec_alloc(e, (size_t)parts * g.m * g.n * 4);
    if (!partial) return fail(e, PSK_E10001, "tensor-core contraction: no memory for the partial sums");
    psk_gemm pg = g;
    pg.out_dtype = PSK_F32; pg.guarded = 0;
    pg.k = kc; pg.batch = parts; pg.batch_lo = parts;
    pg.a_lo = kc; pg.a_hi = 0;                                   // a run of the summed axis further along each row
    pg.b_lo = (g.b_n_major & 1) ? kc * g.b_row : kc; pg.b_hi = 0; // N-major: kc rows down; K-major: kc along each row
    pg.c_row_lo_count = g.m; pg.c_row_lo = g.n; pg.c_row_hi = 0;
    pg.c_col_lo_count = g.n; pg.c_col_hi = 0;
    pg.c_lo = g.m * g.n; pg.c_hi = 0;
    pg.scale_on = 0;
    int r = launch_tc(e, pg, a, b, partial, e->flags);
    if (r == PSK_OK) {
        k_sum_parts<<<grid_for(e, g.m * g.n, 256, 8), 256, 0, e->stream>>>(partial, (int)parts, g.m, g.n, c, g.out_dtype, site_dtype, g.c_row_lo, addend, g.c_row_lo, col_scale, cs_stride, g.guarded, flag);
        e->kernels += 1;
    }
    psk_exec_free(e, partial); // handed out again only to later work of the same stream
    return r;
}

// A tensor map over 8-bit codes: dimensions and strides in elements (= bytes).
bool make_map_u8(psk_exec *e, CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t box0, uint32_t box1)
{
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {s1, s2, s3};
    for (int i = 0; i < 3; ++i) {
        if (dims[i + 1] == 1 && strides[i] == 0) strides[i] = (i == 0 ? (d0 + 15) / 16 * 16 : strides[i - 1] * dims[i]);
        if (strides[i] % 16 != 0 || strides[i] == 0) return false;
    }
    cuuint32_t box[4] = {box0, box1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = e->encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// The integer-sum contraction on the tensor cores (psk_gemm_i8.cuh). PSK_E7001: strides no tensor map takes
// (the caller then runs the scalar kernel). `addend`: a bf16 tensor laid out as a bf16 result, added to the rounded
// product; only the staged stores add it, so other layouts answer PSK_E7001 too.
int launch_i8(psk_exec *e, const GemmMap &g, const DevOperand &A, const DevOperand &B, const DevOperand &O, const psk_operand &out_desc, uint32_t *flag, bool guarded, const void *addend = nullptr)
{
    if (!e->encode) return fail(e, PSK_E10001, "cuTensorMapEncodeTiled is not available from this driver");
    const bool b_n_major = g.b_k != 1;
    const int64_t batch_hi = g.batch / g.batch_lo;
    CUtensorMap ma, mb;
    // tiles of 128 rows with the rescale hidden behind the next tile's products, or of 256 with less traffic from
    // the L2 and the rescale exposed (psk_gemm_i8.cuh); PSK_I8_MT chooses, for measurements
    const char *mt_word = getenv("PSK_I8_MT"); // read at every launch, so that a test can run both forms
    const int mt_env = mt_word ? atoi(mt_word) : 1;
    const int mt_rows = (mt_env == 2 && g.m >= 256 && !addend) ? 2 : 1; // (the addend's instance has tiles of 128 rows)
    if (!make_map_u8(e, &ma, A.p, (uint64_t)g.k, (uint64_t)g.m, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.a_row, (uint64_t)g.a_lo, (uint64_t)g.a_hi, tci8::BKB, (uint32_t)(tci8::BM * mt_rows)))
        return fail(e, PSK_E7001, "integer contraction: operand 0's strides do not make a tensor map");
    const bool okb = b_n_major
        ? make_map_u8(e, &mb, B.p, (uint64_t)g.n, (uint64_t)g.k, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.b_k, (uint64_t)g.b_lo, (uint64_t)g.b_hi, 128, tci8::BKB)
        : make_map_u8(e, &mb, B.p, (uint64_t)g.k, (uint64_t)g.n, (uint64_t)g.batch_lo, (uint64_t)batch_hi, (uint64_t)g.b_n, (uint64_t)g.b_lo, (uint64_t)g.b_hi, tci8::BKB, tci8::BN);
    if (!okb) return fail(e, PSK_E7001, "integer contraction: operand 1's strides do not make a tensor map");
    tci8::Params P;
    memset(&P, 0, sizeof P);
    P.m = g.m; P.n = g.n; P.k = g.k; P.batch = g.batch; P.batch_lo = g.batch_lo;
    P.tiles_m = (g.m + tci8::BM * mt_rows - 1) / (tci8::BM * mt_rows);
    P.tiles_n = (g.n + tci8::BN - 1) / tci8::BN;
    {
        const int64_t col_bytes = (int64_t)tci8::BN * g.k;
        P.panel = std::min<int64_t>(std::max<int64_t>(8, (32ll << 20) / std::max<int64_t>(col_bytes, 1)), P.tiles_n);
    }
    P.c_row_lo_count = g.c_row_lo_count; P.c_row_lo = g.c_row_lo; P.c_row_hi = g.c_row_hi;
    P.c_col_lo_count = g.c_col_lo_count; P.c_col_hi = g.c_col_hi;
    P.c_lo = g.c_lo; P.c_hi = g.c_hi;
    P.c = const_cast<void *>(O.p); P.out_dtype = O.dtype;
    P.out_affine = out_desc.affine; P.out_zero = out_desc.affine_zero; P.out_scale = out_desc.affine_scale;
    P.a_unsigned = A.affine == 2 ? 1 : 0; P.a_zero = A.affine_zero; P.a_scale = A.affine_scale;
    P.b_n_major = b_n_major ? 1 : 0;
    P.col_scale = B.scales; P.col_scale_stride = g.bs_n; P.col_scale_lo = g.bs_lo; P.col_scale_hi = g.bs_hi;
    P.guarded = guarded ? 1 : 0;
    const int64_t va = O.dtype == PSK_F32 ? 4 : 8;
    P.vec_ok = aligned16(O.p) && g.c_row_lo % va == 0 && g.c_row_hi % va == 0 && g.c_col_hi % va == 0 && g.c_lo % va == 0 && g.c_hi % va == 0 && g.c_col_lo_count % 32 == 0 && g.n % va == 0;
    P.ovf = flag; P.status = e->status;
    if (addend) {
        if (!P.vec_ok || O.dtype != PSK_BF16 || out_desc.affine) return fail(e, PSK_E7001, "integer contraction: an addend needs a bf16 result in rows of 16-byte runs");
        P.addend = addend;
    }
    int32_t *colsum = nullptr;
    if (A.affine_zero != 0) {
        colsum = (int32_t *)psk_exec_alloc(e, (size_t)g.n * g.batch * 4);
        if (!colsum) return fail(e, PSK_E10001, "integer contraction: no memory for the weights' column sums");
        CUDA_TRY(e, cudaMemsetAsync(colsum, 0, (size_t)g.n * g.batch * 4, e->stream));
        {
            const int64_t work = g.b_k == 1 ? g.n * g.batch * 32 : g.n * g.batch; // threads: a warp or a thread a column
            dim3 cgrid((unsigned)std::min<int64_t>((work + 255) / 256, 65535), (unsigned)((g.k + tci8::COLSUM_RUN - 1) / tci8::COLSUM_RUN));
            tci8::k_colsum_i8<<<cgrid, 256, 0, e->stream>>>((const int8_t *)B.p, g.n, g.k, g.batch, g.batch_lo, g.b_n, g.b_k, g.b_lo, g.b_hi, colsum);
        }
        e->kernels += 1;
        P.colsum = colsum;
    }
    if (!e->i8_attr_set) {
        CUDA_TRY(e, cudaFuncSetAttribute(tci8::k_gemm_i8<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, tci8::Cfg<1>::SMEM_TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tci8::k_gemm_i8<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, tci8::Cfg<2>::SMEM_TOTAL));
        CUDA_TRY(e, cudaFuncSetAttribute(tci8::k_gemm_i8<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tci8::Cfg<1>::SMEM_TOTAL));
        e->i8_attr_set = true;
    }
    const int64_t tiles = P.tiles_m * P.tiles_n * g.batch;
    const int grid = (int)std::min<int64_t>(tiles, e->sms);
    if (addend) tci8::k_gemm_i8<1, true><<<grid, tci8::THREADS, tci8::Cfg<1>::SMEM_TOTAL, e->stream>>>(ma, mb, P);
    else if (mt_rows == 2) tci8::k_gemm_i8<2><<<grid, tci8::THREADS, tci8::Cfg<2>::SMEM_TOTAL, e->stream>>>(ma, mb, P);
    else tci8::k_gemm_i8<1><<<grid, tci8::THREADS, tci8::Cfg<1>::SMEM_TOTAL, e->stream>>>(ma, mb, P);
    if (colsum) psk_exec_free(e, colsum); // handed out again only to later work of the same stream
    CUDA_TRY(e, cudaGetLastError());
    e->kernels += 1;
    return PSK_OK;
}

// The guard's flags since the last drain: 0, or 1 + the serial number of the first guarded launch whose flag is set.
// Waits for the stream, clears the flags and starts the slots over.
int64_t drain_flags(psk_exec *e)
{
    if (e->guarded_since == 0) return 0;
    cudaSetDevice(e->device);
    std::vector<uint32_t> host(kFlagSlots);
    if (cudaMemcpyAsync(host.data(), e->flags, kFlagSlots * sizeof(uint32_t), cudaMemcpyDeviceToHost, e->stream) != cudaSuccess) return 0;
    cudaStreamSynchronize(e->stream);
    int64_t first = -1;
    const int64_t used = std::min<int64_t>(e->guarded_since, kFlagSlots);
    for (int64_t s = 0; s < used; ++s)
        if (host[s] && (first < 0 || e->flag_serial[s] < first)) first = e->flag_serial[s];
    cudaMemsetAsync(e->flags, 0, kFlagSlots * sizeof(uint32_t), e->stream);
    e->guarded_since = 0;
    return first < 0 ? 0 : first + 1;
}

// A slot of the guard's flags for one guarded launch. A slot is never shared by two launches between two drains:
// when every slot has been handed out the flags are drained first, and an overflow found then is kept
// (`latched_overflow`) for the next psk_exec_overflow, so that the launch it names is the one that overflowed.
uint32_t *next_flag(psk_exec *e, const psk_launch *l)
{
    if (e->guarded_since >= kFlagSlots) {
        const int64_t o = drain_flags(e);
        if (o && !e->latched_overflow) e->latched_overflow = o;
    }
    const int slot = (int)e->guarded_since;
    e->flag_serial[slot] = e->launches;
    e->guarded_since += 1;
    (void)l;
    return e->flags + slot;
}

} // namespace

// ===========================================================================
extern "C" {

psk_exec *psk_exec_create(int device)
{
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || device < 0 || device >= count) {
        g_create_error = err != cudaSuccess ? std::string("no CUDA device: ") + cudaGetErrorString(err) : "no CUDA device of that number";
        return nullptr;
    }
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        g_create_error = "cannot select the CUDA device";
        return nullptr;
    }
    if (prop.major != 10) {
        g_create_error = "this library's kernels are built for sm_100a only; the device is sm_" + std::to_string(prop.major) + std::to_string(prop.minor);
        return nullptr;
    }
    psk_exec *e = new psk_exec;
    e->device = device;
    e->sms = prop.multiProcessorCount;
    bool ok = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) == cudaSuccess
        && cudaMalloc(&e->flags, kFlagSlots * sizeof(uint32_t)) == cudaSuccess
        && cudaMalloc(&e->status, sizeof(uint32_t)) == cudaSuccess
        && cudaMemset(e->flags, 0, kFlagSlots * sizeof(uint32_t)) == cudaSuccess
        && cudaMemset(e->status, 0, sizeof(uint32_t)) == cudaSuccess
        && cudaEventCreate(&e->ev0) == cudaSuccess && cudaEventCreate(&e->ev1) == cudaSuccess;
    if (!ok) {
        g_create_error = std::string("cannot set the executor up: ") + cudaGetErrorString(cudaGetLastError());
        delete e;
        return nullptr;
    }
    e->flag_serial.assign(kFlagSlots, -1);
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
        e->encode = (EncodeTiledFn)fn;
    return e;
}

void psk_exec_destroy(psk_exec *e)
{
    if (!e) return;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    for (auto &kv : e->sizes) cudaFree(kv.first);
    for (auto &kv : e->widened) cudaFree(kv.second);
    if (e->silu_table) cudaFree(e->silu_table);
    cudaFree(e->flags);
    cudaFree(e->status);
    cudaEventDestroy(e->ev0);
    cudaEventDestroy(e->ev1);
    for (auto &r : e->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    for (cudaEvent_t ev : e->event_pool) cudaEventDestroy(ev);
    cudaStreamDestroy(e->stream);
    delete e;
}

const char *psk_exec_name(const psk_exec *) { return "cuda"; }

const char *psk_last_error(const psk_exec *e) { return e ? e->error.c_str() : g_create_error.c_str(); }

void *psk_exec_alloc(psk_exec *e, size_t bytes)
{
    if (bytes == 0) bytes = 16;
    bytes = (bytes + 255) & ~(size_t)255;
    cudaSetDevice(e->device);
    void *p = nullptr;
    auto it = e->pool.find(bytes);
    if (it != e->pool.end() && !it->second.empty()) {
        p = it->second.back();
        it->second.pop_back();
    } else {
        cudaError_t err = cudaMalloc(&p, bytes);
        if (err != cudaSuccess) {
            // give the pool back to the driver and try once more
            for (auto &kv : e->pool) {
                for (void *q : kv.second) { cudaFree(q); e->sizes.erase(q); }
                kv.second.clear();
            }
            cudaGetLastError();
            err = cudaMalloc(&p, bytes);
            if (err != cudaSuccess) {
                fail(e, PSK_E10001, std::string("cudaMalloc of ") + std::to_string(bytes) + " bytes: " + cudaGetErrorString(err));
                cudaGetLastError();
                return nullptr;
            }
        }
        e->sizes[p] = bytes;
    }
    e->live += bytes;
    e->peak = std::max(e->peak, e->live);
    return p;
}

// A widened copy of weights is valid while the codes it was made from are: anything that writes into the
// buffer holding them (an upload, a launch's output) drops it.
static void forget_widened(psk_exec *e, const void *written)
{
    if (e->widened.empty()) return;
    const uint8_t *lo = (const uint8_t *)written, *hi = lo + 1;
    for (auto &kv : e->sizes) {
        const uint8_t *b = (const uint8_t *)kv.first;
        if (lo >= b && lo < b + kv.second) { lo = b; hi = b + kv.second; break; }
    }
    for (auto w = e->widened.begin(); w != e->widened.end();) {
        const uint8_t *q = (const uint8_t *)w->first.first;
        if (q >= lo && q < hi) { cudaFree(w->second); e->live -= (size_t)w->first.second * 2; e->widened_bytes -= (size_t)w->first.second * 2; w = e->widened.erase(w); }
        else ++w;
    }
}

void psk_exec_free(psk_exec *e, void *p)
{
    if (!p) return;
    auto it = e->sizes.find(p);
    if (it == e->sizes.end()) return;
    e->live -= it->second;
    e->causal.erase(p);
    // widened copies of weights that lived in this buffer
    for (auto w = e->widened.begin(); w != e->widened.end();) {
        const uint8_t *q = (const uint8_t *)w->first.first;
        if (q >= (const uint8_t *)p && q < (const uint8_t *)p + it->second) { cudaFree(w->second); e->live -= (size_t)w->first.second * 2; e->widened_bytes -= (size_t)w->first.second * 2; w = e->widened.erase(w); }
        else ++w;
    }
    // The stream is in order and every kernel of this executor runs on it, so
    // a buffer handed out again is written only after its last reader ran.
    e->pool[it->second].push_back(p);
}

int psk_exec_upload(psk_exec *e, void *dst, const void *src_host, size_t bytes)
{
    cudaSetDevice(e->device);
    e->causal.erase(dst);
    forget_widened(e, dst);
    CUDA_TRY(e, cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, e->stream));
    CUDA_TRY(e, cudaStreamSynchronize(e->stream)); // the host buffer is the caller's again
    return PSK_OK;
}

static int check_status(psk_exec *e)
{
    uint32_t st = 0;
    CUDA_TRY(e, cudaMemcpyAsync(&st, e->status, sizeof st, cudaMemcpyDeviceToHost, e->stream));
    CUDA_TRY(e, cudaStreamSynchronize(e->stream));
    if (st) {
        cudaMemsetAsync(e->status, 0, sizeof st, e->stream);
        char buf[256];
        if (st & 0x100u) snprintf(buf, sizeof buf, "a bounded wait ran out in a tensor-core kernel (role 0x%x); its results are not valid", st & 0xffu);
        else if (st & 2u) snprintf(buf, sizeof buf, "an index outside its bound reached a gather");
        else snprintf(buf, sizeof buf, "sin or cos of an argument at or beyond 2^28*pi/2 is not supported by this executor");
        return fail(e, (st & 0x100u) ? PSK_E10001 : PSK_E7001, buf);
    }
    return PSK_OK;
}

// A kernel whose only wait can never be satisfied and is limited to `cycles`: returns what the next sync reports
// (PSK_E10001, "a bounded wait ran out ..."), and leaves the executor usable. For tests of that report.
int psk_exec_wait_selftest(psk_exec *e, int64_t cycles)
{
    cudaSetDevice(e->device);
    if (cycles < 1 || cycles > 400000000ll) return fail(e, PSK_E7001, "psk_exec_wait_selftest: between 1 and 4e8 cycles (a fraction of a second)");
    int *flag = (int *)psk_exec_alloc(e, sizeof(int));
    if (!flag) return PSK_E10001;
    tc::k_wait_runs_out<<<1, 32, 0, e->stream>>>(e->status, (long long)cycles, flag);
    int gave_up = -1;
    cudaError_t err = cudaMemcpyAsync(&gave_up, flag, sizeof gave_up, cudaMemcpyDeviceToHost, e->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
    psk_exec_free(e, flag);
    if (err != cudaSuccess) return fail(e, PSK_E10001, std::string("psk_exec_wait_selftest: ") + cudaGetErrorString(err));
    e->kernels += 1;
    if (gave_up != 1) return fail(e, PSK_E10001, "psk_exec_wait_selftest: the wait did not run out");
    return check_status(e);
}

int64_t psk_exec_overflow(psk_exec *e)
{
    const int64_t now = drain_flags(e);
    if (e->latched_overflow) { // found when the slots ran out: earlier than anything still in the flags
        const int64_t o = e->latched_overflow;
        e->latched_overflow = 0;
        return o;
    }
    return now;
}

int psk_exec_sync(psk_exec *e)
{
    cudaSetDevice(e->device);
    CUDA_TRY(e, cudaStreamSynchronize(e->stream));
    int st = check_status(e);
    if (st != PSK_OK) return st;
    int64_t o = psk_exec_overflow(e);
    if (o) return fail(e, PSK_E7007, "launch " + std::to_string(o - 1) + ": a store rounded a finite value to an infinity");
    return PSK_OK;
}

int psk_exec_download(psk_exec *e, void *dst_host, const void *src, size_t bytes)
{
    cudaSetDevice(e->device);
    CUDA_TRY(e, cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, e->stream));
    CUDA_TRY(e, cudaStreamSynchronize(e->stream));
    return PSK_OK;
}

void psk_exec_memory(const psk_exec *e, size_t *live, size_t *peak)
{
    if (live) *live = e->live;
    if (peak) *peak = e->peak;
}

void psk_exec_counts(const psk_exec *e, int64_t *launches, int64_t *kernels)
{
    if (launches) *launches = e->launches;
    if (kernels) *kernels = e->kernels;
}

void psk_exec_set_profiling(psk_exec *e, int on) { e->profiling = on != 0; }

double psk_exec_last_ms(psk_exec *e)
{
    if (!e->profiling) return -1.0;
    if (cudaEventSynchronize(e->ev1) != cudaSuccess) return -1.0;
    float ms = 0;
    if (cudaEventElapsedTime(&ms, e->ev0, e->ev1) != cudaSuccess) return -1.0;
    return ms;
}

void *psk_exec_stream(psk_exec *e) { return (void *)e->stream; }

const char *psk_exec_profile(psk_exec *e)
{
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    e->prof_text.clear();
    char line[512];
    for (auto &r : e->prof) {
        float ms = -1.0f;
        cudaEventElapsedTime(&ms, r.a, r.b);
        snprintf(line, sizeof line, "%s\t%s\t%.6f\t%.0f\t%.0f\n", r.kernel, r.name.c_str(), ms, r.flops, r.bytes);
        e->prof_text += line;
        e->event_pool.push_back(r.a);
        e->event_pool.push_back(r.b);
    }
    e->prof.clear();
    return e->prof_text.c_str();
}

int psk_exec_gemm(psk_exec *e, const psk_gemm *g, const void *a, const void *b, void *c)
{
    cudaSetDevice(e->device);
    if (g->in_dtype != PSK_BF16 && g->in_dtype != PSK_F16) return fail(e, PSK_E7005, "tensor-core contraction: operands are bf16 or f16");
    if (!aligned16(a) || !aligned16(b)) return fail(e, PSK_E7001, "tensor-core contraction: operands must be 16-byte aligned");
    if (g->out_dtype != PSK_F32 && g->out_dtype != PSK_BF16 && g->out_dtype != PSK_F16 && g->out_dtype != PSK_E8M15)
        return fail(e, PSK_E7005, "tensor-core contraction: the result is stored as f32, bf16, f16 or e8m15");
    if (g->m < 1 || g->n < 1 || g->k < 1 || g->batch < 1 || g->batch_lo < 1 || g->batch % g->batch_lo != 0)
        return fail(e, PSK_E7001, "tensor-core contraction: sizes must be positive and batch a multiple of batch_lo");
    if (g->c_row_lo_count < 1 || g->c_col_lo_count < 1) return fail(e, PSK_E7001, "tensor-core contraction: c_row_lo_count and c_col_lo_count are at least 1");
    if (g->a_row < 0 || g->a_lo < 0 || g->a_hi < 0 || g->b_row < 0 || g->b_lo < 0 || g->b_hi < 0 || g->c_row_lo < 0 || g->c_row_hi < 0 || g->c_col_hi < 0 || g->c_lo < 0 || g->c_hi < 0)
        return fail(e, PSK_E7001, "tensor-core contraction: a negative stride");
    uint32_t *flag = e->flags;
    if (g->guarded) {
        psk_launch dummy;
        flag = next_flag(e, &dummy);
    }
    if (e->profiling) cudaEventRecord(e->ev0, e->stream);
    int r = launch_tc(e, *g, a, b, c, flag);
    if (e->profiling) cudaEventRecord(e->ev1, e->stream);
    e->launches += 1;
    return r;
}

// Integer or e4m3fn weights as the bf16 numbers they are. While the copies kept so far stay within the budget
// (4 GB, or PSK_WIDENED_MB), a copy is made at the weights' first contraction on the tensor cores and kept until the
// codes are written again or freed. Beyond it (a model whose narrow weights are there to save memory) the copy is
// made again for every contraction into a buffer of the pool, which the caller gives back once the contraction is
// queued (`*transient`): the stream is in order, so the next matrix's copy may take the same bytes. That costs a
// read of the codes and a write and a read of the copy a contraction, about 3 ms of a 7B prefill step, and the model
// then holds one byte a weight, not three.
static const void *widened_weights(psk_exec *e, const void *codes, int64_t count, bool int8, bool *transient)
{
    *transient = false;
    auto key = std::make_pair(codes, count);
    auto it = e->widened.find(key);
    if (it != e->widened.end()) return it->second;
    const char *forced = getenv("PSK_WIDENED_MB"); // read at every new copy, so that a test can change it
    const long forced_mb = forced ? atol(forced) : -1;
    const size_t budget = forced_mb >= 0 ? (size_t)forced_mb << 20 : e->widened_budget, bytes = (size_t)count * 2;
    void *wb = nullptr;
    if (e->widened_bytes + bytes > budget) {
        wb = psk_exec_alloc(e, bytes);
        if (!wb) return nullptr;
        *transient = true;
    } else if (cudaMalloc(&wb, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (int8) k_int8_to_bf16<<<grid_for(e, count, 256, 8), 256, 0, e->stream>>>((const int8_t *)codes, (uint16_t *)wb, count);
    else k_e4m3_to_bf16<<<grid_for(e, count, 256, 8), 256, 0, e->stream>>>((const uint8_t *)codes, (uint16_t *)wb, count);
    e->kernels += 1;
    if (!*transient) {
        e->widened.emplace(key, wb);
        e->widened_bytes += bytes;
        e->live += bytes; // the copy is device memory of this executor like any buffer of its pool
        e->peak = std::max(e->peak, e->live);
    }
    return wb;
}

// Whether a group is AdamW's parameter update as the host issues it (inputs m', bc1, v', bc2, eps, θ, λ, lr; steps
// div, div, sqrt, add, div, mul, add, mul, sub) over whole contiguous runs, in an f32 kernel with bf16 or f32 buffers.
static bool adamw_update_program(const psk_launch *l, const DevLaunch &L)
{
    if (l->n_steps != 9 || L.n_in != 8 || L.kdtype != PSK_F32 || L.guarded) return false;
    static const int prim[9] = {PSK_DIV, PSK_DIV, PSK_SQRT, PSK_ADD, PSK_DIV, PSK_MUL, PSK_ADD, PSK_MUL, PSK_SUB};
    static const int nargs[9] = {2, 2, 1, 2, 2, 2, 2, 2, 2};
    static const int src[9][2] = {{0, 1}, {2, 3}, {-2, 0}, {-3, 4}, {-1, -4}, {5, 6}, {-5, -6}, {-7, 7}, {5, -8}};
    for (int s = 0; s < 9; ++s) {
        const psk_step &st = l->steps[s];
        if (st.prim != prim[s] || st.nargs != nargs[s] || st.src[0] != src[s][0] || (nargs[s] == 2 && st.src[1] != src[s][1])) return false;
    }
    const int tensors[3] = {0, 2, 5}, scalars[5] = {1, 3, 4, 6, 7};
    auto run = [&](const DevOperand &o) { // one contiguous run over the whole space, 16-byte aligned
        if (o.affine || (o.dtype != PSK_BF16 && o.dtype != PSK_F32) || !aligned16(o.p)) return false;
        int64_t expect = 1;
        for (int a = L.n_outer - 1; a >= 0; --a) { if (L.dims[a] != 1 && o.stride[a] != expect) return false; expect *= L.dims[a]; }
        return true;
    };
    for (int i : tensors) if (!run(L.in[i])) return false;
    if (!run(L.out)) return false;
    for (int i : scalars) {
        const DevOperand &o = L.in[i];
        if (o.affine || o.dtype == PSK_I8 || o.dtype == PSK_I64 || o.dtype == PSK_F64) return false;
        for (int a = 0; a < L.n_outer; ++a) if (o.stride[a] != 0) return false;
    }
    return L.total % 8 == 0;
}

int psk_exec_run(psk_exec *e, const psk_launch *l, void *const *table)
{
    cudaSetDevice(e->device);
    if (l->n_inputs < 0 || l->n_inputs > PSK_MAX_INPUTS || l->n_outer < 0 || l->n_outer > PSK_MAX_RANK || l->n_inner < 0 || l->n_inner > PSK_MAX_INNER)
        return fail(e, PSK_E7001, std::string(l->name ? l->name : "?") + ": a launch of too many inputs or axes");
    if (l->dtype == PSK_F64 && l->op != PSK_OP_CONVERT)
        return fail(e, PSK_E7005, std::string(l->name ? l->name : "?") + ": this executor computes in f32; a site realised f64 is not runnable by it");
    const int naxes = l->n_outer + l->n_inner;
    if (!e->causal.empty() && l->op != PSK_OP_MAGNITUDE) e->causal.erase(table[l->n_inputs]); // whatever this launch writes is no longer known to be a causal mask
    if (!e->widened.empty() && l->op != PSK_OP_MAGNITUDE && (l->out.dtype == PSK_I8 || l->out.dtype == PSK_E4M3)) forget_widened(e, table[l->n_inputs]);
    DevLaunch L;
    memset(&L, 0, sizeof L);
    L.n_in = l->n_inputs; L.n_outer = l->n_outer; L.n_inner = l->n_inner; L.kdtype = l->dtype;
    L.int_accum = l->int_accum;
    L.chunk = 0;
    if (l->order == PSK_ORDER_CHUNKED && (l->op == PSK_OP_CONTRACT || l->op == PSK_OP_CONTRACT_ADD)) {
        // the reference's chunked(size) (lower.rs:424-457): two operands, one summed axis, on the scalar kernels
        const std::string nm = l->name ? l->name : "?";
        if (l->order_size < 1) return fail(e, PSK_E7001, nm + ": the order chunked(" + std::to_string(l->order_size) + ") has no chunk");
        if (l->n_inner != 1 || l->n_inputs != 2 || l->op != PSK_OP_CONTRACT) return fail(e, PSK_E7005, nm + ": the order chunked(" + std::to_string(l->order_size) + ") sums the product of two operands over one summed axis in chunks");
        if (l->int_accum) return fail(e, PSK_E7005, nm + ": integer sums are exact under every order; state none for them");
        L.chunk = l->order_size;
    }
    L.n_steps = l->n_steps; L.kind = l->kind; L.masked = l->masked; L.guarded = l->guarded && (l->out.dtype == PSK_F16 || l->out.dtype == PSK_E8M15 || l->dtype == PSK_F16 || l->dtype == PSK_E8M15);
    for (int a = 0; a < naxes; ++a) L.dims[a] = l->dims[a];
    int scale_slot = l->n_inputs + 1;
    for (int i = 0; i < l->n_inputs; ++i) {
        const float *sc = nullptr;
        if (l->in[i].dtype == PSK_I8 && !l->in[i].affine) sc = (const float *)table[scale_slot++];
        fill_operand(L.in[i], l->in[i], table[i], sc, naxes);
    }
    fill_operand(L.out, l->out, table[l->n_inputs], nullptr, naxes);
    memcpy(L.steps, l->steps, sizeof(psk_step) * (size_t)std::max(0, std::min(l->n_steps, PSK_MAX_STEPS)));
    for (int i = 0; i < 4; ++i) L.iparam[i] = l->iparam[i];
    L.fparam = (float)l->fparam[0];
    L.status = e->status;
    L.ovf = L.guarded ? next_flag(e, l) : e->flags;
    if (l->op != PSK_OP_EMBED && l->op != PSK_OP_EMBED_VJP && l->op != PSK_OP_IOTA && l->op != PSK_OP_MAGNITUDE && l->op != PSK_OP_ATTENTION && l->op != PSK_OP_RMSNORM && l->op != PSK_OP_ROPE) coalesce_outer(L);
    L.total = 1;
    for (int a = 0; a < L.n_outer; ++a) L.total *= L.dims[a];
    L.inner = 1;
    for (int c = 0; c < L.n_inner; ++c) L.inner *= L.dims[L.n_outer + c];
    const bool device_order = l->order == PSK_ORDER_DEVICE;
    bool any_affine = l->out.affine != 0;
    for (int i = 0; i < l->n_inputs; ++i) any_affine = any_affine || l->in[i].affine != 0;
    const bool affine_norm = l->op == PSK_OP_RMSNORM && l->out.affine != 0 && !l->in[0].affine && !l->in[1].affine && !l->in[2].affine; // the merged norm writing a `scaled` site
    const bool affine_attn = l->op == PSK_OP_ATTENTION && l->out.affine != 0 && !l->in[0].affine && !l->in[1].affine && !l->in[2].affine && !l->in[3].affine && (l->n_inputs < 5 || !l->in[4].affine); // the weighted values into a `scaled` site
    if (any_affine && !affine_norm && !affine_attn && l->op != PSK_OP_FUSED && l->op != PSK_OP_CONTRACT && l->op != PSK_OP_CONVERT && l->op != PSK_OP_CONTRACT_ADD)
        return fail(e, PSK_E7005, std::string(l->name ? l->name : "?") + ": values in an affine format are read and written by elementwise groups, contractions and conversions only");
    bool affine_in = false;
    for (int i = 0; i < l->n_inputs; ++i) affine_in = affine_in || l->in[i].affine != 0;
    if (affine_in && l->op == PSK_OP_CONTRACT && !l->int_accum)
        return fail(e, PSK_E7005, std::string(l->name ? l->name : "?") + ": a contraction over affine values counts its sums in integers (product and accum i32) on this executor");
    cudaEvent_t pa = nullptr, pb = nullptr;
    if (e->profiling) {
        cudaEventRecord(e->ev0, e->stream);
        auto take = [&]() { cudaEvent_t ev; if (e->event_pool.empty()) cudaEventCreate(&ev); else { ev = e->event_pool.back(); e->event_pool.pop_back(); } return ev; };
        pa = take(); pb = take();
        cudaEventRecord(pa, e->stream);
    }
    e->last_kernel = "other";
    e->last_flops = 0;
    int rc = PSK_OK;
    if (L.total == 0 && l->op != PSK_OP_MAGNITUDE && l->op != PSK_OP_EMBED_VJP) {
        // an empty result: nothing to store (embed_vjp still zero-fills its table)
    } else switch (l->op) {
    case PSK_OP_FUSED: {
        e->last_kernel = "k_fused";
        if (l->n_steps < 1 || l->n_steps > PSK_MAX_STEPS) { rc = fail(e, PSK_E7001, "fused: a group of no step or of too many"); break; }
        // silu(g) · u into a `scaled` site (the down-projection's integer-sum operand): bf16 rows in, one-byte codes out,
        // the silu from the table as for a bf16 result
        if (l->out.affine && !l->in[0].affine && L.n_in == 2 && !l->in[1].affine && match_program(l) == EW_SILU_MUL && L.kdtype == PSK_BF16 && !L.guarded
            && L.in[0].dtype == PSK_BF16 && L.in[1].dtype == PSK_BF16 && (L.out.dtype == PSK_I8 || L.out.dtype == PSK_U8) && L.n_outer >= 1 && L.n_outer <= 2
            && L.dims[L.n_outer - 1] % 8 == 0 && L.total / 8 < 0xffffffffll && L.total >= (int64_t)e->sms * 4096 * 8) {
            const int last = L.n_outer - 1;
            bool rows_ok = L.in[0].stride[last] == 1 && L.in[1].stride[last] == 1 && L.out.stride[last] == 1 && aligned16(L.in[0].p) && aligned16(L.in[1].p) && ((uintptr_t)L.out.p % 8) == 0;
            if (L.n_outer == 2) rows_ok = rows_ok && L.in[0].stride[0] % 8 == 0 && L.in[1].stride[0] % 8 == 0 && L.out.stride[0] % 8 == 0;
            if (rows_ok) {
                EwParams E;
                memset(&E, 0, sizeof E);
                for (int i = 0; i < 2; ++i) { E.in[i] = L.in[i].p; E.dt[i] = PSK_BF16; E.cs[i] = 1; E.rs[i] = L.n_outer == 2 ? L.in[i].stride[0] : 0; }
                E.out = const_cast<void *>(L.out.p); E.odt = L.out.dtype; E.kdt = L.kdtype; E.ors = L.n_outer == 2 ? L.out.stride[0] : 0;
                E.rows = L.n_outer == 2 ? (uint32_t)L.dims[0] : 1u; E.colv = (uint32_t)(L.dims[last] / 8); E.n_in = 2;
                E.aff_kind = l->out.affine; E.aff_zero = l->out.affine_zero; E.aff_scale = l->out.affine_scale;
                if (!e->silu_table) {
                    CUDA_TRY(e, cudaMalloc(&e->silu_table, 65536 * sizeof(uint16_t)));
                    k_table_silu<<<64, 1024, 0, e->stream>>>(e->silu_table);
                    CUDA_TRY(e, cudaFuncSetAttribute(k_ew_lut<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
                    CUDA_TRY(e, cudaFuncSetAttribute(k_ew_lut<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
                }
                if (!e->lut_aff_attr_set) {
                    CUDA_TRY(e, cudaFuncSetAttribute(k_ew_lut<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
                    e->lut_aff_attr_set = true;
                }
                k_ew_lut<true, true><<<e->sms, 1024, 65536 * 2, e->stream>>>(E, e->silu_table);
                e->last_kernel = "k_ew_lut_affine";
                e->kernels += 1;
                break;
            }
        }
        bool vec = !any_affine && L.n_outer >= 1 && l->n_steps <= 12 && L.dims[L.n_outer - 1] % 8 == 0 && vec8_operand(L.out, L.dims, L.n_outer, true);
        for (int i = 0; vec && i < L.n_in; ++i) vec = vec8_operand(L.in[i], L.dims, L.n_outer, false);
        bool hot = vec && L.n_outer <= 3 && L.n_in <= 4 && l->n_steps <= 4 && L.total / 8 < 0xffffffffll;
        for (int i = 0; hot && i < L.n_in; ++i) hot = L.in[i].dtype != PSK_I8;
        // three levels (rows in two, e.g. a view of every other run of a row) are taken by the compile-time
        // programs only
        const bool three = L.n_outer == 3;
        if (hot && three) {
            hot = L.out.dtype == PSK_BF16 && L.kdtype == PSK_BF16 && match_program(l) >= 0;
            for (int i = 0; hot && i < L.n_in; ++i)
                hot = L.in[i].dtype == PSK_BF16 || (L.in[i].stride[2] == 0 && (L.in[i].dtype == PSK_F32 || L.in[i].dtype == PSK_F16 || L.in[i].dtype == PSK_E8M15));
        }
        if (hot) {
            EwParams E;
            memset(&E, 0, sizeof E);
            const int last = L.n_outer - 1;
            for (int i = 0; i < L.n_in; ++i) {
                E.in[i] = L.in[i].p; E.dt[i] = L.in[i].dtype; E.cs[i] = (int32_t)L.in[i].stride[last];
                E.rs[i] = L.n_outer >= 2 ? L.in[i].stride[last - 1] : 0;
                E.rs0[i] = three ? L.in[i].stride[0] : 0;
            }
            E.out = const_cast<void *>(L.out.p); E.odt = L.out.dtype; E.kdt = L.kdtype;
            E.ors = L.n_outer >= 2 ? L.out.stride[last - 1] : 0;
            E.ors0 = three ? L.out.stride[0] : 0;
            E.rows = L.n_outer == 2 ? (uint32_t)L.dims[0] : three ? (uint32_t)(L.dims[0] * L.dims[1]) : 1u;
            E.rows1 = three ? (uint32_t)L.dims[1] : 0u;
            E.colv = (uint32_t)(L.dims[last] / 8);
            E.n_in = L.n_in; E.guarded = L.guarded; E.ovf = L.ovf; E.status = L.status;
            for (int k = 0; k < l->n_steps; ++k) E.steps[k] = l->steps[k];
            bool all_bf16 = L.out.dtype == PSK_BF16 && L.kdtype == PSK_BF16;
            for (int i = 0; i < L.n_in; ++i) all_bf16 = all_bf16 && L.in[i].dtype == PSK_BF16;
            const int64_t work = (int64_t)E.rows * E.colv;
            // a compile-time program also takes row-wise scalars of another real type (a norm's f32 root)
            bool prog_ok = L.out.dtype == PSK_BF16 && L.kdtype == PSK_BF16;
            for (int i = 0; i < L.n_in; ++i)
                prog_ok = prog_ok && (L.in[i].dtype == PSK_BF16 || (E.cs[i] == 0 && (L.in[i].dtype == PSK_F32 || L.in[i].dtype == PSK_F16 || L.in[i].dtype == PSK_E8M15)));
            const int prog = prog_ok ? match_program(l) : -1;
            const bool lut = (prog == EW_SILU || prog == EW_SILU_MUL) && all_bf16 && !three && E.cs[0] == 1 && (prog == EW_SILU || E.cs[1] == 1) && work >= (int64_t)e->sms * 4096;
            if (lut) {
                if (!e->silu_table) {
                    CUDA_TRY(e, cudaMalloc(&e->silu_table, 65536 * sizeof(uint16_t)));
                    k_table_silu<<<64, 1024, 0, e->stream>>>(e->silu_table);
                    CUDA_TRY(e, cudaFuncSetAttribute(k_ew_lut<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
                    CUDA_TRY(e, cudaFuncSetAttribute(k_ew_lut<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
                }
                if (prog == EW_SILU) k_ew_lut<false><<<e->sms, 1024, 65536 * 2, e->stream>>>(E, e->silu_table);
                else k_ew_lut<true><<<e->sms, 1024, 65536 * 2, e->stream>>>(E, e->silu_table);
            } else if (prog >= 0) {
                switch (prog) {
                case EW_ADD: launch_prog<EW_ADD>(e, E); break;
                case EW_SUB: launch_prog<EW_SUB>(e, E); break;
                case EW_MUL: launch_prog<EW_MUL>(e, E); break;
                case EW_DIV: launch_prog<EW_DIV>(e, E); break;
                case EW_DIV_MUL: launch_prog<EW_DIV_MUL>(e, E); break;
                case EW_SILU: launch_prog<EW_SILU>(e, E); break;
                case EW_SILU_MUL: launch_prog<EW_SILU_MUL>(e, E); break;
                case EW_MUL_MUL_SUB: launch_prog<EW_MUL_MUL_SUB>(e, E); break;
                default: launch_prog<EW_MUL_MUL_ADD>(e, E); break;
                }
            } else if (all_bf16) {
                const int g = grid_for(e, (work + 3) / 4, 128, 12);
                switch (l->n_steps) {
                case 1: k_ew_bf16<1, 4><<<g, 128, 0, e->stream>>>(E); break;
                case 2: k_ew_bf16<2, 4><<<g, 128, 0, e->stream>>>(E); break;
                case 3: k_ew_bf16<3, 4><<<g, 128, 0, e->stream>>>(E); break;
                default: k_ew_bf16<4, 4><<<g, 128, 0, e->stream>>>(E); break;
                }
            } else {
                const int g = grid_for(e, work, 256, 16);
                switch (l->n_steps) {
                case 1: k_ew<1><<<g, 256, 0, e->stream>>>(E); break;
                case 2: k_ew<2><<<g, 256, 0, e->stream>>>(E); break;
                case 3: k_ew<3><<<g, 256, 0, e->stream>>>(E); break;
                default: k_ew<4><<<g, 256, 0, e->stream>>>(E); break;
                }
            }
        }
        else if (vec && adamw_update_program(l, L)) {
            // the optimizer's nine-step update on runs of bf16 or f32 numbers: its own compile-time kernel
            AdamwUpdate U;
            memset(&U, 0, sizeof U);
            U.m = L.in[0].p; U.v = L.in[2].p; U.theta = L.in[5].p; U.out = const_cast<void *>(L.out.p);
            U.m_bf16 = L.in[0].dtype == PSK_BF16; U.v_bf16 = L.in[2].dtype == PSK_BF16; U.t_bf16 = L.in[5].dtype == PSK_BF16; U.o_bf16 = L.out.dtype == PSK_BF16;
            const int scalars[5] = {1, 3, 4, 6, 7};
            for (int i = 0; i < 5; ++i) { U.sc[i] = L.in[scalars[i]].p; U.sdt[i] = L.in[scalars[i]].dtype; }
            U.nvec = L.total / 8;
            k_adamw_update<<<grid_for(e, U.nvec, 256, 8), 256, 0, e->stream>>>(U);
            e->last_kernel = "k_adamw_update";
        }
        else if (vec && l->n_steps > 8) k_fused_vec8<12><<<grid_for(e, L.total / 8, 256, 8), 256, 0, e->stream>>>(L);
        else if (vec) k_fused_vec8<8><<<grid_for(e, L.total / 8, 256, 8), 256, 0, e->stream>>>(L);
        else k_fused<<<grid_for(e, L.total, 256, 8), 256, 0, e->stream>>>(L);
        e->kernels += 1;
        break;
    }
    case PSK_OP_COPY: {
        e->last_kernel = "k_copy";
        if (L.n_in != 1) { rc = fail(e, PSK_E7001, "copy: one input a launch"); break; }
        bool vec = L.n_outer >= 1 && !L.in[0].is_index && L.dims[L.n_outer - 1] % 8 == 0 && L.in[0].stride[L.n_outer - 1] == 1 && vec8_operand(L.out, L.dims, L.n_outer, true) && vec8_operand(L.in[0], L.dims, L.n_outer, false)
            && (L.in[0].dtype == PSK_BF16 || L.in[0].dtype == PSK_F32 || L.in[0].dtype == PSK_F16) ;
        if (vec) k_copy_vec8<<<grid_for(e, L.total / 8, 256, 8), 256, 0, e->stream>>>(L);
        else k_copy<<<grid_for(e, L.total, 256, 8), 256, 0, e->stream>>>(L);
        e->kernels += 1;
        break;
    }
    case PSK_OP_CONTRACT: {
        if (l->int_accum) {
            bool ok = L.n_in == 2;
            for (int i = 0; ok && i < 2; ++i) ok = L.in[i].affine != 0 || (L.in[i].dtype == PSK_I8 && L.in[i].scales != nullptr);
            if (!ok) { rc = fail(e, PSK_E7005, std::string(l->name ? l->name : "?") + ": integer sums need two operands that are affine values or integer weights"); break; }
            {
                // On the tensor cores (tcgen05 kind::i8) when the operands are an affine activation with its summed
                // axis contiguous and integer weights with a scale a column: 32-bit sums that wrap are
                // associative, so the result is the scalar kernel's under every order. The raw sum of codes must
                // stay inside 32 bits (k <= 65536); 16-byte rows for the tensor maps.
                GemmMap g;
                static const bool i8_tc = getenv("PSK_I8_TC") ? atoi(getenv("PSK_I8_TC")) != 0 : true;
                const DevOperand &A = L.in[0], &B = L.in[1];
                bool fits = i8_tc && e->encode && map_gemm(L, g) && A.affine != 0 && !B.affine && B.dtype == PSK_I8 && B.scales
                    && g.a_k == 1 && (g.b_k == 1 || g.b_n == 1) && g.k >= 16 && g.k <= 65536 && g.c_col_lo == 1 && g.m >= 1 && g.n >= 16
                    && aligned16(A.p) && aligned16(B.p)
                    && (L.out.affine != 0 || L.out.dtype == PSK_F32 || L.out.dtype == PSK_BF16 || L.out.dtype == PSK_F16 || L.out.dtype == PSK_E8M15);
                for (int a = L.n_outer; fits && a < L.n_outer + L.n_inner; ++a) fits = B.sstride[a] == 0;
                if (fits) {
                    if (g.m == 1) g.a_row = (g.k + 15) / 16 * 16;
                    std::string keep = e->error;
                    const int r = launch_i8(e, g, A, B, L.out, l->out, L.ovf, L.guarded);
                    if (r == PSK_OK) {
                        e->last_kernel = "k_gemm_i8";
                        e->last_flops = 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch;
                        break;
                    }
                    if (r != PSK_E7001) { rc = r; break; }
                    e->error = keep; // strides no tensor map takes: the scalar kernel
                }
            }
            k_contract_int<<<grid_for(e, L.total, 128, 16), 128, 0, e->stream>>>(L);
            e->last_kernel = "k_contract_int";
            e->last_flops = 2.0 * (double)L.total * (double)L.inner;
            e->kernels += 1;
            break;
        }
        if (l->out.affine) {
            // Float sums stored into a `scaled` site (the attention's weighted values when its launches run apart):
            // the nest in index order, every order's permitted choice, its binary32 sum stored as the site's code.
            k_contract_generic<<<grid_for(e, L.total, 256, 8), 256, 0, e->stream>>>(L);
            e->last_kernel = "k_contract_generic";
            e->last_flops = 2.0 * (double)L.total * (double)L.inner;
            e->kernels += 1;
            break;
        }
        GemmMap g;
        bool mapped = map_gemm(L, g);
        const DevOperand &A = L.in[0], &B = L.in[1];
        // int8 weights (operand 1) against bf16 activations under the device order: the weights' integers
        // widened to bf16 once, the channel's scale applied to the sum
        const bool w8 = mapped && device_order && e->encode && B.dtype == PSK_I8 && B.scales && !B.affine && A.dtype == PSK_BF16 && !l->int_accum
            && (L.kdtype == PSK_BF16 || L.kdtype == PSK_F32) && g.a_k == 1 && (g.b_k == 1 || g.b_n == 1) && aligned16(A.p) && g.c_col_lo == 1 && g.n >= 8 && g.k >= 8;
        // e4m3fn weights (a `params` entry narrower than the site: the kernel's loads widen them exactly,
        // presk-kernel/src/ir.rs:47-49) against bf16 activations: every e4m3fn number is a bf16 number, so the
        // same widened copy, without a scale
        const bool wf8 = mapped && device_order && e->encode && B.dtype == PSK_E4M3 && !B.affine && A.dtype == PSK_BF16 && !l->int_accum
            && (L.kdtype == PSK_BF16 || L.kdtype == PSK_F32) && g.a_k == 1 && (g.b_k == 1 || g.b_n == 1) && aligned16(A.p) && g.c_col_lo == 1 && g.n >= 8 && g.k >= 8;
        if (w8 || wf8) {
            bool wide_transient = false;
            void *wide = const_cast<void *>(widened_weights(e, B.p, l->in[1].numel, w8, &wide_transient));
            if (wide) {
                psk_gemm pg;
                memset(&pg, 0, sizeof pg);
                pg.in_dtype = PSK_BF16; pg.out_dtype = L.out.dtype; pg.b_n_major = g.b_k == 1 ? 0 : 1; pg.guarded = L.guarded;
                pg.m = g.m; pg.n = g.n; pg.k = g.k; pg.batch = g.batch; pg.batch_lo = g.batch_lo;
                pg.a_row = g.a_row; pg.a_lo = g.a_lo; pg.a_hi = g.a_hi;
                pg.b_row = pg.b_n_major ? g.b_k : g.b_n; pg.b_lo = g.b_lo; pg.b_hi = g.b_hi;
                pg.c_row_lo_count = g.c_row_lo_count; pg.c_row_lo = g.c_row_lo; pg.c_row_hi = g.c_row_hi;
                pg.c_col_lo_count = g.c_col_lo_count; pg.c_col_hi = g.c_col_hi; pg.c_lo = g.c_lo; pg.c_hi = g.c_hi;
                if (g.m == 1) pg.a_row = g.k;
                std::string keep = e->error;
                int r = launch_tc_few_rows(e, pg, A.p, wide, const_cast<void *>(L.out.p), L.ovf, w8 ? B.scales : nullptr, w8 ? g.bs_n : 0, nullptr, L.out.dtype);
                if (r == PSK_E7001) { e->error = keep; r = launch_tc(e, pg, A.p, wide, const_cast<void *>(L.out.p), L.ovf, w8 ? B.scales : nullptr, w8 ? g.bs_n : 0, w8 ? g.bs_lo : 0, w8 ? g.bs_hi : 0); }
                if (wide_transient) psk_exec_free(e, wide); // handed out again only to later work of the same stream
                if (r == PSK_OK) {
                    e->last_kernel = "k_gemm_tc";
                    e->last_flops = 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch;
                    break;
                }
                if (r != PSK_E7001) { rc = r; break; }
                e->error = keep; // strides no tensor map takes: the exact kernel below
            }
        }
        // e8m15 or f32 operands under the device order: each as two or three bf16 planes (exact), every partial
        // product in one tensor-memory accumulator: exact products, f32 sums in the unit's order, as for bf16
        const bool wide_e = A.dtype == PSK_E8M15 && B.dtype == PSK_E8M15 && (L.kdtype == PSK_E8M15 || L.kdtype == PSK_F32);
        const bool wide_f = A.dtype == PSK_F32 && B.dtype == PSK_F32 && L.kdtype == PSK_F32 && 2.0 * (double)g.m * (double)g.n * (double)g.k >= 1e8;
        if (mapped && device_order && e->encode && (wide_e || wide_f)
            && g.batch == 1 && g.a_k == 1 && (g.b_k == 1 || g.b_n == 1) && g.c_col_lo == 1 && g.k % 64 == 0 && g.n % 8 == 0 && g.m >= 1 && g.n >= 8) {
            const bool bnm = g.b_k != 1;
            const int planes = wide_f ? 3 : 2;
            uint16_t *pa = (uint16_t *)psk_exec_alloc(e, (size_t)g.m * planes * g.k * 2), *pb = (uint16_t *)psk_exec_alloc(e, (size_t)g.n * planes * g.k * 2);
            if (pa && pb) {
                if (wide_f) {
                    k_split_f32<<<grid_for(e, g.m * g.k, 256, 8), 256, 0, e->stream>>>((const float *)A.p, g.m, g.k, g.a_row, pa, planes * g.k, g.k);
                    if (bnm) k_split_f32<<<grid_for(e, g.n * g.k, 256, 8), 256, 0, e->stream>>>((const float *)B.p, g.k, g.n, g.b_k, pb, g.n, g.k * g.n);
                    else k_split_f32<<<grid_for(e, g.n * g.k, 256, 8), 256, 0, e->stream>>>((const float *)B.p, g.n, g.k, g.b_n, pb, planes * g.k, g.k);
                } else {
                    k_split_e8m15<<<grid_for(e, g.m * g.k, 256, 8), 256, 0, e->stream>>>((const uint8_t *)A.p, g.m, g.k, g.a_row, pa, planes * g.k, g.k);
                    if (bnm) k_split_e8m15<<<grid_for(e, g.n * g.k, 256, 8), 256, 0, e->stream>>>((const uint8_t *)B.p, g.k, g.n, g.b_k, pb, g.n, g.k * g.n);
                    else k_split_e8m15<<<grid_for(e, g.n * g.k, 256, 8), 256, 0, e->stream>>>((const uint8_t *)B.p, g.n, g.k, g.b_n, pb, planes * g.k, g.k);
                }
                e->kernels += 2;
                psk_gemm pg;
                memset(&pg, 0, sizeof pg);
                pg.in_dtype = PSK_BF16; pg.out_dtype = L.out.dtype; pg.b_n_major = bnm ? 1 : 0; pg.guarded = L.guarded;
                pg.m = g.m; pg.n = g.n; pg.k = (int64_t)planes * planes * g.k; pg.batch = 1; pg.batch_lo = 1;
                pg.a_row = planes * g.k; pg.a_lo = pg.a_hi = 0;
                pg.b_row = bnm ? g.n : planes * g.k; pg.b_lo = pg.b_hi = 0;
                pg.c_row_lo_count = g.c_row_lo_count; pg.c_row_lo = g.c_row_lo; pg.c_row_hi = g.c_row_hi;
                pg.c_col_lo_count = g.c_col_lo_count; pg.c_col_hi = g.c_col_hi; pg.c_lo = g.c_lo; pg.c_hi = g.c_hi;
                std::string keep = e->error;
                int r = launch_tc(e, pg, pa, pb, const_cast<void *>(L.out.p), L.ovf, nullptr, 0, 0, 0, g.k, planes);
                psk_exec_free(e, pa); // the pool hands a buffer out again only to later work of the same stream
                psk_exec_free(e, pb);
                if (r == PSK_OK) {
                    e->last_kernel = "k_gemm_tc";
                    e->last_flops = 2.0 * (double)g.m * (double)g.n * (double)g.k;
                    break;
                }
                if (r != PSK_E7001) { rc = r; break; }
                e->error = keep;
            } else {
                if (pa) psk_exec_free(e, pa);
                if (pb) psk_exec_free(e, pb);
            }
        }
        bool tc_ok = mapped && device_order && e->encode && A.dtype == B.dtype && (A.dtype == PSK_BF16 || A.dtype == PSK_F16)
            && (L.kdtype == A.dtype || L.kdtype == PSK_F32 || (L.kdtype == PSK_E8M15))
            && (g.a_k == 1 || (g.a_row == 1 && g.m >= 8)) && (g.b_k == 1 || g.b_n == 1) && aligned16(A.p) && aligned16(B.p) && g.c_col_lo == 1 && g.m >= 1 && g.n >= 8 && g.k >= 8;
        if (tc_ok) {
            psk_gemm pg;
            memset(&pg, 0, sizeof pg);
            // a first operand whose rows are contiguous along m (x read as xᵀ in dot_vjp_r): the kernel's M-major form
            const bool a_m_major = g.a_k != 1;
            pg.in_dtype = A.dtype; pg.out_dtype = L.out.dtype; pg.b_n_major = (g.b_k == 1 ? 0 : 1) | (a_m_major ? 2 : 0); pg.guarded = L.guarded;
            pg.m = g.m; pg.n = g.n; pg.k = g.k; pg.batch = g.batch; pg.batch_lo = g.batch_lo;
            pg.a_row = a_m_major ? g.a_k : g.a_row; pg.a_lo = g.a_lo; pg.a_hi = g.a_hi;
            pg.b_row = (pg.b_n_major & 1) ? g.b_k : g.b_n; pg.b_lo = g.b_lo; pg.b_hi = g.b_hi;
            pg.c_row_lo_count = g.c_row_lo_count; pg.c_row_lo = g.c_row_lo; pg.c_row_hi = g.c_row_hi;
            pg.c_col_lo_count = g.c_col_lo_count; pg.c_col_hi = g.c_col_hi; pg.c_lo = g.c_lo; pg.c_hi = g.c_hi;
            if (g.m == 1 && !a_m_major) pg.a_row = g.k; // a single row: any stride of 16 bytes will do
            if (g.n == 1) pg.b_row = g.k;
            std::string keep = e->error;
            rc = launch_tc_few_rows(e, pg, A.p, B.p, const_cast<void *>(L.out.p), L.ovf, nullptr, 0, nullptr, L.out.dtype);
            if (rc == PSK_E7001) { e->error = keep; rc = launch_tc(e, pg, A.p, B.p, const_cast<void *>(L.out.p), L.ovf); }
            e->last_kernel = "k_gemm_tc";
            e->last_flops = 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch;
            if (rc == PSK_E7001) { rc = PSK_OK; e->error = keep; tc_ok = false; } // strides no tensor map takes: the exact kernel
        }
        if (!tc_ok && rc == PSK_OK) {
            if (mapped && g.k >= 1) {
                DevGemmExact G;
                memset(&G, 0, sizeof G);
                G.a = A.p; G.b = B.p; G.c = const_cast<void *>(L.out.p);
                G.a_dtype = A.dtype; G.b_dtype = B.dtype; G.c_dtype = L.out.dtype; G.kdtype = L.kdtype;
                G.m = g.m; G.n = g.n; G.k = g.k;
                G.a_i = g.a_row; G.a_k = g.a_k; G.b_k = g.b_k; G.b_j = g.b_n;
                G.batch_lo = g.batch_lo; G.a_lo = g.a_lo; G.a_hi = g.a_hi; G.b_lo = g.b_lo; G.b_hi = g.b_hi; G.c_lo = g.c_lo; G.c_hi = g.c_hi;
                G.c_row_lo_count = g.c_row_lo_count; G.c_row_lo = g.c_row_lo; G.c_row_hi = g.c_row_hi;
                G.c_col_lo_count = g.c_col_lo_count; G.c_col_lo = g.c_col_lo; G.c_col_hi = g.c_col_hi;
                G.b_scales = B.scales; G.b_sj = g.bs_n; G.b_slo = g.bs_lo; G.b_shi = g.bs_hi;
                G.ovf = L.ovf; G.guarded = L.guarded;
                G.chunk = L.chunk;
                dim3 grid((unsigned)((g.n + 63) / 64), (unsigned)((g.m + 63) / 64), (unsigned)g.batch);
                e->last_flops = 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch;
                if (grid.y > 65535 || grid.z > 65535) { k_contract_generic<<<grid_for(e, L.total, 256, 8), 256, 0, e->stream>>>(L); e->last_kernel = "k_contract_generic"; }
                else if (!L.chunk && g.m >= 128 && g.n >= 128 && (A.dtype == PSK_F32 || A.dtype == PSK_BF16) && (B.dtype == PSK_F32 || B.dtype == PSK_BF16) && (g.m + 127) / 128 <= 65535) {
                    dim3 big((unsigned)((g.n + 127) / 128), (unsigned)((g.m + 127) / 128), (unsigned)g.batch);
                    if (A.dtype == PSK_F32 && B.dtype == PSK_F32) k_gemm_exact_big<PSK_F32, PSK_F32><<<big, 256, 0, e->stream>>>(G);
                    else if (A.dtype == PSK_BF16 && B.dtype == PSK_BF16) k_gemm_exact_big<PSK_BF16, PSK_BF16><<<big, 256, 0, e->stream>>>(G);
                    else if (A.dtype == PSK_F32) k_gemm_exact_big<PSK_F32, PSK_BF16><<<big, 256, 0, e->stream>>>(G);
                    else k_gemm_exact_big<PSK_BF16, PSK_F32><<<big, 256, 0, e->stream>>>(G);
                    e->last_kernel = "k_gemm_exact";
                }
                else { k_gemm_exact<<<grid, 256, 0, e->stream>>>(G); e->last_kernel = "k_gemm_exact"; }
            } else {
                k_contract_generic<<<grid_for(e, L.total, 256, 8), 256, 0, e->stream>>>(L);
                e->last_kernel = "k_contract_generic";
                e->last_flops = 2.0 * (double)L.total * (double)L.inner;
            }
            e->kernels += 1;
        }
        break;
    }
    case PSK_OP_REDUCE: {
        e->last_kernel = "k_reduce";
        // Under the device order a sum's terms may be regrouped; `sum_to`, whose running sum the reference keeps in the
        // output's storage, is then summed in f32 and rounded once like any other (a declared difference in order).
        const bool may_regroup = device_order;
        const bool cols = may_regroup && L.n_outer >= 1 && L.n_inner >= 1 && L.inner >= 64 && L.in[0].stride[L.n_outer - 1] == 1 && L.in[0].stride[L.n_outer + L.n_inner - 1] != 1;
        if (may_regroup && L.n_outer == 0 && L.inner >= (1ll << 20)) {
            const int blocks = std::min(e->sms * 2, 1024);
            float *partials = (float *)psk_exec_alloc(e, (size_t)blocks * 4);
            if (!partials) { rc = fail(e, PSK_E10001, "reduce: no memory for the partial sums"); break; }
            // one contiguous run of numbers the kernel reads unrounded: sixteen bytes a load
            const DevOperand &X = L.in[0];
            bool lin = (L.kind == PSK_REDUCE_SUMSQ || L.kind == PSK_REDUCE_SUM) && !X.affine && L.inner % 8 == 0 && aligned16(X.p)
                && ((X.dtype == PSK_BF16 && (L.kdtype == PSK_BF16 || L.kdtype == PSK_F32)) || (X.dtype == PSK_F32 && L.kdtype == PSK_F32));
            {
                int64_t expect = 1;
                for (int a = L.n_inner - 1; a >= 0 && lin; --a) { lin = X.stride[a] == expect; expect *= L.dims[a]; }
            }
            if (lin && X.dtype == PSK_BF16) k_reduce_all_partials_lin<true><<<blocks, 512, 0, e->stream>>>(X.p, L.inner / 8, L.kind == PSK_REDUCE_SUMSQ ? 1 : 0, partials);
            else if (lin) k_reduce_all_partials_lin<false><<<blocks, 512, 0, e->stream>>>(X.p, L.inner / 8, L.kind == PSK_REDUCE_SUMSQ ? 1 : 0, partials);
            else
            k_reduce_all_partials<<<blocks, 1024, 0, e->stream>>>(L, partials);
            k_reduce_all_finish<<<1, 1024, 0, e->stream>>>(L, partials, blocks);
            psk_exec_free(e, partials); // handed out again only to later work of the same stream
            e->kernels += 1;
        }
        else if (may_regroup && L.n_outer == 0) k_reduce_all_tree<<<1, 1024, 0, e->stream>>>(L);
        else if (may_regroup && L.n_inner == 1 && L.in[0].stride[L.n_outer] == 1 && L.inner >= 64 && (L.inner % 8 != 0 || vec8_operand(L.in[0], L.dims, L.n_outer + 1, false) ))
            k_reduce_rows_tree<<<grid_for(e, L.total * 32, 256, 8), 256, 0, e->stream>>>(L);
        else if (cols) k_reduce_cols_tree<<<(int)std::min<int64_t>((L.total + 31) / 32, (int64_t)e->sms * 2), 1024, 0, e->stream>>>(L);
        else if (L.n_inner == 1 && L.inner >= 512 && L.total <= (int64_t)e->sms * 4) k_reduce_seq_staged<<<(int)std::max<int64_t>(1, L.total), 256, 0, e->stream>>>(L); // few long sums
        else k_reduce_seq<<<grid_for(e, L.total, 128, 16), 128, 0, e->stream>>>(L);
        e->kernels += 1;
        break;
    }
    case PSK_OP_SOFTMAX: {
        e->last_kernel = "k_softmax";
        if (L.n_inner != 1) { rc = fail(e, PSK_E7001, "softmax: one axis"); break; }
        if (L.masked) {
            auto it = e->causal.find(table[1]);
            const int64_t n = L.inner;
            bool causal = it != e->causal.end() && it->second == n && l->in[1].offset == 0 && L.in[1].stride[L.n_outer] == 1;
            for (int a = 0; causal && a < L.n_outer; ++a) causal = L.in[1].stride[a] % n == 0 && L.in[1].stride[a] / n <= 1;
            L.iparam[0] = causal ? 1 : 0;
            L.iparam[1] = n;
        }
        const int64_t n = L.inner;
        bool rows = device_order && L.in[0].stride[L.n_outer] == 1 && L.out.stride[L.n_outer] == 1 && n % 8 == 0 && n <= 6144
            && vec8_operand(L.in[0], L.dims, L.n_outer + 1, false) && vec8_operand(L.out, L.dims, L.n_outer + 1, true)
            && (!L.masked || L.iparam[0] == 1 || L.in[1].stride[L.n_outer] == 1);
        if (rows && n * 4 * 4 <= 96 * 1024) {
            // flat rows: every outer axis of the scores walks contiguous rows; the causal mask's row is the
            // position along the last outer axis
            bool flat = L.total < 0x7fffffffll;
            {
                int64_t expect = n;
                for (int a = L.n_outer - 1; a >= 0 && flat; --a) {
                    flat = L.in[0].stride[a] == expect && L.out.stride[a] == expect;
                    expect *= L.dims[a];
                }
                if (flat && L.masked) {
                    flat = L.iparam[0] == 1 && L.n_outer >= 1 && L.in[1].stride[L.n_outer - 1] == n;
                    for (int a = 0; a + 1 < L.n_outer && flat; ++a) flat = L.in[1].stride[a] == 0;
                    L.iparam[3] = L.n_outer >= 1 ? L.dims[L.n_outer - 1] : 1;
                }
            }
            L.iparam[2] = flat ? 1 : 0;
            if (!e->softmax_attr_set) {
                CUDA_TRY(e, cudaFuncSetAttribute(k_softmax_rows_smem<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
                e->softmax_attr_set = true;
            }
            const size_t smem = (size_t)n * 4 * 4;
            const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / std::max<size_t>(smem, 1)));
            k_softmax_rows_smem<4><<<grid_for(e, L.total * 32, 128, per_sm), 128, smem, e->stream>>>(L);
        } else {
            k_softmax_seq<<<grid_for(e, L.total, 128, 16), 128, 0, e->stream>>>(L);
        }
        e->kernels += 1;
        break;
    }
    case PSK_OP_ATTENTION: {
        // (batch, heads, seq, hd | seq2) or (batch, groups, per, seq, hd | seq2); see psk_attn.cuh
        e->last_kernel = l->iparam[0] == 1 ? "k_attn_fwd3" : "k_attn_fwd";
        const std::string nm = l->name ? l->name : "attention";
        if (!device_order) { rc = fail(e, PSK_E7005, nm + ": blockwise attention is a declared order; under the sequential order the four launches run one by one"); break; }
        const int no = L.n_outer;
        if ((no != 4 && no != 5) || L.n_inner != 1 || (L.n_in != 4 && L.n_in != 5)) { rc = fail(e, PSK_E7001, nm + ": q, k, v, the divisor and at most a mask over (batch, [groups,] heads, seq, hd | seq2)"); break; }
        const int ax_hd = no - 1, ax_seq = no - 2, ax_s2 = no, ax_b = 0, ax_g = 1, ax_p = no == 5 ? 2 : -1;
        const int64_t B = L.dims[ax_b], G = L.dims[ax_g], Pn = ax_p >= 0 ? L.dims[ax_p] : 1, T = L.dims[ax_seq], HD = L.dims[ax_hd];
        const bool aff_out = l->out.affine != 0; // the result as one-byte codes of an affine format (the `scaled` site of the weighted values)
        if (T == 1 && L.n_in == 4) {
            // one query position against a cache of keys and values (a decode step): a stream of the cache, see psk_attn_step.cuh
            e->last_kernel = "k_attn_step";
            const int64_t T2 = L.dims[ax_s2];
            const DevOperand &Q = L.in[0], &K = L.in[1], &V = L.in[2], &O = L.out;
            bool ok = HD == attn_step::HD && l->dtype == PSK_BF16 && (aff_out ? (l->out.dtype == PSK_I8 || l->out.dtype == PSK_U8) : l->out.dtype == PSK_BF16) && l->iparam[1] == PSK_BF16 && l->iparam[2] == PSK_BF16 && l->iparam[3] == PSK_BF16
                && T2 >= 1 && T2 <= 49152 && B * G * Pn <= 0x7fffffff && G <= 0x7fffffff && Pn <= 0x7fffffff;
            for (int i = 0; i < 3 && ok; ++i) ok = l->in[i].dtype == PSK_BF16 && L.in[i].stride[ax_hd] == 1 && ((uintptr_t)L.in[i].p % 8) == 0 && L.in[i].stride[ax_b] % 4 == 0 && L.in[i].stride[ax_g] % 4 == 0;
            ok = ok && O.stride[ax_hd] == 1 && K.stride[ax_s2] % 4 == 0 && V.stride[ax_s2] % 4 == 0 && Q.stride[ax_s2] == 0 && O.stride[ax_s2] == 0 && K.stride[ax_seq] == 0 && V.stride[ax_seq] == 0;
            if (ax_p >= 0) ok = ok && K.stride[ax_p] == 0 && V.stride[ax_p] == 0 && Q.stride[ax_p] % 4 == 0;
            if (!ok) { rc = fail(e, PSK_E7005, nm + ": the step's attention runs bf16 sites, hd = 128 and no mask over a cache of at most 49152 positions"); break; }
            attn_step::Params A;
            memset(&A, 0, sizeof A);
            A.q = (const uint16_t *)Q.p; A.k = (const uint16_t *)K.p; A.v = (const uint16_t *)V.p; A.out = (uint16_t *)const_cast<void *>(O.p);
            A.q_b = Q.stride[ax_b]; A.q_g = Q.stride[ax_g]; A.q_p = ax_p >= 0 ? Q.stride[ax_p] : 0;
            A.k_b = K.stride[ax_b]; A.k_g = K.stride[ax_g]; A.k_t = K.stride[ax_s2];
            A.v_b = V.stride[ax_b]; A.v_g = V.stride[ax_g]; A.v_t = V.stride[ax_s2];
            A.o_b = O.stride[ax_b]; A.o_g = O.stride[ax_g]; A.o_p = ax_p >= 0 ? O.stride[ax_p] : 0;
            A.G = (int32_t)G; A.Pn = (int32_t)Pn; A.len = (int32_t)T2;
            A.rt = L.in[3].p; A.rt_dtype = L.in[3].dtype;
            A.aff_kind = l->out.affine; A.aff_zero = l->out.affine_zero; A.aff_scale = l->out.affine_scale;
            const size_t smem = (size_t)T2 * sizeof(float);
            if (smem > 48 * 1024 && !e->attn_step_attr_set) {
                CUDA_TRY(e, cudaFuncSetAttribute(attn_step::k_attn_step, cudaFuncAttributeMaxDynamicSharedMemorySize, 49152 * (int)sizeof(float)));
                e->attn_step_attr_set = true;
            }
            attn_step::k_attn_step<<<(unsigned)(B * G * Pn), attn_step::THREADS, smem, e->stream>>>(A);
            e->last_flops = 4.0 * (double)(B * G * Pn) * (double)T2 * (double)HD;
            e->kernels += 1;
            break;
        }
        // (codes come out of the one-pass kernel only: 16-byte stores of sixteen codes)
        bool fits = HD == attn::HD && T == L.dims[ax_s2] && T % attn::BM == 0 && l->dtype == PSK_BF16
            && (aff_out ? ((l->out.dtype == PSK_I8 || l->out.dtype == PSK_U8) && l->iparam[0] == 1) : l->out.dtype == PSK_BF16)
            && l->iparam[1] == PSK_BF16 && l->iparam[2] == PSK_BF16 && l->iparam[3] == PSK_BF16;
        for (int i = 0; i < 3 && fits; ++i) fits = l->in[i].dtype == PSK_BF16 && L.in[i].stride[ax_hd] == 1 && aligned16(L.in[i].p);
        const DevOperand &Q = L.in[0], &K = L.in[1], &V = L.in[2], &O = L.out;
        const int64_t o_unit = aff_out ? 16 : 8; // elements of a 16-byte store
        fits = fits && O.stride[ax_hd] == 1 && aligned16(O.p) && O.stride[ax_seq] % o_unit == 0 && O.stride[ax_b] % o_unit == 0 && O.stride[ax_g] % o_unit == 0;
        fits = fits && Q.stride[ax_s2] == 0 && K.stride[ax_seq] == 0 && V.stride[ax_seq] == 0 && O.stride[ax_s2] == 0;
        int64_t q_head = Q.stride[ax_g], o_head = O.stride[ax_g];
        if (ax_p >= 0) {
            fits = fits && K.stride[ax_p] == 0 && V.stride[ax_p] == 0 && (Pn == 1 || (Q.stride[ax_g] == Q.stride[ax_p] * Pn && O.stride[ax_g] == O.stride[ax_p] * Pn));
            if (Pn > 1) { q_head = Q.stride[ax_p]; o_head = O.stride[ax_p]; }
        }
        bool causal = false;
        if (fits && L.n_in == 5) {
            auto it = e->causal.find(table[4]);
            causal = it != e->causal.end() && it->second == T && l->in[4].offset == 0 && L.in[4].stride[ax_s2] == 1 && L.in[4].stride[ax_seq] == T && L.in[4].stride[ax_hd] == 0;
            for (int a = 0; a < ax_seq && causal; ++a) causal = L.in[4].stride[a] == 0;
            fits = causal;
        }
        if (!fits) { rc = fail(e, PSK_E7005, nm + ": blockwise attention runs bf16 sites, hd = 128, a sequence that is a multiple of 128 and no mask or the causal one"); break; }
        if (!e->encode) { rc = fail(e, PSK_E10001, "cuTensorMapEncodeTiled is not available from this driver"); break; }
        // two kernels of the same computation: key blocks of 128 and one CTA an SM, or of 64 and two (see psk_attn.cuh)
        static const bool two_a_sm = getenv("PSK_ATTN_KERNEL") ? atoi(getenv("PSK_ATTN_KERNEL")) != 1 : true; // measured: 0.63 ms against 0.74 ms at B = 8, H = 32, T = 2048
        const bool online = l->iparam[0] == 1; // the declared order `attention: online`: one pass, a running reference maximum
        CUtensorMap mq, mk, mv;
        bool ok = make_map(e, &mq, Q.p, 0, (uint64_t)HD, (uint64_t)T, (uint64_t)(G * Pn), (uint64_t)B, (uint64_t)Q.stride[ax_seq], (uint64_t)q_head, (uint64_t)Q.stride[ax_b], 64, attn::BM)
            && make_map(e, &mk, K.p, 0, (uint64_t)HD, (uint64_t)T, (uint64_t)G, (uint64_t)B, (uint64_t)K.stride[ax_s2], (uint64_t)K.stride[ax_g], (uint64_t)K.stride[ax_b], 64, (two_a_sm || online) ? attn::v2::BN2 : attn::BN)
            && make_map(e, &mv, V.p, 0, (uint64_t)HD, (uint64_t)T, (uint64_t)G, (uint64_t)B, (uint64_t)V.stride[ax_s2], (uint64_t)V.stride[ax_g], (uint64_t)V.stride[ax_b], 64, (two_a_sm || online) ? attn::v2::BN2 : attn::BN);
        if (!ok) { rc = fail(e, PSK_E7001, nm + ": an operand's strides do not make a tensor map"); break; }
        attn::Params A;
        memset(&A, 0, sizeof A);
        A.T = T; A.causal = causal ? 1 : 0; A.per = (int32_t)Pn;
        A.out = const_cast<void *>(O.p); A.o_b = O.stride[ax_b]; A.o_g = o_head; A.o_t = O.stride[ax_seq];
        A.rt = L.in[3].p; A.rt_dtype = L.in[3].dtype;
        A.status = e->status;
        A.aff_kind = l->out.affine; A.aff_zero = l->out.affine_zero; A.aff_scale = l->out.affine_scale;
        if (!e->attn_attr_set) {
            CUDA_TRY(e, cudaFuncSetAttribute(attn::k_attn_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_TOTAL));
            CUDA_TRY(e, cudaFuncSetAttribute(attn::v2::k_attn_fwd2, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::v2::SMEM_TOTAL2));
            CUDA_TRY(e, cudaFuncSetAttribute(attn::v3::k_attn_fwd3, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::v3::SMEM_TOTAL3));
            e->attn_attr_set = true;
        }
        const int64_t nqb = T / attn::BM;
        if (G * Pn > 65535 || B > 65535) { rc = fail(e, PSK_E7001, nm + ": more heads or batch entries than a grid holds"); break; }
        dim3 grid((unsigned)nqb, (unsigned)(G * Pn), (unsigned)B);
        if (online) attn::v3::k_attn_fwd3<<<grid, attn::v3::THREADS3, attn::v3::SMEM_TOTAL3, e->stream>>>(mq, mk, mv, A);
        else if (two_a_sm) attn::v2::k_attn_fwd2<<<grid, attn::v2::THREADS2, attn::v2::SMEM_TOTAL2, e->stream>>>(mq, mk, mv, A);
        else attn::k_attn_fwd<<<grid, attn::THREADS, attn::SMEM_TOTAL, e->stream>>>(mq, mk, mv, A);
        const double blocks = causal ? (double)nqb * (double)(nqb + 1) / 2.0 : (double)nqb * (double)nqb;
        e->last_flops = 4.0 * (double)B * (double)(G * Pn) * blocks * 128.0 * 128.0 * (double)HD;
        e->kernels += 1;
        break;
    }
    case PSK_OP_RMSNORM: {
        e->last_kernel = "k_rmsnorm_rows";
        const std::string nm = l->name ? l->name : "rmsnorm";
        const int no = L.n_outer;
        if (no < 1 || L.n_inner != 0 || L.n_in != 3) { rc = fail(e, PSK_E7001, nm + ": x, eps and gamma over the axes of x"); break; }
        const int64_t n = L.dims[no - 1];
        // rows: every leading axis of x and of the result must walk whole rows one after the other
        const bool aff_out = l->out.affine != 0; // the result as one-byte codes of an affine format
        bool fits = device_order && l->dtype == PSK_BF16 && l->in[0].dtype == PSK_BF16 && l->in[2].dtype == PSK_BF16 && (aff_out ? (l->out.dtype == PSK_I8 || l->out.dtype == PSK_U8) : l->out.dtype == PSK_BF16)
            && l->iparam[0] == n && l->iparam[1] == PSK_BF16 && l->iparam[2] == PSK_F32 && l->iparam[3] == PSK_F32
            && n % 256 == 0 && (n / 256 == 1 || n / 256 == 2 || n / 256 == 4 || n / 256 == 8 || n / 256 == 16)
            && L.in[0].stride[no - 1] == 1 && L.out.stride[no - 1] == 1 && L.in[2].stride[no - 1] == 1
            && aligned16(L.in[0].p) && aligned16(L.out.p) && aligned16(L.in[2].p) && !l->in[1].is_index && l->in[1].dtype != PSK_F64 && l->in[1].dtype != PSK_I8;
        int64_t rows = 1, x_row = n, o_row = n;
        for (int a = no - 2; a >= 0 && fits; --a) {
            if (a == no - 2) { x_row = L.in[0].stride[a]; o_row = L.out.stride[a]; }
            else fits = L.in[0].stride[a] == x_row * rows && L.out.stride[a] == o_row * rows;
            fits = fits && L.in[2].stride[a] == 0;
            rows *= L.dims[a];
        }
        fits = fits && x_row % 8 == 0 && o_row % 8 == 0;
        if (!fits) { rc = fail(e, PSK_E7005, nm + ": the merged norm runs under the device order on bf16 rows of 256, 512, 1024, 2048 or 4096 elements with f32 statistics"); break; }
        RmsParams R;
        R.x = (const uint16_t *)L.in[0].p; R.gamma = (const uint16_t *)L.in[2].p; R.eps = L.in[1].p; R.eps_dtype = L.in[1].dtype;
        R.out = (uint16_t *)const_cast<void *>(L.out.p); R.x_row = x_row; R.out_row = o_row; R.rows = rows; R.n = (int32_t)n;
        R.aff_kind = l->out.affine; R.aff_zero = l->out.affine_zero; R.aff_scale = l->out.affine_scale;
        const int g = grid_for(e, rows * 32, 256, 8);
        if (aff_out) {
            switch (n / 256) {
            case 1: k_rmsnorm_rows<1, true><<<g, 256, 0, e->stream>>>(R); break;
            case 2: k_rmsnorm_rows<2, true><<<g, 256, 0, e->stream>>>(R); break;
            case 4: k_rmsnorm_rows<4, true><<<g, 256, 0, e->stream>>>(R); break;
            case 8: k_rmsnorm_rows<8, true><<<g, 256, 0, e->stream>>>(R); break;
            default: k_rmsnorm_rows<16, true><<<g, 256, 0, e->stream>>>(R); break;
            }
        } else
        switch (n / 256) {
        case 1: k_rmsnorm_rows<1><<<g, 256, 0, e->stream>>>(R); break;
        case 2: k_rmsnorm_rows<2><<<g, 256, 0, e->stream>>>(R); break;
        case 4: k_rmsnorm_rows<4><<<g, 256, 0, e->stream>>>(R); break;
        case 8: k_rmsnorm_rows<8><<<g, 256, 0, e->stream>>>(R); break;
        default: k_rmsnorm_rows<16><<<g, 256, 0, e->stream>>>(R); break;
        }
        e->kernels += 1;
        break;
    }
    case PSK_OP_ROPE: {
        e->last_kernel = "k_rope_bf16";
        const std::string nm = l->name ? l->name : "rope";
        const int no = L.n_outer;
        if (no < 3 || L.n_inner != 0 || L.n_in != 3 || L.dims[no - 2] != 2) { rc = fail(e, PSK_E7001, nm + ": x over (.., seq, pair = 2, rot), cos and sin over (seq, rot)"); break; }
        const int64_t rot = L.dims[no - 1], T = L.dims[no - 3];
        bool fits = l->dtype == PSK_BF16 && l->out.dtype == PSK_BF16 && rot % 8 == 0 && rot <= (1 << 20) && T <= 0x7fffffff;
        for (int i = 0; i < 3 && fits; ++i) fits = l->in[i].dtype == PSK_BF16 && aligned16(L.in[i].p) && L.in[i].stride[no - 1] == 1;
        fits = fits && aligned16(L.out.p) && L.out.stride[no - 1] == 1;
        // x and the result: whole rows of 2·rot one after the other; the tables: [seq, rot], broadcast elsewhere
        int64_t expect = 1, rows = 1;
        for (int a = no - 1; a >= 0 && fits; --a) {
            fits = L.in[0].stride[a] == expect && L.out.stride[a] == expect;
            const int64_t tab = a == no - 1 ? 1 : a == no - 3 ? rot : 0;
            fits = fits && L.in[1].stride[a] == tab && L.in[2].stride[a] == tab;
            expect *= L.dims[a];
            if (a <= no - 3) rows *= L.dims[a];
        }
        if (!fits) { rc = fail(e, PSK_E7005, nm + ": the merged rotation runs on contiguous bf16 rows with bf16 tables over (seq, rot)"); break; }
        RopeParams R;
        R.x = (const uint16_t *)L.in[0].p; R.c = (const uint16_t *)L.in[1].p; R.s = (const uint16_t *)L.in[2].p;
        R.out = (uint16_t *)const_cast<void *>(L.out.p); R.rows = rows; R.seq = (int32_t)T; R.rotv = (int32_t)(rot / 8);
        k_rope_bf16<<<grid_for(e, rows * (rot / 8), 256, 8), 256, 0, e->stream>>>(R);
        e->kernels += 1;
        break;
    }
    case PSK_OP_CONTRACT_ADD: {
        const std::string nm = l->name ? l->name : "contract+add";
        if (L.n_in != 3) { rc = fail(e, PSK_E7001, nm + ": two operands of a contraction and an addend"); break; }
        DevLaunch L2 = L;
        L2.n_in = 2;
        GemmMap g;
        const bool mapped = map_gemm(L2, g);
        const DevOperand &A = L.in[0], &B = L.in[1], &X = L.in[2];
        if (l->int_accum) {
            // Integer sums (tcgen05 kind::i8), their rescaled product rounded to bf16, then the addend: both steps are
            // exact per element whatever the order of the sums, so every order takes this path.
            bool fits = mapped && e->encode && A.affine != 0 && !B.affine && B.dtype == PSK_I8 && B.scales && X.dtype == PSK_BF16 && !X.affine && !L.out.affine
                && l->dtype == PSK_BF16 && l->out.dtype == PSK_BF16 && l->iparam[1] == PSK_BF16
                && g.a_k == 1 && (g.b_k == 1 || g.b_n == 1) && g.k >= 16 && g.k <= 65536 && g.c_col_lo == 1 && g.m >= 1 && g.n >= 16
                && aligned16(A.p) && aligned16(B.p) && aligned16(X.p);
            for (int a = L.n_outer; fits && a < L.n_outer + L.n_inner; ++a) fits = B.sstride[a] == 0;
            for (int a = 0; a < L.n_outer && fits; ++a) fits = L.dims[a] == 1 || X.stride[a] == L.out.stride[a];
            if (!fits) { rc = fail(e, PSK_E7005, nm + ": the merged integer contraction and addition take an affine operand, integer weights, a bf16 addend laid out as the bf16 result"); break; }
            if (g.m == 1) g.a_row = (g.k + 15) / 16 * 16;
            const int r = launch_i8(e, g, A, B, L.out, l->out, L.ovf, false, X.p);
            if (r == PSK_E7001) { rc = fail(e, PSK_E7005, nm + ": " + e->error); break; }
            rc = r;
            e->last_kernel = "k_gemm_i8";
            e->last_flops = 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch;
            break;
        }
        const bool b_int8 = B.dtype == PSK_I8 && B.scales, b_e4m3 = B.dtype == PSK_E4M3; // as in a plain contraction: read through a widened copy
        bool fits = mapped && device_order && e->encode && A.dtype == PSK_BF16 && (B.dtype == PSK_BF16 || b_int8 || b_e4m3) && X.dtype == PSK_BF16 && !any_affine
            && l->dtype == PSK_BF16 && l->out.dtype == PSK_BF16 && l->iparam[1] == PSK_BF16
            && g.a_k == 1 && (g.b_k == 1 || g.b_n == 1) && aligned16(A.p) && aligned16(B.p) && aligned16(X.p) && g.c_col_lo == 1 && g.m >= 1 && g.n >= 8 && g.k >= 8;
        for (int a = 0; a < L.n_outer && fits; ++a) fits = L.dims[a] == 1 || X.stride[a] == L.out.stride[a]; // the addend walks the space as the result does
        if (!fits) { rc = fail(e, PSK_E7005, nm + ": the merged contraction and addition run on the tensor cores, bf16 throughout, the addend laid out as the result"); break; }
        psk_gemm pg;
        memset(&pg, 0, sizeof pg);
        pg.in_dtype = PSK_BF16; pg.out_dtype = PSK_BF16; pg.b_n_major = g.b_k == 1 ? 0 : 1; pg.guarded = 0;
        pg.m = g.m; pg.n = g.n; pg.k = g.k; pg.batch = g.batch; pg.batch_lo = g.batch_lo;
        pg.a_row = g.a_row; pg.a_lo = g.a_lo; pg.a_hi = g.a_hi;
        pg.b_row = pg.b_n_major ? g.b_k : g.b_n; pg.b_lo = g.b_lo; pg.b_hi = g.b_hi;
        pg.c_row_lo_count = g.c_row_lo_count; pg.c_row_lo = g.c_row_lo; pg.c_row_hi = g.c_row_hi;
        pg.c_col_lo_count = g.c_col_lo_count; pg.c_col_hi = g.c_col_hi; pg.c_lo = g.c_lo; pg.c_hi = g.c_hi;
        if (g.m == 1) pg.a_row = g.k;
        const void *bp = B.p;
        bool bp_transient = false;
        if (b_int8 || b_e4m3) {
            bp = widened_weights(e, B.p, l->in[1].numel, b_int8, &bp_transient);
            if (!bp) { rc = fail(e, PSK_E7005, nm + ": no memory for the weights' bf16 copy"); break; }
        }
        std::string keep_err = e->error;
        int r = launch_tc_few_rows(e, pg, A.p, bp, const_cast<void *>(L.out.p), L.ovf, b_int8 ? B.scales : nullptr, b_int8 ? g.bs_n : 0, X.p, (int)l->iparam[1]);
        if (r == PSK_E7001) { e->error = keep_err; r = launch_tc(e, pg, A.p, bp, const_cast<void *>(L.out.p), L.ovf, b_int8 ? B.scales : nullptr, b_int8 ? g.bs_n : 0, b_int8 ? g.bs_lo : 0, b_int8 ? g.bs_hi : 0, 0, 2, X.p); }
        if (bp_transient) psk_exec_free(e, const_cast<void *>(bp));
        if (r == PSK_E7001) { rc = fail(e, PSK_E7005, nm + ": " + e->error); break; } // strides no tensor map or staged epilogue takes: the caller's two launches
        rc = r;
        e->last_kernel = "k_gemm_tc";
        e->last_flops = 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch;
        break;
    }
    case PSK_OP_XENT: {
        e->last_kernel = "k_xent";
        if (L.n_inner != 1 || L.n_in != 2) { rc = fail(e, PSK_E7001, "cross_entropy: logits and labels"); break; }
        bool vec_ok = L.in[0].stride[L.n_outer] != 1 || L.inner % 8 != 0 || vec8_operand(L.in[0], L.dims, L.n_outer + 1, false);
        if (device_order && L.inner >= 256 && vec_ok) k_xent_rows_tree<<<(int)std::min<int64_t>(L.total, (int64_t)e->sms * 8), 256, 0, e->stream>>>(L);
        else k_xent_seq<<<grid_for(e, L.total, 128, 16), 128, 0, e->stream>>>(L);
        e->kernels += 1;
        break;
    }
    case PSK_OP_XENT_VJP: {
        e->last_kernel = "k_xent_vjp";
        if (L.n_inner != 1 || L.n_in != 3) { rc = fail(e, PSK_E7001, "cross_entropy_vjp: logits, labels and a cotangent"); break; }
        if (device_order && L.inner >= 256) k_xent_vjp_rows_tree<<<(int)std::min<int64_t>(L.total, (int64_t)e->sms * 8), 256, 0, e->stream>>>(L);
        else k_xent_vjp_rows<<<(int)std::min<int64_t>((L.total + 3) / 4, (int64_t)e->sms * 16), 128, 0, e->stream>>>(L);
        e->kernels += 1;
        break;
    }
    case PSK_OP_EMBED_VJP: {
        e->last_kernel = "k_embed_vjp";
        if (L.n_inner != 0 || L.n_in != 3 || L.n_outer < 2 || l->iparam[0] < 0) { rc = fail(e, PSK_E7001, "embed_vjp: a table, indices with an axis and a cotangent"); break; }
        if (l->iparam[0] > 0) {
            k_embed_vjp<<<(int)std::min<int64_t>(l->iparam[0], (int64_t)e->sms * 8), 256, 0, e->stream>>>(L);
            e->kernels += 1;
        }
        break;
    }
    case PSK_OP_ARGMAX:
        k_argmax<<<grid_for(e, L.total, 128, 16), 128, 0, e->stream>>>(L);
        e->kernels += 1;
        break;
    case PSK_OP_EMBED: {
        e->last_kernel = "k_embed";
        const int last = L.n_outer - 1;
        int64_t work = L.total / (L.dims[last] % 8 == 0 ? 8 : 1);
        k_embed<<<grid_for(e, work, 256, 8), 256, 0, e->stream>>>(L);
        e->kernels += 1;
        break;
    }
    case PSK_OP_IOTA:
        k_iota<<<grid_for(e, L.total, 256, 8), 256, 0, e->stream>>>(L);
        e->kernels += 1;
        if (l->kind == PSK_IOTA_CAUSAL && l->out.offset == 0) e->causal[table[l->n_inputs]] = l->dims[1];
        break;
    case PSK_OP_CONVERT: {
        int64_t n = L.total;
        k_convert<<<grid_for(e, n, 256, 8), 256, 0, e->stream>>>(L.in[0].p, L.in[0].dtype, const_cast<void *>(L.out.p), L.out.dtype, n, L.guarded, L.ovf, L.in[0].affine, L.in[0].affine_zero, L.in[0].affine_scale);
        e->kernels += 1;
        break;
    }
    case PSK_OP_MAGNITUDE: {
        // the input is read flat: its `numel` elements from its offset
        const int64_t n = l->in[0].numel;
        if (n > 0) k_magnitude<<<grid_for(e, n, 256, 8), 256, 0, e->stream>>>(L.in[0].p, L.in[0].dtype, n, (uint32_t *)const_cast<void *>(L.out.p));
        e->kernels += 1;
        break;
    }
    default:
        rc = fail(e, PSK_E7001, std::string(l->name ? l->name : "?") + ": no such operation");
    }
    if (rc == PSK_OK) {
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) rc = fail(e, PSK_E10001, std::string(l->name ? l->name : "?") + ": " + cudaGetErrorString(err));
    }
    if (e->profiling) {
        cudaEventRecord(e->ev1, e->stream);
        cudaEventRecord(pb, e->stream);
        // algorithmic bytes: every operand once at its stored width (the reference's Q, presk-kernel/src/cost.rs:92-95)
        double bytes = (double)l->out.numel * (double)elem_bytes(l->out.dtype);
        for (int i = 0; i < l->n_inputs; ++i) bytes += (double)l->in[i].numel * (double)elem_bytes(l->in[i].dtype);
        e->prof.push_back({l->name ? l->name : "?", e->last_kernel, e->last_flops, bytes, pa, pb});
    }
    e->launches += 1;
    return rc;
}

// ---- helpers of the host program that are device work -----------------------
int psk_exec_quantize(psk_exec *e, const void *w, int from, int8_t *q, float *s, int64_t outer, int64_t k, int64_t inner)
{
    cudaSetDevice(e->device);
    forget_widened(e, q); // codes written anew: a bf16 copy of what the buffer held before is stale
    k_quant_scales<<<grid_for(e, outer * inner, 256, 8), 256, 0, e->stream>>>(w, from, s, outer, k, inner);
    k_quant_codes<<<grid_for(e, outer * k * inner, 256, 8), 256, 0, e->stream>>>(w, from, s, q, outer, k, inner);
    CUDA_TRY(e, cudaGetLastError());
    e->kernels += 2;
    return PSK_OK;
}

int psk_exec_init_normal(psk_exec *e, void *dst, int to, int64_t n, uint64_t seed, double std)
{
    cudaSetDevice(e->device);
    k_init_normal<<<grid_for(e, n, 256, 8), 256, 0, e->stream>>>(dst, to, n, seed, (float)std);
    CUDA_TRY(e, cudaGetLastError());
    e->kernels += 1;
    return PSK_OK;
}

// `presk solve --measure` on the device: the gap between a candidate realization's result and the reference
// realization's, without bringing either to the host.
int psk_exec_gap(psk_exec *e, const void *a, int32_t a_dtype, const void *b, int32_t b_dtype, int64_t n, double *gap, double *max_abs)
{
    cudaSetDevice(e->device);
    auto real = [](int d) { return d == PSK_F64 || d == PSK_F32 || d == PSK_BF16 || d == PSK_F16 || d == PSK_E8M15 || d == PSK_E4M3; };
    if (!real(a_dtype) || !real(b_dtype) || n < 0) return fail(e, PSK_E7001, "psk_exec_gap: two buffers of reals of the same number of elements");
    unsigned long long *out = (unsigned long long *)psk_exec_alloc(e, 16);
    if (!out) return PSK_E10001;
    unsigned long long host[2] = {0, 0};
    cudaError_t err = cudaMemsetAsync(out, 0, 16, e->stream);
    if (err == cudaSuccess && n > 0) {
        k_gap<<<grid_for(e, n, 256, 8), 256, 0, e->stream>>>(a, a_dtype, b, b_dtype, n, out);
        e->kernels += 1;
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaMemcpyAsync(host, out, 16, cudaMemcpyDeviceToHost, e->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
    psk_exec_free(e, out);
    if (err != cudaSuccess) return fail(e, PSK_E10001, std::string("psk_exec_gap: ") + cudaGetErrorString(err));
    double g, m;
    memcpy(&g, &host[0], 8);
    memcpy(&m, &host[1], 8);
    if (gap) *gap = g;
    if (max_abs) *max_abs = m;
    return PSK_OK;
}

// ---- the executor as a table -------------------------------------------------
static const char *vt_name(void *s) { return psk_exec_name((psk_exec *)s); }
static void *vt_alloc(void *s, size_t b) { return psk_exec_alloc((psk_exec *)s, b); }
static void vt_free(void *s, void *p) { psk_exec_free((psk_exec *)s, p); }
static int vt_upload(void *s, void *d, const void *h, size_t b) { return psk_exec_upload((psk_exec *)s, d, h, b); }
static int vt_download(void *s, void *h, const void *d, size_t b) { return psk_exec_download((psk_exec *)s, h, d, b); }
static int vt_run(void *s, const psk_launch *l, void *const *t) { return psk_exec_run((psk_exec *)s, l, t); }
static int vt_sync(void *s) { return psk_exec_sync((psk_exec *)s); }
static int64_t vt_overflow(void *s) { return psk_exec_overflow((psk_exec *)s); }
static const char *vt_error(void *s) { return psk_last_error((psk_exec *)s); }
static int vt_quantize(void *s, const void *w, int from, int8_t *q, float *sc, int64_t outer, int64_t k, int64_t inner) { return psk_exec_quantize((psk_exec *)s, w, from, q, sc, outer, k, inner); }
static int vt_init_normal(void *s, void *dst, int to, int64_t n, uint64_t seed, double std) { return psk_exec_init_normal((psk_exec *)s, dst, to, n, seed, std); }

void psk_exec_as_vtable(psk_exec *e, psk_exec_vtable *out)
{
    out->self = e;
    out->name = vt_name;
    out->alloc = vt_alloc;
    out->free = vt_free;
    out->upload = vt_upload;
    out->download = vt_download;
    out->run = vt_run;
    out->sync = vt_sync;
    out->overflow = vt_overflow;
    out->last_error = vt_error;
    out->quantize = vt_quantize;
    out->init_normal = vt_init_normal;
}

} // extern "C"
