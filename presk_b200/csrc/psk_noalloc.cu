// psk_gemm_noalloc: the tensor-core contraction for a caller that may not
// allocate device memory.
//
// Who that is: a host that hands this library a fixed arena and forbids any
// other allocation while an entry runs (the reference's own exported C host
// works that way: one block sized ahead of time, "nothing is allocated from
// the system during a call"); a server whose memory budget is fixed at start;
// a thread that holds a lock under which the driver's allocator must not be
// entered. psk_exec_create allocates (its guard flags, its status word, its
// buffer pool), so such a caller cannot use an executor at all. This entry
// point needs none: the two kinds of scratch the kernel writes besides its
// output - the status word of its bounded waits and the overflow guard's
// flags - live in a file-scope array on the device.
//
// What that costs: the array exists once per device and every call uses it.
// Calls are serialised by the entry point itself (it waits for the stream
// before it returns, because it reads the flags back), but two host threads
// calling at once on one device, or a call overlapping on the GPU with another
// through some other route, race on the flags. The array keeps the last
// call's contents, so each call clears the words it will read before it
// launches.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>

#include "../../include/presk_cuda.h"
#include "psk_gemm_tc.cuh"

using namespace psk;

// Word 0: the kernel's status. Words 1 .. batch: one guard flag a batch entry.
static __device__ __align__(256) uint32_t g_noalloc_scratch[1 + PSK_NOALLOC_MAX_BATCH];

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kMaxDevices = 64;

// What the first call on a device finds out, kept for the later ones.
struct DeviceSetup {
    bool done = false;
    uint32_t *scratch = nullptr; // the DEVICE address of g_noalloc_scratch on this device
    int sms = 0;
    EncodeTiledFn encode = nullptr;
};
DeviceSetup g_setup[kMaxDevices];

int say(char *err, size_t cap, int code, const char *fmt, const char *detail = "")
{
    if (err && cap) snprintf(err, cap, fmt, detail);
    return code;
}

bool make_map(EncodeTiledFn encode, CUtensorMap *map, const void *base, bool f16, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t box0, uint32_t box1)
{
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {s1 * 2, s2 * 2, s3 * 2};
    for (int i = 0; i < 3; ++i) {
        if (dims[i + 1] == 1 && strides[i] == 0) strides[i] = (i == 0 ? d0 * 2 : strides[i - 1] * dims[i]);
        if (strides[i] % 16 != 0 || strides[i] == 0) return false;
    }
    cuuint32_t box[4] = {box0, box1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

extern "C" int psk_gemm_noalloc(const psk_gemm *g, const void *a, const void *b, void *c, void *stream_, int64_t *overflowed_batch, char *err, size_t err_cap)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (overflowed_batch) *overflowed_batch = -1;
    if (!g || !a || !b || !c) return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: a null argument");
    if (g->in_dtype != PSK_BF16 && g->in_dtype != PSK_F16) return say(err, err_cap, PSK_E7005, "psk_gemm_noalloc: operands are bf16 or f16");
    if (g->batch < 1 || g->batch > PSK_NOALLOC_MAX_BATCH) {
        char msg[160];
        snprintf(msg, sizeof msg, "psk_gemm_noalloc: batch %lld is beyond the %d guard flags the static scratch holds", (long long)g->batch, PSK_NOALLOC_MAX_BATCH);
        return say(err, err_cap, PSK_E7001, "%s", msg);
    }
    if (g->m < 1 || g->n < 1 || g->k < 1 || g->batch_lo < 1 || g->batch % g->batch_lo != 0) return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: sizes must be positive and batch a multiple of batch_lo");
    if (((uintptr_t)a & 15u) || ((uintptr_t)b & 15u)) return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: operands must be 16-byte aligned");
    // the result's side of the descriptor: the kernel divides by the two counts and adds the strides to `c`
    if (g->out_dtype != PSK_F32 && g->out_dtype != PSK_BF16 && g->out_dtype != PSK_F16 && g->out_dtype != PSK_E8M15)
        return say(err, err_cap, PSK_E7005, "psk_gemm_noalloc: the result is stored as f32, bf16, f16 or e8m15");
    if (g->c_row_lo_count < 1 || g->c_col_lo_count < 1) return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: c_row_lo_count and c_col_lo_count are at least 1");
    if (g->a_row < 0 || g->a_lo < 0 || g->a_hi < 0 || g->b_row < 0 || g->b_lo < 0 || g->b_hi < 0 || g->c_row_lo < 0 || g->c_row_hi < 0 || g->c_col_hi < 0 || g->c_lo < 0 || g->c_hi < 0)
        return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: a negative stride");

    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: no current CUDA device");
    DeviceSetup &S = g_setup[device];
    if (!S.done) {
        // Once per device, with that device current. In host code the array's name is only a
        // stand-in; the address a kernel can use is what the runtime reports for it here.
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess || prop.major != 10) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: the kernels are built for sm_100a only");
        void *p = nullptr;
        cudaError_t rc = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (rc != cudaSuccess || !p) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(rc));
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: the driver has no cuTensorMapEncodeTiled");
        rc = cudaFuncSetAttribute(tc::k_gemm_tc<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<256>::TOTAL);
        if (rc == cudaSuccess) rc = cudaFuncSetAttribute(tc::k_gemm_tc<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::Smem<128>::TOTAL);
        if (rc != cudaSuccess) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: cudaFuncSetAttribute: %s", cudaGetErrorString(rc));
        S.scratch = (uint32_t *)p;
        S.sms = prop.multiProcessorCount;
        S.encode = (EncodeTiledFn)fn;
        S.done = true;
    }

    if (g->b_n_major & ~1) return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: the first operand is read k-contiguous here");
    const bool f16 = g->in_dtype == PSK_F16;
    const int bn = g->n >= 256 || g->n % 128 != 0 ? 256 : 128;
    const int64_t batch_hi = g->batch / g->batch_lo;
    CUtensorMap ma, mb;
    if (!make_map(S.encode, &ma, a, f16, (uint64_t)g->k, (uint64_t)g->m, (uint64_t)g->batch_lo, (uint64_t)batch_hi, (uint64_t)g->a_row, (uint64_t)g->a_lo, (uint64_t)g->a_hi, tc::BK, tc::BM))
        return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: operand 0's strides do not make a tensor map");
    const bool okb = g->b_n_major
        ? make_map(S.encode, &mb, b, f16, (uint64_t)g->n, (uint64_t)g->k, (uint64_t)g->batch_lo, (uint64_t)batch_hi, (uint64_t)g->b_row, (uint64_t)g->b_lo, (uint64_t)g->b_hi, 64, tc::BK)
        : make_map(S.encode, &mb, b, f16, (uint64_t)g->k, (uint64_t)g->n, (uint64_t)g->batch_lo, (uint64_t)batch_hi, (uint64_t)g->b_row, (uint64_t)g->b_lo, (uint64_t)g->b_hi, tc::BK, (uint32_t)bn);
    if (!okb) return say(err, err_cap, PSK_E7001, "psk_gemm_noalloc: operand 1's strides do not make a tensor map");

    tc::Params P;
    memset(&P, 0, sizeof P);
    P.m = g->m; P.n = g->n; P.k = g->k; P.batch = g->batch; P.batch_lo = g->batch_lo;
    P.tiles_m = (g->m + tc::BM - 1) / tc::BM;
    P.tiles_n = (g->n + bn - 1) / bn;
    P.panel = P.tiles_n < 8 ? P.tiles_n : 8;
    P.c_row_lo_count = g->c_row_lo_count; P.c_row_lo = g->c_row_lo; P.c_row_hi = g->c_row_hi;
    P.c_col_lo_count = g->c_col_lo_count; P.c_col_hi = g->c_col_hi;
    P.c_lo = g->c_lo; P.c_hi = g->c_hi;
    P.c = c; P.out_dtype = g->out_dtype; P.in_f16 = f16; P.b_n_major = g->b_n_major; P.guarded = g->guarded;
    const int64_t va = g->out_dtype == PSK_F32 ? 4 : 8;
    P.vec_ok = (((uintptr_t)c & 15u) == 0) && g->c_row_lo % va == 0 && g->c_row_hi % va == 0 && g->c_col_hi % va == 0 && g->c_lo % va == 0 && g->c_hi % va == 0
        && g->c_col_lo_count % (g->out_dtype == PSK_F32 ? 32 : 64) == 0 && g->n % va == 0 && g->out_dtype != PSK_E8M15;
    P.scale = g->scale; P.scale_on = g->scale_on;
    P.status = S.scratch;
    P.ovf = S.scratch + 1;

    // the words this call will read must start at zero: the array holds the last call's
    const size_t words = 1 + (size_t)g->batch;
    cudaError_t rc = cudaMemsetAsync(S.scratch, 0, words * sizeof(uint32_t), stream);
    if (rc != cudaSuccess) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(rc));
    const int64_t tiles = P.tiles_m * P.tiles_n * g->batch;
    const int grid = (int)(tiles < S.sms ? tiles : S.sms);
    if (bn == 256) tc::k_gemm_tc<256, true><<<grid, tc::THREADS, tc::Smem<256>::TOTAL, stream>>>(ma, mb, P);
    else tc::k_gemm_tc<128, true><<<grid, tc::THREADS, tc::Smem<128>::TOTAL, stream>>>(ma, mb, P);
    rc = cudaGetLastError();
    if (rc != cudaSuccess) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: launch: %s", cudaGetErrorString(rc));

    uint32_t host_words[1 + PSK_NOALLOC_MAX_BATCH];
    rc = cudaMemcpyAsync(host_words, S.scratch, words * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
    if (rc == cudaSuccess) rc = cudaStreamSynchronize(stream);
    if (rc != cudaSuccess) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: %s", cudaGetErrorString(rc));
    if (host_words[0]) return say(err, err_cap, PSK_E10001, "psk_gemm_noalloc: a bounded wait ran out in the kernel; the result is not valid");
    if (g->guarded)
        for (int64_t i = 0; i < g->batch; ++i)
            if (host_words[1 + i]) {
                if (overflowed_batch) *overflowed_batch = i;
                char msg[160];
                snprintf(msg, sizeof msg, "psk_gemm_noalloc: batch entry %lld: a store rounded a finite value to an infinity", (long long)i);
                return say(err, err_cap, PSK_E7007, "%s", msg);
            }
    return PSK_OK;
}
