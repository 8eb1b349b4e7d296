// The device-side form of a launch, shared by the kernels of this library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/presk_cuda.h"
#include "psk_formats.cuh"
#include "psk_libm.cuh"

namespace psk {

// An operand with its offset folded into the pointer.
struct DevOperand {
    const void *p;
    const float *scales; // integer weights: one f32 per channel
    int32_t dtype;
    int32_t is_index;
    int32_t affine; // 0, or 1 (i8/sat) / 2 (u8/sat): codes q denoting (q - zero)·scale
    int32_t affine_zero;
    float affine_scale;
    int32_t pad;
    int64_t stride[PSK_MAX_AXES];
    int64_t sstride[PSK_MAX_AXES];
};

struct DevLaunch {
    int32_t n_in, n_outer, n_inner, kdtype;
    int32_t n_steps, kind, masked, guarded;
    int32_t int_accum, chunk; // chunk: 0, or the length of a chunk of a contraction's sum (PSK_ORDER_CHUNKED)
    int64_t dims[PSK_MAX_AXES];
    int64_t total; // product of the outer dims
    int64_t inner; // product of the inner dims
    DevOperand in[PSK_MAX_INPUTS];
    DevOperand out;
    psk_step steps[PSK_MAX_STEPS];
    int64_t iparam[4];
    float fparam;
    uint32_t *ovf;    // the overflow guard's flag word of this launch
    uint32_t *status; // bit 0: an argument of sin/cos beyond the supported range
};

// The multi-index of linear position `lin` over dims[first .. first+n), and
// with it an operand's element offset.
struct Offsets {
    int64_t v[PSK_MAX_INPUTS + 1];
};

PSK_DEV int64_t operand_offset(const DevOperand &o, const int64_t *dims, int first, int n, int64_t lin)
{
    int64_t off = 0;
    for (int a = first + n - 1; a >= first; --a) {
        int64_t d = dims[a];
        int64_t i = lin % d;
        lin /= d;
        off += i * o.stride[a];
    }
    return off;
}

// A load as the kernel of type kdtype sees it (psk_formats.cuh `edge_round`),
// an index as a real, an integer weight times its channel's scale in one f32
// multiplication (presk-rt/src/quant.rs:250-252).
PSK_DEV int affine_code_at(const DevOperand &o, int64_t off)
{
    return o.affine == 2 ? (int)((const uint8_t *)o.p)[off] : (int)((const int8_t *)o.p)[off];
}

PSK_DEV float load_operand(const DevOperand &o, int64_t off, int64_t soff, int kdtype, uint32_t *ovf)
{
    if (o.affine) // (q - z)·s is exact in a double; a nest that computes in f32 reads it rounded to f32
        return (float)((double)(affine_code_at(o, off) - o.affine_zero) * (double)o.affine_scale);
    if (o.dtype == PSK_I8)
        return (float)((const int8_t *)o.p)[off] * o.scales[soff];
    float x = load_real(o.p, o.dtype, off);
    return edge_round(x, kdtype, o.dtype, ovf);
}

PSK_DEV int64_t scale_offset(const DevOperand &o, const int64_t *dims, int first, int n, int64_t lin)
{
    if (o.dtype != PSK_I8) return 0;
    int64_t off = 0;
    for (int a = first + n - 1; a >= first; --a) {
        int64_t d = dims[a];
        int64_t i = lin % d;
        lin /= d;
        off += i * o.sstride[a];
    }
    return off;
}

} // namespace psk
