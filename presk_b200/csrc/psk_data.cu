// psk_data_*: samples of a .psk.d file read straight into device buffers.
//
// The format is presk-data's, as the reference's C runtime states and reads it (presk-export-c/c/presk_rt.c:8-33,
// presk_open :295-460, presk_read :462-520): "PSKD", a u16 version (1, 2 or 3), the sample type as text, a u64
// count, from version 2 a byte of encoding a leaf (0 f64, 1 f32, 2 bf16; in version 3 also 3 = a float format given
// by six more bytes, of which binary16 and e8m15 are held), then the samples back to back, each the type's leaves
// in order: an idx[N] element as the smallest of u8/u16/u32/u64 that holds N - 1, a real in its encoding, all
// little-endian. The header is parsed and checked on the host with the reference reader's checks and error codes
// (9002 not such a file or a format not held, 9003 truncated, 9005 another type or another length). The samples'
// bytes then go to the device as they are (through one pinned staging buffer) and a kernel a leaf takes them
// apart: leaf i of `count` samples becomes one dense [count, n_i] buffer, an index widened to i64 and tested
// against its bound (9004, naming the first offender in file order, as presk_read does), a real rounded once to
// the buffer's type as the reference's store_real rounds (presk_rt.c:107-129: f32 by the machine's conversion,
// bf16 by way of f32, binary16 and e8m15 directly from the double).
#include <cuda_runtime.h>
#include <algorithm>
#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/presk_cuda.h"
#include "psk_formats.cuh"

using namespace psk;

namespace {

enum { ENC_F64 = 0, ENC_F32 = 1, ENC_BF16 = 2, ENC_FORMAT = 3, ENC_F16 = 4, ENC_E8M15 = 5 };

// The six bytes that describe a float format in a version 3 header (p, emin i16, emax i16, flags).
const unsigned char kF16Desc[6] = {11, 0xf2, 0xff, 15, 0, 0x01};
const unsigned char kE8m15Desc[6] = {16, 0x82, 0xff, 127, 0, 0x01};

unsigned idx_width(uint64_t bound)
{
    const uint64_t m = bound - 1;
    return m <= 0xffu ? 1u : m <= 0xffffu ? 2u : m <= 0xffffffffu ? 4u : 8u;
}

unsigned enc_width(int enc)
{
    switch (enc) {
    case ENC_F32: return 4;
    case ENC_BF16: case ENC_F16: return 2;
    case ENC_E8M15: return 3;
    default: return 8;
    }
}

uint64_t get_le(const unsigned char *b, unsigned w)
{
    uint64_t x = 0;
    for (unsigned i = w; i-- > 0;) x = x << 8 | b[i];
    return x;
}

// ---- device side -----------------------------------------------------------

__device__ __forceinline__ uint64_t dev_get_le(const uint8_t *p, int w)
{
    uint64_t x = 0;
    for (int i = w - 1; i >= 0; --i) x = x << 8 | p[i];
    return x;
}

// The code, in the IEEE format of t trailing bits and w exponent bits (w <= 8), of the double with bits b rounded
// once, ties to even; a NaN quiet with the top t - 1 bits of its payload; a subnormal double is a zero.
__device__ uint32_t narrow_f64(uint64_t b, int t, int w)
{
    const uint64_t sign = (b >> 63) << (t + w), inf = ((1ull << w) - 1) << t, mag = b & ~(1ull << 63);
    if (mag > (0x7ffull << 52)) return (uint32_t)(sign | inf | 1ull << (t - 1) | ((mag >> (52 - t)) & ((1ull << (t - 1)) - 1)));
    const int field = (int)(mag >> 52);
    if (field == 0) return (uint32_t)sign;
    const uint64_t sig = (mag & ((1ull << 52) - 1)) | 1ull << 52; // |x| = sig · 2^(lead - 52)
    const int lead = field - 1023, bias = (1 << (w - 1)) - 1, emin = 1 - bias;
    const int drop = 52 - t + (emin > lead ? emin - lead : 0);    // bits of sig below the result's last place
    uint64_t kept = 0;
    if (drop <= 63) {
        const uint64_t below = sig & ((1ull << drop) - 1), half = 1ull << (drop - 1);
        kept = sig >> drop;
        kept += (below > half || (below == half && (kept & 1ull))) ? 1ull : 0ull;
    }
    // a normal result: the leading one of `kept` adds into the exponent field, and a carry moves it along
    const uint64_t code = lead >= emin ? ((uint64_t)(lead + bias - 1) << t) + kept : kept;
    return (uint32_t)(sign | (code < inf ? code : inf));
}

// A double to f32 as the machine's conversion does it: nearest, ties to even; a NaN quiet, its sign and the top of
// its payload kept.
__device__ __forceinline__ float f64_to_f32_keep_nan(uint64_t b)
{
    if ((b & ~(1ull << 63)) > (0x7ffull << 52)) return bits_f32((uint32_t)(b >> 63) << 31 | 0x7fc00000u | (uint32_t)((b >> 29) & 0x3fffffu));
    return __double2float_rn(__longlong_as_double((long long)b));
}

struct LeafJob {
    const uint8_t *raw;  // the samples of this piece, as in the file
    uint64_t per;        // bytes a sample
    uint64_t off;        // where this leaf starts in a sample
    uint64_t n;          // elements of the leaf
    uint64_t samples;    // samples in this piece
    uint64_t bound;      // of an index leaf, else 0
    uint64_t ordinal;    // the leaf's first element, counted over a sample's elements (for the error's position)
    uint64_t per_elems;  // elements a sample, all leaves
    uint64_t first;      // the piece's first sample within the read
    void *dst;           // [samples of the whole read, n]
    int32_t width, enc, dtype;
    unsigned long long *bad; // the least position (sample · per_elems + element) of an index not below its bound
};

__global__ void __launch_bounds__(256) k_data_leaf(const LeafJob J)
{
    const uint64_t total = J.samples * J.n, step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += step) {
        const uint64_t s = e / J.n, k = e - s * J.n;
        const uint64_t x = dev_get_le(J.raw + s * J.per + J.off + k * (uint64_t)J.width, J.width);
        const int64_t o = (int64_t)((J.first + s) * J.n + k);
        if (J.bound) {
            if (x >= J.bound) atomicMin(J.bad, (unsigned long long)((J.first + s) * J.per_elems + J.ordinal + k));
            else ((int64_t *)J.dst)[o] = (int64_t)x;
            continue;
        }
        if (J.enc == ENC_F64) {
            switch (J.dtype) {
            case PSK_F32: ((float *)J.dst)[o] = f64_to_f32_keep_nan(x); break;
            case PSK_BF16: ((uint16_t *)J.dst)[o] = f32_to_bf16(f64_to_f32_keep_nan(x)); break;
            case PSK_F16: ((uint16_t *)J.dst)[o] = (uint16_t)narrow_f64(x, 10, 5); break;
            default: store_e8m15((uint8_t *)J.dst, o, narrow_f64(x, 15, 8)); break;
            }
            continue;
        }
        // the narrower encodings are exact in f32; a NaN of a format's code is the NaN of its sign, whatever its
        // payload, and an f32's or a bf16's NaN is made quiet (it passes through a double in the reference)
        float g;
        if (J.enc == ENC_F32) g = bits_f32((uint32_t)x);
        else if (J.enc == ENC_BF16) g = bits_f32((uint32_t)x << 16);
        else if (J.enc == ENC_F16) g = f16_to_f32((uint16_t)x);
        else g = e8m15_to_f32((uint32_t)x);
        if (g != g) {
            const uint32_t gb = f32_bits(g);
            g = (J.enc == ENC_F16 || J.enc == ENC_E8M15) ? bits_f32((gb & 0x80000000u) | 0x7fc00000u) : bits_f32(gb | 0x00400000u);
        }
        store_real(J.dst, J.dtype, o, g);
    }
}

} // namespace

struct psk_data {
    FILE *f = nullptr;
    std::vector<psk_data_leaf> leaves;
    std::vector<int> enc;       // a leaf's encoding (ENC_F64 for every index leaf and in version 1)
    std::vector<unsigned> width;
    std::vector<uint64_t> off, ordinal;
    uint64_t count = 0, per = 0, per_elems = 0, head = 0;
    void *staging = nullptr;    // pinned
    size_t staging_bytes = 0;
    std::string error;
};

static int data_fail(std::string *into, char *err, size_t cap, int code, const char *fmt, ...)
{
    char buf[1024];
    int n = snprintf(buf, sizeof buf, "[E%d] ", code);
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf + n, sizeof buf - (size_t)n, fmt, ap);
    va_end(ap);
    if (into) *into = buf;
    if (err && cap) snprintf(err, cap, "%s", buf);
    return code;
}

static std::string format_name(const unsigned char *d)
{
    static const struct { const char *name; unsigned char d[6]; } known[] = {
        {"f16", {11, 0xf2, 0xff, 15, 0, 0x01}}, {"e8m15", {16, 0x82, 0xff, 127, 0, 0x01}}, {"e5m2", {3, 0xf2, 0xff, 15, 0, 0x01}},
        {"e4m3fn", {4, 0xfa, 0xff, 8, 0, 0x0b}}, {"e2m1", {2, 0, 0, 2, 0, 0x15}}};
    for (const auto &k : known)
        if (memcmp(d, k.d, 6) == 0) return k.name;
    char buf[96];
    snprintf(buf, sizeof buf, "float(p=%u,emin=%d,emax=%d,flags=0x%02x)", d[0], (int)(int16_t)(uint16_t)(d[1] | d[2] << 8), (int)(int16_t)(uint16_t)(d[3] | d[4] << 8), d[5]);
    return buf;
}

extern "C" int psk_data_open(const char *path, const char *type, const psk_data_leaf *leaves, size_t nleaves, psk_data **out, char *err, size_t err_cap)
{
    if (out) *out = nullptr;
    if (!path || !type || (!leaves && nleaves) || !out) return data_fail(nullptr, err, err_cap, PSK_E7001, "psk_data_open: a null argument");
    FILE *f = fopen(path, "rb");
    if (!f) return data_fail(nullptr, err, err_cap, PSK_E9002, "%s: %s", path, strerror(errno));
    psk_data *d = new psk_data;
    d->f = f;
    auto bail = [&](int code) { fclose(f); delete d; return code; };
    unsigned char b[8];
    if (fread(b, 1, 4, f) != 4) return bail(data_fail(nullptr, err, err_cap, PSK_E9002, "%s: not a .psk.d file (too short)", path));
    if (memcmp(b, "PSKD", 4) != 0) return bail(data_fail(nullptr, err, err_cap, PSK_E9002, "%s: not a .psk.d file (bad magic)", path));
    if (fread(b, 1, 2, f) != 2) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated header", path));
    const unsigned version = (unsigned)get_le(b, 2);
    if (version < 1 || version > 3) return bail(data_fail(nullptr, err, err_cap, PSK_E9002, "%s: .psk.d version %u, this reader reads versions 1, 2 and 3", path, version));
    if (fread(b, 1, 4, f) != 4) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated header", path));
    const uint64_t tlen_file = get_le(b, 4);
    const size_t tlen = strlen(type);
    std::string found((size_t)std::min<uint64_t>(tlen_file, 1u << 20), '\0');
    if (tlen_file > (1u << 20) || fread(&found[0], 1, found.size(), f) != found.size()) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated header", path));
    if (found.size() != tlen || memcmp(found.data(), type, tlen) != 0) return bail(data_fail(nullptr, err, err_cap, PSK_E9005, "%s holds samples of `%s`, the program reads `%s`", path, found.c_str(), type));
    if (fread(b, 1, 8, f) != 8) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated header", path));
    d->count = get_le(b, 8);
    d->head = 4 + 2 + 4 + tlen + 8;
    d->leaves.assign(leaves, leaves + nleaves);
    d->enc.assign(nleaves, ENC_F64);
    if (version >= 2) {
        if (fread(b, 1, 4, f) != 4) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated header", path));
        const uint64_t n = get_le(b, 4);
        if (n != nleaves) return bail(data_fail(nullptr, err, err_cap, PSK_E9005, "%s: %llu encodings for the %zu leaves of `%s`", path, (unsigned long long)n, nleaves, type));
        for (size_t i = 0; i < nleaves; ++i) {
            unsigned char c, desc[6];
            if (fread(&c, 1, 1, f) != 1) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated header", path));
            int e = c;
            if (c == ENC_FORMAT && version == 3) {
                if (fread(desc, 1, 6, f) != 6) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated header", path));
                d->head += 6;
                if (memcmp(desc, kF16Desc, 6) == 0) e = ENC_F16;
                else if (memcmp(desc, kE8m15Desc, 6) == 0) e = ENC_E8M15;
                else return bail(data_fail(nullptr, err, err_cap, PSK_E9002, "%s: leaf %zu is in %s, a format this program does not hold (it holds f64, f32, bf16, f16 and e8m15)", path, i, format_name(desc).c_str()));
            } else if (c > ENC_BF16) {
                return bail(data_fail(nullptr, err, err_cap, PSK_E9002, "%s: leaf %zu: unknown encoding %u", path, i, (unsigned)c));
            }
            if (leaves[i].bound && e != ENC_F64) return bail(data_fail(nullptr, err, err_cap, PSK_E9005, "%s: leaf %zu holds indices and has a real encoding %u", path, i, (unsigned)c));
            d->enc[i] = e;
        }
        d->head += 4 + nleaves;
    }
    d->width.resize(nleaves);
    d->off.resize(nleaves);
    d->ordinal.resize(nleaves);
    bool overflowed = false;
    for (size_t i = 0; i < nleaves; ++i) {
        const unsigned w = leaves[i].bound ? idx_width(leaves[i].bound) : enc_width(d->enc[i]);
        d->width[i] = w;
        d->off[i] = d->per;
        d->ordinal[i] = d->per_elems;
        if (leaves[i].n > (UINT64_MAX - 1 - d->per) / w) { overflowed = true; break; }
        d->per += leaves[i].n * w;
        d->per_elems += leaves[i].n;
    }
    if (overflowed || (d->per > 0 && d->count > (UINT64_MAX - d->head) / d->per))
        return bail(data_fail(nullptr, err, err_cap, PSK_E9005, "%s: %llu samples of this type overflow a file", path, (unsigned long long)d->count));
    const uint64_t need = d->head + d->count * d->per;
    long end;
    if (fseek(f, 0, SEEK_END) != 0 || (end = ftell(f)) < 0) return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: %s", path, strerror(errno)));
    if ((uint64_t)end < need)
        return bail(data_fail(nullptr, err, err_cap, PSK_E9003, "%s: truncated: %llu samples of %llu bytes announced, %llu bytes of data present", path, (unsigned long long)d->count, (unsigned long long)d->per, (unsigned long long)((uint64_t)end - d->head)));
    if ((uint64_t)end > need)
        return bail(data_fail(nullptr, err, err_cap, PSK_E9005, "%s: %llu bytes of data where %llu samples of %llu bytes were expected: the file holds a sample of other dimensions", path, (unsigned long long)((uint64_t)end - d->head), (unsigned long long)d->count, (unsigned long long)d->per));
    *out = d;
    return PSK_OK;
}

extern "C" uint64_t psk_data_count(const psk_data *d) { return d ? d->count : 0; }
extern "C" uint64_t psk_data_sample_bytes(const psk_data *d) { return d ? d->per : 0; }
extern "C" const char *psk_data_error(const psk_data *d) { return d ? d->error.c_str() : ""; }

extern "C" void psk_data_close(psk_data *d)
{
    if (!d) return;
    if (d->f) fclose(d->f);
    if (d->staging) cudaFreeHost(d->staging);
    delete d;
}

extern "C" int psk_data_read(psk_data *d, psk_exec *e, uint64_t first, uint64_t count, void *const *dst, const int32_t *dtypes)
{
    if (!d || !e || (!dst && !d->leaves.empty()) || (!dtypes && !d->leaves.empty())) return PSK_E7001;
    d->error.clear();
    if (first > d->count || count > d->count - first)
        return data_fail(&d->error, nullptr, 0, PSK_E9003, "sample %llu requested, %llu in the file", (unsigned long long)(first + count - (count ? 1 : 0)), (unsigned long long)d->count);
    const size_t nl = d->leaves.size();
    for (size_t i = 0; i < nl; ++i) {
        const bool idx = d->leaves[i].bound != 0;
        if (idx != (dtypes[i] == PSK_I64))
            return data_fail(&d->error, nullptr, 0, PSK_E9005, "leaf %zu: %s, but the program holds it as %s", i, idx ? "indices" : "reals", dtypes[i] == PSK_I64 ? "indices" : "reals");
        if (!idx && dtypes[i] != PSK_F32 && dtypes[i] != PSK_BF16 && dtypes[i] != PSK_F16 && dtypes[i] != PSK_E8M15)
            return data_fail(&d->error, nullptr, 0, PSK_E7005, "leaf %zu: this executor holds reals as f32, bf16, f16 or e8m15", i);
    }
    if (count == 0 || d->per == 0) return PSK_OK;
    cudaStream_t stream = (cudaStream_t)psk_exec_stream(e);
    // pieces of whole samples, 32 MB or one sample at the least
    const uint64_t piece_samples = std::max<uint64_t>(1, (32ull << 20) / d->per);
    const size_t piece_bytes = (size_t)(std::min<uint64_t>(piece_samples, count) * d->per);
    if (d->staging_bytes < piece_bytes) {
        if (d->staging) cudaFreeHost(d->staging);
        d->staging = nullptr;
        d->staging_bytes = 0;
        if (cudaHostAlloc(&d->staging, piece_bytes, cudaHostAllocDefault) != cudaSuccess) {
            cudaGetLastError();
            return data_fail(&d->error, nullptr, 0, PSK_E10001, "no pinned memory for %zu bytes of samples", piece_bytes);
        }
        d->staging_bytes = piece_bytes;
    }
    uint8_t *raw = (uint8_t *)psk_exec_alloc(e, piece_bytes);
    unsigned long long *bad = (unsigned long long *)psk_exec_alloc(e, sizeof(unsigned long long));
    if (!raw || !bad) {
        if (raw) psk_exec_free(e, raw);
        if (bad) psk_exec_free(e, bad);
        return data_fail(&d->error, nullptr, 0, PSK_E10001, "no device memory for %zu bytes of samples", piece_bytes);
    }
    int rc = PSK_OK;
    cudaError_t ce = cudaMemsetAsync(bad, 0xff, sizeof(unsigned long long), stream);
    for (uint64_t done = 0; done < count && rc == PSK_OK && ce == cudaSuccess; done += piece_samples) {
        const uint64_t ns = std::min<uint64_t>(piece_samples, count - done);
        // the staging buffer is free again once the copy before has been made
        ce = cudaStreamSynchronize(stream);
        if (ce != cudaSuccess) break;
        if (fseek(d->f, (long)(d->head + (first + done) * d->per), SEEK_SET) != 0 || fread(d->staging, 1, (size_t)(ns * d->per), d->f) != (size_t)(ns * d->per)) {
            rc = data_fail(&d->error, nullptr, 0, PSK_E9003, "truncated at sample %llu", (unsigned long long)(first + done));
            break;
        }
        ce = cudaMemcpyAsync(raw, d->staging, (size_t)(ns * d->per), cudaMemcpyHostToDevice, stream);
        for (size_t i = 0; i < nl && ce == cudaSuccess; ++i) {
            if (d->leaves[i].n == 0) continue;
            LeafJob J;
            J.raw = raw; J.per = d->per; J.off = d->off[i]; J.n = d->leaves[i].n; J.samples = ns; J.bound = d->leaves[i].bound;
            J.ordinal = d->ordinal[i]; J.per_elems = d->per_elems; J.first = done; J.dst = dst[i];
            J.width = (int32_t)d->width[i]; J.enc = d->enc[i]; J.dtype = dtypes[i]; J.bad = bad;
            const uint64_t total = ns * J.n;
            const unsigned grid = (unsigned)std::min<uint64_t>((total + 255) / 256, 148u * 8u);
            k_data_leaf<<<grid, 256, 0, stream>>>(J);
            ce = cudaGetLastError();
        }
    }
    unsigned long long worst = ~0ull;
    if (ce == cudaSuccess && rc == PSK_OK) ce = cudaMemcpyAsync(&worst, bad, sizeof worst, cudaMemcpyDeviceToHost, stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream);
    psk_exec_free(e, raw);
    psk_exec_free(e, bad);
    if (ce != cudaSuccess) {
        cudaGetLastError();
        return data_fail(&d->error, nullptr, 0, PSK_E10001, "reading samples: %s", cudaGetErrorString(ce));
    }
    if (rc == PSK_OK && worst != ~0ull) {
        // which element that was, and its value, from the file
        const uint64_t s = worst / d->per_elems, pos = worst % d->per_elems;
        size_t i = 0;
        while (i + 1 < nl && d->ordinal[i + 1] <= pos) ++i;
        const uint64_t k = pos - d->ordinal[i];
        unsigned char b[8] = {0};
        uint64_t x = 0;
        if (fseek(d->f, (long)(d->head + (first + s) * d->per + d->off[i] + k * d->width[i]), SEEK_SET) == 0 && fread(b, 1, d->width[i], d->f) == d->width[i]) x = get_le(b, d->width[i]);
        rc = data_fail(&d->error, nullptr, 0, PSK_E9004, "sample %llu, leaf %zu, element %llu: index %llu is not below the bound %llu", (unsigned long long)(first + s), i, (unsigned long long)k, (unsigned long long)x, (unsigned long long)d->leaves[i].bound);
    }
    return rc;
}
