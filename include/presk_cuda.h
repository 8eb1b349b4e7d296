/* presk_cuda.h: the C ABI of the B200 executor for Presk's realized kernels.
 *
 * What this boundary replaces in the reference (paths within presk-lang/presk):
 *
 *   - the inner seam, `trait KernelExec` (crates/presk-kernel/src/host.rs:28-95):
 *     `run(idx, &Kernel, inputs: &[&Buf], out: &mut Buf) -> Result<()>`, called
 *     by one host thread, one launch per fusion group or tensor primitive;
 *   - the raw kernel signature of the native executor,
 *     `KernelFn = extern "C" fn(*const *mut u8, i64, i64)`
 *     (crates/presk-cranelift/src/lib.rs:42) with its pointer-table order
 *     (inputs, output, one scales pointer per quantised input, overflow flag:
 *     lib.rs:1609-1629), which `psk_exec_run` keeps;
 *   - the outer seam, `trait Backend { prepare; call }`
 *     (crates/presk-rt/src/lib.rs:1274-1303), which `psk_host_*` stands in for.
 *
 * A launch is described by `psk_launch`, the resolved form of the reference's
 * `Kernel` (crates/presk-kernel/src/ir.rs:300-322): the lowering table of
 * crates/presk-kernel/src/lower.rs decides, per primitive, an iteration space
 * (the output's axes, then the summed axes) and how each operand is indexed
 * in it; here that indexing is carried as element strides, so that axis names
 * are a matter of the host alone and an executor is name-free.
 *
 * Everything is plain C: pointers, sizes, fixed-size structs. No type of
 * PyTorch or of the CUDA runtime appears in a signature.
 */
#ifndef PRESK_CUDA_H
#define PRESK_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PSK_MAX_RANK 8    /* axes of the output of a launch */
#define PSK_MAX_INNER 4   /* summed axes of a launch */
#define PSK_MAX_AXES (PSK_MAX_RANK + PSK_MAX_INNER)
#define PSK_MAX_INPUTS 8
#define PSK_MAX_STEPS 64  /* the reference's MAX_TREE, presk-core/src/fusion.rs:79 */

/* Machine types of a buffer. 0..5 are the reference's `presk_dtype`
 * (crates/presk-export-c/c/presk_rt.h, "The machine type of a buffer"), in
 * its order; the rest are storage formats of the realization's `quant` and
 * `params` maps (presk-rt/src/quant.rs, presk-format/src/lib.rs:136). */
typedef enum {
    PSK_F64 = 0,
    PSK_F32 = 1,
    PSK_BF16 = 2,
    PSK_I64 = 3,
    PSK_F16 = 4,
    PSK_E8M15 = 5, /* three bytes an element, little-endian */
    PSK_I8 = 6,    /* integer weights (the scales travel beside them), or the codes of an affine i8 format */
    PSK_E4M3 = 7,  /* e4m3fn codes, one byte */
    PSK_U8 = 8     /* the codes of an affine u8 format */
} psk_dtype;

/* Status of a call: the reference's RtError codes (presk-rt/src/lib.rs:971-981). */
typedef enum {
    PSK_OK = 0,
    PSK_E7001 = 7001,  /* runtime error (bad descriptor, shapes) */
    PSK_E7005 = 7005,  /* a realization this executor does not run */
    PSK_E7006 = 7006,  /* a scaled site whose scale is not computed yet */
    PSK_E7007 = 7007,  /* the overflow guard: a store rounded a finite value to an infinity */
    PSK_E9002 = 9002,  /* psk_data: not a .psk.d file of version 1, 2 or 3, or a leaf in a format not held */
    PSK_E9003 = 9003,  /* psk_data: truncated */
    PSK_E9004 = 9004,  /* psk_data: an index not below its bound */
    PSK_E9005 = 9005,  /* psk_data: another sample type, or a length that is not the layout's */
    PSK_E10001 = 10001 /* internal error of the backend (a CUDA call failed, a wait ran out) */
} psk_status;

/* What a launch computes. Each is a family of the reference's lowerings. */
typedef enum {
    PSK_OP_FUSED = 0,    /* lower.rs:309-372: a fusion group, a unary or a binary primitive */
    PSK_OP_CONTRACT = 1, /* lower.rs:384-636, 906-1139: dot, ein, dot_vjp_l/r */
    PSK_OP_REDUCE = 2,   /* lower.rs:1221-1255, 1693: sum, mean, sum_squares */
    PSK_OP_SOFTMAX = 3,  /* lower.rs:1274-1419: softmax over one axis, masked or not */
    PSK_OP_XENT = 4,     /* lower.rs:1459: cross_entropy */
    PSK_OP_ARGMAX = 5,   /* lower.rs:1490 */
    PSK_OP_EMBED = 6,    /* lower.rs:1421 */
    PSK_OP_COPY = 7,     /* lower.rs:1554-1667: slice, concat, split_heads, merge_heads, index, broadcast_like */
    PSK_OP_IOTA = 8,     /* lower.rs:1706-1750: positions, causal_mask, one_hot, fill */
    PSK_OP_CONVERT = 9,  /* host.rs:809-829: Buf::of(to, b.to_f64()) at a kernel's edge */
    PSK_OP_MAGNITUDE = 10, /* presk-precision/src/envelope.rs:29-127: a site's max |x|, least non-zero |x|, least
                             and greatest x. Output: four u32 words, merged into what they hold (so that one
                             slot collects several launches and several ranks): [0] bits of max |x|, start 0;
                             [1] bits of the least non-zero |x|, start 0x7f800000; [2], [3] least and greatest
                             x under the order-preserving map u = b ^ (b >> 31 ? 0xffffffff : 0x80000000) of
                             its bits b, start 0xff800000 and 0x007fffff. NaNs are passed over. No counterpart
                             among the reference's kernels: it measures envelopes on its exact interpreter. */
    PSK_OP_ATTENTION = 11, /* four launches of an attention function as one (examples/coverage/llama.psk:100-102):
                             scores = ein(q*k) over hd, scores / rt, softmax over seq2 where mask, ein(a*v) over
                             seq2. Space: outer axes (..., seq, hd), one inner axis seq2. Inputs: q (stride 0 on
                             seq2), k and v (stride 0 on seq; hd and seq2 both walked), rt (rank 0), and the mask
                             over (seq, seq2) when n_inputs is 5. iparam[1..3]: the storage types of the three
                             sites in between. iparam[0]: how an executor may fuse them: 0 blockwise (two passes
                             over the keys, each stored site's rounding kept in registers), 1 online (one pass
                             against a running reference maximum, the sites in between not rounded). The value is
                             DEFINED as that of the four launches run one after the other; an executor may only fuse
                             them under PSK_ORDER_DEVICE, and then agrees with them within a tolerance. The result
                             may be a `scaled` site (out.affine): the last launch's binary32 sum stored as its code. No counterpart among the reference's kernels: its
                             fusion (presk-core/src/fusion.rs) never crosses a contraction or a softmax. */
    PSK_OP_RMSNORM = 12,  /* the four launches of RMSNorm.apply as one (examples/coverage/llama.psk:34-40): x*x, its
                             mean over the last axis, sqrt(mean + eps), x / root * gamma. Space: the axes of x, no
                             inner axis. Inputs: x, eps (rank 0), gamma (over the last axis). iparam[0]: the length
                             of the last axis; iparam[1..3]: the storage types of the square's, the mean's and the
                             root's sites; dtype: the result's. The value is DEFINED as that of the four launches run
                             one after the other under the launch's order (the oracle runs exactly those); an
                             executor that takes it must give their bits. No counterpart among the reference's
                             kernels: its groups never cross a reduction. */
    PSK_OP_ROPE = 13,     /* the rotation of `rope` (examples/coverage/llama.psk:66-72) as one launch: with x read as
                             (.., seq, pair = 2, rot) and c, s over (seq, rot),
                               out[.., 0, r] = x[.., 0, r]*c - x[.., 1, r]*s,  out[.., 1, r] = x[.., 1, r]*c + x[.., 0, r]*s,
                             every product rounded to f32 before the sum, the sums rounded once to the result's
                             type: the reference's two slices, two groups of three steps and concatenation, for the
                             case that all of their sites are stored in x's type (the host offers nothing else).
                             Space: the axes of the result. Inputs: x, c, s. */
    PSK_OP_CONTRACT_ADD = 14, /* a contraction and the addition of a third operand to its result as one launch: the
                             reference's `ein`/`dot` followed by a residual `add` (examples/coverage/llama.psk:117-118).
                             Inputs 0 and 1 as in PSK_OP_CONTRACT, input 2 over the outer axes. iparam[1]: the storage
                             type of the contraction's own site; dtype: the sum's. The value is DEFINED as that of the
                             two launches (contraction stored in its type, then in[2] + it); an executor that takes
                             it must give their bits under the launch's order. With int_accum the contraction counts
                             in integers as PSK_OP_CONTRACT does (inputs 0 and 1 affine values or integer weights). */
    PSK_OP_XENT_VJP = 15, /* lower.rs:1472-1488: cross_entropy_vjp. Space as PSK_OP_XENT (outer axes, one inner axis:
                             the classes). Inputs: logits, labels, the cotangent over the outer axes. Output over the
                             whole space: (exp(x - m) / z - [k == y]) * ct, m and z as in PSK_OP_XENT (the maximum from
                             the row's first element, z summed in index order), each operation rounded. */
    PSK_OP_EMBED_VJP = 16 /* lower.rs:1444-1457: embed_vjp. Space as PSK_OP_EMBED: (the indices' axes..., d). Inputs: the
                             table (its shape only: never read), the indices, the cotangent over the space. Output: a
                             table of iparam[0] rows (strides in out.stride[0], out.stride[1]), zero-filled, then
                             row idx[iv] += ct[iv, :] for every iv in index order, each sum kept in the output's
                             storage type (rounded there after every addition). */
} psk_op;

/* Elementary operations of a fusion group's steps (lower.rs:184-226). */
typedef enum {
    PSK_ADD = 0, PSK_SUB, PSK_MUL, PSK_DIV, PSK_MAX, PSK_MIN,
    PSK_NEG, PSK_EXP, PSK_LOG, PSK_TANH, PSK_SQRT, PSK_SIN, PSK_COS, PSK_ABS,
    PSK_GELU, PSK_GELU_DERIV, PSK_RELU, PSK_HEAVISIDE, PSK_SIGN, PSK_SIGMOID,
    PSK_POW, /* by repeated multiplication, exponent in `imm` */
    PSK_REAL, /* identity on a real; an index read as a real */
    PSK_DIV_N, /* x / n with n = `imm` a constant of the kernel in its arithmetic type (lower.rs:1257-1270 `mean_vjp`:
                  the cotangent of a mean, broadcast, divided by the count) */
    PSK_ROUND /* the value as a store into the type `imm` (a psk_dtype without a guard: f32, bf16) and a load back
                 would leave it. No primitive of the reference: it stands where two of its groups, each with its
                 result stored in its site's type, run as one launch (realization `launches: merged`). */
} psk_prim;

/* One step of a group (presk-core/src/fusion.rs:19-59): an operation on one or
 * two sources, each an input of the launch (src >= 0) or an earlier step
 * (src = -1 - step). */
typedef struct {
    int32_t prim;  /* psk_prim */
    int32_t nargs; /* 1 or 2 */
    int32_t src[2];
    int32_t imm;   /* PSK_POW's exponent */
} psk_step;

/* How a sum is accumulated: the realization's `order`
 * (presk-rt/src/lib.rs:251-285). SEQUENTIAL is the reference's default and is
 * bit-defining; DEVICE is this executor's declared reassociation (tensor-core
 * tiles for contractions, shuffle trees for row reductions), as `chunked` and
 * `interleaved` are the reference's. */
typedef enum {
    PSK_ORDER_SEQUENTIAL = 0,
    PSK_ORDER_DEVICE = 1,
    PSK_ORDER_CHUNKED = 2 /* the reference's `chunked(size)` (presk-rt/src/lib.rs:264-269; the nest at
                             presk-kernel/src/lower.rs:424-457): a contraction over ONE summed axis adds its terms in
                             chunks of `order_size` consecutive ones, each chunk from zero in index order, the chunks'
                             sums then in order from zero, the last chunk shorter. Exact on this executor's scalar
                             kernels: the reference's bits. Every other operation keeps the sequential order, as in
                             the reference (lower.rs:262-266). */
} psk_order;

typedef enum {
    PSK_REDUCE_SUM = 0, PSK_REDUCE_MEAN = 1, PSK_REDUCE_SUMSQ = 2,
    PSK_REDUCE_SUM_STORED = 3 /* lower.rs:1670-1680 `sum_to`: the sum is kept in the output buffer, so every partial sum
                                 is rounded to the output's type (and tested by the guard) before the next term is
                                 added; terms in row-major order of the summed axes. Under PSK_ORDER_DEVICE an
                                 executor may sum it like PSK_REDUCE_SUM (f32 partial sums in its own order, one
                                 rounding): the declared difference of that order */
} psk_reduce_kind;

typedef enum {
    PSK_IOTA_POSITIONS = 0, PSK_IOTA_CAUSAL = 1, PSK_IOTA_ONE_HOT = 2, PSK_IOTA_FILL = 3
} psk_iota_kind;

/* An operand as the launch indexes it: the element of the iteration point
 * (o_0 .. o_{n_outer-1}, c_0 .. c_{n_inner-1}) is at
 * offset + sum_a index_a * stride[a], in elements. A broadcast axis has
 * stride 0. For integer weights (`quant`), `scale_stride` indexes the f32
 * scales the same way (quant.rs:227-278: the scale is constant along the
 * contracted axis). */
typedef struct {
    int32_t dtype;              /* psk_dtype of the stored elements */
    int32_t is_index;           /* 1: an idx tensor (i64), read as an integer */
    int64_t offset;
    int64_t stride[PSK_MAX_AXES];
    int64_t scale_stride[PSK_MAX_AXES];
    int64_t numel;              /* elements of the whole buffer, for checks */
    /* A value stored in an affine format (the realization's `scaled` map, presk-rt/src/lib.rs:287-360;
     * presk-format/src/lib.rs:865-954): codes q of dtype PSK_I8 (`i8/sat`, affine = 1) or PSK_U8
     * (`u8/sat`, affine = 2) denoting (q - zero)·scale, the scale a positive normal f32. 0: not affine. */
    int32_t affine;
    int32_t affine_zero;
    float affine_scale;
    int32_t reserved;
} psk_operand;

typedef struct {
    const char *name;   /* the reference's kernel name: "dot", "ein[batch, seq, model]", "fused 2 steps" */
    int32_t op;         /* psk_op */
    int32_t dtype;      /* the kernel's type: its output's storage type; it computes in f32
                           (presk-rt/src/lib.rs:147-152) */
    int32_t order;      /* psk_order */
    int32_t guarded;    /* 1: test f16/e8m15 stores for overflow (host.rs:144-177) */
    int32_t n_inputs;
    int32_t n_outer;    /* axes of the output */
    int32_t n_inner;    /* summed axes, after the outer ones in every stride array */
    int64_t dims[PSK_MAX_AXES];
    psk_operand in[PSK_MAX_INPUTS];
    psk_operand out;    /* stride over the outer axes; row-major unless the launch writes a part */
    int32_t n_steps;
    psk_step steps[PSK_MAX_STEPS];
    int32_t kind;       /* psk_reduce_kind or psk_iota_kind */
    int32_t masked;     /* softmax: input 1 is the mask */
    int32_t int_accum;  /* contraction: 1 = `product: i32, accum: i32` (presk-kernel/src/exec.rs:493-526): both
                           operands are read as integer counts in their scales' unit, the products and the
                           sum are exact integers wrapped to 32 bits, and the store rounds the exact value
                           sum·s0·s1 once into the output's format */
    int32_t order_size; /* PSK_ORDER_CHUNKED: the chunk's length (at least 1) */
    int64_t iparam[4];  /* reduce: the divisor of a mean; copy/iota: see psk_host.cpp */
    double fparam[2];   /* fill: the value */
} psk_launch;

/* Sizes of this header's structs as the library was compiled with them, for a
 * binding in another language to check its own layout against: 0 psk_launch,
 * 1 psk_operand, 2 psk_step, 3 psk_gemm, 4 psk_value, 5 psk_exec_vtable. */
size_t psk_abi_sizeof(int which);

/* ---------------------------------------------------------------------------
 * The executor (KernelExec). One per device and host thread.
 * ------------------------------------------------------------------------- */
typedef struct psk_exec psk_exec;

/* An executor on CUDA device `device`. NULL when the device cannot be used;
 * psk_last_error(NULL) then says why. Never falls back to the CPU. */
psk_exec *psk_exec_create(int device);
void psk_exec_destroy(psk_exec *e);

/* KernelExec::name, workers, emulates, codes (host.rs:28-95): "cuda"; no host
 * workers; runs the native float types and their codes, emulates nothing. */
const char *psk_exec_name(const psk_exec *e);

/* The message of the last call that did not return PSK_OK. */
const char *psk_last_error(const psk_exec *e);

/* Device buffers. Contents of a fresh buffer are arbitrary, as the
 * reference's pooled buffers are (presk-rt/src/elems.rs:57-72). */
void *psk_exec_alloc(psk_exec *e, size_t bytes);
void psk_exec_free(psk_exec *e, void *p);
int psk_exec_upload(psk_exec *e, void *dst, const void *src_host, size_t bytes);
int psk_exec_download(psk_exec *e, void *dst_host, const void *src, size_t bytes);
int psk_exec_sync(psk_exec *e);
/* Bytes in use and the most there have been (presk-kernel/src/memory.rs). */
void psk_exec_memory(const psk_exec *e, size_t *live, size_t *peak);

/* KernelExec::run. `table` is the native executor's pointer table
 * (presk-cranelift/src/lib.rs:1609-1629): the n_inputs inputs, the output,
 * then one `const float *` of scales for each input that holds integer weights
 * (dtype PSK_I8, not affine), in input order. All are device pointers of this executor. The launch is
 * queued on the executor's stream; PSK_E7007 of a guarded launch is
 * reported by the next psk_exec_sync, psk_exec_download or psk_exec_overflow,
 * naming the first launch whose store overflowed, and later launches still
 * run (presk_rt.h:296-310). */
int psk_exec_run(psk_exec *e, const psk_launch *l, void *const *table);

/* The overflow guard's flag since the last call, cleared by it: 0, or
 * 1 + the serial number of the first guarded launch that overflowed. */
int64_t psk_exec_overflow(psk_exec *e);
/* Every wait of a kernel of this library on a barrier is limited (about two seconds); when one runs out the kernel
 * records where, leaves its loops, frees what it holds and returns, and the next psk_exec_sync reports PSK_E10001.
 * This runs a kernel whose only wait cannot be satisfied, limited to `cycles` SM cycles (at most 4e8), and returns
 * what the host reports for it: PSK_E10001 with the message in psk_last_error. The executor stays usable. */
int psk_exec_wait_selftest(psk_exec *e, int64_t cycles);

/* Launches queued, and how many kernels of this library they started. */
void psk_exec_counts(const psk_exec *e, int64_t *launches, int64_t *kernels);

/* KernelExec::set_profiling / overhead (host.rs:45): device time of the last
 * psk_exec_run in milliseconds, timed with events on the stream, or < 0. */
void psk_exec_set_profiling(psk_exec *e, int on);
double psk_exec_last_ms(psk_exec *e);

/* While profiling is on every psk_exec_run is bracketed by two events on the
 * stream. This waits for the stream and returns one line a launch since the
 * last call: kernel family, the launch's name, milliseconds, its floating-point
 * operations (contractions) and its algorithmic bytes (each operand once at
 * its stored width, the reference's Q, presk-kernel/src/cost.rs:92-95),
 * tab-separated. The text belongs to the executor until the next call. */
const char *psk_exec_profile(psk_exec *e);

/* The raw CUDA stream the executor launches on (a cudaStream_t), for a
 * caller that times it with its own events. */
void *psk_exec_stream(psk_exec *e);

/* `presk solve --measure` without the host in the loop: the gap between two results that stay on the device
 * (presk-driver/src/gap.rs:35-64, `leaf_gap` and `leaf_max`): *gap = the largest |a[i] - b[i]|, *max_abs = the
 * largest |a[i]|, both in binary64 over the exactly widened elements, an element that is not finite counting as
 * +infinity (so that a realization that overflowed is never measured on the rest). `a` is the reference result
 * (budget_abs = budget x *max_abs, gap.rs:35), `b` the candidate's; any two real storage types. Sixteen bytes
 * come back to the host. */
int psk_exec_gap(psk_exec *e, const void *a, int32_t a_dtype, const void *b, int32_t b_dtype, int64_t n, double *gap, double *max_abs);

/* A tensor-core contraction on its own, outside a launch: C[b] = A[b]·B[b]
 * with bf16/f16 operands and f32 sums; what PSK_OP_CONTRACT dispatches to
 * under PSK_ORDER_DEVICE. See psk_gemm in csrc/gemm_tc.cuh. */
typedef struct {
    int32_t in_dtype;  /* PSK_BF16 or PSK_F16, both operands */
    int32_t out_dtype; /* PSK_F32, PSK_BF16, PSK_F16 or PSK_E8M15 */
    int32_t b_n_major; /* bit 0: 0 B[batch][n][k], k contiguous; 1 B[batch][k][n], n contiguous.
                          bit 1: 0 A[batch][m][k], k contiguous (a_row: a row's stride); 1 A[batch][k][m], m contiguous
                          (a_row: the stride between two k) */
    int32_t guarded;
    int64_t m, n, k;
    int64_t batch, batch_lo;                 /* batch index = hi * batch_lo + lo */
    int64_t a_row, a_lo, a_hi;               /* element strides of A: row, batch lo, batch hi */
    int64_t b_row, b_lo, b_hi;
    int64_t c_row_lo_count, c_row_lo, c_row_hi; /* row r at (r / count) * hi + (r % count) * lo */
    int64_t c_col_lo_count, c_col_hi;        /* col c at (c / count) * hi + (c % count) */
    int64_t c_lo, c_hi;                      /* batch strides of C */
    float scale;                             /* the output is acc * scale when scale_on (a fused `div`/`mul`) */
    int32_t scale_on;
} psk_gemm;
int psk_exec_gemm(psk_exec *e, const psk_gemm *g, const void *a, const void *b, void *c);

/* The tensor-core contraction for a caller that may not allocate device
 * memory at all: one that gave this library a fixed arena, runs under a fixed
 * memory budget, or calls from a place where the driver's allocator must not
 * be entered. An executor allocates when it is created (guard flags, status
 * word, buffer pool), so such a caller cannot have one; this entry point
 * needs none. It has no counterpart in the reference.
 *
 * Same arithmetic and the same kernel as psk_exec_gemm, so the same bytes in
 * `c`. The scratch the kernel writes besides `c` (its status word and the
 * overflow guard's flags, here one flag a batch entry) lives in one static
 * array of 1 + PSK_NOALLOC_MAX_BATCH words on each device that loads the
 * library, held until the process exits; a `batch` above that maximum is
 * refused with PSK_E7001. `a`, `b`, `c` are device pointers the caller owns;
 * `stream` is a cudaStream_t (NULL: the default stream). The call clears the
 * words it uses, launches, copies them back and waits for the stream, so it
 * is synchronous; it calls no cudaMalloc, cudaFree or allocating library
 * routine. Returns PSK_OK, or PSK_E7007 with `*overflowed_batch` the first
 * batch entry a guarded store overflowed in (else -1), or another status
 * with a message in `err` (may be NULL).
 *
 * The array is shared by every call on a device and keeps the last call's
 * contents: two calls that overlap on one GPU (two host threads, or a second
 * route to the same kernel) race on it. The first call on a device looks the
 * array's device address up and sets the kernel's attributes; make that first
 * call before any stream capture begins. Every call, the first included, waits
 * for `stream` and copies the flags back to the host before it returns, so the
 * entry point is not callable while the stream is capturing.
 *
 * The descriptor is checked before anything is launched: out_dtype one of
 * PSK_F32, PSK_BF16, PSK_F16, PSK_E8M15; c_row_lo_count and c_col_lo_count at
 * least 1 (the kernel divides by them); no negative stride. Anything else is
 * PSK_E7001 (PSK_E7005 for a type the kernel does not store). */
#define PSK_NOALLOC_MAX_BATCH 1023
int psk_gemm_noalloc(const psk_gemm *g, const void *a, const void *b, void *c, void *stream, int64_t *overflowed_batch, char *err, size_t err_cap);

/* ---- the exchange step of a sharded call -------------------------------------------------------------------
 * The path shards by the batch axis: every rank (one process a GPU) runs the same launches on its rows, and
 * nothing crosses between GPUs until the end of a call, where the loss (and, under `presk calibrate`, each
 * site's magnitudes) is combined. No counterpart in the reference, whose executors are single-process: these
 * stand where its `Backend` reads a scalar back (presk-kernel/src/host.rs:1584, 1844). NCCL over NVLink;
 * looked up at run time (libnccl.so.2), so that the library loads where NCCL is absent. */
#define PSK_COMM_ID_BYTES 128
#define PSK_COMM_U32 100 /* raw 32-bit words, compared as unsigned integers (dtype argument) */
typedef enum { PSK_COMM_SUM = 0, PSK_COMM_MAX = 1, PSK_COMM_MIN = 2 } psk_comm_op;
typedef struct psk_comm psk_comm;
/* Rank 0 makes an id and gives it to the others by whatever route started them (a file, a socket, MPI). */
int psk_comm_unique_id(uint8_t id[PSK_COMM_ID_BYTES]);
/* Collective: every rank calls it with the same id. NULL on failure; psk_comm_error(NULL) says why. */
psk_comm *psk_comm_create(psk_exec *e, int32_t nranks, int32_t rank, const uint8_t id[PSK_COMM_ID_BYTES]);
void psk_comm_destroy(psk_comm *c);
const char *psk_comm_error(const psk_comm *c);
int32_t psk_comm_rank(const psk_comm *c);
int32_t psk_comm_size(const psk_comm *c);
/* In place, on the executor's stream, ordered after the launches queued before it; `dtype` is PSK_F32, PSK_F64,
 * PSK_I64 or PSK_COMM_U32. */
int psk_comm_allreduce(psk_comm *c, void *device_buf, int64_t count, int32_t dtype, int32_t op);

/* ---------------------------------------------------------------------------
 * From the reference's kernel to a launch. `KernelExec::run` receives `(idx, &Kernel, inputs, out)`
 * (crates/presk-kernel/src/host.rs:30), and a `Kernel` prints itself as text (its `Display`,
 * crates/presk-kernel/src/ir.rs:495-596): `kernel NAME (%0 : T[..], ..) -> %N : T[..] { loop nest }`. This reads
 * the first kernel of `kernel_text` and fills `*out` with the launch that computes it: the iteration space, each
 * buffer's element strides in it, the steps of an elementwise group. The pointer table of psk_exec_run is then
 * the kernel's inputs in order, its output, and the scales of each `intB/OVER` input.
 *
 * Recognised by structure: a perfect nest around one store (PSK_OP_FUSED, PSK_OP_COPY); sums kept in a scalar or
 * in the output over the loops that do not index the output (PSK_OP_CONTRACT, PSK_OP_REDUCE). Recognised by name
 * and buffers, the body's layout being free: `dot` in any tiling, `softmax axis A [where]`, `cross_entropy`,
 * `argmax`, `embed`. Anything else is refused with PSK_E7005 and a message in `err`; text that is not the
 * grammar, with PSK_E7001. `order` is the psk_order to run it under (the nest itself states the sequential one).
 * `name` (may be NULL) receives the kernel's name, which `out->name` then points at; `*rest` (may be NULL) is
 * left after the kernel read, for a listing of several. */
int psk_describe(const char *kernel_text, int32_t order, psk_launch *out, char *name, size_t name_cap, const char **rest, char *err, size_t err_cap);

/* ---------------------------------------------------------------------------
 * Samples of a .psk.d file, read into device buffers (presk-data's container; the reference's C reader is
 * presk_open / presk_read / presk_close, presk-export-c/c/presk_rt.c:295-530, whose header checks, error codes
 * and conversions these keep). `leaves` are the sample type's leaves in order, as the reference's exports state
 * them (presk_leaf, presk_rt.h:432-435): `bound` > 0 for idx[bound] elements, 0 for reals; `n` elements.
 * psk_data_open parses and checks the header on the host (no GPU needed; errors 9002, 9003, 9005 with the
 * reference's messages in `err`). psk_data_read moves samples first .. first + count - 1 to the device as the
 * file holds them and takes them apart there: dst[i] (a device buffer of the executor, count x leaves[i].n
 * elements of dtypes[i], dense, sample-major) receives leaf i of every sample; an index leaf's dtype is PSK_I64,
 * a real leaf's PSK_F32, PSK_BF16, PSK_F16 or PSK_E8M15, each real rounded once from the file's encoding as the
 * reference's store_real rounds. An index not below its bound: PSK_E9004 naming the first one in file order
 * (that element is not written). The call returns when the buffers are complete. Messages: psk_data_error.
 * ------------------------------------------------------------------------- */
typedef struct psk_data psk_data;
typedef struct {
    uint64_t bound;
    uint64_t n;
} psk_data_leaf;
int psk_data_open(const char *path, const char *type, const psk_data_leaf *leaves, size_t nleaves, psk_data **out, char *err, size_t err_cap);
uint64_t psk_data_count(const psk_data *d);
uint64_t psk_data_sample_bytes(const psk_data *d);
int psk_data_read(psk_data *d, psk_exec *e, uint64_t first, uint64_t count, void *const *dst, const int32_t *dtypes);
const char *psk_data_error(const psk_data *d);
void psk_data_close(psk_data *d);

/* ---------------------------------------------------------------------------
 * The executor as a table of functions, so that the host program can run
 * over another one (KernelBackend::with_exec, host.rs:466). The library's
 * own is the CUDA executor; tests hand the host a CPU one.
 * ------------------------------------------------------------------------- */
typedef struct {
    void *self;
    const char *(*name)(void *self);
    void *(*alloc)(void *self, size_t bytes);
    void (*free)(void *self, void *p);
    int (*upload)(void *self, void *dst, const void *src_host, size_t bytes);
    int (*download)(void *self, void *dst_host, const void *src, size_t bytes);
    int (*run)(void *self, const psk_launch *l, void *const *table);
    int (*sync)(void *self);
    int64_t (*overflow)(void *self);
    const char *(*last_error)(void *self);
    /* Integer weights made from reals on the executor (presk-rt/src/quant.rs:128-167):
     * w is outer x k x inner reals of type `from` (PSK_F32 or PSK_F64), q its
     * int8 codes, s one f32 scale per (outer, inner) channel, absmax scheme. */
    int (*quantize)(void *self, const void *w, int32_t from, int8_t *q, float *s, int64_t outer, int64_t k, int64_t inner);
    /* n elements of type `to` drawn on the executor; may be NULL. */
    int (*init_normal)(void *self, void *dst, int32_t to, int64_t n, uint64_t seed, double std);
} psk_exec_vtable;

/* The two device helpers of the table, on the CUDA executor. */
int psk_exec_quantize(psk_exec *e, const void *w, int32_t from, int8_t *q, float *s, int64_t outer, int64_t k, int64_t inner);
int psk_exec_init_normal(psk_exec *e, void *dst, int32_t to, int64_t n, uint64_t seed, double std);

/* The CUDA executor `e` as such a table. */
void psk_exec_as_vtable(psk_exec *e, psk_exec_vtable *out);

/* ---------------------------------------------------------------------------
 * The host program (Backend: prepare, call). It walks a model's lets in the
 * reference's order, one launch per fusion group or tensor primitive
 * (presk-kernel/src/host.rs:887-1039), each at its site's storage type
 * (Realization::dtype_at, presk-rt/src/lib.rs:459-471).
 * ------------------------------------------------------------------------- */
typedef struct psk_host psk_host;

/* A host over an executor. `realization` is the text of a realization file
 * (presk-rt/src/lib.rs:374-434): {"default": "bf16", "storage": {site: type},
 * "params": {path: type}, "quant": {path: {"bits": 8, "over": -2}},
 * "order": {"kind": "sequential" | "device"}}, or a bare type name as
 * `--realize f32` gives. NULL on a realization that does not parse;
 * psk_host_error(NULL) says why. */
psk_host *psk_host_create(const psk_exec_vtable *exec, const char *realization);
void psk_host_destroy(psk_host *h);
const char *psk_host_error(const psk_host *h);

/* The models of the five benchmark configurations. `model` is one of
 * "mlp" (Linear{784,256}, ReLU, Linear{256,10}, cross-entropy loss),
 * "gpt" (examples/corpus/nlp/05_gpt.psk), "llama" (examples/coverage/llama.psk),
 * "contract_ln" (x·w then LayerNorm), "layernorm", "rmsnorm"
 * (examples/spec/layernorm/layernorm.psk). `consts` are the program's
 * constants and dimensions as "V=32000 D=4096 H=32 G=32 FF=11008 L=32 B=8 T=2048".
 * Backend::prepare (presk-rt/src/lib.rs:1276). */
int psk_host_prepare(psk_host *h, const char *model, const char *consts);

/* Parameters, by path ("blocks.attn.wq", "tok"; a stacked parameter's
 * leading axis is its layers), given as f64 or f32 host reals and stored as
 * the realization says (Realization::store_params, lib.rs:711): rounded once
 * to the path's `params` type, quantised per channel under `quant`, else the
 * default type. Parameters stay on the executor across calls. */
int psk_host_set_param(psk_host *h, const char *path, const void *host, int32_t host_dtype, const int64_t *dims, int32_t rank);
/* The same, drawn on the executor's side of the boundary from a seed:
 * normal(0, std) or, std < 0, ones. For models whose parameters would not
 * fit a host copy in reasonable time. The draw is a counter-based hash, not
 * the reference's ChaCha keys. */
int psk_host_init_param(psk_host *h, const char *path, uint64_t seed, double std, const int64_t *dims, int32_t rank);

/* Backend::call on `entry` ("apply", "loss"): inputs are host buffers in the
 * entry's order (reals as f32 or f64, indices as i64), the result is written
 * to a host buffer of `out_dtype` (PSK_F32 or PSK_F64). Host-to-device and
 * device-to-host copies happen inside. Returns a psk_status. */
typedef struct {
    const void *data;
    int32_t dtype;
    int32_t rank;
    int64_t dims[PSK_MAX_RANK];
} psk_value;
int psk_host_call(psk_host *h, const char *entry, const psk_value *inputs, int32_t n_inputs, void *out_host, int32_t out_dtype, int64_t out_capacity, int64_t *out_numel);
/* A leaf of the last call's result when the entry returns a tree of the parameters' shape (a gradient,
 * `grad(..)(θ)`: presk-rt/src/lib.rs `Value::Record`): `path` is the parameter's, as in psk_host_set_param. */
int psk_host_result(psk_host *h, const char *path, void *out_host, int32_t out_dtype, int64_t out_capacity, int64_t *out_numel);
/* Gives the host a leaf of a gradient in place of one a call computed: `adamw.step` takes its `g` as an argument
 * (presk-core/src/lower/optim.rs:8). f32 or f64 reals of the parameter's size; stored at the default type. */
int psk_host_set_result(psk_host *h, const char *path, const void *data, int32_t dtype, const int64_t *dims, int32_t rank);

/* The optimizer of a training run: the functions presk-core/src/lower/optim.rs:118-330 builds from an
 * `optimizer adamw { … }` block. `hyperparameters` is NAME=VALUE words: lr (1e-3), beta1 (0.9), beta2 (0.999),
 * eps (1e-8), weight_decay (0), grad_clip (none), schedule (constant | linear | cosine), warmup (steps); the
 * block's defaults in brackets. Setting them forgets the moments (`adamw.init`: zeros). */
int psk_host_adamw(psk_host *h, const char *hyperparameters);
/* `adamw.step(θ, (m, v), g, t, total)`: g = the leaves the last gradient call (or psk_host_set_result) left, one a
 * parameter; t counts from 1. The parameters and moments are replaced; psk_host_result then reads θ' under a
 * parameter's path and the moments under "m:" + path and "v:" + path. */
int psk_host_adamw_step(psk_host *h, int64_t t, int64_t total);
/* `adamw.lr(t, total)`: the schedule's learning rate, computed by the executor in the `adamw.lr` sites' type. */
int psk_host_adamw_lr(psk_host *h, int64_t t, int64_t total, double *out);

/* The same with the inputs already on the executor (`inputs[i].data` is a
 * device pointer of the host's executor) and the result left there: what a
 * caller that shards a batch over several executors times. `*out` points at
 * the result, which belongs to the host until its next call. The launches are
 * queued, not waited for: psk_exec_sync (or the table's `sync`) ends them and
 * reports the overflow guard. */
int psk_host_call_device(psk_host *h, const char *entry, const psk_value *inputs, int32_t n_inputs, void **out, int32_t *out_dtype, int64_t *out_numel);

/* `presk calibrate` on this executor (presk-driver/src/precision.rs:65-117 measures on the exact
 * interpreter; this measures the values of the realization being run): while on, every launch's
 * real output is folded into its site's magnitudes. psk_host_envelope returns one line a site,
 * "site\tmax|x|\tmin non-zero |x|\tlo\thi", sorted by site, of everything seen since calibration was
 * switched on; the text belongs to the host until the next call. Ranks that shard a batch merge
 * their envelopes with one max-reduction (presk_b200/shard.py). */
void psk_host_set_calibrating(psk_host *h, int on);
const char *psk_host_envelope(psk_host *h);

/* Launch statistics of the last call (Backend::launch_stats): launches, and
 * the kernel names in order, newline-separated (for the launch-list tests). */
int64_t psk_host_launches(const psk_host *h);
const char *psk_host_launch_log(const psk_host *h);
void psk_host_set_logging(psk_host *h, int on);

/* The mean over all ranks' rows of a per-rank mean that stays on the executor (a loss from psk_host_call_device):
 * sum over ranks, divided by the number of ranks (equal rows a rank), read back as f64. */
int psk_host_mean_over_ranks(psk_host *h, psk_comm *c, const void *device_scalar, int32_t dtype, double *out);
/* Merges the magnitudes psk_host_envelope reports over the ranks: one max-reduction (the minima travel
 * complemented). After it every rank's envelope is that of the whole batch. */
int psk_host_envelope_allreduce(psk_host *h, psk_comm *c);
/* A training step over a sharded batch: every rank holds the gradient of the mean loss over its own rows (as many
 * rows on every rank); this sums each leaf of the last gradient over the ranks (NCCL, in the leaf's storage type, on
 * the executor's stream) and divides by their number, so that psk_host_adamw_step takes the same step everywhere:
 * the gradient all-reduce a data-parallel `presk train` needs. */
int psk_host_grads_allreduce(psk_host *h, psk_comm *c);

#ifdef __cplusplus
}
#endif
#endif
