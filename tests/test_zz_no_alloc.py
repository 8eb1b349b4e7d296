"""psk_gemm_noalloc: the tensor-core contraction for callers that cannot allocate on the device
(a fixed arena, a fixed memory budget, a context where the driver's allocator must not be entered).

It runs the same kernel as psk_exec_gemm with its scratch (status word, one overflow-guard flag a
batch entry) in a static device array instead of memory an executor allocated, so its output must
be the executor's, byte for byte. Two calls in a row share that array: the second must not see the
first's flags. The buffers here are made by the test through an executor; the entry point under
test allocates nothing itself.

This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import numpy as np
import pytest

from presk_b200 import abi

pytestmark = pytest.mark.gpu


def gemm_desc(m, n, k, batch, in_dtype, out_dtype, b_n_major=0):
    g = abi.Gemm()
    g.in_dtype, g.out_dtype, g.b_n_major, g.guarded = in_dtype, out_dtype, b_n_major, 1
    g.m, g.n, g.k, g.batch, g.batch_lo = m, n, k, batch, batch
    g.a_row, g.a_lo, g.a_hi = k, m * k, m * k * batch
    g.b_row, g.b_lo, g.b_hi = (n if b_n_major else k), n * k, n * k * batch
    g.c_row_lo_count, g.c_row_lo, g.c_col_lo_count = m, n, n
    g.c_lo, g.c_hi = m * n, m * n * batch
    return g


def call_noalloc(cuda, g, pa, pb, pc):
    err = C.create_string_buffer(256)
    where = C.c_int64(-2)
    rc = cuda.lib.psk_gemm_noalloc(C.byref(g), pa, pb, pc, cuda.stream(), C.byref(where), err, 256)
    return rc, where.value, err.value.decode()


def both_ways(cuda, oracle, g, a32, b32):
    """The executor's entry point and the one that allocates nothing, on the same operands."""
    a, b = oracle.convert(a32, g.in_dtype), oracle.convert(b32, g.in_dtype)
    pa, pb = cuda.upload(a), cuda.upload(b)
    nbytes = g.batch * g.m * g.n * abi.DTYPE_BYTES[g.out_dtype]
    pc1, pc2 = cuda.alloc(nbytes), cuda.alloc(nbytes)
    cuda.gemm(g, pa, pb, pc1)
    overflow_exec = cuda.overflow() != 0
    cuda.sync()
    rc, where, msg = call_noalloc(cuda, g, pa, pb, pc2)
    out1, out2 = cuda.download(pc1, nbytes), cuda.download(pc2, nbytes)
    for p in (pa, pb, pc1, pc2):
        cuda.free(p)
    return out1, out2, overflow_exec, rc, where, msg


def test_same_bytes_as_the_executor_on_two_calls_in_a_row(cuda, oracle):
    rng = np.random.default_rng(0)
    # first call: binary16 output, and batch entry 2 holds operands large enough to overflow its store
    g = gemm_desc(256, 256, 128, 4, abi.F16, abi.F16)
    a = rng.standard_normal((4, 256, 128)).astype(np.float32)
    b = rng.standard_normal((4, 256, 128)).astype(np.float32)
    a[2] *= 200.0
    b[2] *= 200.0
    out1, out2, ovf, rc, where, msg = both_ways(cuda, oracle, g, a, b)
    assert np.array_equal(out1, out2)
    assert ovf and rc == abi.E7007 and where == 2, (ovf, rc, where, msg)
    # second call, straight after: other sizes, bf16, N-major second operand, nothing overflows.
    # The static array still holds the first call's flags unless the entry point cleared them.
    g = gemm_desc(384, 512, 192, 3, abi.BF16, abi.BF16, b_n_major=1)
    a = rng.standard_normal((3, 384, 192)).astype(np.float32)
    b = rng.standard_normal((3, 192, 512)).astype(np.float32)
    out1, out2, ovf, rc, where, msg = both_ways(cuda, oracle, g, a, b)
    assert np.array_equal(out1, out2)
    assert not ovf and rc == abi.OK and where == -1, (ovf, rc, where, msg)
    # and the numbers are a matrix product
    av = oracle.widen(oracle.convert(a, abi.BF16), abi.BF16, a.size).reshape(a.shape).astype(np.float64)
    bv = oracle.widen(oracle.convert(b, abi.BF16), abi.BF16, b.size).reshape(b.shape).astype(np.float64)
    got = oracle.widen(out2, abi.BF16, 3 * 384 * 512).reshape(3, 384, 512)
    want = np.einsum("bmk,bkn->bmn", av, bv)
    assert np.abs(got - want).max() <= 2.0**-7 * np.abs(want).max()


def test_sizes_beyond_the_static_scratch_are_refused(cuda):
    g = gemm_desc(128, 128, 64, 1024, abi.BF16, abi.BF16)
    rc, where, msg = call_noalloc(cuda, g, 16, 16, 16)  # refused before any pointer is touched
    assert rc == abi.E7001 and "beyond" in msg and "1023" in msg


def test_a_descriptor_the_kernel_cannot_index_with_is_refused(cuda):
    """The result's side of the descriptor is checked before any launch: the kernel divides by the two
    counts and adds the strides to the caller's pointer, so a zero count or a negative stride never reaches it."""
    for field, value, code in (("c_row_lo_count", 0, abi.E7001), ("c_col_lo_count", 0, abi.E7001), ("c_row_lo", -256, abi.E7001), ("out_dtype", 77, abi.E7005)):
        g = gemm_desc(128, 256, 64, 1, abi.BF16, abi.BF16)
        setattr(g, field, value)
        rc, where, msg = call_noalloc(cuda, g, 16, 16, 16)
        assert rc == code and msg, (field, rc, msg)
