"""The tcgen05 contraction on its own, through psk_exec_gemm: both layouts of the second
operand, batches, ragged edges, every output type, against f32 arithmetic on exact products."""
import ctypes as C

import numpy as np
import pytest

from presk_b200 import abi

pytestmark = pytest.mark.gpu


def to_bits(oracle, a, dtype):
    return oracle.convert(np.ascontiguousarray(a, np.float32), dtype)


def run_gemm(cuda, oracle, m, n, k, batch=1, b_n_major=0, in_dtype=abi.BF16, out_dtype=abi.F32, seed=0):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((batch, m, k)).astype(np.float32)
    b = rng.standard_normal((batch, k, n) if b_n_major else (batch, n, k)).astype(np.float32)
    ab, bb = to_bits(oracle, a, in_dtype), to_bits(oracle, b, in_dtype)
    av = oracle.widen(ab, in_dtype, a.size).reshape(a.shape).astype(np.float64)
    bv = oracle.widen(bb, in_dtype, b.size).reshape(b.shape).astype(np.float64)
    want = np.einsum("bmk,bkn->bmn", av, bv) if b_n_major else np.einsum("bmk,bnk->bmn", av, bv)
    pa, pb = cuda.upload(ab), cuda.upload(bb)
    pc = cuda.alloc(batch * m * n * abi.DTYPE_BYTES[out_dtype])
    g = abi.Gemm()
    g.in_dtype, g.out_dtype, g.b_n_major, g.guarded = in_dtype, out_dtype, b_n_major, 1
    g.m, g.n, g.k, g.batch, g.batch_lo = m, n, k, batch, batch
    g.a_row, g.a_lo, g.a_hi = k, m * k, m * k * batch
    g.b_row, g.b_lo, g.b_hi = (n if b_n_major else k), n * k, n * k * batch
    g.c_row_lo_count, g.c_row_lo, g.c_row_hi = m, n, 0
    g.c_col_lo_count, g.c_col_hi = n, 0
    g.c_lo, g.c_hi = m * n, m * n * batch
    cuda.gemm(g, pa, pb, pc)
    cuda.sync()
    raw = cuda.download(pc, batch * m * n * abi.DTYPE_BYTES[out_dtype])
    got = oracle.widen(raw, out_dtype, batch * m * n).reshape(batch, m, n)
    for p in (pa, pb, pc):
        cuda.free(p)
    return got, want


@pytest.mark.parametrize("b_n_major", [0, 1])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (256, 512, 256), (384, 768, 1024), (100, 200, 72), (2048, 2048, 128), (1, 256, 64), (130, 264, 8)])
def test_gemm_bf16_f32(cuda, oracle, m, n, k, b_n_major):
    if b_n_major and n % 8:
        pytest.skip("row stride of B must be a multiple of 16 bytes")
    got, want = run_gemm(cuda, oracle, m, n, k, 1, b_n_major)
    # exact products, f32 sums in some order: the error of a sum of k terms of size ~1
    assert np.abs(got - want).max() <= 4e-6 * k + 1e-5, (m, n, k)


@pytest.mark.parametrize("b_n_major", [0, 1])
def test_gemm_batched(cuda, oracle, b_n_major):
    got, want = run_gemm(cuda, oracle, 256, 128, 192, batch=6, b_n_major=b_n_major, seed=1)
    assert np.abs(got - want).max() <= 1e-3


@pytest.mark.parametrize("in_dtype,out_dtype,tol", [(abi.BF16, abi.BF16, 2.0**-8), (abi.F16, abi.F16, 2.0**-10), (abi.F16, abi.F32, 1e-6), (abi.BF16, abi.E8M15, 2.0**-15)])
def test_gemm_output_types_round_once(cuda, oracle, in_dtype, out_dtype, tol):
    got, want = run_gemm(cuda, oracle, 256, 256, 256, 1, 0, in_dtype, out_dtype, seed=2)
    assert np.abs(got - want).max() <= tol * np.abs(want).max() + 1e-4
    # and the stored value is the nearest number of the format to the f32 sum, for almost every element:
    # round the exact result the same way and count disagreements (a sum's last bit may flip a tie)
    if out_dtype == abi.F32:
        return
    raw = oracle.convert(want.astype(np.float32), out_dtype)
    rounded = oracle.widen(raw, out_dtype, want.size).reshape(want.shape)
    assert np.mean(got != rounded) < 0.02
