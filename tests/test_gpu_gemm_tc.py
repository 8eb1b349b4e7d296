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


@pytest.mark.parametrize("m,n,k,b_n_major", [(256, 256, 128, True), (384, 1000 // 8 * 8, 512, False), (1024, 1024, 1024, True)])
def test_e8m15_contraction_on_tensor_cores(cuda, oracle, m, n, k, b_n_major):
    """e8m15 operands under the device order: two bf16 planes each (x = hi + lo exactly), four partial products
    summed in one f32 accumulator. The products are exact, so the result differs from the oracle's sequential
    f32 sum only by the order of the additions: the f32 tolerance of the bf16 contractions, then one rounding
    to e8m15 (2^-16 relative)."""
    from presk_b200 import abi, launch_desc
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n) if b_n_major else (n, k)).astype(np.float32)
    a.ravel()[:4] = [0.0, -0.0, 1.0 + 2.0**-15, 3.0e-30]
    a8, b8 = oracle.convert(a, abi.E8M15), oracle.convert(b, abi.E8M15)
    l = launch_desc(abi.OP_CONTRACT, abi.E8M15, [m, n], [k], order=abi.ORDER_DEVICE)
    l.n_inputs = 2
    l.inputs[0].dtype, l.inputs[0].numel = abi.E8M15, m * k
    l.inputs[0].stride[0], l.inputs[0].stride[2] = k, 1
    l.inputs[1].dtype, l.inputs[1].numel = abi.E8M15, n * k
    if b_n_major:
        l.inputs[1].stride[1], l.inputs[1].stride[2] = 1, n
    else:
        l.inputs[1].stride[1], l.inputs[1].stride[2] = k, 1
    l.out.dtype, l.out.numel = abi.E8M15, m * n
    l.out.stride[0], l.out.stride[1] = n, 1
    pa, pb, pc = cuda.upload(a8), cuda.upload(b8), cuda.alloc(m * n * 3)
    cuda.set_profiling(True)
    cuda.run(l, [pa, pb, pc])
    cuda.sync()
    assert any(rec[0] == "k_gemm_tc" for rec in cuda.profile()), "the launch did not reach the tensor-core kernel"
    cuda.set_profiling(False)
    got8 = cuda.download(pc, m * n * 3)
    for p in (pa, pb, pc):
        cuda.free(p)
    want8 = np.zeros(m * n * 3, np.uint8)
    ls = launch_desc(abi.OP_CONTRACT, abi.E8M15, [m, n], [k])
    ls.n_inputs = 2
    for i in range(2):
        ls.inputs[i] = l.inputs[i]
    ls.out = l.out
    oracle.run(ls, [np.ascontiguousarray(a8), np.ascontiguousarray(b8), want8])

    def widen(u8):
        t = np.ascontiguousarray(u8).view(np.uint8).reshape(-1, 3).astype(np.uint32)
        return ((t[:, 0] | (t[:, 1] << 8) | (t[:, 2] << 16)) << 8).view(np.float32)

    got, want = widen(got8), widen(want8)
    assert np.abs(got - want).max() <= 4e-6 * k + 1e-5 + 2.0**-15 * np.abs(want).max()
    # and against the exact sum of the same e8m15 inputs in f64
    af, bf = widen(a8).reshape(m, k).astype(np.float64), widen(b8).reshape(b.shape).astype(np.float64)
    exact = (af @ bf if b_n_major else af @ bf.T).ravel()
    assert np.abs(got - exact).max() <= 4e-6 * k + 1e-5 + 2.0**-15 * np.abs(exact).max()


@pytest.mark.parametrize("m,n,k,b_n_major", [(512, 512, 256, True), (384, 1000 // 8 * 8, 512, False), (1024, 1024, 1024, True)])
def test_f32_contraction_on_tensor_cores(cuda, oracle, m, n, k, b_n_major):
    """f32 operands under the device order: three bf16 planes each (x = hi + mid + lo exactly), nine partial products
    in one f32 accumulator. Exact products; the result differs from the sequential f32 sum by the order of the
    additions only."""
    from presk_b200 import abi, launch_desc
    rng = np.random.default_rng(m * 3 + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n) if b_n_major else (n, k)).astype(np.float32)
    a.ravel()[:5] = [0.0, -0.0, 1.0 + 2.0**-23, 3.0e-30, -1.7e10]
    l = launch_desc(abi.OP_CONTRACT, abi.F32, [m, n], [k], order=abi.ORDER_DEVICE)
    l.n_inputs = 2
    l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = abi.F32, m * k, k, 1
    l.inputs[1].dtype, l.inputs[1].numel = abi.F32, n * k
    if b_n_major:
        l.inputs[1].stride[1], l.inputs[1].stride[2] = 1, n
    else:
        l.inputs[1].stride[1], l.inputs[1].stride[2] = k, 1
    l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = abi.F32, m * n, n, 1
    pa, pb, pc = cuda.upload(a), cuda.upload(b), cuda.alloc(m * n * 4)
    cuda.set_profiling(True)
    cuda.run(l, [pa, pb, pc])
    cuda.sync()
    assert any(rec[0] == "k_gemm_tc" for rec in cuda.profile()), "the launch did not reach the tensor-core kernel"
    cuda.set_profiling(False)
    got = cuda.download(pc, m * n * 4).view(np.float32)
    for p in (pa, pb, pc):
        cuda.free(p)
    exact = (a.astype(np.float64) @ b.astype(np.float64) if b_n_major else a.astype(np.float64) @ b.astype(np.float64).T).ravel()
    scale = np.abs(a).max() * np.abs(b).max()
    assert np.abs(got - exact).max() <= (4e-6 * k + 1e-5) * max(1.0, scale / 16)
    # the nine partial products must all be there: an f32-accurate result, far below a bf16-plane's 2^-8
    row = slice(5 * n, 6 * n)
    assert np.abs(got[row] - exact[row]).max() <= 1e-4 * np.abs(exact[row]).max() + 1e-4


@pytest.mark.parametrize("dt", ["f32", "bf16", "mixed"])
@pytest.mark.parametrize("m,n,k,b_n_major", [(300, 260, 70, True), (257, 384, 200, False), (128, 128, 16, True), (513, 129, 33, False)])
def test_exact_contraction_of_large_operands_is_the_oracle_s_bits(cuda, oracle, dt, m, n, k, b_n_major):
    """Sequential order, operands of 128 rows and columns or more: the 128 x 128 tile kernel (`k_gemm_exact_big`), ragged
    edges and both layouts of the second operand. Every result adds its products in increasing k: the oracle's bits."""
    from presk_b200 import abi, launch_desc
    rng = np.random.default_rng(m + 7 * n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n) if b_n_major else (n, k)).astype(np.float32)
    a.ravel()[:3] = [-0.0, 0.0, 1e-30]
    da = abi.F32 if dt == "f32" else abi.BF16
    db = abi.BF16 if dt == "bf16" else abi.F32
    kd = abi.F32 if dt != "bf16" else abi.BF16
    ab = a if da == abi.F32 else oracle.convert(a, abi.BF16)
    bb = b if db == abi.F32 else oracle.convert(b, abi.BF16)
    l = launch_desc(abi.OP_CONTRACT, kd, [m, n], [k])
    l.n_inputs = 2
    l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = da, m * k, k, 1
    l.inputs[1].dtype, l.inputs[1].numel = db, n * k
    if b_n_major:
        l.inputs[1].stride[1], l.inputs[1].stride[2] = 1, n
    else:
        l.inputs[1].stride[1], l.inputs[1].stride[2] = k, 1
    l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = kd, m * n, n, 1
    nbytes = m * n * abi.DTYPE_BYTES[kd]
    pa, pb, pc = cuda.upload(np.ascontiguousarray(ab)), cuda.upload(np.ascontiguousarray(bb)), cuda.alloc(nbytes)
    cuda.run(l, [pa, pb, pc])
    cuda.sync()
    got = cuda.download(pc, nbytes)
    for p in (pa, pb, pc):
        cuda.free(p)
    want = np.zeros(nbytes, np.uint8)
    oracle.run(l, [np.ascontiguousarray(ab), np.ascontiguousarray(bb), want])
    assert np.array_equal(got, want)


@pytest.mark.parametrize("b_n_major", [0, 1])
@pytest.mark.parametrize("out_dtype", [abi.BF16, abi.F32])
def test_gemm_long_summed_axis_takes_the_256_row_tiles(cuda, oracle, b_n_major, out_dtype):
    """K >= 8192: tiles of 256 rows, two accumulators multiplying one tile of B; 640 rows leave the last tile half
    empty, 520 columns the last column tile ragged."""
    got, want = run_gemm(cuda, oracle, 640, 520, 8192, 1, b_n_major, abi.BF16, out_dtype, seed=9)
    tol = 4e-6 * 8192 + 1e-5 if out_dtype == abi.F32 else 2.0**-8 * np.abs(want).max() + 1e-3
    assert np.abs(got - want).max() <= tol


def test_contract_add_and_integer_weights_on_the_256_row_tiles(cuda, oracle):
    """The epilogue's extras on the long-K form of the kernel: a residual addend (the same bits as the contraction
    followed by the addition on this executor) and integer weights with one scale a column (within the bf16
    tolerance of the oracle's sequential result)."""
    from presk_b200 import launch_desc
    m, n, k = 512, 256, 8192
    rng = np.random.default_rng(17)
    a = oracle.convert((rng.standard_normal((m, k)) * 0.1).astype(np.float32), abi.BF16)
    w = oracle.convert((rng.standard_normal((k, n)) * 0.1).astype(np.float32), abi.BF16)
    x = oracle.convert(rng.standard_normal((m, n)).astype(np.float32), abi.BF16)

    def contract(op, n_inputs):
        l = launch_desc(op, abi.BF16, [m, n], [k], order=abi.ORDER_DEVICE)
        l.n_inputs = n_inputs
        l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = abi.BF16, m * k, k, 1
        l.inputs[1].dtype, l.inputs[1].numel, l.inputs[1].stride[1], l.inputs[1].stride[2] = abi.BF16, n * k, 1, n
        l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = abi.BF16, m * n, n, 1
        return l

    pa, pw, px = cuda.upload(a), cuda.upload(w), cuda.upload(x)
    pc, ps, pf = cuda.alloc(m * n * 2), cuda.alloc(m * n * 2), cuda.alloc(m * n * 2)
    cuda.run(contract(abi.OP_CONTRACT, 2), [pa, pw, pc])
    add = launch_desc(abi.OP_FUSED, abi.BF16, [m, n], order=abi.ORDER_DEVICE)
    add.n_inputs, add.n_steps = 2, 1
    add.steps[0].prim, add.steps[0].nargs, add.steps[0].src[0], add.steps[0].src[1] = abi.ADD, 2, 0, 1
    for o in (add.inputs[0], add.inputs[1], add.out):
        o.dtype, o.numel, o.stride[0], o.stride[1] = abi.BF16, m * n, n, 1
    cuda.run(add, [px, pc, ps])
    fused = contract(abi.OP_CONTRACT_ADD, 3)
    fused.iparam[1] = abi.BF16
    fused.inputs[2].dtype, fused.inputs[2].numel, fused.inputs[2].stride[0], fused.inputs[2].stride[1] = abi.BF16, m * n, n, 1
    cuda.run(fused, [pa, pw, px, pf])
    cuda.sync()
    assert np.array_equal(cuda.download(pf, m * n * 2), cuda.download(ps, m * n * 2))
    # integer weights: codes and one f32 scale a column
    q = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    sc = (rng.uniform(0.5, 2.0, n) * 1e-3).astype(np.float32)
    lq = contract(abi.OP_CONTRACT, 2)
    lq.inputs[1].dtype = abi.I8
    lq.inputs[1].scale_stride[1] = 1
    pq, psc = cuda.upload(q), cuda.upload(sc)
    cuda.run(lq, [pa, pq, pc, psc])
    cuda.sync()
    got = (cuda.download(pc, m * n * 2).view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    want_b = np.zeros(m * n * 2, np.uint8)
    ls = contract(abi.OP_CONTRACT, 2)
    ls.order = abi.ORDER_SEQUENTIAL
    ls.inputs[1].dtype = abi.I8
    ls.inputs[1].scale_stride[1] = 1
    oracle.run(ls, [np.ascontiguousarray(a), np.ascontiguousarray(q), want_b, np.ascontiguousarray(sc)])
    want = (want_b.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    assert np.abs(got - want).max() <= 2.0**-7 * np.abs(want).max()
    for p in (pa, pw, px, pc, ps, pf, pq, psc):
        cuda.free(p)


def _narrow_weight_launch(m, n, k, wdtype, order):
    from presk_b200 import launch_desc
    l = launch_desc(abi.OP_CONTRACT, abi.BF16, [m, n], [k], order=order)
    l.n_inputs = 2
    l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = abi.BF16, m * k, k, 1
    l.inputs[1].dtype, l.inputs[1].numel, l.inputs[1].stride[1], l.inputs[1].stride[2] = wdtype, n * k, 1, n
    l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = abi.BF16, m * n, n, 1
    if wdtype == abi.I8:
        l.inputs[1].scale_stride[1] = 1
    return l


def _bf16_values(raw):
    return (np.frombuffer(raw, np.uint16).astype(np.uint32) << 16).view(np.float32)


def test_integer_weights_widened_once_follow_their_codes(cuda, oracle):
    """Integer weights reach the tensor-core kernel as a bf16 copy made once and kept; the copy is dropped when
    the codes are written again. 328 columns: five whole groups of 64 (the epilogue's path with the scales of
    a group loaded as vectors) and a ragged one of 8."""
    m, n, k = 512, 328, 256
    rng = np.random.default_rng(23)
    a = oracle.convert((rng.standard_normal((m, k)) * 0.1).astype(np.float32), abi.BF16)
    sc = (rng.uniform(0.5, 2.0, n) * 1e-3).astype(np.float32)
    pa, psc, pc = cuda.upload(a), cuda.upload(sc), cuda.alloc(m * n * 2)
    pq = cuda.alloc(k * n)
    for seed in (1, 2):
        q = np.random.default_rng(seed).integers(-127, 128, size=(k, n), dtype=np.int8)
        cuda._check(cuda.lib.psk_exec_upload(cuda.handle, pq, q.ctypes.data_as(C.c_void_p), q.nbytes))
        cuda.set_profiling(True)
        cuda.run(_narrow_weight_launch(m, n, k, abi.I8, abi.ORDER_DEVICE), [pa, pq, pc, psc])
        cuda.sync()
        assert any(rec[0] == "k_gemm_tc" for rec in cuda.profile()), "the launch did not reach the tensor-core kernel"
        cuda.set_profiling(False)
        got = _bf16_values(cuda.download(pc, m * n * 2))
        want_b = np.zeros(m * n * 2, np.uint8)
        oracle.run(_narrow_weight_launch(m, n, k, abi.I8, abi.ORDER_SEQUENTIAL), [np.ascontiguousarray(a), np.ascontiguousarray(q), want_b, sc])
        want = _bf16_values(want_b)
        assert np.abs(got - want).max() <= 2.0**-7 * np.abs(want).max(), seed
    for p in (pa, psc, pc, pq):
        cuda.free(p)


@pytest.mark.parametrize("m,n,k", [(512, 256, 512), (130, 264, 72)])
def test_e4m3_weights_on_tensor_cores(cuda, oracle, m, n, k):
    """Weights stored e4m3fn under a bf16 site (a `params` entry narrower than the site): widened exactly, once,
    to the bf16 numbers they are; products exact, sums in the unit's order, within the bf16 tolerance of the
    oracle's sequential result."""
    rng = np.random.default_rng(29)
    a = oracle.convert((rng.standard_normal((m, k)) * 0.1).astype(np.float32), abi.BF16)
    w = oracle.convert(rng.standard_normal((k, n)).astype(np.float32), abi.E4M3)
    assert w.dtype == np.uint8 and w.size == k * n
    pa, pw, pc = cuda.upload(a), cuda.upload(w), cuda.alloc(m * n * 2)
    cuda.set_profiling(True)
    cuda.run(_narrow_weight_launch(m, n, k, abi.E4M3, abi.ORDER_DEVICE), [pa, pw, pc])
    cuda.sync()
    assert any(rec[0] == "k_gemm_tc" for rec in cuda.profile()), "the launch did not reach the tensor-core kernel"
    cuda.set_profiling(False)
    got = _bf16_values(cuda.download(pc, m * n * 2))
    want_b = np.zeros(m * n * 2, np.uint8)
    oracle.run(_narrow_weight_launch(m, n, k, abi.E4M3, abi.ORDER_SEQUENTIAL), [np.ascontiguousarray(a), np.ascontiguousarray(w), want_b])
    want = _bf16_values(want_b)
    assert np.isfinite(want).all() and np.abs(want).max() > 0.1
    assert np.abs(got - want).max() <= 2.0**-7 * np.abs(want).max()
    # and the sequential order on the device is the oracle's bits
    cuda.run(_narrow_weight_launch(m, n, k, abi.E4M3, abi.ORDER_SEQUENTIAL), [pa, pw, pc])
    cuda.sync()
    assert np.array_equal(np.frombuffer(cuda.download(pc, m * n * 2), np.uint8), want_b)
    for p in (pa, pw, pc):
        cuda.free(p)


@pytest.mark.parametrize("b_n_major", [0, 1])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (640, 520, 1024), (136, 264, 72), (4096, 1024, 2048)])
def test_gemm_first_operand_m_major(cuda, oracle, m, n, k, b_n_major):
    """The first operand stored [k][m], m contiguous (x read as its transpose: a weight's gradient xᵀ·ct), through
    both tile forms (640 and 4096 rows take the 256-row one), ragged edges included."""
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal((k, m)).astype(np.float32)
    b = rng.standard_normal((k, n) if b_n_major else (n, k)).astype(np.float32)
    ab, bb = to_bits(oracle, a, abi.BF16), to_bits(oracle, b, abi.BF16)
    av = oracle.widen(ab, abi.BF16, a.size).reshape(a.shape).astype(np.float64)
    bv = oracle.widen(bb, abi.BF16, b.size).reshape(b.shape).astype(np.float64)
    want = av.T @ (bv if b_n_major else bv.T)
    pa, pb, pc = cuda.upload(ab), cuda.upload(bb), cuda.alloc(m * n * 4)
    g = abi.Gemm()
    g.in_dtype, g.out_dtype, g.b_n_major, g.guarded = abi.BF16, abi.F32, b_n_major | 2, 1
    g.m, g.n, g.k, g.batch, g.batch_lo = m, n, k, 1, 1
    g.a_row, g.a_lo, g.a_hi = m, m * k, m * k
    g.b_row, g.b_lo, g.b_hi = (n if b_n_major else k), n * k, n * k
    g.c_row_lo_count, g.c_row_lo, g.c_row_hi = m, n, 0
    g.c_col_lo_count, g.c_col_hi = n, 0
    g.c_lo, g.c_hi = m * n, m * n
    cuda.gemm(g, pa, pb, pc)
    cuda.sync()
    got = np.frombuffer(cuda.download(pc, m * n * 4), np.float32).reshape(m, n)
    for p in (pa, pb, pc):
        cuda.free(p)
    assert np.abs(got - want).max() <= 4e-6 * k + 1e-5


def test_weight_gradient_contraction_reaches_the_tensor_cores(cuda, oracle):
    """dot_vjp_r as a launch: out[model, ff] = Σ over (batch, seq) of x[batch, seq, model] · ct[batch, seq, ff] under the
    device order: the transposed first operand goes to the tensor-core kernel's M-major form."""
    from presk_b200 import launch_desc
    bsz, t, d, ff = 2, 256, 192, 320
    rng = np.random.default_rng(31)
    x = oracle.convert((rng.standard_normal((bsz, t, d)) * 0.5).astype(np.float32), abi.BF16)
    ct = oracle.convert((rng.standard_normal((bsz, t, ff)) * 0.5).astype(np.float32), abi.BF16)

    def launch(order):
        l = launch_desc(abi.OP_CONTRACT, abi.BF16, [d, ff], [bsz, t], order=order)
        l.n_inputs = 2
        l.inputs[0].dtype, l.inputs[0].numel = abi.BF16, x.size // 2
        l.inputs[0].stride[0], l.inputs[0].stride[2], l.inputs[0].stride[3] = 1, t * d, d
        l.inputs[1].dtype, l.inputs[1].numel = abi.BF16, ct.size // 2
        l.inputs[1].stride[1], l.inputs[1].stride[2], l.inputs[1].stride[3] = 1, t * ff, ff
        l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = abi.BF16, d * ff, ff, 1
        return l

    px, pct, pc = cuda.upload(x), cuda.upload(ct), cuda.alloc(d * ff * 2)
    cuda.set_profiling(True)
    cuda.run(launch(abi.ORDER_DEVICE), [px, pct, pc])
    cuda.sync()
    assert any(rec[0] == "k_gemm_tc" for rec in cuda.profile()), "the launch did not reach the tensor-core kernel"
    cuda.set_profiling(False)
    got = _bf16_values(cuda.download(pc, d * ff * 2))
    want_b = np.zeros(d * ff * 2, np.uint8)
    oracle.run(launch(abi.ORDER_SEQUENTIAL), [x, ct, want_b])
    want = _bf16_values(want_b)
    assert np.abs(got - want).max() <= 2.0**-7 * np.abs(want).max()
    for p in (px, pct, pc):
        cuda.free(p)


@pytest.fixture(params=[1, 2])
def i8_tile_form(request):
    """Both forms of the integer kernel: tiles of 128 rows (the rescale hidden behind the next tile) and of 256."""
    import os
    before = os.environ.get("PSK_I8_MT")
    os.environ["PSK_I8_MT"] = str(request.param)
    yield request.param
    if before is None:
        del os.environ["PSK_I8_MT"]
    else:
        os.environ["PSK_I8_MT"] = before


@pytest.mark.parametrize("m,k,n,b_n_major", [(300, 576, 272, True), (300, 576, 272, False), (512, 4096, 256, True), (129, 160, 48, True), (1, 1024, 512, True), (64, 65536, 32, False), (2600, 160, 2096, True)])
def test_integer_sums_on_the_tensor_cores_are_exact(cuda, oracle, i8_tile_form, m, k, n, b_n_major):
    """`product: i32, accum: i32` at contraction scale: affine activations (u8 with a zero point, i8 without and
    with one) times int8 weights with a scale a column, on tcgen05's 8-bit integer kind. Sums modulo 2^32 are
    associative and the store rounds the exact value once, so every output is the oracle's, bit for bit, for every
    result type (bf16, f32, f16, e8m15, affine i8): ragged edges, a summed axis that is no multiple of the tile,
    the longest sum the kernel takes (65536 terms of the largest codes, which stays inside 32 bits)."""
    from presk_b200 import abi, launch_desc
    rng = np.random.default_rng(m * 7 + k + n)
    cases = [(2, 37, abi.BF16), (1, 0, abi.F32), (1, -5, abi.BF16), (2, 255, abi.F16), (1, 0, abi.E8M15), (2, 128, "affine")]
    for kind, zero, store in cases:
        lo, hi = (0, 255) if kind == 2 else (-128, 127)
        codes = rng.integers(lo, hi + 1, size=(m, k)).astype(np.uint8 if kind == 2 else np.int8)
        qw = rng.integers(-127, 128, size=(k, n) if b_n_major else (n, k)).astype(np.int8)
        if k == 65536:  # the extreme: every product the largest there is
            codes[:] = hi
            qw[:] = 127 if kind == 2 else -127
        s_a = np.float32(rng.uniform(1.0, 2.0) * 2.0 ** int(rng.integers(-10, -2)))
        sw = (rng.uniform(1.0, 2.0, size=n) * 2.0 ** rng.integers(-12, -4, size=n)).astype(np.float32)
        l = launch_desc(abi.OP_CONTRACT, abi.F32, [m, n], [k], name=b"dot")
        l.n_inputs, l.int_accum = 2, 1
        l.inputs[0].dtype = abi.U8 if kind == 2 else abi.I8
        l.inputs[0].affine, l.inputs[0].affine_zero, l.inputs[0].affine_scale = kind, zero, float(s_a)
        l.inputs[0].stride[0], l.inputs[0].stride[2], l.inputs[0].numel = k, 1, m * k
        l.inputs[1].dtype, l.inputs[1].numel = abi.I8, k * n
        if b_n_major:
            l.inputs[1].stride[1], l.inputs[1].stride[2] = 1, n
        else:
            l.inputs[1].stride[1], l.inputs[1].stride[2] = k, 1
        l.inputs[1].scale_stride[1] = 1
        l.out.stride[0], l.out.stride[1], l.out.numel = n, 1, m * n
        if store == "affine":
            l.out.dtype, l.out.affine, l.out.affine_zero = abi.I8, 1, 3
            l.out.affine_scale = float(np.float32(float(s_a) * float(sw.mean()) * np.sqrt(k) * 40.0))
            out_bytes = m * n
        else:
            l.dtype = l.out.dtype = store
            out_bytes = m * n * abi.DTYPE_BYTES[store]
        dev = [cuda.upload(codes), cuda.upload(qw)]
        pout, psw = cuda.alloc(out_bytes), cuda.upload(sw)
        cuda.set_profiling(True)
        cuda.run(l, dev + [pout, psw])
        cuda.overflow()
        cuda.sync()
        kinds = [rec[0] for rec in cuda.profile()]
        cuda.set_profiling(False)
        assert kinds == ["k_gemm_i8"], kinds  # the tensor-core kernel took it
        got = cuda.download(pout, out_bytes)
        for p in dev + [pout, psw]:
            cuda.free(p)
        want = np.zeros(out_bytes, np.uint8)
        oracle.run(l, [codes, qw, want, sw])
        bad = np.nonzero(got != want)[0]
        assert bad.size == 0, (kind, zero, store, bad.size, bad[:4], got[bad[:4]], want[bad[:4]])
        if store == abi.F32:  # and the oracle's integer is the one numpy's 64-bit sum wraps to
            acc = (codes.astype(np.int64) - zero) @ (qw.astype(np.int64) if b_n_major else qw.astype(np.int64).T)
            acc = ((acc + 2**31) % 2**32) - 2**31
            ref = acc.astype(np.float64) * float(s_a) * sw.astype(np.float64)[None, :]
            np.testing.assert_allclose(got.view(np.float32).reshape(m, n), ref, rtol=1e-6)


@pytest.mark.parametrize("m,k,n,b_n_major,inner", [(300, 576, 288, True, None), (512, 4096, 256, False, None), (129, 384, 64, True, (2, 3, 64)), (1, 1024, 512, True, None)])
def test_integer_sums_take_a_residual_along(cuda, oracle, m, k, n, b_n_major, inner):
    """PSK_OP_CONTRACT_ADD with `product: i32, accum: i32`: the W8A8 projections that end in a residual addition
    (out-projection, down-projection), as one launch of the integer tensor-core kernel. The sums are exact, their
    rescaled value is rounded once to bf16, and the addition rounds once more, so every bit is the oracle's two
    launches' under any order; ragged rows and columns, both layouts of the weights, a summed axis given as three
    (groups, per, hd), one row. A result whose rows are not made of 16-byte runs is refused (E7005) and left to the
    caller's two launches."""
    from presk_b200 import PreskError, abi, launch_desc
    rng = np.random.default_rng(m + k + n)
    for kind, zero in ((1, 0), (2, 77)):
        lo, hi = (0, 255) if kind == 2 else (-128, 127)
        codes = rng.integers(lo, hi + 1, size=(m, k)).astype(np.uint8 if kind == 2 else np.int8)
        qw = rng.integers(-127, 128, size=(k, n) if b_n_major else (n, k)).astype(np.int8)
        s_a = np.float32(rng.uniform(1.0, 2.0) * 2.0**-6)
        sw = (rng.uniform(1.0, 2.0, size=n) * 2.0**-9).astype(np.float32)
        x = oracle.convert((rng.standard_normal((m, n)) * 4.0).astype(np.float32), abi.BF16)

        def launch(n_cols):
            dims_in = list(inner) if inner else [k]
            l = launch_desc(abi.OP_CONTRACT_ADD, abi.BF16, [m, n_cols], dims_in, order=abi.ORDER_DEVICE, name=b"dot+add")
            l.n_inputs, l.int_accum = 3, 1
            l.iparam[1] = abi.BF16
            l.inputs[0].dtype = abi.U8 if kind == 2 else abi.I8
            l.inputs[0].affine, l.inputs[0].affine_zero, l.inputs[0].affine_scale = kind, zero, float(s_a)
            l.inputs[0].stride[0], l.inputs[0].numel = k, m * k
            l.inputs[1].dtype, l.inputs[1].numel = abi.I8, k * n
            l.inputs[1].stride[1] = 1 if b_n_major else k
            run = 1  # the summed axes, innermost last, walk k as one
            for a in range(len(dims_in) - 1, -1, -1):
                l.inputs[0].stride[2 + a] = run
                l.inputs[1].stride[2 + a] = run * (n if b_n_major else 1)
                run *= dims_in[a]
            l.inputs[1].scale_stride[1] = 1
            l.inputs[2].dtype, l.inputs[2].numel, l.inputs[2].stride[0], l.inputs[2].stride[1] = abi.BF16, m * n, n, 1
            l.out.dtype, l.out.stride[0], l.out.stride[1], l.out.numel = abi.BF16, n, 1, m * n
            return l

        l = launch(n)
        dev = [cuda.upload(codes), cuda.upload(qw), cuda.upload(x)]
        pout, psw = cuda.alloc(m * n * 2), cuda.upload(sw)
        cuda.set_profiling(True)
        cuda.run(l, dev + [pout, psw])
        cuda.sync()
        kinds = [rec[0] for rec in cuda.profile()]
        cuda.set_profiling(False)
        assert kinds[-1] == "k_gemm_i8", kinds
        got = cuda.download(pout, m * n * 2)
        want = np.zeros(m * n * 2, np.uint8)
        oracle.run(l, [codes, qw, np.ascontiguousarray(x), want, sw])
        bad = np.nonzero(got.view(np.uint16) != want.view(np.uint16))[0]
        assert bad.size == 0, (kind, zero, bad.size, bad[:4])
        assert np.any(want)
        if n > 20:  # the first 20 columns of the same buffers: rows of 40 bytes, no 16-byte runs
            with pytest.raises(PreskError, match="E7005"):
                cuda.run(launch(20), dev + [pout, psw])
        for p in dev + [pout, psw]:
            cuda.free(p)
