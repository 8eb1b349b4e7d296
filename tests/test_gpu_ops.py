"""Single launches through psk_exec_run against the oracle's psk_oracle_run on the same
descriptor and the same bytes: elementwise steps (every primitive, the device library's
transcendental functions), conversions of every storage format, reductions, softmax,
cross-entropy, gathers and copies; empty and ragged shapes."""
import ctypes as C

import numpy as np
import pytest

from presk_b200 import abi, launch_desc

pytestmark = pytest.mark.gpu


def contiguous(shape):
    s, acc = [], 1
    for d in reversed(shape):
        s.append(acc)
        acc *= d
    return list(reversed(s))


def set_operand(op, dtype, shape, positions, offset=0, is_index=False):
    """`shape` contiguous; axis i of it sits at iteration axis positions[i]."""
    op.dtype = abi.I64 if is_index else dtype
    op.is_index = 1 if is_index else 0
    op.offset = offset
    n = 1
    for d in shape:
        n *= d
    op.numel = n
    for st, p in zip(contiguous(shape), positions):
        op.stride[p] += st


def run_both(cuda, oracle, l, host_inputs, out_bytes):
    """Runs `l` on the GPU and on the oracle; returns (gpu bytes, oracle bytes, gpu flag, oracle flag)."""
    dev = [cuda.upload(a) for a in host_inputs]
    pout = cuda.alloc(max(out_bytes, 1))
    cuda.run(l, dev + [pout])
    flag = cuda.overflow()
    cuda.sync()
    got = cuda.download(pout, out_bytes)
    for p in dev + [pout]:
        cuda.free(p)
    want = np.full(out_bytes, 0xA5, dtype=np.uint8)
    oflag = oracle.run(l, [np.ascontiguousarray(a) for a in host_inputs] + [want])
    return got, want, 1 if flag else 0, oflag


UNARY = [abi.NEG, abi.EXP, abi.LOG, abi.TANH, abi.SQRT, abi.SIN, abi.COS, abi.ABS, abi.GELU, abi.GELU_DERIV, abi.RELU, abi.HEAVISIDE, abi.SIGN, abi.SIGMOID, abi.REAL]


@pytest.mark.parametrize("prim", UNARY)
def test_unary_primitives_bit_exact_on_many_inputs(cuda, oracle, prim):
    rng = np.random.default_rng(prim)
    n = 1 << 20
    x = np.concatenate([
        rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32).view(np.float32),
        rng.uniform(-100, 100, size=n).astype(np.float32),
        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.0, -1.0, 88.7, -104.0], np.float32),
    ])
    if prim in (abi.SIN, abi.COS):
        x = x[np.abs(x) < 4e8]  # beyond 2^28·π/2 the executor declines (reported, never wrong)
    x = np.ascontiguousarray(x[: (x.size // 8) * 8 + 1])  # an odd length: the scalar kernel
    for count in (x.size, (x.size // 8) * 8):
        l = launch_desc(abi.OP_FUSED, abi.F32, [count])
        l.n_inputs, l.n_steps = 1, 1
        l.steps[0].prim, l.steps[0].nargs, l.steps[0].src[0] = prim, 1, 0
        set_operand(l.inputs[0], abi.F32, [count], [0])
        set_operand(l.out, abi.F32, [count], [0])
        got, want, _, _ = run_both(cuda, oracle, l, [x[:count]], count * 4)
        a, b = got.view(np.uint32), want.view(np.uint32)
        nan = np.isnan(got.view(np.float32)) & np.isnan(want.view(np.float32))
        bad = np.nonzero((a != b) & ~nan)[0]
        assert bad.size == 0, f"{bad.size} differ; x={x[bad[0]]!r}: {a[bad[0]]:#x} vs {b[bad[0]]:#x}"


@pytest.mark.parametrize("prim", [abi.ADD, abi.SUB, abi.MUL, abi.DIV, abi.MAX, abi.MIN])
def test_binary_primitives_with_broadcast(cuda, oracle, prim):
    rng = np.random.default_rng(prim + 50)
    a = rng.standard_normal((6, 5, 24)).astype(np.float32)
    b = rng.standard_normal((5, 1)).astype(np.float32)  # broadcast over the first and the last axis
    a.ravel()[:7] = [0.0, -0.0, np.inf, -np.inf, 1e-45, -1e-45, 3.0]
    l = launch_desc(abi.OP_FUSED, abi.F32, [6, 5, 24])
    l.n_inputs, l.n_steps = 2, 1
    l.steps[0].prim, l.steps[0].nargs, l.steps[0].src[0], l.steps[0].src[1] = prim, 2, 0, 1
    set_operand(l.inputs[0], abi.F32, [6, 5, 24], [0, 1, 2])
    set_operand(l.inputs[1], abi.F32, [5], [1])
    set_operand(l.out, abi.F32, [6, 5, 24], [0, 1, 2])
    got, want, _, _ = run_both(cuda, oracle, l, [a, b], a.size * 4)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("to", [abi.F32, abi.BF16, abi.F16, abi.E8M15, abi.E4M3])
@pytest.mark.parametrize("frm", [abi.F32, abi.F64, abi.BF16, abi.F16, abi.E8M15])
def test_conversions_of_every_storage_format(cuda, oracle, frm, to):
    rng = np.random.default_rng(frm * 10 + to)
    n = 1 << 18
    if frm == abi.F64:
        src = np.concatenate([rng.standard_normal(n) * 10.0 ** rng.integers(-42, 39, n), [1.0 + 2.0**-11 + 2.0**-40, 65519.999, 65520.0, 1e-50, 1e300, np.inf, -np.inf, 0.0, -0.0]])
    else:
        f = rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32).view(np.float32)
        f = f[~np.isnan(f)]  # payloads of NaNs are compared in the CPU suite; here numbers and infinities
        src = f if frm == abi.F32 else np.frombuffer(oracle.convert(f, frm).tobytes(), dtype=np.uint8)
    count = src.size if frm in (abi.F32, abi.F64) else src.size // abi.DTYPE_BYTES[frm]
    l = launch_desc(abi.OP_CONVERT, to, [count])
    l.n_inputs = 1
    set_operand(l.inputs[0], frm, [count], [0])
    set_operand(l.out, to, [count], [0])
    got, want, gf, of = run_both(cuda, oracle, l, [np.ascontiguousarray(src)], count * abi.DTYPE_BYTES[to])
    assert np.array_equal(got, want)
    assert gf == of


@pytest.mark.parametrize("order", [abi.ORDER_SEQUENTIAL, abi.ORDER_DEVICE])
@pytest.mark.parametrize("shape,axis", [((7, 33), 1), ((4, 2048), 1), ((3, 5, 64), 1), ((16, 4096), 1), ((5, 0), 1), ((9, 1), 1)])
def test_reduce_axis(cuda, oracle, shape, axis, order):
    rng = np.random.default_rng(11)
    x = rng.standard_normal(shape).astype(np.float32)
    outer = [d for i, d in enumerate(shape) if i != axis]
    for kind in (abi.REDUCE_SUM, abi.REDUCE_MEAN):
        l = launch_desc(abi.OP_REDUCE, abi.F32, outer, [shape[axis]], order=order)
        l.n_inputs, l.kind = 1, kind
        l.iparam[0] = shape[axis]
        pos = []
        o = 0
        for i in range(len(shape)):
            if i == axis:
                pos.append(len(outer))
            else:
                pos.append(o)
                o += 1
        set_operand(l.inputs[0], abi.F32, list(shape), pos)
        set_operand(l.out, abi.F32, outer, list(range(len(outer))))
        nout = int(np.prod(outer))
        got, want, _, _ = run_both(cuda, oracle, l, [x], nout * 4)
        g, w = got.view(np.float32), want.view(np.float32)
        if order == abi.ORDER_SEQUENTIAL:
            # the mean of no element is 0/0: a NaN whose sign is the machine's
            both_nan = np.isnan(g) & np.isnan(w)
            assert np.array_equal(got.view(np.uint32)[~both_nan], want.view(np.uint32)[~both_nan])
        else:
            np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-5, equal_nan=True)


@pytest.mark.parametrize("dtype", [abi.F32, abi.BF16])
@pytest.mark.parametrize("order", [abi.ORDER_SEQUENTIAL, abi.ORDER_DEVICE])
@pytest.mark.parametrize("masked", [0, 1, 2])
@pytest.mark.parametrize("rows,n", [(5, 8), (64, 256), (33, 2048), (3, 40), (2, 1)])
def test_softmax(cuda, oracle, rows, n, masked, order, dtype):
    """masked: 0 no mask, 1 a random mask with an empty row, 2 the causal mask a `causal_mask` launch wrote."""
    rng = np.random.default_rng(rows * 31 + n)
    if masked == 2:
        rows = n
    x32 = (rng.standard_normal((2, rows, n)) * 4).astype(np.float32)
    x = x32 if dtype == abi.F32 else np.frombuffer(oracle.convert(x32, dtype).tobytes(), dtype=np.uint16).reshape(x32.shape)
    l = launch_desc(abi.OP_SOFTMAX, dtype, [2, rows], [n], order=order)
    l.n_inputs, l.masked = (2 if masked else 1), (1 if masked else 0)
    set_operand(l.inputs[0], dtype, [2, rows, n], [0, 1, 2])
    set_operand(l.out, dtype, [2, rows, n], [0, 1, 2])
    ins = [x]
    dev_mask = None
    if masked == 1:
        m = (rng.uniform(size=(rows, n)) < 0.7).astype(np.int64)
        m[0, :] = 0  # a row the mask empties gives zeros
        set_operand(l.inputs[1], abi.I64, [rows, n], [1, 2], is_index=True)
        ins.append(m)
    elif masked == 2:
        m = np.tril(np.ones((n, n), np.int64))
        set_operand(l.inputs[1], abi.I64, [n, n], [1, 2], is_index=True)
        ins.append(m)
    nbytes = x.size * abi.DTYPE_BYTES[dtype]
    if masked == 2:
        # let the executor write the mask itself, so that it knows it for the causal one
        lm = launch_desc(abi.OP_IOTA, abi.F32, [n, n])
        lm.kind = abi.IOTA_CAUSAL
        set_operand(lm.out, abi.I64, [n, n], [0, 1], is_index=True)
        dev_mask = cuda.alloc(n * n * 8)
        cuda.run(lm, [dev_mask])
        px, pout = cuda.upload(x), cuda.alloc(nbytes)
        cuda.run(l, [px, dev_mask, pout])
        cuda.sync()
        got = cuda.download(pout, nbytes)
        assert np.array_equal(cuda.download(dev_mask, n * n * 8).view(np.int64).reshape(n, n), m)
        for p in (px, pout, dev_mask):
            cuda.free(p)
        want = np.zeros(nbytes, np.uint8)
        oracle.run(l, [x, m, want])
    else:
        got, want, _, _ = run_both(cuda, oracle, l, ins, nbytes)
    if order == abi.ORDER_SEQUENTIAL:
        assert np.array_equal(got, want)
    else:
        g = oracle.widen(got, dtype, x.size)
        w = oracle.widen(want, dtype, x.size)
        # the row's sum is a tree, not a chain: its last bits differ, by a relative 2048·2^-24 at the very most
        tol = 3e-5 if dtype == abi.F32 else 2.0**-8
        assert np.abs(g - w).max() <= tol * max(float(w.max()), 1e-3)


@pytest.mark.parametrize("order", [abi.ORDER_SEQUENTIAL, abi.ORDER_DEVICE])
@pytest.mark.parametrize("rows,v", [(64, 10), (16, 1000), (8, 32000), (3, 65)])
def test_cross_entropy(cuda, oracle, rows, v, order):
    rng = np.random.default_rng(v)
    x = (rng.standard_normal((rows, v)) * 3).astype(np.float32)
    y = rng.integers(0, v, size=(rows,), dtype=np.int64)
    l = launch_desc(abi.OP_XENT, abi.F32, [rows], [v], order=order)
    l.n_inputs = 2
    set_operand(l.inputs[0], abi.F32, [rows, v], [0, 1])
    set_operand(l.inputs[1], abi.I64, [rows], [0], is_index=True)
    set_operand(l.out, abi.F32, [rows], [0])
    got, want, _, _ = run_both(cuda, oracle, l, [x, y], rows * 4)
    if order == abi.ORDER_SEQUENTIAL:
        assert np.array_equal(got, want)
    else:
        # z is a sum of v terms: a chain and a tree differ by up to ~v·2^-24 relative, and ln z by as much absolutely
        np.testing.assert_allclose(got.view(np.float32), want.view(np.float32), rtol=3e-5, atol=3e-5)


def test_embed_and_argmax(cuda, oracle):
    rng = np.random.default_rng(12)
    for d in (24, 30):
        table = rng.standard_normal((50, d)).astype(np.float32)
        ids = rng.integers(0, 50, size=(3, 7), dtype=np.int64)
        l = launch_desc(abi.OP_EMBED, abi.F32, [3, 7, d])
        l.n_inputs = 2
        l.iparam[0] = 50
        l.inputs[0].dtype, l.inputs[0].numel = abi.F32, table.size
        l.inputs[0].stride[0], l.inputs[0].stride[1] = d, 1
        set_operand(l.inputs[1], abi.I64, [3, 7], [0, 1], is_index=True)
        set_operand(l.out, abi.F32, [3, 7, d], [0, 1, 2])
        got, want, _, _ = run_both(cuda, oracle, l, [table, ids], 3 * 7 * d * 4)
        assert np.array_equal(got, want)
        assert np.array_equal(got.view(np.float32).reshape(3, 7, d), table[ids])
    x = rng.integers(0, 4, size=(9, 17)).astype(np.float32)  # many ties: the last maximum wins
    l = launch_desc(abi.OP_ARGMAX, abi.F32, [9], [17])
    l.n_inputs = 1
    set_operand(l.inputs[0], abi.F32, [9, 17], [0, 1])
    set_operand(l.out, abi.I64, [9], [0], is_index=True)
    got, want, _, _ = run_both(cuda, oracle, l, [x], 9 * 8)
    assert np.array_equal(got, want)
    assert np.array_equal(got.view(np.int64), 16 - np.argmax(x[:, ::-1], axis=1))


def test_contraction_exact_generic_strides(cuda, oracle):
    """A generic `ein` with permuted operands, and a matrix product with ragged edges: bit-exact."""
    rng = np.random.default_rng(13)
    # out[b, g, s, h] = sum_m x[b, s, m] * w[m, g, h]   (llama's key projection)
    B, S, M, G, H = 2, 9, 20, 3, 5
    x = rng.standard_normal((B, S, M)).astype(np.float32)
    w = rng.standard_normal((M, G, H)).astype(np.float32)
    l = launch_desc(abi.OP_CONTRACT, abi.F32, [B, G, S, H], [M])
    l.n_inputs = 2
    set_operand(l.inputs[0], abi.F32, [B, S, M], [0, 2, 4])
    set_operand(l.inputs[1], abi.F32, [M, G, H], [4, 1, 3])
    set_operand(l.out, abi.F32, [B, G, S, H], [0, 1, 2, 3])
    got, want, _, _ = run_both(cuda, oracle, l, [x, w], B * G * S * H * 4)
    assert np.array_equal(got, want)
    np.testing.assert_allclose(got.view(np.float32).reshape(B, G, S, H), np.einsum("bsm,mgh->bgsh", x, w), rtol=1e-5, atol=1e-5)
    # an outer product: no summed axis
    a, b = rng.standard_normal(13).astype(np.float32), rng.standard_normal(6).astype(np.float32)
    l = launch_desc(abi.OP_CONTRACT, abi.F32, [13, 6], [])
    l.n_inputs = 2
    set_operand(l.inputs[0], abi.F32, [13], [0])
    set_operand(l.inputs[1], abi.F32, [6], [1])
    set_operand(l.out, abi.F32, [13, 6], [0, 1])
    got, want, _, _ = run_both(cuda, oracle, l, [a, b], 13 * 6 * 4)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("order", [abi.ORDER_SEQUENTIAL, abi.ORDER_DEVICE])
@pytest.mark.parametrize("dtype", [abi.BF16, abi.F32])
def test_float_sums_into_a_scaled_site(cuda, oracle, dtype, order):
    """A contraction that sums in floats and stores into a `scaled` site (exec.rs:758-782 stores any kernel's value
    through its output's format): the binary32 sum of the index-order nest, stored as clamp(rne(x / s) + z). The
    oracle's codes, every one, under both orders (the executor runs the index-order nest for it whatever the order);
    i8 without and u8 with a zero point, a scale that saturates some of them, two summed axes."""
    rng = np.random.default_rng(int(dtype) * 2 + int(order))
    B, S, M, N = 3, 17, 40, 24
    x = rng.standard_normal((B, S, 5, M // 5)).astype(np.float32)
    w = rng.standard_normal((5, M // 5, N)).astype(np.float32)
    if dtype == abi.BF16:
        x, w = bf16_of(oracle, x), bf16_of(oracle, w)
    for kind, zero, scale in ((1, 0, 0.11), (2, 131, 0.05), (1, -7, 0.02)):
        l = launch_desc(abi.OP_CONTRACT, dtype, [B, S, N], [5, M // 5], order=order)
        l.n_inputs = 2
        set_operand(l.inputs[0], dtype, [B, S, 5, M // 5], [0, 1, 3, 4])
        set_operand(l.inputs[1], dtype, [5, M // 5, N], [3, 4, 2])
        set_operand(l.out, abi.U8 if kind == 2 else abi.I8, [B, S, N], [0, 1, 2])
        l.out.affine, l.out.affine_zero, l.out.affine_scale = kind, zero, scale
        got, want, _, _ = run_both(cuda, oracle, l, [x, w], B * S * N)
        assert np.array_equal(got, want), (kind, zero, scale, np.nonzero(got != want)[0][:5])
        codes = want.view(np.uint8 if kind == 2 else np.int8)
        assert len(np.unique(codes)) > 20
        if scale <= 0.05:
            assert (codes == codes.max()).sum() > 1 and int(codes.max()) == (255 if kind == 2 else 127)


def test_integer_sums_over_scaled_values_are_exact(cuda, oracle):
    """`product: i32, accum: i32`: affine activations times int8 weights summed in 32 bits that wrap,
    stored once from the exact value into f16, bf16, f32, e8m15 or an affine format: the bits of
    exact arithmetic written out in Python integers (tests/exact.py), 120 random trials."""
    import w8a8_cases
    rng = np.random.default_rng(0x180004)
    for trial in range(120):
        l, ins, sw, out_bytes, view, want = w8a8_cases.make_case(rng, trial)
        dev = [cuda.upload(a) for a in ins]
        pout, psw = cuda.alloc(out_bytes), cuda.upload(sw)
        cuda.run(l, dev + [pout, psw])
        cuda.overflow()
        cuda.sync()
        got = w8a8_cases.decode(cuda.download(pout, out_bytes), view, *want.shape)
        for p in dev + [pout, psw]:
            cuda.free(p)
        assert np.array_equal(got, want), f"trial {trial}"


def bf16_of(oracle, x):
    return np.frombuffer(oracle.convert(np.ascontiguousarray(x, np.float32), abi.BF16).tobytes(), dtype=np.uint16).reshape(x.shape)


def bf16_value(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("online", [0, 1, 2])
@pytest.mark.parametrize("B,G,P,T,causal", [(2, 2, 2, 384, True), (1, 3, 1, 256, True), (1, 1, 2, 128, False), (1, 2, 1, 1024, True), (1, 2, 1, 512, False)])
def test_blockwise_attention_against_its_four_launches(cuda, oracle, B, G, P, T, causal, online):
    """PSK_OP_ATTENTION under the device order (one tcgen05 kernel, scores never stored) against the
    oracle's four launches with bf16 sites. Tolerance: the result is a bf16 number of magnitude up to
    max|v|; the fused kernel rounds the unnormalised exponentials where the four launches round the
    normalised ones, so an element may differ by a couple of bf16 units (2^-8 relative each).
    `online` = 1, 2: the one-pass kernel (`attention: online`, iparam[0] = 1), which takes the exponentials against
    a running reference maximum and does not round the scores in between; 2 makes the keys grow along the
    sequence so that rows' maxima keep rising and the accumulator in tensor memory is rescaled many times.
    Its tolerance is stated further down, against float64 first: the roundings it leaves out are the four launches'
    own distance from the exact attention."""
    HD = 128
    rng = np.random.default_rng(B * 1000 + T)
    q = bf16_of(oracle, rng.standard_normal((B, G, P, T, HD)) * 1.5)
    kf = rng.standard_normal((B, G, T, HD)) * 1.5
    if online == 2:
        kf = kf * (0.25 + 3.0 * np.arange(T)[None, None, :, None] / T)
    k = bf16_of(oracle, kf)
    v = bf16_of(oracle, rng.standard_normal((B, T, G, HD)))
    rt = bf16_of(oracle, np.array(np.sqrt(np.float32(HD)), np.float32).reshape(()))
    l = launch_desc(abi.OP_ATTENTION, abi.BF16, [B, G, P, T, HD], [T], order=abi.ORDER_DEVICE, name=b"attention[blockwise]")
    l.n_inputs = 5 if causal else 4
    l.masked = 1 if causal else 0
    l.iparam[0] = 1 if online else 0
    l.iparam[1] = l.iparam[2] = l.iparam[3] = abi.BF16
    set_operand(l.inputs[0], abi.BF16, [B, G, P, T, HD], [0, 1, 2, 3, 4])
    set_operand(l.inputs[1], abi.BF16, [B, G, T, HD], [0, 1, 5, 4])
    set_operand(l.inputs[2], abi.BF16, [B, T, G, HD], [0, 5, 1, 4])
    set_operand(l.inputs[3], abi.BF16, [], [])
    set_operand(l.out, abi.BF16, [B, T, G, P, HD], [0, 3, 1, 2, 4])
    host_in = [q, k, v, rt]
    dev = [cuda.upload(a) for a in host_in]
    if causal:
        set_operand(l.inputs[4], abi.I64, [T, T], [3, 5], is_index=True)
        mask_dev = cuda.alloc(T * T * 8)
        m = launch_desc(abi.OP_IOTA, abi.BF16, [T, T], name=b"causal_mask seq")
        m.kind = abi.IOTA_CAUSAL
        set_operand(m.out, abi.I64, [T, T], [0, 1], is_index=True)
        cuda.run(m, [mask_dev])
        dev.append(mask_dev)
        host_in.append(np.tril(np.ones((T, T), np.int64)))
    out_bytes = B * T * G * P * HD * 2
    pout = cuda.alloc(out_bytes)
    cuda.set_profiling(True)
    cuda.run(l, dev + [pout])
    cuda.sync()
    assert [rec[0] for rec in cuda.profile()] == ["k_attn_fwd3" if online else "k_attn_fwd"]
    cuda.set_profiling(False)
    got = bf16_value(cuda.download(pout, out_bytes).view(np.uint16))
    for p in dev + [pout]:
        cuda.free(p)
    want_b = np.zeros(out_bytes, np.uint8)
    oracle.run(l, [np.ascontiguousarray(a) for a in host_in] + [want_b])
    want = bf16_value(want_b.view(np.uint16))
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    # against the exact statement in f64 over the same bf16 inputs
    qf, kf, vf = bf16_value(q).astype(np.float64), bf16_value(k).astype(np.float64), bf16_value(v).astype(np.float64)
    s = np.einsum("bgpsh,bgth->bgpst", qf, kf) / np.sqrt(HD)
    if causal:
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
    a = np.exp(s - s.max(-1, keepdims=True))
    a /= a.sum(-1, keepdims=True)
    exact = np.einsum("bgpst,btgh->bsgph", a, vf).reshape(-1)
    exact_err = np.abs(got - exact)
    if not online:
        assert err.max() <= 2.0**-6 * np.abs(want).max(), (err.max(), np.abs(want).max())
        assert err.mean() <= 2.0**-8 * np.abs(want).mean(), (err.mean(), np.abs(want).mean())  # on average well within one bf16 unit of an element
        assert exact_err.max() <= 0.03 * np.abs(exact).max()
    else:
        # The one-pass kernel leaves out the four launches' roundings of the scores (bf16 of a score of up to 75 here
        # moves it by up to 0.15, and the scaled score's by another 0.016: an exponential by a few percent), so it is
        # NEARER the exact attention than they are and further from them than the two-pass kernel, which repeats
        # those roundings. Stated for each: within 2^-7 of the scale of the exact result (its own roundings: P and
        # the output to bf16), and of the four launches within what they themselves are of the exact result.
        oracle_err = np.abs(want - exact)
        assert exact_err.max() <= 2.0**-7 * np.abs(exact).max(), (exact_err.max(), np.abs(exact).max())
        assert exact_err.mean() <= 1.25 * oracle_err.mean() + 2.0**-10 * np.abs(exact).mean(), (exact_err.mean(), oracle_err.mean())
        assert err.max() <= 1.5 * oracle_err.max() + 2.0**-7 * np.abs(exact).max(), (err.max(), oracle_err.max())
        assert err.mean() <= 1.5 * oracle_err.mean() + 2.0**-9 * np.abs(exact).mean(), (err.mean(), oracle_err.mean())


@pytest.mark.parametrize("B,G,P,T2", [(2, 2, 2, 1), (1, 2, 1, 7), (3, 2, 4, 1000), (1, 1, 2, 13001)])
def test_one_position_against_a_cache(cuda, oracle, B, G, P, T2):
    """PSK_OP_ATTENTION with seq = 1 and no mask (a decode step: `k_attn_step`) against the oracle's four launches.
    The kernel keeps their three roundings (score, scaled score and normalised weight to bf16) and their exp; only
    the order of the three sums differs, so the result is within a bf16 unit or two of an element: 2^-7 of the
    result's scale at most, 2^-9 of the mean magnitude on average. Cache lengths of one position, of a few, of a
    thousand and of more than fit the default 48 KB of shared memory; keys and values strided as a cache holds them
    (a view of the first T2 positions of a longer buffer)."""
    HD, TMAX = 128, T2 + 5
    rng = np.random.default_rng(T2)
    q = bf16_of(oracle, rng.standard_normal((B, G, P, 1, HD)) * 1.5)
    kbuf = bf16_of(oracle, rng.standard_normal((B, G, TMAX, HD)) * 1.5)
    vbuf = bf16_of(oracle, rng.standard_normal((B, TMAX, G, HD)))
    rt = bf16_of(oracle, np.array(np.sqrt(np.float32(HD)), np.float32).reshape(()))
    l = launch_desc(abi.OP_ATTENTION, abi.BF16, [B, G, P, 1, HD], [T2], order=abi.ORDER_DEVICE, name=b"attention[online]")
    l.n_inputs, l.masked = 4, 0
    l.iparam[0] = 1
    l.iparam[1] = l.iparam[2] = l.iparam[3] = abi.BF16
    set_operand(l.inputs[0], abi.BF16, [B, G, P, 1, HD], [0, 1, 2, 3, 4])
    # the cache's views: the buffers' strides, T2 of their TMAX positions
    for op, strides, n in ((l.inputs[1], {0: G * TMAX * HD, 1: TMAX * HD, 5: HD, 4: 1}, B * G * TMAX * HD), (l.inputs[2], {0: TMAX * G * HD, 5: G * HD, 1: HD, 4: 1}, B * TMAX * G * HD)):
        op.dtype, op.numel = abi.BF16, n
        for ax, st in strides.items():
            op.stride[ax] = st
    set_operand(l.inputs[3], abi.BF16, [], [])
    set_operand(l.out, abi.BF16, [B, 1, G, P, HD], [0, 3, 1, 2, 4])
    host_in = [q, kbuf, vbuf, rt]
    dev = [cuda.upload(a) for a in host_in]
    out_bytes = B * G * P * HD * 2
    pout = cuda.alloc(out_bytes)
    cuda.set_profiling(True)
    cuda.run(l, dev + [pout])
    cuda.sync()
    assert [rec[0] for rec in cuda.profile()] == ["k_attn_step"]
    cuda.set_profiling(False)
    got = bf16_value(cuda.download(pout, out_bytes).view(np.uint16))
    for p_ in dev + [pout]:
        cuda.free(p_)
    want_b = np.zeros(out_bytes, np.uint8)
    oracle.run(l, [np.ascontiguousarray(a) for a in host_in] + [want_b])
    want = bf16_value(want_b.view(np.uint16))
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    assert err.max() <= 2.0**-7 * np.abs(want).max(), (err.max(), np.abs(want).max())
    assert err.mean() <= 2.0**-9 * np.abs(want).mean(), (err.mean(), np.abs(want).mean())
    if T2 == 1:  # one position: its weight is 1 and the result is that position's values, exactly
        assert np.array_equal(got.reshape(B, G, P, HD), np.broadcast_to(bf16_value(vbuf[:, 0])[:, :, None, :], (B, G, P, HD)))


@pytest.mark.parametrize("B,G,P,T,T2,kind,zero,shrink", [(1, 2, 2, 256, 256, 1, 0, 1.0), (2, 1, 1, 384, 384, 2, 131, 0.6), (2, 2, 2, 1, 777, 1, 0, 1.0), (1, 1, 4, 1, 40, 2, 120, 0.5)])
def test_attention_into_a_scaled_site(cuda, oracle, B, G, P, T, T2, kind, zero, shrink):
    """The weighted values stored as one-byte codes of an affine format (a `scaled` site: the W8A8 out-projection's
    operand): the one-pass kernel over a window (causal) and the decode step's kernel over a cache, each writing
    clamp(rne(x / s) + z) of its binary32 result x as the oracle's last launch stores its sum (the one-pass kernel
    takes the quotient by a reciprocal, a few binary32 units off: inside its tolerance). `shrink` < 1 makes
    the scale too small for the largest values, so that codes saturate at both ends. Stated against the exact
    attention in f64: a decoded code is within half a step plus the kernel's own distance (2^-7 of the scale, as for
    the bf16 result), or saturated where the exact value is past the format's end; and against the oracle's codes,
    which differ by what its bf16 roundings of the scores move a value."""
    HD = 128
    rng = np.random.default_rng(T * 31 + T2 + kind)
    step = T == 1
    q = bf16_of(oracle, rng.standard_normal((B, G, P, T, HD)) * 1.5)
    k = bf16_of(oracle, rng.standard_normal((B, G, T2, HD)) * 1.5)
    v = bf16_of(oracle, rng.standard_normal((B, T2, G, HD)))
    rt = bf16_of(oracle, np.array(np.sqrt(np.float32(HD)), np.float32).reshape(()))
    qf, kf, vf = bf16_value(q).astype(np.float64), bf16_value(k).astype(np.float64), bf16_value(v).astype(np.float64)
    sc = np.einsum("bgpsh,bgth->bgpst", qf, kf) / np.sqrt(HD)
    if not step:
        sc = np.where(np.tril(np.ones((T, T), bool)), sc, -np.inf)
    a = np.exp(sc - sc.max(-1, keepdims=True))
    a /= a.sum(-1, keepdims=True)
    exact = np.einsum("bgpst,btgh->bsgph", a, vf).reshape(-1)
    lo, hi = (0, 255) if kind == 2 else (-128, 127)
    scale = np.float32(np.abs(exact).max() / 127.0 * shrink)
    l = launch_desc(abi.OP_ATTENTION, abi.BF16, [B, G, P, T, HD], [T2], order=abi.ORDER_DEVICE, name=b"attention[online]")
    l.n_inputs = 4 if step else 5
    l.masked = 0 if step else 1
    l.iparam[0] = 1
    l.iparam[1] = l.iparam[2] = l.iparam[3] = abi.BF16
    set_operand(l.inputs[0], abi.BF16, [B, G, P, T, HD], [0, 1, 2, 3, 4])
    set_operand(l.inputs[1], abi.BF16, [B, G, T2, HD], [0, 1, 5, 4])
    set_operand(l.inputs[2], abi.BF16, [B, T2, G, HD], [0, 5, 1, 4])
    set_operand(l.inputs[3], abi.BF16, [], [])
    set_operand(l.out, abi.U8 if kind == 2 else abi.I8, [B, T, G, P, HD], [0, 3, 1, 2, 4])
    l.out.affine, l.out.affine_zero, l.out.affine_scale = kind, zero, float(scale)
    host_in = [q, k, v, rt]
    dev = [cuda.upload(x) for x in host_in]
    if not step:
        set_operand(l.inputs[4], abi.I64, [T, T], [3, 5], is_index=True)
        mask_dev = cuda.alloc(T * T * 8)
        m = launch_desc(abi.OP_IOTA, abi.BF16, [T, T], name=b"causal_mask seq")
        m.kind = abi.IOTA_CAUSAL
        set_operand(m.out, abi.I64, [T, T], [0, 1], is_index=True)
        cuda.run(m, [mask_dev])
        dev.append(mask_dev)
        host_in.append(np.tril(np.ones((T, T), np.int64)))
    out_bytes = B * T * G * P * HD
    pout = cuda.alloc(out_bytes)
    cuda.set_profiling(True)
    cuda.run(l, dev + [pout])
    cuda.sync()
    assert [rec[0] for rec in cuda.profile()] == ["k_attn_step" if step else "k_attn_fwd3"]
    cuda.set_profiling(False)
    code_type = np.uint8 if kind == 2 else np.int8
    got = cuda.download(pout, out_bytes).view(code_type).astype(np.int64)
    for p_ in dev + [pout]:
        cuda.free(p_)
    want_b = np.zeros(out_bytes, np.uint8)
    oracle.run(l, [np.ascontiguousarray(x) for x in host_in] + [want_b])
    want = want_b.view(code_type).astype(np.int64)
    s64 = float(scale)
    slack = 2.0**-7 * np.abs(exact).max()
    ideal = exact / s64 + zero  # the exact value on the codes' axis
    inside = (ideal > lo) & (ideal < hi)
    assert np.all(np.abs(got - ideal)[inside] <= 0.5 + slack / s64 + 1e-6), np.abs(got - ideal)[inside].max()
    assert np.all(got[ideal >= hi + 0.5 + slack / s64] == hi) and np.all(got[ideal <= lo - 0.5 - slack / s64] == lo)
    if shrink < 1.0:
        assert (got == hi).any() and (got == lo).any()
    oracle_off = np.abs(np.clip(ideal, lo, hi) - want).max()  # the four launches' own distance, in steps
    diff = np.abs(got - want)
    assert diff.max() <= oracle_off + 0.5 + slack / s64 + 1e-6, (diff.max(), oracle_off)
    assert diff.mean() <= 0.6, diff.mean()
    assert (diff == 0).mean() >= (0.9 if step else 0.4), (diff == 0).mean()  # (the step's kernel keeps the launches' roundings)


def test_blockwise_attention_is_refused_where_it_does_not_apply(cuda):
    """Under the sequential order, or with a head dimension other than 128, the launch is refused with
    E7005 and nothing runs: the host then keeps the four launches apart."""
    from presk_b200 import PreskError
    B, G, P, T, HD = 1, 1, 1, 128, 64
    for order, hd in ((abi.ORDER_SEQUENTIAL, 128), (abi.ORDER_DEVICE, 64)):
        l = launch_desc(abi.OP_ATTENTION, abi.BF16, [B, G, P, T, hd], [T], order=order, name=b"attention[blockwise]")
        l.n_inputs = 4
        l.iparam[1] = l.iparam[2] = l.iparam[3] = abi.BF16
        set_operand(l.inputs[0], abi.BF16, [B, G, P, T, hd], [0, 1, 2, 3, 4])
        set_operand(l.inputs[1], abi.BF16, [B, G, T, hd], [0, 1, 5, 4])
        set_operand(l.inputs[2], abi.BF16, [B, T, G, hd], [0, 5, 1, 4])
        set_operand(l.inputs[3], abi.BF16, [], [])
        set_operand(l.out, abi.BF16, [B, T, G, P, hd], [0, 3, 1, 2, 4])
        bufs = [cuda.alloc(T * hd * 2) for _ in range(3)] + [cuda.alloc(16), cuda.alloc(T * hd * 2)]
        with pytest.raises(PreskError) as e:
            cuda.run(l, bufs)
        assert e.value.code == 7005
        for p in bufs:
            cuda.free(p)


@pytest.mark.parametrize("with_mul", [False, True])
def test_tabulated_silu_is_the_exact_one(cuda, oracle, with_mul):
    """A bf16 silu group over enough elements is read from a table of all 65 536 codes that the device
    computed with its exact function; with the product by a second operand it is the merged group
    [sigmoid; mul; round to bf16; mul]. Every code occurs in the input, NaNs and infinities included:
    the bits must be the oracle's."""
    rows, cols = 2560, 2048  # 5.2 M elements: above the size from which the table is used
    rng = np.random.default_rng(21)
    g = rng.integers(0, 65536, size=(rows, cols), dtype=np.uint16)
    g.ravel()[:65536] = np.arange(65536, dtype=np.uint16)
    u = bf16_of(oracle, rng.standard_normal((rows, cols)) * 3.0)
    l = launch_desc(abi.OP_FUSED, abi.BF16, [rows, cols])
    if with_mul:
        l.n_inputs, l.n_steps = 2, 4
        steps = [(abi.SIGMOID, 1, 0, 0, 0), (abi.MUL, 2, 0, -1, 0), (abi.ROUND, 1, -2, 0, abi.BF16), (abi.MUL, 2, -3, 1, 0)]
    else:
        l.n_inputs, l.n_steps = 1, 2
        steps = [(abi.SIGMOID, 1, 0, 0, 0), (abi.MUL, 2, 0, -1, 0)]
    for k, (prim, nargs, a, b, imm) in enumerate(steps):
        l.steps[k].prim, l.steps[k].nargs, l.steps[k].src[0], l.steps[k].src[1], l.steps[k].imm = prim, nargs, a, b, imm
    set_operand(l.inputs[0], abi.BF16, [rows, cols], [0, 1])
    if with_mul:
        set_operand(l.inputs[1], abi.BF16, [rows, cols], [0, 1])
    set_operand(l.out, abi.BF16, [rows, cols], [0, 1])
    got, want, _, _ = run_both(cuda, oracle, l, [g, u] if with_mul else [g], rows * cols * 2)
    a, b = got.view(np.uint16), want.view(np.uint16)
    # a NaN is a NaN on both sides; which NaN the hardware's arithmetic makes of one is not the host's choice
    nan = ((a & 0x7fff) > 0x7f80) & ((b & 0x7fff) > 0x7f80)
    bad = np.nonzero((a != b) & ~nan)[0]
    assert bad.size == 0, f"{bad.size} differ; first: code {g.ravel()[bad[0]]:#x}: {a[bad[0]]:#x} vs {b[bad[0]]:#x}"


@pytest.mark.parametrize("kind,zero,scale", [(1, 0, 0.05), (2, 117, 0.0173), (1, -20, 3.0e-3)])
def test_silu_times_up_into_an_affine_site(cuda, oracle, kind, zero, scale):
    """The merged silu group writing a `scaled` site (the down-projection's integer-sum operand): bf16 rows in,
    one-byte codes clamp(rne(x / s) + z) out. The kernel takes the quotient by a reciprocal and sends what lies near
    a tie through the exact routine; every code of `gate` occurs, and `up` is laid out so that many products fall on
    exact ties of the scale. The codes must be the oracle's, every one."""
    rows, cols = 2560, 2048
    rng = np.random.default_rng(kind * 100 + zero + 5)
    g = rng.integers(0, 65536, size=(rows, cols), dtype=np.uint16)
    g.ravel()[:65536] = np.arange(65536, dtype=np.uint16)
    u = rng.standard_normal((rows, cols)) * 3.0
    u[1::7] = 1.0   # silu(g) itself, a bf16 number: quotients by the scale of every kind, ties among them
    u[2::7] = np.float32(scale) * 0.5
    u = bf16_of(oracle, u)
    l = launch_desc(abi.OP_FUSED, abi.BF16, [rows, cols], order=abi.ORDER_DEVICE)
    l.n_inputs, l.n_steps = 2, 4
    steps = [(abi.SIGMOID, 1, 0, 0, 0), (abi.MUL, 2, 0, -1, 0), (abi.ROUND, 1, -2, 0, abi.BF16), (abi.MUL, 2, -3, 1, 0)]
    for k, (prim, nargs, a, b, imm) in enumerate(steps):
        l.steps[k].prim, l.steps[k].nargs, l.steps[k].src[0], l.steps[k].src[1], l.steps[k].imm = prim, nargs, a, b, imm
    set_operand(l.inputs[0], abi.BF16, [rows, cols], [0, 1])
    set_operand(l.inputs[1], abi.BF16, [rows, cols], [0, 1])
    set_operand(l.out, abi.I8 if kind == 1 else abi.U8, [rows, cols], [0, 1])
    l.out.affine, l.out.affine_zero, l.out.affine_scale = kind, zero, scale
    cuda.set_profiling(True)
    got, want, _, _ = run_both(cuda, oracle, l, [g, u], rows * cols)
    assert [rec[0] for rec in cuda.profile()] == ["k_ew_lut_affine"]
    cuda.set_profiling(False)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, f"{bad.size} differ; first: gate {g.ravel()[bad[0]]:#x}, up {u.ravel()[bad[0]]:#x}: {got[bad[0]]} vs {want[bad[0]]}"
    assert len(np.unique(want)) > 100  # the codes spread over the format


@pytest.mark.parametrize("with_mul", [False, True])
def test_division_by_a_row_scalar_is_the_ieee_division(cuda, oracle, with_mul):
    """bf16 rows divided by one f32 value a row (a norm's root, rounded to bf16 at the kernel's edge), then
    optionally scaled by a bf16 vector: the program kernel divides by the reciprocal with one correction.
    Every bf16 code as a numerator against 4 096 divisors of every magnitude: the oracle's bits."""
    rows, cols = 4096, 65536 // 16
    rng = np.random.default_rng(31)
    codes = np.arange(65536, dtype=np.uint16)
    a = np.stack([np.roll(codes, int(s))[:cols] for s in rng.integers(0, 65536, rows)])
    a[:16] = codes.reshape(16, cols)
    div = (rng.standard_normal(rows) * 10.0 ** rng.integers(-30, 30, rows)).astype(np.float32)
    div[:8] = [1.0, -3.0, 11.3125, 2.0**-100, 2.0**100, 1e-38, 3e38, 0.1]
    gamma = bf16_of(oracle, rng.standard_normal(cols) + 1.0)
    l = launch_desc(abi.OP_FUSED, abi.BF16, [rows, cols])
    l.n_inputs, l.n_steps = (3, 2) if with_mul else (2, 1)
    l.steps[0].prim, l.steps[0].nargs, l.steps[0].src[0], l.steps[0].src[1] = abi.DIV, 2, 0, 1
    if with_mul:
        l.steps[1].prim, l.steps[1].nargs, l.steps[1].src[0], l.steps[1].src[1] = abi.MUL, 2, -1, 2
        set_operand(l.inputs[2], abi.BF16, [cols], [1])
    set_operand(l.inputs[0], abi.BF16, [rows, cols], [0, 1])
    set_operand(l.inputs[1], abi.F32, [rows], [0])
    set_operand(l.out, abi.BF16, [rows, cols], [0, 1])
    got, want, _, _ = run_both(cuda, oracle, l, [a, div, gamma] if with_mul else [a, div], rows * cols * 2)
    x, y = got.view(np.uint16), want.view(np.uint16)
    nan = ((x & 0x7fff) > 0x7f80) & ((y & 0x7fff) > 0x7f80)
    bad = np.nonzero((x != y) & ~nan)[0]
    assert bad.size == 0, f"{bad.size} differ; first: {a.ravel()[bad[0]]:#x} / {div[bad[0] // cols]!r}: {x[bad[0]]:#x} vs {y[bad[0]]:#x}"


def test_a_wait_that_runs_out_is_reported_and_the_executor_lives_on(cuda):
    """Every barrier wait in the tensor-core kernels is bounded. A kernel whose only wait cannot be satisfied
    (limited to 2e7 cycles, about 10 ms) gives up, records where, and the host reports E10001; the next launch on the
    same executor runs normally."""
    rc = cuda.lib.psk_exec_wait_selftest(cuda.handle, 20_000_000)
    assert rc == abi.E10001
    assert b"bounded wait ran out" in cuda.lib.psk_last_error(cuda.handle)
    x = np.arange(64, dtype=np.float32)
    l = launch_desc(abi.OP_FUSED, abi.F32, [64])
    l.n_inputs, l.n_steps = 1, 1
    l.steps[0].prim, l.steps[0].nargs, l.steps[0].src[0] = abi.NEG, 1, 0
    set_operand(l.inputs[0], abi.F32, [64], [0])
    set_operand(l.out, abi.F32, [64], [0])
    p, q = cuda.upload(x), cuda.alloc(256)
    cuda.run(l, [p, q])
    cuda.sync()
    assert np.array_equal(cuda.download(q, 256).view(np.float32), -x)
    cuda.free(p)
    cuda.free(q)


@pytest.mark.parametrize("dtype", [abi.F32, abi.BF16])
@pytest.mark.parametrize("rows,v", [(64, 10), (16, 1000), (5, 4099), (3, 65)])
def test_cross_entropy_vjp_bit_exact(cuda, oracle, rows, v, dtype):
    """(softmax(x) - onehot(y)) * ct a row: the maximum and z in index order, every operation rounded; one label
    outside the classes (no class is hot: the comparison of the two integers simply fails)."""
    rng = np.random.default_rng(v + rows)
    x = oracle.convert((rng.standard_normal((rows, v)) * 3).astype(np.float32), dtype)
    ct = oracle.convert(rng.standard_normal(rows).astype(np.float32), dtype)
    y = rng.integers(0, v, size=(rows,), dtype=np.int64)
    y[0] = v + 3
    l = launch_desc(abi.OP_XENT_VJP, dtype, [rows], [v])
    l.n_inputs = 3
    set_operand(l.inputs[0], dtype, [rows, v], [0, 1])
    set_operand(l.inputs[1], abi.I64, [rows], [0], is_index=True)
    set_operand(l.inputs[2], dtype, [rows], [0])
    set_operand(l.out, dtype, [rows, v], [0, 1])
    nbytes = rows * v * abi.DTYPE_BYTES[dtype]
    got, want, _, _ = run_both(cuda, oracle, l, [x, y, ct], nbytes)
    assert np.array_equal(got, want)
    g = oracle.widen(got, dtype, rows * v).reshape(rows, v).astype(np.float64)
    xv = oracle.widen(x, dtype, rows * v).reshape(rows, v).astype(np.float64)
    sm = np.exp(xv - xv.max(1, keepdims=True))
    sm /= sm.sum(1, keepdims=True)
    hot = np.zeros_like(sm)
    hot[np.arange(1, rows), y[1:]] = 1.0
    ref = (sm - hot) * oracle.widen(ct, dtype, rows).astype(np.float64)[:, None]
    assert np.abs(g - ref).max() <= (1e-5 if dtype == abi.F32 else 2.0**-7) * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("dtype", [abi.F32, abi.BF16])
@pytest.mark.parametrize("shape,vocab,d", [((3, 7), 50, 24), ((2, 300), 17, 30), ((1, 1), 5, 8), ((0, 4), 6, 8)])
def test_embed_vjp_bit_exact(cuda, oracle, shape, vocab, d, dtype):
    """The table's gradient: zeros, then one row of the cotangent added per index in index order, the running sum
    kept in the output's type (bf16: rounded after every addition; 600 indices into 17 rows make long chains).
    No index at all still leaves a table of zeros."""
    rng = np.random.default_rng(vocab)
    n = int(np.prod(shape))
    ids = rng.integers(0, vocab, size=shape, dtype=np.int64)
    ct = oracle.convert(rng.standard_normal(shape + (d,)).astype(np.float32), dtype)
    table = np.zeros(vocab * d * abi.DTYPE_BYTES[dtype], np.uint8)
    l = launch_desc(abi.OP_EMBED_VJP, dtype, list(shape) + [d])
    l.n_inputs = 3
    l.iparam[0] = vocab
    l.inputs[0].dtype, l.inputs[0].numel = dtype, vocab * d
    l.inputs[0].stride[0], l.inputs[0].stride[1] = d, 1
    set_operand(l.inputs[1], abi.I64, list(shape), [0, 1], is_index=True)
    set_operand(l.inputs[2], dtype, list(shape) + [d], [0, 1, 2])
    l.out.dtype, l.out.numel = dtype, vocab * d
    l.out.stride[0], l.out.stride[1] = d, 1
    nbytes = vocab * d * abi.DTYPE_BYTES[dtype]
    got, want, _, _ = run_both(cuda, oracle, l, [table, ids, ct if n else np.zeros(1, np.uint8)], nbytes)
    assert np.array_equal(got, want)
    g = oracle.widen(got, dtype, vocab * d).reshape(vocab, d).astype(np.float64)
    ref = np.zeros((vocab, d))
    if n:
        np.add.at(ref, ids.reshape(-1), oracle.widen(ct, dtype, n * d).reshape(n, d).astype(np.float64))
    assert np.abs(g - ref).max() <= (1e-5 if dtype == abi.F32 else 0.1) * max(1.0, np.abs(ref).max())


def test_gap_between_two_results_on_the_device(cuda, oracle):
    """`presk solve --measure`'s gap (presk-driver/src/gap.rs:35-64) without bringing the results back: max |a - b| and
    max |a| in binary64 over exactly widened elements of any two storage types; one element that is not finite
    makes the gap infinite."""
    rng = np.random.default_rng(57)
    n = 1_000_003
    a = rng.standard_normal(n).astype(np.float32)
    b16 = oracle.convert(a, abi.BF16)
    bv = oracle.widen(b16, abi.BF16, n)
    pa, pb = cuda.upload(a), cuda.upload(b16)
    gap, mx = cuda.gap(pa, abi.F32, pb, abi.BF16, n)
    assert gap == float(np.abs(a.astype(np.float64) - bv.astype(np.float64)).max())
    assert mx == float(np.abs(a).astype(np.float64).max())
    a[12345] = np.inf
    cuda.free(pa)
    pa = cuda.upload(a)
    gap, mx = cuda.gap(pa, abi.F32, pb, abi.BF16, n)
    assert gap == np.inf and mx == np.inf
    assert cuda.gap(pa, abi.F32, pb, abi.BF16, 0) == (0.0, 0.0)
    cuda.free(pa)
    cuda.free(pb)
