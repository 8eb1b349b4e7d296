"""Parity at the shapes the throughput number is quoted on.

The other GPU suites compare small models; these run the widths and tile paths of the timed step itself:
  * one Llama layer of the 7B width (d 4096, 32 heads of 128, FFN 11008, vocabulary 32000) under the benchmark's
    realization against the oracle's sequential, unmerged run, with bf16, int8 and e4m3fn weights;
  * the blockwise attention kernel at sequence 2048 with 32 heads against the oracle's four launches on a sample
    of heads;
  * one tensor-core contraction of [16384, 4096] x [4096, 11008] (256-row tiles, panels of 16 tile-columns, the
    last panel narrower) against float64 on sampled rows and every column;
  * the contraction-plus-LayerNorm workload at N = 4096 and 8192 in f16 and e8m15, and the e8m15 store's guard.
"""
import numpy as np
import pytest

import headline
import models
from presk_b200 import Host, PreskError, abi, launch_desc
from test_gpu_ops import bf16_of, bf16_value, set_operand

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def wide_params():
    return headline.llama_params_f32(dict(headline.WIDTH_7B, L=1), seed=0)


@pytest.mark.parametrize("weights", ["bf16", "int8", "e4m3fn"])
def test_one_layer_of_the_7b_width_under_the_benchmarks_realization(cuda, oracle, wide_params, weights):
    """B = 2, T = 256 (512 rows: the 256-row tiles of the contraction kernel), every launch the timed step issues:
    merged norms and rotations, q/k/v/out projections, the blockwise attention kernel, SwiGLU with the tabulated
    silu, residual additions in the contractions' epilogues, the f32 head, cross-entropy and the mean."""
    r = headline.llama_width_parity(cuda, oracle, B=2, T=256, weights=weights, params=wide_params, want_loss=(weights == "bf16"))
    log = r["gpu_launch_log"]
    assert "attention[blockwise]" in log and "rmsnorm[merged]" in log and "rope[merged]" in log and any(n.endswith("+add") for n in log), log
    assert r["finite"]
    tol = headline.LOGITS_TOL * (2.0 if weights != "bf16" else 1.0)  # narrow weights: the scale multiplies a reordered sum once more
    summary = {k: v for k, v in r.items() if k != "gpu_launch_log"}
    assert r["logits_max_err"] <= tol * r["logits_scale"], summary
    assert r["logits_mean_err"] <= headline.LOGITS_MEAN_TOL * (2.0 if weights != "bf16" else 1.0) * r["logits_scale"], summary
    if weights == "bf16":
        assert abs(r["loss_gpu"] - r["loss_oracle"]) <= headline.LOSS_RTOL * abs(r["loss_oracle"]), summary


def test_the_7b_width_under_the_sequential_order_is_the_oracles_bits(cuda, oracle, wide_params):
    """The same layer of the full width (d 4096, FFN 11008, vocabulary 32000), B = 1, T = 128, under the reference's
    own order on both sides: every logit bit for bit, through the exact contraction kernels at their largest tiles."""
    from presk_b200 import Host
    c = dict(headline.WIDTH_7B, L=1)
    rng = np.random.default_rng(9)
    ids = rng.integers(0, c["V"], size=(1, 128), dtype=np.int64)
    outs = []
    for ex in (cuda, oracle.vtable()):
        h = headline.give(Host(ex, headline.realization(wide_params, headline.ORACLE_ORDER)).prepare("llama", **c), wide_params)
        outs.append(h.call("apply", [ids], (1, 128, c["V"])))
        h.close()
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))


@pytest.mark.parametrize("attention", ["online"])
def test_one_layer_of_the_7b_width_with_the_one_pass_attention(cuda, oracle, wide_params, attention):
    """The benchmark's default realization: as above with `attention: online`."""
    r = headline.llama_width_parity(cuda, oracle, B=2, T=256, weights="bf16", params=wide_params, order=dict(headline.BENCH_ORDER, attention=attention))
    summary = {k: v for k, v in r.items() if k != "gpu_launch_log"}
    assert "attention[online]" in r["gpu_launch_log"]
    assert r["finite"]
    assert r["logits_max_err"] <= headline.LOGITS_TOL * r["logits_scale"], summary
    assert r["logits_mean_err"] <= headline.LOGITS_MEAN_TOL * 1.5 * r["logits_scale"], summary
    assert abs(r["loss_gpu"] - r["loss_oracle"]) <= headline.LOSS_RTOL * abs(r["loss_oracle"]), summary


def test_blockwise_attention_at_the_benchmarks_sequence(cuda, oracle):
    """B = 1, 32 heads, T = 2048, hd = 128, causal: the kernel's 16 query blocks a head and up to 32 key blocks a
    row, against the oracle's four launches (scores, division, masked softmax, values; bf16 sites) on three of the
    heads, and against float64 on the same. Tolerance as for the small shapes: the largest difference within
    2^-6 of the result's scale (a couple of bf16 units: the kernel rounds unnormalised exponentials where the
    four launches round normalised ones), the mean difference within 2^-8 of the mean magnitude."""
    B, G, P, T, HD = 1, 32, 1, 2048, 128
    rng = np.random.default_rng(2048)
    q = bf16_of(oracle, rng.standard_normal((B, G, P, T, HD)) * 1.5)
    k = bf16_of(oracle, rng.standard_normal((B, G, T, HD)) * 1.5)
    v = bf16_of(oracle, rng.standard_normal((B, T, G, HD)))
    rt = bf16_of(oracle, np.array(np.sqrt(np.float32(HD)), np.float32).reshape(()))

    def desc(g):
        l = launch_desc(abi.OP_ATTENTION, abi.BF16, [B, g, P, T, HD], [T], order=abi.ORDER_DEVICE, name=b"attention[blockwise]")
        l.n_inputs, l.masked = 5, 1
        l.iparam[1] = l.iparam[2] = l.iparam[3] = abi.BF16
        set_operand(l.inputs[0], abi.BF16, [B, g, P, T, HD], [0, 1, 2, 3, 4])
        set_operand(l.inputs[1], abi.BF16, [B, g, T, HD], [0, 1, 5, 4])
        set_operand(l.inputs[2], abi.BF16, [B, T, g, HD], [0, 5, 1, 4])
        set_operand(l.inputs[3], abi.BF16, [], [])
        set_operand(l.inputs[4], abi.I64, [T, T], [3, 5], is_index=True)
        set_operand(l.out, abi.BF16, [B, T, g, P, HD], [0, 3, 1, 2, 4])
        return l

    l = desc(G)
    dev = [cuda.upload(a) for a in (q, k, v, rt)]
    mask_dev = cuda.alloc(T * T * 8)
    m = launch_desc(abi.OP_IOTA, abi.BF16, [T, T], name=b"causal_mask seq")
    m.kind = abi.IOTA_CAUSAL
    set_operand(m.out, abi.I64, [T, T], [0, 1], is_index=True)
    cuda.run(m, [mask_dev])
    out_bytes = B * T * G * P * HD * 2
    pout = cuda.alloc(out_bytes)
    cuda.run(l, dev + [mask_dev, pout])
    cuda.sync()
    got = bf16_value(cuda.download(pout, out_bytes).view(np.uint16)).reshape(B, T, G, P, HD)
    for p in dev + [mask_dev, pout]:
        cuda.free(p)
    assert np.isfinite(got).all()
    tril = np.tril(np.ones((T, T), np.int64))
    for g in (0, 13, 31):
        q1, k1, v1 = np.ascontiguousarray(q[:, g:g + 1]), np.ascontiguousarray(k[:, g:g + 1]), np.ascontiguousarray(v[:, :, g:g + 1])
        want_b = np.zeros(B * T * P * HD * 2, np.uint8)
        oracle.run(desc(1), [q1, k1, v1, rt, tril, want_b])
        want = bf16_value(want_b.view(np.uint16)).reshape(B, T, 1, P, HD)
        mine = got[:, :, g:g + 1]
        err = np.abs(mine - want)
        assert err.max() <= 2.0**-6 * np.abs(want).max(), (g, err.max(), np.abs(want).max())
        assert err.mean() <= 2.0**-8 * np.abs(want).mean(), (g, err.mean(), np.abs(want).mean())
        qf, kf, vf = bf16_value(q1).astype(np.float64), bf16_value(k1).astype(np.float64), bf16_value(v1).astype(np.float64)
        s = np.einsum("bgpsh,bgth->bgpst", qf, kf) / np.sqrt(HD)
        s = np.where(tril.astype(bool), s, -np.inf)
        a = np.exp(s - s.max(-1, keepdims=True))
        a /= a.sum(-1, keepdims=True)
        exact = np.einsum("bgpst,btgh->bsgph", a, vf)
        assert np.abs(mine - exact).max() <= 0.03 * np.abs(exact).max()


@pytest.mark.parametrize("addend", [False, True])
def test_the_ffn_contraction_of_the_timed_step(cuda, oracle, addend):
    """x[16384, 4096] · w[4096, 11008] as the step's gate and up projections issue it (w read as stored, n
    contiguous; bf16 result): 64 x 43 tiles of 256 x 256, handed out in panels of 16 tile-columns, the last of 11.
    With `addend`: down-projection shape [16384, 11008] · [11008, 4096] plus a residual in the epilogue
    (PSK_OP_CONTRACT_ADD). 96 sampled rows (first and last tiles among them) against float64 on the exactly
    widened operands, every column: one bf16 rounding (2^-9 relative) plus the f32 accumulation's error."""
    m, k, n = (16384, 11008, 4096) if addend else (16384, 4096, 11008)
    rng = np.random.default_rng(11008 + addend)
    x = bf16_of(oracle, rng.standard_normal((m, k), dtype=np.float32))
    w = bf16_of(oracle, rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02))
    res = bf16_of(oracle, rng.standard_normal((m, n), dtype=np.float32)) if addend else None
    l = launch_desc(abi.OP_CONTRACT_ADD if addend else abi.OP_CONTRACT, abi.BF16, [m, n], [k], order=abi.ORDER_DEVICE, name=b"dot+add" if addend else b"dot")
    l.n_inputs = 3 if addend else 2
    l.iparam[1] = abi.BF16
    set_operand(l.inputs[0], abi.BF16, [m, k], [0, 2])
    set_operand(l.inputs[1], abi.BF16, [k, n], [2, 1])
    if addend:
        set_operand(l.inputs[2], abi.BF16, [m, n], [0, 1])
    set_operand(l.out, abi.BF16, [m, n], [0, 1])
    dev = [cuda.upload(a) for a in ([x, w, res] if addend else [x, w])]
    pout = cuda.alloc(m * n * 2)
    cuda.set_profiling(True)
    cuda.run(l, dev + [pout])
    cuda.sync()
    assert [rec[0] for rec in cuda.profile()] == ["k_gemm_tc"]
    cuda.set_profiling(False)
    got = bf16_value(cuda.download(pout, m * n * 2).view(np.uint16)).reshape(m, n)
    for p in dev + [pout]:
        cuda.free(p)
    rows = np.unique(np.concatenate([np.arange(0, 8), np.arange(m - 8, m), [127, 128, 255, 256, 257, 8191, 8192], rng.integers(0, m, 73)]))
    xf, wf = bf16_value(x[rows]).astype(np.float64), bf16_value(w).astype(np.float64)
    exact = xf @ wf
    if addend:
        # the product is rounded to bf16 as its own site stores it, then added to the residual and rounded again
        prod = bf16_value(bf16_of(oracle, exact.astype(np.float32))).astype(np.float64)
        exact = prod + bf16_value(res[rows]).astype(np.float64)
    err = np.abs(got[rows] - exact)
    scale = np.abs(exact).max()
    # bf16 keeps eight significant bits: a rounding moves a value by at most 2^-8 of its binade's top, and with a
    # residual there are two of them (the product to its site, then the sum); plus the f32 accumulation's error
    assert err.max() <= (2.0**-7 if addend else 2.0**-8) * scale + 4e-6 * np.sqrt(k), (err.max(), scale)
    # and per entry, relative to the entry itself, for entries not far below the tensor's scale
    rel = err / np.maximum(np.abs(exact), 2.0**-4 * scale)
    assert rel.max() <= (2.0**-5 if addend else 2.0**-7), rel.max()


def e8m15_value(u8):
    t = np.ascontiguousarray(u8).view(np.uint8).reshape(-1, 3).astype(np.uint32)
    return ((t[:, 0] | (t[:, 1] << 8) | (t[:, 2] << 16)) << 8).view(np.float32)


def f16_value(u8):
    return np.ascontiguousarray(u8).view(np.float16).astype(np.float32)


@pytest.mark.parametrize("n", [4096, 8192])
@pytest.mark.parametrize("dtype", ["f16", "e8m15"])
def test_contract_ln_at_the_stated_sizes(cuda, oracle, dtype, n):
    """x·w then a row LayerNorm with M = N = K = n, operands normal(0, 1), every site stored f16 or e8m15, under
    the device order. The contraction (f16: one tensor-core product; e8m15: two bf16 planes an operand, four
    partial products in one accumulator) against float64 on the exactly widened operands for 48 sampled rows; the
    LayerNorm's rows against the oracle's LayerNorm (sequential order) fed the very rows the GPU's contraction
    stored, which isolates the norm's reordered row sums."""
    code = abi.F16 if dtype == "f16" else abi.E8M15
    value = f16_value if dtype == "f16" else e8m15_value
    eb = abi.DTYPE_BYTES[code]
    rng = np.random.default_rng(n)
    x = rng.standard_normal((n, n), dtype=np.float32)
    w = rng.standard_normal((n, n), dtype=np.float32)
    xs, ws = oracle.convert(x, code), oracle.convert(w, code)
    l = launch_desc(abi.OP_CONTRACT, code, [n, n], [n], order=abi.ORDER_DEVICE, name=b"dot")
    l.n_inputs = 2
    set_operand(l.inputs[0], code, [n, n], [0, 2])
    set_operand(l.inputs[1], code, [n, n], [2, 1])
    set_operand(l.out, code, [n, n], [0, 1])
    pa, pb, pc = cuda.upload(xs), cuda.upload(ws), cuda.alloc(n * n * eb)
    cuda.set_profiling(True)
    cuda.run(l, [pa, pb, pc])
    cuda.sync()
    assert any(rec[0] == "k_gemm_tc" for rec in cuda.profile()), "the contraction did not reach the tensor-core kernel"
    cuda.set_profiling(False)
    dot_raw = cuda.download(pc, n * n * eb)
    for p in (pa, pb, pc):
        cuda.free(p)
    dot = value(dot_raw).reshape(n, n)
    rows = np.unique(np.concatenate([[0, 1, 127, 128, 255, 256, n - 1], rng.integers(0, n, 41)]))
    xf, wf = value(xs).reshape(n, n)[rows].astype(np.float64), value(ws).reshape(n, n).astype(np.float64)
    exact = xf @ wf
    ulp = 2.0**-11 if dtype == "f16" else 2.0**-16
    err = np.abs(dot[rows] - exact)
    # one rounding to the site's type of a sum of n products of unit normals (magnitude about sqrt(n)), plus the
    # f32 accumulation's error
    assert err.max() <= ulp * np.abs(exact).max() + 4e-6 * n + 1e-5, (err.max(), np.abs(exact).max())
    # the whole workload through the host program
    params = {"ln.γ": np.ones(n, np.float32), "ln.β": np.zeros(n, np.float32)}
    # binary16 cannot hold the squared deviations of such rows (up to about 25·n > 65504): all-f16 stops with E7007, on
    # the reference too; that site is f32 here, as a solved realization would have it
    # (and their mean, which an f16 kernel would read rounded to binary16 at its edge)
    sites = {"LayerNorm.apply/%5": "f32", "LayerNorm.apply/%6": "f32"} if dtype == "f16" else {}
    if dtype == "f16":
        hf = models.give(Host(cuda, {"default": "f16", "order": {"kind": "device"}}).prepare("contract_ln"), params)
        with pytest.raises(PreskError) as e:
            hf.call("apply", [x, w], (n, n))
        assert e.value.code == 7007
        hf.close()
    h = models.give(Host(cuda, {"default": dtype, "order": {"kind": "device"}, "storage": sites}).prepare("contract_ln"), params)
    got = h.call("apply", [x, w], (n, n))
    h.close()
    ho = models.give(Host(oracle.vtable(), {"default": dtype, "order": {"kind": "sequential"}, "storage": sites}).prepare("layernorm"), {"γ": params["ln.γ"], "β": params["ln.β"]})
    want = ho.call("apply", [np.ascontiguousarray(dot[rows])], (len(rows), n))
    ho.close()
    # LayerNorm outputs are O(1) (up to about 4.5 at these widths); the row sums are regrouped, every site rounds
    tol = 2.0**-8 if dtype == "f16" else 2.0**-12
    assert np.abs(got[rows] - want).max() <= tol * max(1.0, np.abs(want).max())
    z = (exact - exact.mean(1, keepdims=True)) / np.sqrt(exact.var(1, keepdims=True) + 1e-5)
    assert np.abs(got[rows] - z).max() <= 4 * tol * max(1.0, np.abs(z).max())


@pytest.mark.parametrize("order", ["sequential", "device"])
def test_the_e8m15_store_guard_trips(cuda, oracle, order):
    """Scaling unit-normal inputs by 2^20 overflows binary16 and leaves e8m15 (eight exponent bits) far from its
    limit, so the e8m15 guard needs a sum placed on purpose: row 0 of x holds 2^64 and 2^56, column 0 of w holds
    (2 - 2^-15)·2^63 and 2^55, and their products add up to (2 - 2^-16)·2^127, finite in f32 and a tie that e8m15's
    16 significant bits round to infinity. Both orders stop with E7007; the same data with the small term
    left out (sum (2 - 2^-15)·2^127, an e8m15 number) runs."""
    n = 256
    rng = np.random.default_rng(64)
    x = rng.standard_normal((n, n)).astype(np.float32)
    w = rng.standard_normal((n, n)).astype(np.float32)
    x[0, :] = 0.0
    w[:, 0] = 0.0
    x[0, 0], w[0, 0] = 2.0**64, (2.0 - 2.0**-15) * 2.0**63
    x[0, 1], w[1, 0] = 2.0**56, 2.0**55
    params = {"ln.γ": np.ones(n, np.float32), "ln.β": np.zeros(n, np.float32)}
    rz = {"default": "e8m15", "order": {"kind": order}}
    h = models.give(Host(cuda, rz).prepare("contract_ln"), params)
    with pytest.raises(PreskError) as e:
        h.call("apply", [x, w], (n, n))
    assert e.value.code == 7007
    h.close()
    ho = models.give(Host(oracle.vtable(), {"default": "e8m15", "order": {"kind": "sequential"}}).prepare("contract_ln"), params)
    with pytest.raises(PreskError) as eo:
        ho.call("apply", [x, w], (n, n))
    assert eo.value.code == 7007
    ho.close()
    # the contraction alone, with and without the term that makes the tie: the flag is the store's, not the sum's
    for small, want_flag in ((True, True), (False, False)):
        xs = x.copy()
        xs[0, 1] = 2.0**56 if small else 0.0
        l = launch_desc(abi.OP_CONTRACT, abi.E8M15, [n, n], [n], order=abi.ORDER_DEVICE if order == "device" else abi.ORDER_SEQUENTIAL, name=b"dot")
        l.n_inputs = 2
        set_operand(l.inputs[0], abi.E8M15, [n, n], [0, 2])
        set_operand(l.inputs[1], abi.E8M15, [n, n], [2, 1])
        set_operand(l.out, abi.E8M15, [n, n], [0, 1])
        pa, pb, pc = cuda.upload(oracle.convert(xs, abi.E8M15)), cuda.upload(oracle.convert(w, abi.E8M15)), cuda.alloc(n * n * 3)
        cuda.run(l, [pa, pb, pc])
        flagged = cuda.overflow() != 0
        cuda.sync()
        first = e8m15_value(cuda.download(pc, 3))[0]
        for p in (pa, pb, pc):
            cuda.free(p)
        assert flagged == want_flag
        assert np.isinf(first) if small else first == np.float32((2.0 - 2.0**-15) * 2.0**127)
