"""Parity of the CUDA executor with the CPU oracle through the host program:
the same model, realization, parameters and seeded inputs run over both.
Under `order: sequential` the results must be the same bits; under
`order: device` (tensor-core contractions, tree row sums) within the stated
tolerance of the oracle."""
import numpy as np
import pytest

import models
from presk_b200 import Host, PreskError

pytestmark = pytest.mark.gpu


def both(cuda, oracle, realization, model, consts, params, entry, inputs, out_shape):
    outs = []
    for ex in (cuda, oracle.vtable()):
        h = models.give(Host(ex, realization).prepare(model, **consts), params)
        outs.append(h.call(entry, inputs, out_shape))
    return outs


def assert_same_bits(got, want):
    a, b = np.ascontiguousarray(got).view(np.uint32), np.ascontiguousarray(want).view(np.uint32)
    bad = np.nonzero(a != b)
    assert bad[0].size == 0, f"{bad[0].size} of {a.size} elements differ, first at {tuple(x[0] for x in bad)}: {got[tuple(x[0] for x in bad)]!r} vs {want[tuple(x[0] for x in bad)]!r}"


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16", "e8m15"])
@pytest.mark.parametrize("model", ["layernorm", "rmsnorm"])
def test_norms_bit_exact(cuda, oracle, model, dtype):
    rng = np.random.default_rng(7)
    for shape in [(3, 8), (5, 7, 40), (2, 1000), (1, 4096)]:
        d = shape[-1]
        x = rng.standard_normal(shape).astype(np.float32)
        params = {"γ": rng.standard_normal(d).astype(np.float32)}
        if model == "layernorm":
            params["β"] = rng.standard_normal(d).astype(np.float32)
        got, want = both(cuda, oracle, dtype, model, {}, params, "apply", [x], shape)
        assert_same_bits(got, want)


def test_mlp_config1_bit_exact(cuda, oracle):
    """The MLP classifier workload at full size: Linear{784,256} · ReLU · Linear{256,10} + cross-entropy, B = 4096, all f32."""
    p = models.mlp_params()
    x, y = models.mlp_inputs(4096)
    got, want = both(cuda, oracle, "f32", "mlp", {}, p, "apply", [x], (4096, 10))
    assert_same_bits(got, want)
    got, want = both(cuda, oracle, "f32", "mlp", {}, p, "loss", [x, y], ())
    assert_same_bits(got, want)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16", "e8m15"])
def test_llama_tiny_bit_exact_under_sequential_order(cuda, oracle, dtype):
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, c["V"], size=(2, 16), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(2, 16), dtype=np.int64)
    got, want = both(cuda, oracle, dtype, "llama", c, p, "apply", [ids], (2, 16, c["V"]))
    assert_same_bits(got, want)
    got, want = both(cuda, oracle, dtype, "llama", c, p, "loss", [ids, y], ())
    assert_same_bits(got, want)


def test_llama_gqa_and_int8_bit_exact(cuda, oracle):
    c = dict(V=64, D=64, H=4, G=2, FF=96, L=2)
    p = models.llama_params(c)
    ids = np.random.default_rng(4).integers(0, c["V"], size=(3, 24), dtype=np.int64)
    q = {k: {"bits": 8, "over": -2} for k in ("blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w")}
    rz = {"default": "bf16", "storage": {"RMSNorm.apply/%3": "f32", "RMSNorm.apply/%7": "f32"}, "params": {"tok": "bf16", "head": "bf16"}, "quant": q}
    got, want = both(cuda, oracle, rz, "llama", c, p, "apply", [ids], (3, 24, c["V"]))
    assert_same_bits(got, want)


def test_llama_device_order_within_tolerance(cuda, oracle):
    """Tensor-core contractions and tree sums: bf16 sites, shapes that reach the tcgen05 kernel
    (every contracted axis a multiple of 8, hd = 64)."""
    c = dict(V=512, D=256, H=4, G=4, FF=512, L=2)
    p = models.llama_params(c)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, c["V"], size=(2, 128), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(2, 128), dtype=np.int64)
    rz = {"default": "bf16", "order": {"kind": "device"}, "params": {k: "bf16" for k in p}, "storage": {"Llama.apply/%11": "f32", "loss/%5": "f32", "loss/%6": "f32"}}
    rs = dict(rz, order={"kind": "sequential"})
    outs = []
    for ex, r in ((cuda, rz), (oracle.vtable(), rs)):
        h = models.give(Host(ex, r).prepare("llama", **c), p)
        outs.append((h.call("apply", [ids], (2, 128, c["V"])), h.call("loss", [ids, y], ())))
    (lg, ls), (lw, lsw) = outs
    # bf16 activations: an element of a site may land on the neighbouring bf16 number when a sum's
    # last bits differ; across two layers that is within a few bf16 ulps of the logits' scale
    assert np.abs(lg - lw).max() <= 2.0**-6 * np.abs(lw).max()
    assert abs(float(ls) - float(lsw)) <= 2e-3 * abs(float(lsw))
    # and both stay close to the exact model
    want = models.llama_numpy(p, c, ids)
    assert np.abs(lg - want).max() <= 0.05 * np.abs(want).max()


@pytest.mark.parametrize("dtype,scale,overflows", [("f16", 1.0, False), ("f16", 2.0**20, True), ("e8m15", 2.0**20, False)])
@pytest.mark.parametrize("order", ["sequential", "device"])
def test_contract_ln_config3_and_overflow_guard(cuda, oracle, dtype, scale, overflows, order):
    """The contraction-plus-LayerNorm workload at N = 1024: x·w stored in f16 / e8m15 then a row LayerNorm; inputs scaled
    by 2^20 overflow the f16 store of the `dot` and stop the run with E7007."""
    n = 1024 if order == "device" else 256
    rng = np.random.default_rng(6)
    x, w = (rng.standard_normal((n, n)) * scale).astype(np.float32), (rng.standard_normal((n, n)) * scale).astype(np.float32)
    params = {"ln.γ": np.ones(n, np.float32), "ln.β": np.zeros(n, np.float32)}
    rz = {"default": dtype, "order": {"kind": order}}
    if overflows:
        h = models.give(Host(cuda, rz).prepare("contract_ln"), params)
        with pytest.raises(PreskError, match="E7007"):
            h.call("apply", [x, w], (n, n))
        return
    rs = {"default": dtype, "order": {"kind": "sequential"}}
    h = models.give(Host(cuda, rz).prepare("contract_ln"), params)
    got = h.call("apply", [x, w], (n, n))
    h = models.give(Host(oracle.vtable(), rs).prepare("contract_ln"), params)
    want = h.call("apply", [x, w], (n, n))
    if order == "sequential":
        assert_same_bits(got, want)
    else:
        # LayerNorm outputs are O(1); the dot's sums differ in their last bits and each site rounds to 11 or 16 bits
        tol = 2.0**-8 if dtype == "f16" else 2.0**-12
        assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_gpt_config2_bit_exact_under_sequential_order(cuda, oracle, dtype):
    """The GPT workload's program (05_gpt.psk) at reduced constants; its full shape runs under device order below."""
    c = models.GPT_TINY
    T = 16
    p = models.gpt_params(c, T)
    rng = np.random.default_rng(8)
    ids = rng.integers(0, c["V"], size=(3, T), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(3, T), dtype=np.int64)
    got, want = both(cuda, oracle, dtype, "gpt", c, p, "apply", [ids], (3, T, c["V"]))
    assert_same_bits(got, want)
    got, want = both(cuda, oracle, dtype, "gpt", c, p, "loss", [ids, y], ())
    assert_same_bits(got, want)


def test_gpt_config2_full_shape_mixed_realization(cuda, oracle):
    """Config 2 at its stated shape: 4 layers, d_model 128, 4 heads, ctx 64, vocab 65, batch 256 (a
    quarter of it on the CPU side of the comparison), a mixed bf16/f32 assignment, device order."""
    c = dict(V=65, D=128, H=4, L=4)
    T, B = 64, 256
    p = models.gpt_params(c, T)
    rng = np.random.default_rng(2)
    ids = rng.integers(0, c["V"], size=(B, T), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(B, T), dtype=np.int64)
    rz = {"default": "bf16", "order": {"kind": "device"}, "storage": {"LayerNorm.apply/%2": "f32", "LayerNorm.apply/%5": "f32", "LayerNorm.apply/%10": "f32", "GPT.apply/%24": "f32", "loss/%6": "f32", "loss/%7": "f32"}}
    h = models.give(Host(cuda, rz).prepare("gpt", **c), p)
    loss = float(h.call("loss", [ids, y], ()))
    logits = h.call("apply", [ids[:64]], (64, T, c["V"]))
    ho = models.give(Host(oracle.vtable(), dict(rz, order={"kind": "sequential"})).prepare("gpt", **c), p)
    want = ho.call("apply", [ids[:64]], (64, T, c["V"]))
    assert np.abs(logits - want).max() <= 2.0**-5 * np.abs(want).max()
    exact = models.gpt_numpy(p, c, ids[:16])
    assert np.abs(logits[:16] - exact).max() <= 1e-3 * max(1.0, np.abs(exact).max()) * 50  # the budget's order of magnitude at bf16
    assert abs(loss - float(models.gpt_numpy(p, c, ids[:64], y[:64]))) < 0.05


def test_calibrate_envelope_matches_the_oracle(cuda, oracle):
    """The magnitudes of every site, measured on the GPU, are the oracle's (order-free reductions of equal values)."""
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    ids = np.random.default_rng(3).integers(0, c["V"], size=(2, 16), dtype=np.int64)
    envs = []
    for ex in (cuda, oracle.vtable()):
        h = models.give(Host(ex, "bf16").prepare("llama", **c), p)
        h.set_calibrating(True)
        h.call("apply", [ids], (2, 16, c["V"]))
        envs.append(h.envelope())
    assert envs[0] == envs[1] and len(envs[0]) > 25


def test_w8a8_dense_is_exact_on_the_gpu(cuda, oracle):
    """examples/tests/formats/w8a8.psk under w8a8.json with static scales: the integer path end to end."""
    from test_oracle_w8a8 import w8a8_dense_case
    for seed, shape in [(0, (4, 16, 8)), (1, (33, 130, 17))]:
        rz, x, w, want = w8a8_dense_case(seed, *shape)
        h = Host(cuda, rz).prepare("dense")
        h.set_param("w", w)
        got = h.call("apply", [x], want.shape, np.float64)
        assert np.array_equal(got, want)


def test_llama_int8_weights_on_tensor_cores(cuda, oracle):
    """The int8 workload's shape of program at small constants: int8 projection and FFN weights with one
    f32 scale a channel, bf16 activations, device order: the weights' integers go through the tensor
    cores as bf16 numbers and the scale multiplies the sum. Against the oracle's sequential
    sum of x·(q·s) the difference is a reassociation: a few bf16 ulps after two layers."""
    c = dict(V=512, D=256, H=4, G=4, FF=512, L=2)
    p = models.llama_params(c)
    ids = np.random.default_rng(5).integers(0, c["V"], size=(2, 128), dtype=np.int64)
    q = {k: {"bits": 8, "over": -2} for k in ("blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w")}
    rz = {"default": "bf16", "order": {"kind": "device"}, "params": {"tok": "bf16", "head": "bf16", "norm.γ": "bf16", "blocks.n1.γ": "bf16", "blocks.n2.γ": "bf16"}, "quant": q, "storage": {"Llama.apply/%11": "f32"}}
    ex_before = cuda.counts()
    cuda.set_profiling(True)
    h = models.give(Host(cuda, rz).prepare("llama", **c), p)
    got = h.call("apply", [ids], (2, 128, c["V"]))
    kinds = [r[0] for r in cuda.profile() if r[1] in ("dot", "ein[batch, seq, model]")]
    cuda.set_profiling(False)
    assert kinds and all(k == "k_gemm_tc" for k in kinds), kinds
    ho = models.give(Host(oracle.vtable(), dict(rz, order={"kind": "sequential"})).prepare("llama", **c), p)
    want = ho.call("apply", [ids], (2, 128, c["V"]))
    assert np.abs(got - want).max() <= 2.0**-6 * np.abs(want).max()


@pytest.mark.parametrize("G", [4, 2])
def test_llama_blockwise_attention_within_tolerance(cuda, oracle, G):
    """hd = 128, T = 256: the fused attention kernel inside the whole model (GQA when G < H), against the
    oracle's unfused sequential run."""
    c = dict(V=512, D=512, H=4, G=G, FF=512, L=2)
    p = models.llama_params(c)
    rng = np.random.default_rng(6)
    ids = rng.integers(0, c["V"], size=(2, 256), dtype=np.int64)
    rz = {"default": "bf16", "order": {"kind": "device", "attention": "blockwise"}, "params": {k: "bf16" for k in p}, "storage": {"Llama.apply/%11": "f32"}}
    rs = dict(rz, order={"kind": "sequential"})
    h = models.give(Host(cuda, rz).prepare("llama", **c), p)
    h.set_logging(True)
    lg = h.call("apply", [ids], (2, 256, c["V"]))
    assert h.launch_log().count("attention[blockwise]") == c["L"]
    lw = models.give(Host(oracle.vtable(), rs).prepare("llama", **c), p).call("apply", [ids], (2, 256, c["V"]))
    assert np.abs(lg - lw).max() <= 2.0**-6 * np.abs(lw).max()
    want = models.llama_numpy(p, c, ids)
    assert np.abs(lg - want).max() <= 0.05 * np.abs(want).max()


@pytest.mark.parametrize("kind", ["sequential", "device"])
def test_merged_launches_keep_every_bit_on_the_gpu(cuda, oracle, kind):
    """`launches: merged` (slices as views, concatenation halves written in place, rotary tables once a call,
    silu and the product with `up` as one group) changes which launches run, not one bit of any value."""
    c = dict(V=512, D=256, H=4, G=2, FF=512, L=2)
    p = models.llama_params(c)
    ids = np.random.default_rng(10).integers(0, c["V"], size=(2, 128), dtype=np.int64)
    outs = []
    for extra in ({}, {"launches": "merged"}):
        rz = {"default": "bf16", "order": dict(kind=kind, **extra), "params": {k: "bf16" for k in p}, "storage": {"Llama.apply/%11": "f32"}}
        h = models.give(Host(cuda, rz).prepare("llama", **c), p)
        h.set_logging(True)
        outs.append(h.call("apply", [ids], (2, 128, c["V"])))
        log = h.launch_log()
    assert "fused 4 steps" in log and not any(n.startswith("slice") for n in log)
    assert_same_bits(outs[1], outs[0])
    if kind == "sequential":
        rz = {"default": "bf16", "order": {"kind": "sequential"}, "params": {k: "bf16" for k in p}, "storage": {"Llama.apply/%11": "f32"}}
        want = models.give(Host(oracle.vtable(), rz).prepare("llama", **c), p).call("apply", [ids], (2, 128, c["V"]))
        assert_same_bits(outs[1], want)


NARROW = ("blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w")


@pytest.mark.parametrize("weights", ["int8", "e4m3fn"])
def test_narrow_weights_through_the_model(cuda, oracle, weights):
    """Projection and FFN weights as int8 codes with a scale a channel (`quant`) or stored e4m3fn (`params`), bf16
    activations. Sequential order: the oracle's bits. Device order: the contractions run on the tensor cores from a
    bf16 copy of the codes, merged launches (the residual additions in the contractions' epilogues among them) keep
    the bits of the unmerged list, and the logits stay within the bf16 tolerance of the sequential result."""
    c = dict(V=512, D=256, H=4, G=2, FF=512, L=2)
    p = models.llama_params(c)
    ids = np.random.default_rng(12).integers(0, c["V"], size=(2, 128), dtype=np.int64)

    def rz(order):
        r = {"default": "bf16", "order": order, "storage": {"Llama.apply/%11": "f32"}}
        if weights == "int8":
            r["params"] = {k: "bf16" for k in p if k not in NARROW}
            r["quant"] = {k: {"bits": 8, "over": -2} for k in NARROW}
        else:
            r["params"] = {k: ("e4m3fn" if k in NARROW else "bf16") for k in p}
        return r

    want = models.give(Host(oracle.vtable(), rz({"kind": "sequential"})).prepare("llama", **c), p).call("apply", [ids], (2, 128, c["V"]))
    got = models.give(Host(cuda, rz({"kind": "sequential"})).prepare("llama", **c), p).call("apply", [ids], (2, 128, c["V"]))
    assert_same_bits(got, want)
    outs = []
    for extra in ({}, {"launches": "merged"}):
        h = models.give(Host(cuda, rz(dict(kind="device", **extra))).prepare("llama", **c), p)
        h.set_logging(True)
        cuda.set_profiling(True)
        outs.append(h.call("apply", [ids], (2, 128, c["V"])))
        prof = cuda.profile()
        cuda.set_profiling(False)
        log = h.launch_log()
        assert sum(1 for rec in prof if rec[0] == "k_gemm_tc") >= 7 * c["L"], "the narrow weights did not reach the tensor-core kernel"
    assert any(n.endswith("+add") for n in log), log
    assert_same_bits(outs[1], outs[0])
    assert np.abs(outs[1] - want).max() <= 2.0**-5 * np.abs(want).max()
    # with no room to keep the bf16 copies (a model whose narrow weights are there to save memory) each is made
    # for its contraction only, from the pool: the same bits, and the executor's memory stays that of the codes
    import os
    before = os.environ.get("PSK_WIDENED_MB")
    os.environ["PSK_WIDENED_MB"] = "0"
    try:
        h = models.give(Host(cuda, rz(dict(kind="device", launches="merged"))).prepare("llama", **c), p)
        cuda.set_profiling(True)
        lean = h.call("apply", [ids], (2, 128, c["V"]))
        prof = cuda.profile()
        cuda.set_profiling(False)
        h.close()
    finally:
        if before is None:
            del os.environ["PSK_WIDENED_MB"]
        else:
            os.environ["PSK_WIDENED_MB"] = before
    assert sum(1 for rec in prof if rec[0] == "k_gemm_tc") >= 7 * c["L"]
    assert_same_bits(lean, outs[1])


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("d,b", [(4, 2), (64, 48)])
def test_mlp_gradient_bit_exact(cuda, oracle, dtype, d, b):
    """The reverse-mode program of examples/spec/mlp/mlp.psk (`mse_grad`: sum_to, dot_vjp_l, dot_vjp_r,
    mean_vjp, gelu', tree additions): every leaf of the gradient, the oracle's bits."""
    rng = np.random.default_rng(d)
    bound = np.sqrt(6.0 / (5 * d))
    params = {"l1.w": rng.uniform(-bound, bound, (d, 4 * d)), "l1.b": rng.standard_normal(4 * d) * 0.1,
              "l2.w": rng.uniform(-bound, bound, (4 * d, d)), "l2.b": rng.standard_normal(d) * 0.1}
    x, y = rng.standard_normal((b, d)), rng.standard_normal((b, d))
    leaves = []
    for ex in (cuda, oracle.vtable()):
        h = Host(ex, dtype).prepare("mlp_spec", D=d)
        for k, v in params.items():
            h.set_param(k, v)
        loss = h.call("mse", [x, y], (), np.float32)
        h.call("mse_grad", [x, y], (d, 4 * d), np.float32)
        leaves.append([loss] + [h.result(k, np.shape(v), np.float32) for k, v in params.items()])
    for got, want in zip(*leaves):
        assert_same_bits(np.atleast_1d(got), np.atleast_1d(want))


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_attention_entry_bit_exact(cuda, oracle, dtype):
    """The attention function alone on given activations (the entry the rope golden is checked through)."""
    c = dict(V=8, D=64, H=4, G=2, FF=8, L=1)
    rng = np.random.default_rng(12)
    params = {"blocks.attn." + n: rng.standard_normal((1, 64, 64 if n in ("wq", "wo") else 32)) * 0.05 for n in ("wq", "wk", "wv", "wo")}
    x = rng.standard_normal((3, 24, 64))
    outs = []
    for ex in (cuda, oracle.vtable()):
        h = Host(ex, dtype).prepare("llama", **c)
        for k, v in params.items():
            h.set_param(k, v)
        outs.append(h.call("attention", [x], (3, 24, 64), np.float32))
    assert_same_bits(*outs)


def test_toy_loss_bit_exact(cuda, oracle):
    """examples/spec/concat/concat.psk `loss` (index slices, concatenated weights, min/max/clamp, cross-entropy)."""
    v, d = 64, 16
    rng = np.random.default_rng(14)
    params = {"tok": rng.standard_normal((v, d)) * 0.5, "qkv.wq": rng.standard_normal((d, d)), "qkv.wk": rng.standard_normal((d, d)),
              "qkv.wv": rng.standard_normal((d, d)), "head": rng.standard_normal((d, v)) * 0.3}
    w = rng.integers(0, v, size=(5, 33), dtype=np.int64)
    for dtype in ("f32", "bf16"):
        outs = []
        for ex in (cuda, oracle.vtable()):
            h = Host(ex, dtype).prepare("toy", V=v, D=d)
            for k, p in params.items():
                h.set_param(k, p)
            outs.append(h.call("loss", [w], (), np.float32))
        assert_same_bits(np.atleast_1d(outs[0]), np.atleast_1d(outs[1]))


@pytest.mark.parametrize("v,d,b,t", [(64, 16, 5, 33), (300, 96, 4, 64)])
def test_toy_loss_gradient_bit_exact(cuda, oracle, v, d, b, t):
    """examples/spec/concat/concat.psk `loss_grad`: cross_entropy_vjp, dot_vjp_l/r, the max/min rule (ties go to the
    second operand: weights of 1 make q hit the clamp's bounds exactly), slice_vjp, embed_vjp with repeated tokens:
    every leaf of the gradient, the oracle's bits, in f32, bf16 and f16."""
    rng = np.random.default_rng(v)
    params = {"tok": np.round(rng.standard_normal((v, d)) * 2) / 4, "qkv.wq": np.eye(d), "qkv.wk": rng.standard_normal((d, d)) * 0.3,
              "qkv.wv": np.diag(np.where(np.arange(d) % 2, 0.5, 1.0)), "head": rng.standard_normal((d, v)) * 0.3}  # v == q in every other column
    w = rng.integers(0, v // 2, size=(b, t + 1), dtype=np.int64)
    for dtype in ("f32", "bf16", "f16"):
        leaves = []
        for ex in (cuda, oracle.vtable()):
            h = Host(ex, dtype).prepare("toy", V=v, D=d)
            for k, p in params.items():
                h.set_param(k, p)
            h.call("loss_grad", [w], (v, d), np.float32)
            leaves.append([h.result(k, np.shape(p), np.float32) for k, p in params.items()])
        for k, got, want in zip(params, *leaves):
            assert_same_bits(got, want)
            assert np.isfinite(want).all() and (np.abs(want).max() > 0), k


@pytest.mark.parametrize("d,L,b", [(3, 3, 2), (64, 4, 40)])
def test_tower_gradient_through_the_fold_bit_exact(cuda, oracle, d, L, b):
    """examples/tests/data/stack_grad.psk `loss` and `loss_grad`: a fold over a stacked parameter tree and its
    reverse pass (layers read as views of [L, D, D] and [L, D], each layer's leaves placed at l of the stacked
    gradient): the oracle's bits in f32, bf16 and f16."""
    rng = np.random.default_rng(d)
    params = {"blocks.w": rng.uniform(-1, 1, (L, d, d)) * np.sqrt(3.0 / d), "blocks.b": rng.standard_normal((L, d)) * 0.5}
    x, scale = rng.standard_normal((b, d)), np.float64(0.7)
    for dtype in ("f32", "bf16", "f16"):
        leaves = []
        for ex in (cuda, oracle.vtable()):
            h = Host(ex, dtype).prepare("tower", D=d, L=L)
            for k, p in params.items():
                h.set_param(k, p)
            loss = h.call("loss", [x, scale], (), np.float32)
            h.call("loss_grad", [x, scale], (L, d, d), np.float32)
            leaves.append([np.atleast_1d(loss)] + [h.result(k, np.shape(p), np.float32) for k, p in params.items()])
        for got, want in zip(*leaves):
            assert_same_bits(got, want)
            assert np.isfinite(want).all() and np.abs(want).max() > 0


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_training_steps_bit_exact(cuda, oracle, dtype):
    """Five steps of `loss_grad` + `adamw.step` (decay, cosine schedule with warm-up) on the tower and on the concat
    toy: parameters, both moments and the loss after the last step, the oracle's bits."""
    rng = np.random.default_rng(21)
    d, L, b = 32, 3, 24
    tower = ("tower", dict(D=d, L=L), {"blocks.w": rng.uniform(-1, 1, (L, d, d)) * np.sqrt(3.0 / d), "blocks.b": rng.standard_normal((L, d)) * 0.5},
             [rng.standard_normal((b, d)), np.float64(0.7)], (L, d, d))
    v, dt = 64, 16
    toy = ("toy", dict(V=v, D=dt), {"tok": rng.standard_normal((v, dt)) * 0.5, "qkv.wq": rng.standard_normal((dt, dt)) * 0.3, "qkv.wk": rng.standard_normal((dt, dt)) * 0.3,
                                    "qkv.wv": rng.standard_normal((dt, dt)) * 0.3, "head": rng.standard_normal((dt, v)) * 0.3},
           [rng.integers(0, v, size=(4, 17), dtype=np.int64)], (v, dt))
    for model, consts, params, inputs, first_shape in (tower, toy):
        runs = []
        for ex in (cuda, oracle.vtable()):
            h = Host(ex, dtype).prepare(model, **consts).adamw(lr=1e-2, beta2=0.95, weight_decay=0.1, grad_clip=0.5, schedule="cosine", warmup=2)
            for k, p in params.items():
                h.set_param(k, p)
            for t in range(1, 6):
                h.call("loss_grad", inputs, first_shape)
                h.adamw_step(t, 5)
            leaves = [h.result(pre + k, np.shape(p)) for k, p in params.items() for pre in ("", "m:", "v:")]
            leaves.append(np.atleast_1d(h.call("loss", inputs, ())))
            runs.append(leaves)
        for got, want in zip(*runs):
            assert_same_bits(got, want)
            assert np.isfinite(want).all()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_llama_gradient_bit_exact(cuda, oracle, dtype):
    """examples/coverage/llama.psk `loss_grad` (grouped-query attention, three blocks): every leaf of the gradient,
    the oracle's bits under the sequential order; then two training steps with AdamW, parameters still bit-equal."""
    c = dict(V=50, D=32, H=4, G=2, FF=48, L=3)
    p = models.llama_params(c, seed=4, std=0.2)
    rng = np.random.default_rng(6)
    ids = rng.integers(0, c["V"] // 2, size=(2, 12), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(2, 12), dtype=np.int64)
    runs = []
    for ex in (cuda, oracle.vtable()):
        # the optimizer's own sites stay f32, as a solved realization keeps them: in bf16 its β₂ = 0.999 is 1 and
        # the bias correction 1 - β₂ᵗ is 0
        rz = {"default": dtype, "functions": {"adamw.step": "f32", "adamw.lr": "f32"}}
        h = models.give(Host(ex, rz).prepare("llama", **c), p).adamw(lr=1e-2, weight_decay=0.1, grad_clip=1.0)
        h.call("loss_grad", [ids, y], p["tok"].shape)
        leaves = [h.result(k, np.shape(v)) for k, v in p.items()]
        for t in (1, 2):
            if ex is cuda:
                cuda.set_profiling(True)
            h.adamw_step(t, 2)
            if ex is cuda:
                # the nine-step update of every leaf ran as its compile-time kernel (the bits below are the generic group's)
                assert sum(1 for rec in cuda.profile() if rec[0] == "k_adamw_update") == len(p)
                cuda.set_profiling(False)
            h.call("loss_grad", [ids, y], p["tok"].shape)
        leaves += [h.result(k, np.shape(v)) for k, v in p.items()]
        runs.append(leaves)
    for got, want in zip(*runs):
        assert_same_bits(got, want)
        assert np.isfinite(want).all() and np.abs(want).max() > 0


def test_llama_gradient_device_order_within_tolerance(cuda, oracle):
    """The same program under the device order at a size whose contractions reach the tensor cores (bf16 storage):
    every leaf within a bf16 tolerance of the oracle's sequential gradient under the same storage types (the sums'
    order is all that differs; every value between the loss and a leaf is rounded to bf16 some dozens of times),
    relative to the leaf's largest entry."""
    c = dict(V=512, D=256, H=4, G=2, FF=512, L=2)
    p = models.llama_params(c, seed=5, std=0.05)
    rng = np.random.default_rng(9)
    ids = rng.integers(0, c["V"], size=(2, 128), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(2, 128), dtype=np.int64)
    rz = {"default": "bf16", "order": {"kind": "device"}, "params": {k: "bf16" for k in p}, "storage": {"Llama.apply/%11": "f32", "loss/%5": "f32"}}
    want_h = models.give(Host(oracle.vtable(), dict(rz, order={"kind": "sequential"})).prepare("llama", **c), p)
    want_h.call("loss_grad", [ids, y], p["tok"].shape)
    h = models.give(Host(cuda, rz).prepare("llama", **c), p)
    cuda.set_profiling(True)
    h.call("loss_grad", [ids, y], p["tok"].shape)
    prof = cuda.profile()
    cuda.set_profiling(False)
    assert sum(1 for rec in prof if rec[0] == "k_gemm_tc") >= 10 * c["L"], "the reverse pass's contractions did not reach the tensor-core kernel"
    for k, v in p.items():
        want, got = want_h.result(k, np.shape(v)), h.result(k, np.shape(v))
        assert np.isfinite(got).all(), k
        assert np.abs(got - want).max() <= 0.06 * np.abs(want).max(), (k, np.abs(got - want).max(), np.abs(want).max())


def test_step_after_prefill_on_the_gpu(cuda, oracle):
    """Generation with a cache of keys and values on the CUDA executor. Sequential order: `prefill` then three
    `step`s give the oracle's bits, which are those of recomputing the whole window (tests/test_host_cpu.py).
    Device order at a width where a step's contractions are cut along the summed axis (k >= 1024, a few rows
    against a large weight matrix, partial sums added in the runs' order): within the bf16 tolerance of the
    sequential result, with bf16, int8 and e4m3fn weights."""
    c = dict(V=512, D=1024, H=8, G=4, FF=2048, L=2)
    p = models.llama_params(c)
    rng = np.random.default_rng(21)
    ids = rng.integers(0, c["V"], size=(4, 131), dtype=np.int64)
    base = {"default": "bf16", "params": {k: "bf16" for k in p}, "storage": {"Llama.apply/%11": "f32", "RMSNorm.apply/%3": "f32", "RMSNorm.apply/%7": "f32"}}

    def run(ex, rz):
        h = models.give(Host(ex, rz).prepare("llama", TMAX=256, **c), p)
        outs = [h.call("prefill", [ids[:, :128]], (4, 128, c["V"]))[:, -1:, :]]
        for t in range(128, 131):
            outs.append(h.call("step", [ids[:, t:t + 1]], (4, 1, c["V"])))
        return np.concatenate(outs, axis=1)

    want = run(oracle.vtable(), dict(base, order={"kind": "sequential"}))
    got = run(cuda, dict(base, order={"kind": "sequential"}))
    assert_same_bits(got, want)
    cuda.set_profiling(True)
    dev = run(cuda, dict(base, order={"kind": "device", "attention": "blockwise", "launches": "merged"}))
    prof = cuda.profile()
    cuda.set_profiling(False)
    assert sum(1 for rec in prof if rec[0] == "k_gemm_tc") > 7 * c["L"] * 4
    assert sum(1 for rec in prof if rec[0] == "k_attn_step") == 3 * c["L"]  # a step's attention: one stream of the cache a layer
    assert np.abs(dev - want).max() <= 2.0**-6 * np.abs(want).max()
    for weights in ("int8", "e4m3fn"):
        rz = dict(base, order={"kind": "sequential"})
        if weights == "int8":
            rz["params"] = {k: "bf16" for k in p if k not in NARROW}
            rz["quant"] = {k: {"bits": 8, "over": -2} for k in NARROW}
        else:
            rz["params"] = {k: ("e4m3fn" if k in NARROW else "bf16") for k in p}
        w_want = run(oracle.vtable(), rz)
        w_dev = run(cuda, dict(rz, order={"kind": "device", "launches": "merged"}))
        assert np.abs(w_dev - w_want).max() <= 2.0**-5 * np.abs(w_want).max(), weights


def test_w8a8_llama_on_the_integer_tensor_cores(cuda, oracle):
    """The W8A8 realization of the Llama program (tests/headline.py): the norm and the silu group write i8 codes
    with static scales (from a calibration on this executor), q, k, v, gate, up, down and the head are integer-sum
    contractions on tcgen05's 8-bit kind, the out-projection reads bf16 against int8 weights. Sequential order: the
    oracle's bits, the scalar integer kernel's among them. Device order: the merged launches (the norm and the silu
    group writing their codes themselves) keep every bit of the unmerged list, and the logits stay within the bf16
    tolerance of the sequential result (the integer sums are exact either way; what is reordered are the
    out-projection's and the statistics' sums)."""
    import headline
    c = dict(V=512, D=256, H=2, G=2, FF=512, L=2)
    p = models.llama_params(c)
    ids = np.random.default_rng(14).integers(0, c["V"], size=(2, 128), dtype=np.int64)
    h = models.give(Host(cuda, headline.realization(p, {"kind": "device"})).prepare("llama", **c), p)
    h.set_calibrating(True)
    h.call("apply", [ids], (2, 128, c["V"]))
    scales = headline.w8a8_scales(h.envelope())
    h.close()

    def run(ex, order):
        hw = models.give(Host(ex, headline.w8a8_realization(p, order, scales)).prepare("llama", **c), p)
        hw.set_logging(True)
        out = hw.call("apply", [ids], (2, 128, c["V"]))
        log = hw.launch_log()
        hw.close()
        return out, log

    want, _ = run(oracle.vtable(), {"kind": "sequential"})
    got, _ = run(cuda, {"kind": "sequential"})
    assert_same_bits(got, want)
    cuda.set_profiling(True)
    plain, plain_log = run(cuda, {"kind": "device"})
    cuda.profile()
    merged, merged_log = run(cuda, {"kind": "device", "attention": "online", "launches": "merged"})
    prof = [rec[0] for rec in cuda.profile()]
    cuda.set_profiling(False)
    assert prof.count("k_gemm_i8") >= 6 * c["L"] + 1, prof
    assert merged_log.count("rmsnorm[merged]") == 2 * c["L"] + 1 and len(merged_log) < len(plain_log)
    unfused, _ = run(cuda, {"kind": "device", "launches": "merged"})  # the attention's four launches: merged launches alone keep every bit
    assert_same_bits(unfused, plain)
    # An i8 code is a step of 1/127 of its site's largest magnitude (2^-7): a sum reordered upstream moves a value
    # across a code's boundary now and then, and that whole step then goes through the next contraction. Stated
    # accordingly: 2^-4 of the logits' scale at most (seen: 0.051 of a scale of 1.52 with the one-pass attention
    # kernel), 2^-7 on average.
    for out in (merged, plain):
        assert np.abs(out - want).max() <= 2.0**-4 * np.abs(want).max()
        assert np.abs(out - want).mean() <= 2.0**-7 * np.abs(want).max()


def test_gap_of_a_candidate_realization_measured_on_the_device(cuda):
    """What `presk solve --measure` does for every candidate (presk-driver/src/gap.rs): the same entry under the
    reference realization and under a candidate's, the largest difference of the results against budget x max |y|.
    Both results stay on the executor; psk_exec_gap returns the two numbers, equal to numpy's on the downloads."""
    from presk_b200 import abi
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    ids = np.random.default_rng(3).integers(0, c["V"], size=(2, 16), dtype=np.int64)
    pid = cuda.upload(ids)
    outs = {}
    hosts = []
    for name, rz in (("reference", "f32"), ("candidate", {"default": "bf16", "order": {"kind": "device"}})):
        h = models.give(Host(cuda, rz).prepare("llama", **c), p)
        hosts.append(h)
        outs[name] = h.call_device("apply", [(pid, abi.I64, (2, 16))])
    (pa, da, na), (pb, db, nb) = outs["reference"], outs["candidate"]
    assert na == nb == 2 * 16 * c["V"] and da == abi.F32 and db == abi.BF16
    gap, mx = cuda.gap(pa, da, pb, db, na)
    a = cuda.download(pa, na * 4).view(np.float32).astype(np.float64)
    b = (cuda.download(pb, nb * 2).view(np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert gap == np.abs(a - b).max() and mx == np.abs(a).max()
    assert 0 < gap <= 3e-2 * mx  # the bf16 candidate sits inside a 3e-2 budget, as against the exact evaluator
    cuda.free(pid)


def test_w8a8_llama_with_the_attention_result_in_codes(cuda, oracle):
    """The fuller W8A8 form (tests/headline.py, `attn_out`): the weighted values are a scaled site too, written by the
    one-pass attention kernel as i8 codes, and the out-projection counts its sums in i32 like the other six; it and
    the down-projection take their residual along in the integer kernel's epilogue. Sequential order (the launches
    apart, the weighted values' float sums stored as codes by the index-order nest): the oracle's bits. The
    benchmark's order against that, within the W8A8 tolerance (one more i8 site than the other form), and the device
    order with the reference's launch list likewise."""
    import headline
    c = dict(V=512, D=256, H=2, G=2, FF=512, L=2)
    p = models.llama_params(c)
    ids = np.random.default_rng(15).integers(0, c["V"], size=(2, 128), dtype=np.int64)
    h = models.give(Host(cuda, headline.realization(p, {"kind": "device"})).prepare("llama", **c), p)
    h.set_calibrating(True)
    h.call("apply", [ids], (2, 128, c["V"]))
    scales = headline.w8a8_scales(h.envelope())
    h.close()
    assert scales[headline.W8A8_ATTN_OUT_SITE] > 0

    def run(ex, order):
        hw = models.give(Host(ex, headline.w8a8_realization(p, order, scales, attn_out=True)).prepare("llama", **c), p)
        hw.set_logging(True)
        try:
            return hw.call("apply", [ids], (2, 128, c["V"])), hw.launch_log()
        finally:
            hw.close()

    want, _ = run(oracle.vtable(), {"kind": "sequential"})
    seq, _ = run(cuda, {"kind": "sequential"})
    assert_same_bits(seq, want)
    cuda.set_profiling(True)
    cuda.profile()
    got, log = run(cuda, {"kind": "device", "attention": "online", "launches": "merged"})
    prof = [rec[0] for rec in cuda.profile()]
    cuda.set_profiling(False)
    assert log.count("attention[online]") == c["L"] and sum(1 for n in log if n.endswith("+add")) == 2 * c["L"], log
    assert prof.count("k_gemm_i8") == 7 * c["L"] + 1 and prof.count("k_attn_fwd3") == c["L"], prof
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2.0**-3.5 * np.abs(want).max(), (np.abs(got - want).max(), np.abs(want).max())
    assert np.abs(got - want).mean() <= 2.0**-6.5 * np.abs(want).max(), (np.abs(got - want).mean(), np.abs(want).max())
    plain, _ = run(cuda, {"kind": "device"})
    assert np.abs(plain - want).max() <= 2.0**-3.5 * np.abs(want).max()
    assert np.abs(plain - want).mean() <= 2.0**-6.5 * np.abs(want).max()


def test_w8a8_merged_launches_keep_every_bit_at_the_7b_width(cuda):
    """The kernels that write a scaled site's codes themselves (the merged norm over rows of 4096 elements, sixteen
    vectors a lane, and the silu-times-up group) against the reference's launch list on this executor, one layer of
    the 7B model's width: the same logits, bit for bit."""
    import headline
    c = dict(V=256, D=4096, H=32, G=32, FF=512, L=1)
    p = models.llama_params(c)
    ids = np.random.default_rng(16).integers(0, c["V"], size=(1, 128), dtype=np.int64)
    h = models.give(Host(cuda, headline.realization(p, {"kind": "device"})).prepare("llama", **c), p)
    h.set_calibrating(True)
    h.call("apply", [ids], (1, 128, c["V"]))
    scales = headline.w8a8_scales(h.envelope())
    h.close()
    outs = []
    for order in ({"kind": "device"}, {"kind": "device", "launches": "merged"}):
        hw = models.give(Host(cuda, headline.w8a8_realization(p, order, scales)).prepare("llama", **c), p)
        hw.set_logging(True)
        outs.append(hw.call("apply", [ids], (1, 128, c["V"])))
        log = hw.launch_log()
        hw.close()
    assert log.count("rmsnorm[merged]") == 2 * c["L"] + 1
    assert np.isfinite(outs[0]).all() and np.abs(outs[0]).max() > 0
    assert_same_bits(outs[1], outs[0])
