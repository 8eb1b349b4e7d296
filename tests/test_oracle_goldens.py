"""Known answers of the reference pin the oracle and the host program:

  - the first four normal draws of the key seed 0 names and the FNV fold of the
    next 100 000 (crates/presk-interp/src/key.rs:86-93) pin the build of the
    reference's C runtime in oracle/_ref (ChaCha keys, musl log and cos);
  - the seed-0 outputs of `LayerNorm{8}.apply` and `RMSNorm{8}.apply` at
    batch 3 from the exact interpreter (tests/run/*.snap, 12 digits) pin the
    launch sequences of the host program and the oracle's kernels: an f32
    realization must agree with the exact reals to f32 accuracy.
"""
import ctypes as C
import json
import os

import numpy as np
import pytest

import models
from presk_b200 import Host, abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = json.load(open(os.path.join(ROOT, "tests", "golden", "reference_vectors.json")))


def normals(ref, seed, split_of, index, n):
    out = np.empty(n, dtype=np.float64)
    ref.ref_normals.argtypes = [C.c_uint64, C.c_int, C.c_int, C.c_void_p, C.c_size_t]
    ref.ref_normals(seed, split_of, index, out.ctypes.data, n)
    return out


def test_key_draws_are_the_reference_s(ref):
    x = normals(ref, 0, 0, 0, 100_004)
    assert [int(b) for b in x[:4].view(np.uint64)] == GOLD["seed0_first_normals_bits"]
    h = 0xCBF29CE484222325
    for b in x[4:].view(np.uint64).tolist():
        h = ((h ^ b) * 0x00000100000001B3) & 0xFFFFFFFFFFFFFFFF
    assert h == GOLD["seed0_next_100000_fnv"]


@pytest.mark.parametrize("model,key", [("layernorm", "layernorm_apply"), ("rmsnorm", "rmsnorm_apply")])
def test_norm_goldens_on_the_oracle(oracle, ref, model, key):
    want = np.array(GOLD[key]["values"])
    b, d = GOLD[key]["shape"]
    # the entry's parameters are (θ, x, eps): x is drawn from the second of three keys
    x = normals(ref, 0, 3, 1, b * d).reshape(b, d)
    h = Host(oracle.vtable(), "f32").prepare(model)
    h.set_param("γ", np.ones(d))
    if model == "layernorm":
        h.set_param("β", np.zeros(d))
    h.set_logging(True)
    got = h.call("apply", [x], (b, d), np.float32)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-6)
    log = h.launch_log()
    if model == "layernorm":
        # crates/presk-core/tests/snapshots/lower__core_minigpt.snap + fusion.rs: five launches
        assert log == ["mean axis model", "fused 2 steps", "mean axis model", "fused 2 steps", "fused 4 steps"]
    else:
        assert log == ["pow 2", "mean axis model", "fused 2 steps", "fused 2 steps"]


def test_bf16_storage_rounds_every_site(oracle, ref):
    """Under `--realize bf16` each launch's output is a bf16 number (storage rounding at every site)."""
    b, d = 3, 8
    x = normals(ref, 0, 3, 1, b * d).reshape(b, d)
    h = Host(oracle.vtable(), "bf16").prepare("rmsnorm")
    h.set_param("γ", np.ones(d))
    got = h.call("apply", [x], (b, d), np.float32)
    bits = got.view(np.uint32)
    assert np.all(bits & 0xFFFF == 0)
    want = np.array(GOLD["rmsnorm_apply"]["values"])
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)


def draws_at(ref, kind, seed, path, n):
    out = np.empty(n, dtype=np.float64)
    p = (C.c_int * len(path))(*path)
    fn = ref.ref_uniforms_at if kind == "uniform" else ref.ref_normals_at
    fn.argtypes = [C.c_uint64, C.POINTER(C.c_int), C.c_int, C.c_void_p, C.c_size_t]
    fn(seed, p, len(path), out.ctypes.data, n)
    return out


def spec_mlp_seed0(ref, d=4, b=2):
    """The arguments `presk run examples/spec/mlp/mlp.psk --entry mse --const D=4 --const B=2` synthesizes from
    seed 0 (crates/presk-interp/src/run.rs:73-101, 315-366): the entry's three arguments θ, x, y take the three
    children of the master key; θ is MLP.init of its key (split in two for l1, l2; each Linear.init splits its key
    in two and draws w from the first by xavier_uniform, host.rs:1641-1657; b is zeros); x and y are normal draws."""
    bound = np.sqrt(6.0 / (d + 4 * d))
    params = {
        "l1.w": ((2.0 * draws_at(ref, "uniform", 0, [0, 0, 0], d * 4 * d) - 1.0) * bound).reshape(d, 4 * d),
        "l1.b": np.zeros(4 * d),
        "l2.w": ((2.0 * draws_at(ref, "uniform", 0, [0, 1, 0], d * 4 * d) - 1.0) * bound).reshape(4 * d, d),
        "l2.b": np.zeros(d),
    }
    x = draws_at(ref, "normal", 0, [1], b * d).reshape(b, d)
    y = draws_at(ref, "normal", 0, [2], b * d).reshape(b, d)
    return params, x, y


def test_mlp_loss_and_gradient_goldens_on_the_oracle(oracle, ref):
    """tests/run/mlp_mse.snap and mlp_mse_grad.snap (exact interpreter, 12 digits): the forward pass and the
    reverse-mode program of crates/presk-core/tests/snapshots/ad__ad_mlp.snap, launch by launch, in f32."""
    params, x, y = spec_mlp_seed0(ref)
    h = Host(oracle.vtable(), "f32").prepare("mlp_spec", D=4)
    for k, v in params.items():
        h.set_param(k, v)
    h.set_logging(True)
    loss = h.call("mse", [x, y], (), np.float32)
    assert abs(float(loss) - GOLD["mlp_mse"]) <= 2e-6
    assert h.launch_log() == ["dot", "add", "gelu", "dot", "add", "fused 2 steps", "mean"]
    h.call("mse_grad", [x, y], (4, 16), np.float32)
    linear_bwd = ["sum_to", "dot_vjp_l", "dot_vjp_r", "add", "add"]
    assert h.launch_log() == (["dot", "add", "gelu", "dot", "add", "sub", "mean_vjp", "fused 3 steps", "sum_to"]
                              + linear_bwd + ["fused 2 steps"] + linear_bwd + ["add"] * 4)
    for path, g in GOLD["mlp_mse_grad"].items():
        got = h.result(path, tuple(g["shape"]), np.float32)
        np.testing.assert_allclose(got, np.array(g["values"]), rtol=0, atol=2e-6, err_msg=path)


@pytest.mark.parametrize("entry,key", [("attention", "rope_attention2"), ("attention3", "rope_attention3")])
def test_rope_attention_golden_on_the_oracle(oracle, ref, entry, key):
    """tests/run/rope_attention2.snap (and rope_attention3.snap: the base 500 000 with Llama 3's frequency scaling): causal attention with rotary embeddings (examples/spec/rope/rope.psk
    `attention2`, H = 2, HD = 8, B = 2, T = 8, seed 0) from the exact interpreter. The host's Llama attention
    with G = H is the same function (llama.psk's `per` axis has length 1); its parameters are the four children of
    θ's key drawn normal(std = 0.02) in declaration order, x the second argument's key."""
    g = GOLD[key]
    b, t, d = g["shape"]
    h = Host(oracle.vtable(), "f32").prepare("llama", V=8, D=d, H=2, G=2, FF=8, L=1)
    for i, name in enumerate(("wq", "wk", "wv", "wo")):
        h.set_param("blocks.attn." + name, (draws_at(ref, "normal", 0, [0, i], d * d) * 0.02).reshape(1, d, d))
    x = draws_at(ref, "normal", 0, [1], b * t * d).reshape(b, t, d)
    got = h.call(entry, [x], (b, t, d), np.float32)
    want = np.array(g["values"])
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-8)  # outputs are of magnitude 8e-3: f32 accuracy


def indices_at(ref, seed, path, bound, n):
    """Indices below `bound` as an idx input is synthesized (run.rs:327-333): floor(uniform · bound)."""
    return (draws_at(ref, "uniform", seed, path, n) * bound).astype(np.int64)


def test_concat_loss_golden_on_the_oracle(oracle, ref):
    """tests/run/concat_loss.snap: examples/spec/concat/concat.psk `loss` at B = 2, T = 8, seed 0 (slices of an index
    window, concatenated weights, min/max/clamp groups, embed, cross-entropy, mean). θ is the first argument's key
    through Toy.init (its own parameters tok and head first, then the module it uses, whose init draws wq, wk, wv),
    the window the second's."""
    v, d, b, t = 64, 16, 2, 8
    h = Host(oracle.vtable(), "f32").prepare("toy", V=v, D=d)
    h.set_param("tok", (draws_at(ref, "normal", 0, [0, 0], v * d) * 0.02).reshape(v, d))
    for i, name in enumerate(("wq", "wk", "wv")):
        h.set_param("qkv." + name, (draws_at(ref, "normal", 0, [0, 2, i], d * d) * 0.02).reshape(d, d))
    h.set_param("head", (draws_at(ref, "normal", 0, [0, 1], d * v) * 0.02).reshape(d, v))
    w = indices_at(ref, 0, [1], v, b * (t + 1)).reshape(b, t + 1)
    got = float(h.call("loss", [w], (), np.float32))
    assert abs(got - GOLD["concat_loss"]) <= 2e-6 * GOLD["concat_loss"], (got, GOLD["concat_loss"])


def test_concat_loss_grad_golden_on_the_oracle(oracle, ref):
    """tests/run/concat_loss_grad.snap: the gradient of the same loss, every leaf (tok, head, qkv.wq, qkv.wk, qkv.wv):
    cross_entropy_vjp, dot_vjp_l/r, the max/min rule at q, k and v, slice_vjp, the concatenation's cotangent cut
    in two, embed_vjp. wk's leaf is of magnitude 4e-7 (it flows through leaky's 0.01 and k's small values): an
    absolute tolerance scaled to each leaf."""
    v, d, b, t = 64, 16, 2, 8
    h = Host(oracle.vtable(), "f32").prepare("toy", V=v, D=d)
    h.set_param("tok", (draws_at(ref, "normal", 0, [0, 0], v * d) * 0.02).reshape(v, d))
    for i, name in enumerate(("wq", "wk", "wv")):
        h.set_param("qkv." + name, (draws_at(ref, "normal", 0, [0, 2, i], d * d) * 0.02).reshape(d, d))
    h.set_param("head", (draws_at(ref, "normal", 0, [0, 1], d * v) * 0.02).reshape(d, v))
    w = indices_at(ref, 0, [1], v, b * (t + 1)).reshape(b, t + 1)
    h.set_logging(True)
    h.call("loss_grad", [w], (v, d), np.float32)
    log = h.launch_log()
    assert log.count("cross_entropy_vjp") == 1 and log.count("embed_vjp") == 1 and log.count("dot_vjp_l") == 2 and log.count("dot_vjp_r") == 2
    assert sum(1 for n in log if n.startswith("slice_vjp out")) == 3 and log.count("heaviside") == 4
    for path, g in GOLD["concat_loss_grad"].items():
        want = np.array(g["values"])
        got = h.result(path, tuple(g["shape"]), np.float32)
        np.testing.assert_allclose(got, want, rtol=0, atol=3e-6 * np.abs(want).max(), err_msg=path)
    # rows of tokens the window does not hold stay zero
    tok = h.result("tok", (v, d), np.float32)
    absent = np.setdiff1d(np.arange(v), w[:, :t])
    assert absent.size and not tok[absent].any()


def test_stack_grad_golden_on_the_oracle(oracle, ref):
    """tests/run/stack_grad.snap: examples/tests/data/stack_grad.psk `loss_grad` at B = 2, seed 0: the gradient through
    a fold over a stacked parameter tree (three blocks x + tanh(x·w + b) * scale, the loss mean(y^2)). Tower.init
    splits θ's key once (its one `use`), the stack splits that in L, each block's init in two: w xavier_uniform
    (fan_in = fan_out = 3: bound 1), b normal(std = 0.5); x and the rank-0 scale are the second and third
    arguments' keys."""
    L, d, b = 3, 3, 2
    h = Host(oracle.vtable(), "f32").prepare("tower", D=d, L=L)
    w = np.stack([(2.0 * draws_at(ref, "uniform", 0, [0, 0, l, 0], d * d) - 1.0).reshape(d, d) for l in range(L)])
    bias = np.stack([draws_at(ref, "normal", 0, [0, 0, l, 1], d) * 0.5 for l in range(L)])
    h.set_param("blocks.w", w)
    h.set_param("blocks.b", bias)
    x = draws_at(ref, "normal", 0, [1], b * d).reshape(b, d)
    scale = draws_at(ref, "normal", 0, [2], 1).reshape(())
    h.set_logging(True)
    h.call("loss_grad", [x, scale], (L, d, d), np.float32)
    log = h.launch_log()
    assert log.count("dot_vjp_l") == L and log.count("dot_vjp_r") == L and log.count("sum_to") == L and log.count("scatter_params") == 2 * L
    for path, g in GOLD["stack_grad"].items():
        want = np.array(g["values"])
        got = h.result(path, tuple(g["shape"]), np.float32)
        np.testing.assert_allclose(got, want, rtol=0, atol=3e-6 * np.abs(want).max(), err_msg=path)
    # and the loss the gradient belongs to, against a central difference in f64 of the same function
    def loss_at(wv):
        y = x.astype(np.float64)
        for l in range(L):
            y = y + np.tanh(y @ wv[l] + bias[l]) * float(scale)
        return np.mean(y * y)
    got_loss = float(h.call("loss", [x, scale], (), np.float32))
    assert abs(got_loss - loss_at(w)) <= 2e-6 * abs(loss_at(w))


def test_minigpt_zero_head_goldens_on_the_oracle(oracle):
    """tests/run/minigpt_forward.snap and minigpt_loss.snap (examples/spec/minigpt, V = 64, D = 16, H = 2, L = 2,
    B = 2, T = 8, seed 0): MiniGPT's head is initialised to zeros, so every logit is exactly 0 and the loss is ln 64
    whatever the other parameters are. The host's GPT (examples/corpus/nlp/05_gpt.psk, the same decoder with learned
    positions) under the same constants and a zero head must give the same two values: what this pins is the head
    contraction on exact zeros, cross_entropy's `ln z + m - x[y]` and the mean, not the key derivation."""
    g = GOLD["minigpt_forward"]
    assert g["all_equal_to"] == 0 and g["distinct"] == 1
    c = dict(V=64, D=16, H=2, L=2)
    b, t, v = g["shape"]
    p = models.gpt_params(c, t)
    p["head"] = np.zeros_like(p["head"])
    rng = np.random.default_rng(0)
    ids = rng.integers(0, c["V"], size=(b, t), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(b, t), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("gpt", **c), p)
    logits = h.call("apply", [ids], (b, t, v))
    assert np.all(logits == 0.0)
    loss = float(h.call("loss", [ids, y], ()))
    assert abs(loss - GOLD["minigpt_loss"]) <= 1e-6
