"""The host program over the CPU oracle: launch sequences, realizations, errors.
No GPU: the executor under the host is the oracle's table of functions."""
import numpy as np
import pytest

import models
from presk_b200 import Host, PreskError, abi


def test_llama_tiny_matches_an_independent_numpy_statement(oracle):
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, c["V"], size=(2, 16), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(2, 16), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), p)
    logits = h.call("apply", [ids], (2, 16, c["V"]))
    want = models.llama_numpy(p, c, ids)
    np.testing.assert_allclose(logits, want, rtol=0, atol=2e-5 * np.abs(want).max() + 1e-6)
    loss = h.call("loss", [ids, y], ())
    np.testing.assert_allclose(loss, models.llama_numpy(p, c, ids, y), rtol=2e-6)


def test_llama_launch_list(oracle):
    """The launches of one call, by the reference's kernel names: prologue, 2 blocks, epilogue."""
    c = models.LLAMA_TINY
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), models.llama_params(c))
    h.set_logging(True)
    ids = np.zeros((2, 16), np.int64)
    h.call("apply", [ids], (2, 16, c["V"]))
    log = h.launch_log()
    norm = ["mul", "mean axis model", "fused 2 steps", "fused 2 steps"]
    rope = ["slice pair: 0..1", "slice pair: 1..2", "cos", "sin", "fused 3 steps", "fused 3 steps", "concat pair"]
    block = (norm + ["ein[batch, groups, per, seq, hd]"] + rope + ["ein[batch, groups, seq, hd]"] + rope + ["dot"]
             + ["ein[batch, groups, per, seq, seq2]", "sqrt", "div", "softmax axis seq2 where", "ein[batch, seq, groups, per, hd]", "ein[batch, seq, model]", "add"]
             + norm + ["dot", "fused 2 steps", "dot", "mul", "dot", "add"])
    prologue = ["causal_mask seq", "embed", "positions seq", "real", "neg", "positions rot", "real", "log", "fused 4 steps", "ein[seq, rot]"]
    assert log == prologue + block * c["L"] + norm + ["dot"]
    assert h.launches() == len(log)


def test_mixed_realization_sites(oracle):
    """A site named in `storage` is stored in its own type; the rest in the default."""
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    ids = np.arange(32, dtype=np.int64).reshape(2, 16) % c["V"]
    rz = {"default": "bf16", "order": {"kind": "sequential"}, "storage": {"RMSNorm.apply/%3": "f32", "RMSNorm.apply/%7": "f32", "Llama.apply/%11": "f32"},
          "params": {k: "bf16" for k in p}}
    h = models.give(Host(oracle.vtable(), rz).prepare("llama", **c), p)
    logits = h.call("apply", [ids], (2, 16, c["V"]))
    want = models.llama_numpy(p, c, ids)
    assert np.abs(logits - want).max() < 0.05 * np.abs(want).max()
    assert np.any(logits.view(np.uint32) & 0xFFFF)  # the logits site is f32: not every value is a bf16 number


def test_int8_weights(oracle):
    """`quant` paths are stored as int8 with one f32 scale a channel (quant.rs:128-167)."""
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    ids = np.arange(32, dtype=np.int64).reshape(2, 16) % c["V"]
    q = {k: {"bits": 8, "over": -2} for k in ("blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w")}
    h = models.give(Host(oracle.vtable(), {"default": "f32", "quant": q}).prepare("llama", **c), p)
    logits = h.call("apply", [ids], (2, 16, c["V"]))
    # against numpy with the weights dequantised by the same rule
    pq = dict(p)
    for k in q:
        w = p[k].astype(np.float64)
        s = (np.abs(w).max(axis=-2, keepdims=True) / 127.0).astype(np.float32)
        codes = np.clip(np.rint(w / s.astype(np.float64)), -127, 127)
        pq[k] = (codes.astype(np.float32) * s).astype(np.float32)
    want = models.llama_numpy(pq, c, ids)
    np.testing.assert_allclose(logits, want, rtol=0, atol=3e-5 * np.abs(want).max() + 1e-6)


def test_realization_errors(oracle):
    with pytest.raises(PreskError, match="no type"):
        Host(oracle.vtable(), "f33")
    with pytest.raises(PreskError, match="E7005"):
        Host(oracle.vtable(), {"default": "f32", "order": {"kind": "interleaved", "partials": 4}})
    with pytest.raises(PreskError, match="E7005"):
        Host(oracle.vtable(), {"default": "f32", "accum": {"Dense.apply/%3": "i32"}})
    # quant entries the reference accepts and this host does not run: a power-of-two scheme (quant.rs:30-38) and an
    # axis given by name (quant.rs:46-49); both refused, neither read as something else
    with pytest.raises(PreskError, match="E7005.*pow2"):
        Host(oracle.vtable(), {"default": "f32", "quant": {"blocks.attn.wq": {"bits": 8, "over": -2, "scheme": "pow2"}}})
    with pytest.raises(PreskError, match="E7005.*by position"):
        Host(oracle.vtable(), {"default": "f32", "quant": {"blocks.attn.wq": {"bits": 8, "over": "model"}}})
    Host(oracle.vtable(), {"default": "f32", "quant": {"blocks.attn.wq": {"bits": 8, "over": -2, "scheme": "absmax"}}}).close()
    h = Host(oracle.vtable(), {"default": "f32", "params": {"blocks.attn.wz": "bf16"}})
    with pytest.raises(PreskError, match="no parameter of Llama"):
        h.prepare("llama", **models.LLAMA_TINY)
    h = Host(oracle.vtable(), "f32").prepare("mlp")
    with pytest.raises(PreskError, match="was not given"):
        h.call("apply", [np.zeros((4, 784), np.float32)], (4, 10))


def test_overflow_guard_stops_the_run(oracle):
    """Inputs scaled by 2^20 overflow the binary16 store of the `dot` (the contraction-plus-LayerNorm workload): E7007."""
    rng = np.random.default_rng(5)
    n = 64
    x, w = rng.standard_normal((n, n)).astype(np.float32), rng.standard_normal((n, n)).astype(np.float32)
    for dtype, scale, overflows in [("f16", 1.0, False), ("f16", 2.0**20, True), ("e8m15", 2.0**20, False), ("bf16", 2.0**20, False)]:
        h = Host(oracle.vtable(), dtype).prepare("contract_ln")
        h.set_param("ln.γ", np.ones(n, np.float32))
        h.set_param("ln.β", np.zeros(n, np.float32))
        if overflows:
            with pytest.raises(PreskError, match="E7007"):
                h.call("apply", [x * scale, w * scale], (n, n))
        else:
            out = h.call("apply", [x * scale, w * scale], (n, n))
            assert np.all(np.isfinite(out))


def test_mlp_config1_shapes(oracle):
    p = models.mlp_params()
    x, y = models.mlp_inputs(64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("mlp"), p)
    h.set_logging(True)
    loss = h.call("loss", [x, y], ())
    assert h.launch_log() == ["dot", "add", "relu", "dot", "add", "cross_entropy", "mean"]
    hid = np.maximum(x.astype(np.float64) @ p["l1.w"], 0)
    lg = hid @ p["l2.w"]
    want = (np.log(np.exp(lg - lg.max(-1, keepdims=True)).sum(-1)) + lg.max(-1) - lg[np.arange(64), y]).mean()
    np.testing.assert_allclose(loss, want, rtol=1e-5)


def test_gpt_config2_matches_numpy_and_its_launch_list(oracle):
    """examples/corpus/nlp/05_gpt.psk at small constants: LayerNorm, biased linear maps, split_heads and
    merge_heads, masked softmax, GELU, learned positions, dropout masks of ones."""
    c = models.GPT_TINY
    T = 16
    p = models.gpt_params(c, T)
    rng = np.random.default_rng(8)
    ids = rng.integers(0, c["V"], size=(3, T), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(3, T), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("gpt", **c), p)
    h.set_logging(True)
    logits = h.call("apply", [ids], (3, T, c["V"]))
    want = models.gpt_numpy(p, c, ids)
    np.testing.assert_allclose(logits, want, rtol=0, atol=3e-5 * np.abs(want).max() + 1e-6)
    ln = ["mean axis model", "fused 2 steps", "mean axis model", "fused 2 steps", "fused 4 steps"]
    lin = ["dot", "add"]
    block = (ln + (lin + ["split_heads 4x8"]) * 3 + ["ein[batch, heads, seq, seq2]", "sqrt", "div", "softmax axis seq2 where", "mul", "ein[batch, heads, seq, hd]", "merge_heads 4x8"]
             + lin + ["fused 2 steps"] + ln + lin + ["gelu"] + lin + ["fused 2 steps"])
    assert h.launch_log() == ["causal_mask seq", "embed", "positions seq", "embed", "fused 2 steps"] + block * c["L"] + ln + ["dot"]
    loss = h.call("loss", [ids, y], ())
    np.testing.assert_allclose(loss, models.gpt_numpy(p, c, ids, y), rtol=3e-6)


def test_calibrate_envelope(oracle):
    """`presk calibrate` on the executor: per-site max |x|, least non-zero |x| and range of what was run."""
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    ids = np.random.default_rng(3).integers(0, c["V"], size=(2, 16), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), p)
    h.set_calibrating(True)
    logits = h.call("apply", [ids], (2, 16, c["V"]))
    env = h.envelope()
    mx, mn, lo, hi = env["Llama.apply/%11"]
    assert mx == np.abs(logits).max() and lo == logits.min() and hi == logits.max()
    assert mn == np.abs(logits)[logits != 0].min()
    emb = p["tok"][ids]
    assert env["Llama.apply/%4"][0] == np.abs(emb).max()
    # a site run once per layer holds the largest of its launches; the softmax's values lie in [0, 1]
    assert env["Attention.apply/%21"][2] == 0.0 and 0.99 < env["Attention.apply/%21"][3] <= 1.0
    assert len(env) > 25
    # a second call folds into the same envelope
    h.call("apply", [(ids + 1) % c["V"]], (2, 16, c["V"]))
    assert h.envelope()["Llama.apply/%11"][0] >= mx


def test_blockwise_attention_is_its_four_launches_on_the_oracle(oracle):
    """`order: {kind: device, attention: blockwise}` makes one launch of scores, division, softmax and
    weighted values; its value is defined as that of the four, so over the oracle the bits agree."""
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    ids = np.random.default_rng(8).integers(0, c["V"], size=(2, 16), dtype=np.int64)
    outs, logs = [], []
    for order in ({"kind": "device"}, {"kind": "device", "attention": "blockwise"}, {"kind": "device", "attention": "online"}):
        h = models.give(Host(oracle.vtable(), {"default": "bf16", "order": order}).prepare("llama", **c), p)
        h.set_logging(True)
        outs.append(h.call("apply", [ids], (2, 16, c["V"])))
        logs.append(h.launch_log())
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    assert logs[1].count("attention[blockwise]") == c["L"]
    assert "softmax axis seq2 where" in logs[0] and "softmax axis seq2 where" not in logs[1]
    assert len(logs[0]) - len(logs[1]) == 3 * c["L"]
    # `attention: online` is the same launch with another way of fusing it allowed: the same definition, the same bits here
    assert np.array_equal(outs[0].view(np.uint32), outs[2].view(np.uint32))
    assert logs[2].count("attention[online]") == c["L"] and len(logs[2]) == len(logs[1])
    with pytest.raises(PreskError) as e:
        Host(oracle.vtable(), {"default": "bf16", "order": {"kind": "sequential", "attention": "blockwise"}})
    assert e.value.code == 7005


def test_merged_launches_keep_every_bit(oracle):
    """`launches: merged` reads slices as views, writes a concatenation's halves in place and computes the
    rotary cos/sin once a call: fewer launches, the same bits, under either order and with GQA."""
    c = dict(models.LLAMA_TINY, G=1)
    p = models.llama_params(c)
    ids = np.random.default_rng(9).integers(0, c["V"], size=(2, 16), dtype=np.int64)
    for default in ("f32", "bf16"):
        outs, logs = [], []
        for order in ({"kind": "sequential"}, {"kind": "sequential", "launches": "merged"}, {"kind": "device", "launches": "merged"}):
            h = models.give(Host(oracle.vtable(), {"default": default, "order": order}).prepare("llama", **c), p)
            h.set_logging(True)
            outs.append(h.call("apply", [ids], (2, 16, c["V"])))
            outs.append(h.call("apply", [ids], (2, 16, c["V"])))  # a second call: nothing kept from the first
            logs.append(h.launch_log())
        # under the device order the norm's four launches are offered as one too (the oracle runs the four)
        assert logs[2].count("rmsnorm[merged]") == 2 * c["L"] + 1 and "mean axis model" not in logs[2]
        for o in outs[1:]:
            assert np.array_equal(outs[0].view(np.uint32), o.view(np.uint32))
        assert not any(n.startswith("slice") or n.startswith("concat") for n in logs[1])
        assert logs[1].count("cos") == 1 and logs[0].count("cos") == 2 * c["L"]  # the log is that of the last call
        assert len(logs[1]) < len(logs[0])


def test_e4m3_weights_are_the_bf16_model_on_rounded_weights(oracle):
    """`params: e4m3fn` under bf16 sites: the kernels' loads widen the codes exactly, so the call is, bit for bit,
    the bf16 model run on weights rounded to e4m3fn beforehand."""
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    narrow = ("blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w")
    ids = np.random.default_rng(3).integers(0, c["V"], size=(2, 16), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), {"default": "bf16", "params": {k: "e4m3fn" for k in narrow}}).prepare("llama", **c), p)
    got = h.call("apply", [ids], (2, 16, c["V"]))
    rounded = dict(p)
    for k in narrow:
        w = np.asarray(p[k], np.float32)
        rounded[k] = oracle.widen(oracle.convert(w, abi.E4M3), abi.E4M3, w.size).reshape(w.shape)
    want = models.give(Host(oracle.vtable(), {"default": "bf16"}).prepare("llama", **c), rounded).call("apply", [ids], (2, 16, c["V"]))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    plain = models.give(Host(oracle.vtable(), {"default": "bf16"}).prepare("llama", **c), p).call("apply", [ids], (2, 16, c["V"]))
    assert not np.array_equal(plain, want)


@pytest.mark.parametrize("rz", ["f32", "bf16", {"default": "bf16", "order": {"kind": "sequential", "launches": "merged"}}])
def test_step_after_prefill_is_the_whole_window_recomputed(oracle, rz):
    """Generation with a cache of keys and values: `prefill` on a window, then `step` a new position at a time. The
    reference recomputes the whole window for every token (presk-serve/src/lib.rs:241); under the sequential order
    the cached step must give the bits of that recompute's last row, and `prefill` those of `apply`. GQA (G < H)."""
    c = dict(V=100, D=32, H=4, G=2, FF=64, L=2)
    p = models.llama_params(c)
    rng = np.random.default_rng(12)
    ids = rng.integers(0, c["V"], size=(3, 16), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), rz).prepare("llama", TMAX=16, **c), p)
    ref = models.give(Host(oracle.vtable(), rz).prepare("llama", **c), p)
    first = h.call("prefill", [ids[:, :11]], (3, 11, c["V"]))
    assert np.array_equal(first.view(np.uint32), ref.call("apply", [ids[:, :11]], (3, 11, c["V"])).view(np.uint32))
    for t in range(11, 16):
        got = h.call("step", [ids[:, t:t + 1]], (3, 1, c["V"]))
        want = ref.call("apply", [ids[:, :t + 1]], (3, t + 1, c["V"]))[:, -1:, :]
        assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(want).view(np.uint32)), t
    with pytest.raises(PreskError, match="used up"):
        h.call("step", [ids[:, :1]], (3, 1, c["V"]))
    with pytest.raises(PreskError, match="no `prefill`"):
        ref.prepare("llama", TMAX=8, **c).call("step", [ids[:, :1]], (3, 1, c["V"]))


def test_w8a8_step_after_prefill_is_the_whole_window_recomputed(oracle):
    """The same with the W8A8 realization in its fuller form (tests/headline.py, `attn_out`: the weighted values a
    scaled site, every projection's sums in i32): static scales make a position's codes independent of the window's
    other positions, so a cached step is still the recompute's last row, bit for bit, with the launches apart and
    with the attention issued as one launch that writes the codes."""
    import headline
    c = dict(V=100, D=32, H=4, G=2, FF=64, L=2)
    p = models.llama_params(c)
    ids = np.random.default_rng(13).integers(0, c["V"], size=(2, 12), dtype=np.int64)
    cal = models.give(Host(oracle.vtable(), headline.realization(p, {"kind": "sequential"})).prepare("llama", **c), p)
    cal.set_calibrating(True)
    cal.call("apply", [ids], (2, 12, c["V"]))
    scales = headline.w8a8_scales(cal.envelope())
    for order in ({"kind": "sequential"}, {"kind": "device", "attention": "online", "launches": "merged"}):
        rz = headline.w8a8_realization(p, order, scales, attn_out=True)
        h = models.give(Host(oracle.vtable(), rz).prepare("llama", TMAX=12, **c), p)
        ref = models.give(Host(oracle.vtable(), rz).prepare("llama", **c), p)
        h.set_logging(True)
        first = h.call("prefill", [ids[:, :8]], (2, 8, c["V"]))
        assert np.array_equal(first.view(np.uint32), ref.call("apply", [ids[:, :8]], (2, 8, c["V"])).view(np.uint32))
        for t in range(8, 12):
            got = h.call("step", [ids[:, t:t + 1]], (2, 1, c["V"]))
            want = ref.call("apply", [ids[:, :t + 1]], (2, t + 1, c["V"]))[:, -1:, :]
            assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(want).view(np.uint32)), (order, t)
        if order["kind"] == "device":
            assert h.launch_log().count("attention[online]") == c["L"]  # the step's attention is one launch, codes out


def test_w8a8_llama_merged_launches_keep_every_bit(oracle):
    """The W8A8 realization of the Llama program (tests/headline.py: i8 activations at the projections' inputs with
    static scales from a calibration, int8 weights, i32 sums): under `launches: merged` the norm and the silu group
    write their `scaled` sites themselves, and the logits are the bits of the reference's launch list."""
    import headline
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    ids = np.random.default_rng(3).integers(0, c["V"], size=(2, 16), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), headline.realization(p, {"kind": "sequential"})).prepare("llama", **c), p)
    h.set_calibrating(True)
    h.call("apply", [ids], (2, 16, c["V"]))
    scales = headline.w8a8_scales(h.envelope())
    assert all(s > 0 for s in scales.values())
    outs, logs = [], []
    for order in ({"kind": "sequential"}, {"kind": "device"}, {"kind": "device", "launches": "merged"}):
        hw = models.give(Host(oracle.vtable(), headline.w8a8_realization(p, order, scales)).prepare("llama", **c), p)
        hw.set_logging(True)
        outs.append(hw.call("apply", [ids], (2, 16, c["V"])))
        logs.append(hw.launch_log())
    assert np.isfinite(outs[0]).all() and np.abs(outs[0]).max() > 0
    assert np.array_equal(outs[1].view(np.uint32), outs[2].view(np.uint32))
    assert logs[2].count("rmsnorm[merged]") == 2 * c["L"] + 1 and len(logs[2]) < len(logs[1])
    # against the bf16 realization: the quantisation's error, a few percent of the logits' scale
    ref = models.give(Host(oracle.vtable(), headline.realization(p, {"kind": "sequential"})).prepare("llama", **c), p).call("apply", [ids], (2, 16, c["V"]))
    assert np.abs(outs[0] - ref).max() <= 0.1 * np.abs(ref).max()
    # The fuller form: the weighted values a scaled site too, the out-projection's sums in i32. Merged, the
    # out-projection and the down-projection each take their residual along (one launch with the integer sums), and
    # the fused attention writes the codes: the same bits as the launch list.
    outs2, logs2 = [], []
    for order in ({"kind": "device"}, {"kind": "device", "launches": "merged", "attention": "blockwise"}):
        hw = models.give(Host(oracle.vtable(), headline.w8a8_realization(p, order, scales, attn_out=True)).prepare("llama", **c), p)
        hw.set_logging(True)
        outs2.append(hw.call("apply", [ids], (2, 16, c["V"])))
        logs2.append(hw.launch_log())
    assert np.array_equal(outs2[0].view(np.uint32), outs2[1].view(np.uint32))
    assert sum(1 for n in logs2[1] if n.endswith("+add")) == 2 * c["L"] and logs2[1].count("attention[blockwise]") == c["L"]
    assert not np.array_equal(outs2[0], outs[1]) # (another realization: the out-projection's operand is rounded to codes)
    assert np.abs(outs2[0] - ref).max() <= 0.1 * np.abs(ref).max()
