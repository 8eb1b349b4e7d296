"""The benchmark's own widths, at sizes the CPU oracle finishes in seconds.

The throughput number is quoted on a Llama-7B-shaped prefill (d 4096, 32 heads of 128, SwiGLU 11008,
vocabulary 32000, 32 layers, sequence 2048). The oracle cannot run that whole, but it runs one layer of that
width on a short sequence; the functions here build such a case once and run it over both executors, for
tests/test_gpu_headline.py and for bench.py's parity pre-flight (outside its timed region; the oracle is the
checker there, never the thing measured).

TEST INFRASTRUCTURE: nothing under presk_b200/ imports this module.
"""
import numpy as np

WIDTH_7B = dict(V=32000, D=4096, H=32, G=32, FF=11008)
QUANTISED = ("blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w")
F32_SITES = {"RMSNorm.apply/%3": "f32", "RMSNorm.apply/%7": "f32", "Llama.apply/%11": "f32", "loss/%5": "f32", "loss/%6": "f32"}


def llama_params_f32(c, seed=0, std=0.02):
    """normal(0, std) weights and unit norms, drawn in float32 (a 7B-wide layer is half a billion numbers)."""
    rng = np.random.default_rng(seed)
    V, D, FF, L, H = c["V"], c["D"], c["FF"], c["L"], c["H"]
    G = c.get("G", H)
    HD = D // H

    def n(*s):
        a = rng.standard_normal(s, dtype=np.float32)
        a *= np.float32(std)
        return a

    return {
        "tok": n(V, D), "head": n(D, V), "norm.γ": np.ones(D, np.float32),
        "blocks.n1.γ": np.ones((L, D), np.float32), "blocks.n2.γ": np.ones((L, D), np.float32),
        "blocks.attn.wq": n(L, D, D), "blocks.attn.wk": n(L, D, G * HD), "blocks.attn.wv": n(L, D, G * HD), "blocks.attn.wo": n(L, D, D),
        "blocks.ff.gate.w": n(L, D, FF), "blocks.ff.up.w": n(L, D, FF), "blocks.ff.down.w": n(L, FF, D),
    }


def realization(paths, order, weights="bf16"):
    """The benchmark's realization (bf16 sites, f32 norm statistics, logits and loss) under `order`;
    `weights`: "bf16", "int8" (a `quant` entry a projection) or "e4m3fn" (a `params` entry)."""
    rz = {"default": "bf16", "order": order, "storage": dict(F32_SITES)}
    rz["params"] = {p: ("e4m3fn" if weights == "e4m3fn" and p in QUANTISED else "bf16") for p in paths if not (weights == "int8" and p in QUANTISED)}
    if weights == "int8":
        rz["quant"] = {p: {"bits": 8, "over": -2} for p in QUANTISED}
    return rz


# W8A8: the activations that feed the projections stored as i8 codes with a static scale (`scaled` sites: the norm's
# result and silu(gate)·up), every projection's weights and the head's as int8 (`quant`), and those contractions'
# products and sums counted in i32 (`product`, `accum`), as examples/tests/formats/w8a8.json declares them for a Dense
# layer. In the first form the attention's result stays bf16, so the out-projection reads it against int8 weights
# widened exactly; with `attn_out` the weighted values are a scaled site too and the out-projection counts in i32 like
# the other six.
W8A8_SCALED_SITES = ("RMSNorm.apply/%10", "SwiGLU.apply/%7")
W8A8_INT_SUMS = ("Attention.apply/%7", "Attention.apply/%11", "Attention.apply/%14", "Dense.apply/%3", "Llama.apply/%11")
W8A8_ATTN_OUT_SITE, W8A8_ATTN_OUT_SUMS = "Attention.apply/%22", "Attention.apply/%26"
W8A8_QUANTISED = QUANTISED + ("head",)


def w8a8_realization(paths, order, scales, attn_out=False):
    """`scales`: {site: scale} of the scaled sites (from an envelope: largest magnitude / 127)."""
    scaled = W8A8_SCALED_SITES + ((W8A8_ATTN_OUT_SITE,) if attn_out else ())
    sums = W8A8_INT_SUMS + ((W8A8_ATTN_OUT_SUMS,) if attn_out else ())
    rz = {"default": "bf16", "order": order, "storage": dict(F32_SITES)}
    rz["params"] = {p: "bf16" for p in paths if p not in W8A8_QUANTISED}
    rz["quant"] = {p: {"bits": 8, "over": -2} for p in W8A8_QUANTISED}
    rz["scaled"] = {site: {"int": "i8/sat", "scale": float(np.float32(scales[site])), "zero": 0} for site in scaled}
    rz["product"] = {site: "i32" for site in sums}
    rz["accum"] = {site: "i32" for site in sums}
    return rz


def w8a8_scales(envelope):
    """A static scale a scaled site from a calibration's envelope {site: (max |x|, ...)}: absmax / 127, as `presk
    scales` computes an absmax scheme's (presk-rt/src/lib.rs:287-360)."""
    return {site: float(np.float32(envelope[site][0]) / np.float32(127.0)) for site in W8A8_SCALED_SITES + (W8A8_ATTN_OUT_SITE,)}


BENCH_ORDER = {"kind": "device", "attention": "blockwise", "launches": "merged"}
ORACLE_ORDER = {"kind": "sequential"}


def give(host, params):
    for k, v in params.items():
        host.set_param(k, v)
    return host


def llama_width_parity(cuda_executor, oracle, B=1, T=256, weights="bf16", consts=None, seed=0, want_loss=True, params=None, order=None):
    """One layer of the 7B width over both executors: the CUDA one under the benchmark's order (tensor-core
    contractions, the blockwise attention kernel, merged launches), the oracle under the sequential order with
    the reference's launch list. Returns a dict with the logits' largest difference, their scale, and both losses."""
    from presk_b200 import Host
    c = dict(consts or WIDTH_7B, L=1)
    p = params if params is not None else llama_params_f32(c, seed)
    rng = np.random.default_rng(seed + 1)
    ids = rng.integers(0, c["V"], size=(B, T), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(B, T), dtype=np.int64)
    out = {"shape": f"llama L=1 V={c['V']} D={c['D']} H={c['H']} G={c['G']} FF={c['FF']} B={B} T={T}, weights {weights}"}
    res = {}
    make = lambda how: realization(p, how, weights)
    if weights in ("w8a8", "w8a8_attn_out"):
        # static scales from a calibration of the bf16 realization on the CUDA executor; both sides then run the same
        # W8A8 realization
        hc = give(Host(cuda_executor, realization(p, {"kind": "device"})).prepare("llama", **c), p)
        hc.set_calibrating(True)
        hc.call("apply", [ids], (B, T, c["V"]))
        scales = w8a8_scales(hc.envelope())
        hc.close()
        make = lambda how: w8a8_realization(p, how, scales, attn_out=weights == "w8a8_attn_out")
    for name, ex, how in (("gpu", cuda_executor, order or BENCH_ORDER), ("oracle", oracle.vtable(), ORACLE_ORDER)):
        h = give(Host(ex, make(how)).prepare("llama", **c), p)
        if name == "gpu":
            h.set_logging(True)
        logits = h.call("apply", [ids], (B, T, c["V"]))
        loss = float(h.call("loss", [ids, y], ())) if want_loss else None
        if name == "gpu":
            out["gpu_launch_log"] = h.launch_log()
        res[name] = (logits, loss)
        h.close()
    (lg, ls), (lw, lsw) = res["gpu"], res["oracle"]
    out["logits_max_err"] = float(np.abs(lg - lw).max())
    out["logits_scale"] = float(np.abs(lw).max())
    out["logits_mean_err"] = float(np.abs(lg - lw).mean())
    out["finite"] = bool(np.isfinite(lg).all())
    out["loss_gpu"], out["loss_oracle"] = ls, lsw
    return out


# What the comparison above may differ by, and why it is stated against the tensor's scale and not entry by entry:
# a logit is a sum of 4096 products of mixed sign, so an entry near zero carries the same absolute error as the
# largest one (cancellation), and a per-entry relative bound would be violated by design. Every bf16 site rounds to
# 2^-9 relative; sums reordered on the tensor cores move an element of a site to the neighbouring bf16 number now and
# then, and one layer plus the head passes about ten such sites.
# Measured at this width (B = 1, T = 256; 8.2 million logits of scale 6.85, standard deviation 1.28), against the
# oracle's sequential run, the CUDA executor's sequential run being its bits:
#   order device, the reference's launches, attention unfused   max 2^-6.1 of the scale   mean 2^-10.1
#   + the two-pass attention kernel (blockwise), merged launches   max 2^-6.0             mean 2^-9.7
#   + the one-pass attention kernel (online)                       max 2^-5.9             mean 2^-9.0
# so the reordering alone gives 2^-6.1: the bound is 2^-5 (twice the largest seen), the mean 2^-8.5.
LOGITS_TOL = 2.0**-5
LOGITS_MEAN_TOL = 2.0**-8.5
LOSS_RTOL = 2e-3
