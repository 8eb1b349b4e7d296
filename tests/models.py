"""Inputs and parameters of the test models, seeded, as numpy arrays."""
import numpy as np

LLAMA_TINY = dict(V=100, D=32, H=2, G=2, FF=64, L=2)  # the reference's own small constants (presk-cranelift/tests/codes.rs:397)


def llama_params(c, seed=0, std=0.02):
    rng = np.random.default_rng(seed)
    V, D, FF, L = c["V"], c["D"], c["FF"], c["L"]
    G, H = c.get("G", c["H"]), c["H"]
    HD = D // H
    n = lambda *s: (rng.standard_normal(s) * std).astype(np.float32)
    return {
        "tok": n(V, D), "head": n(D, V), "norm.γ": np.ones(D, np.float32),
        "blocks.n1.γ": np.ones((L, D), np.float32), "blocks.n2.γ": np.ones((L, D), np.float32),
        "blocks.attn.wq": n(L, D, D), "blocks.attn.wk": n(L, D, G * HD), "blocks.attn.wv": n(L, D, G * HD), "blocks.attn.wo": n(L, D, D),
        "blocks.ff.gate.w": n(L, D, FF), "blocks.ff.up.w": n(L, D, FF), "blocks.ff.down.w": n(L, FF, D),
    }


def llama_numpy(p, c, ids, y=None):
    """Llama in float64 numpy, straight from examples/coverage/llama.psk: an independent
    statement of the model (not of the kernels) to hold the host program against."""
    D, H, L = c["D"], c["H"], c["L"]
    G = c.get("G", H)
    HD, P = D // H, H // G
    B, T = ids.shape
    f = lambda a: np.asarray(a, np.float64)
    x = f(p["tok"])[ids]
    rms = lambda g, x: x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * f(g)
    freq = np.exp(-2.0 * np.arange(HD // 2) / HD * np.log(1e4))
    phi = np.arange(T)[:, None] * freq[None, :]
    cs, sn = np.cos(phi), np.sin(phi)

    def rope(x):  # [..., T, HD]
        x0, x1 = x[..., : HD // 2], x[..., HD // 2:]
        return np.concatenate([x0 * cs - x1 * sn, x1 * cs + x0 * sn], -1)

    mask = np.tril(np.ones((T, T), bool))
    for l in range(L):
        h = rms(p["blocks.n1.γ"][l], x)
        q = (h @ f(p["blocks.attn.wq"][l])).reshape(B, T, G, P, HD).transpose(0, 2, 3, 1, 4)
        k = (h @ f(p["blocks.attn.wk"][l])).reshape(B, T, G, HD).transpose(0, 2, 1, 3)
        v = (h @ f(p["blocks.attn.wv"][l])).reshape(B, T, G, HD)
        q, k = rope(q), rope(k)
        s = np.einsum("bgpsh,bgth->bgpst", q, k) / np.sqrt(HD)
        s = np.where(mask, s, -np.inf)
        a = np.exp(s - s.max(-1, keepdims=True))
        a = a / a.sum(-1, keepdims=True)
        o = np.einsum("bgpst,btgh->bsgph", a, v).reshape(B, T, D)
        x = x + o @ f(p["blocks.attn.wo"][l])
        h = rms(p["blocks.n2.γ"][l], x)
        g = h @ f(p["blocks.ff.gate.w"][l])
        x = x + ((g / (1 + np.exp(-g))) * (h @ f(p["blocks.ff.up.w"][l]))) @ f(p["blocks.ff.down.w"][l])
    logits = rms(p["norm.γ"], x) @ f(p["head"])
    if y is None:
        return logits
    m = logits.max(-1, keepdims=True)
    lse = np.log(np.exp(logits - m).sum(-1)) + m[..., 0]
    return (lse - np.take_along_axis(logits, y[..., None], -1)[..., 0]).mean()


def mlp_params(seed=0, d_in=784, d_h=256, d_out=10):
    """xavier_uniform weights, zero biases (the MLP classifier workload)."""
    rng = np.random.default_rng(seed)
    xav = lambda i, o: rng.uniform(-np.sqrt(6.0 / (i + o)), np.sqrt(6.0 / (i + o)), size=(i, o)).astype(np.float32)
    return {"l1.w": xav(d_in, d_h), "l1.b": np.zeros(d_h, np.float32), "l2.w": xav(d_h, d_out), "l2.b": np.zeros(d_out, np.float32)}


def mlp_inputs(batch, seed=0, d_in=784, d_out=10):
    rng = np.random.default_rng(seed + 1)
    return rng.uniform(-1, 1, size=(batch, d_in)).astype(np.float32), rng.integers(0, d_out, size=(batch,), dtype=np.int64)


def give(host, params):
    for k, v in params.items():
        host.set_param(k, v)
    return host


GPT_TINY = dict(V=65, D=32, H=4, L=2)


def gpt_params(c, T, seed=0):
    """examples/corpus/nlp/05_gpt.psk's parameters: normal(0.02) tables, xavier linear maps, zero biases;
    the head drawn normal(0.02) too so that the logits are not all zero (the GPT workload)."""
    rng = np.random.default_rng(seed)
    V, D, L = c["V"], c["D"], c["L"]
    n = lambda *s: (rng.standard_normal(s) * 0.02).astype(np.float32)

    def xav(*s):
        b = np.sqrt(6.0 / (s[-2] + s[-1]))
        return rng.uniform(-b, b, size=s).astype(np.float32)

    p = {"tok": n(V, D), "pos": n(T, D), "head": n(D, V), "lnf.γ": np.ones(D, np.float32), "lnf.β": np.zeros(D, np.float32)}
    for ln in ("ln1", "ln2"):
        p[f"blocks.{ln}.γ"] = (1 + 0.1 * rng.standard_normal((L, D))).astype(np.float32)
        p[f"blocks.{ln}.β"] = (0.1 * rng.standard_normal((L, D))).astype(np.float32)
    for w in ("wq", "wk", "wv", "wo"):
        p[f"blocks.attn.{w}.w"] = xav(L, D, D)
        p[f"blocks.attn.{w}.b"] = (0.01 * rng.standard_normal((L, D))).astype(np.float32)
    p["blocks.ff.up.w"], p["blocks.ff.up.b"] = xav(L, D, 4 * D), np.zeros((L, 4 * D), np.float32)
    p["blocks.ff.down.w"], p["blocks.ff.down.b"] = xav(L, 4 * D, D), np.zeros((L, D), np.float32)
    return p


def gpt_numpy(p, c, ids, y=None):
    """05_gpt.psk in float64 numpy (outside training: dropout is the identity)."""
    from math import erf
    D, H, L = c["D"], c["H"], c["L"]
    HD = D // H
    B, T = ids.shape
    f = lambda a: np.asarray(a, np.float64)

    def ln(g, b, x):
        mu = x.mean(-1, keepdims=True)
        var = ((x - mu) ** 2).mean(-1, keepdims=True)
        return (x - mu) / np.sqrt(var + 1e-5) * f(g) + f(b)

    verf = np.vectorize(erf)
    x = f(p["tok"])[ids] + f(p["pos"])[np.arange(T)]
    mask = np.tril(np.ones((T, T), bool))
    for l in range(L):
        h = ln(p["blocks.ln1.γ"][l], p["blocks.ln1.β"][l], x)
        lin = lambda w, z: z @ f(p[f"blocks.attn.{w}.w"][l]) + f(p[f"blocks.attn.{w}.b"][l])
        sh = lambda z: z.reshape(B, T, H, HD).transpose(0, 2, 1, 3)
        q, k, v = sh(lin("wq", h)), sh(lin("wk", h)), sh(lin("wv", h))
        s = np.einsum("bhsd,bhtd->bhst", q, k) / np.sqrt(HD)
        s = np.where(mask, s, -np.inf)
        a = np.exp(s - s.max(-1, keepdims=True))
        a = a / a.sum(-1, keepdims=True)
        o = np.einsum("bhst,bhtd->bhsd", a, v).transpose(0, 2, 1, 3).reshape(B, T, D)
        x = x + lin("wo", o)
        h = ln(p["blocks.ln2.γ"][l], p["blocks.ln2.β"][l], x)
        u = h @ f(p["blocks.ff.up.w"][l]) + f(p["blocks.ff.up.b"][l])
        g = u * (1 + verf(u / np.sqrt(2.0))) / 2
        x = x + g @ f(p["blocks.ff.down.w"][l]) + f(p["blocks.ff.down.b"][l])
    logits = ln(p["lnf.γ"], p["lnf.β"], x) @ f(p["head"])
    if y is None:
        return logits
    m = logits.max(-1, keepdims=True)
    lse = np.log(np.exp(logits - m).sum(-1)) + m[..., 0]
    return (lse - np.take_along_axis(logits, y[..., None], -1)[..., 0]).mean()
