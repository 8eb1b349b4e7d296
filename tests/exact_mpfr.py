"""An exact evaluator over MPFR for the budget assertions.

The reference's exact interpreter evaluates a program over `rug::Float` (MPFR) at 256 bits
(crates/presk-interp/src/real.rs; `ein`, `softmax` and the masked softmax at crates/presk-interp/src/prims.rs:820-924:
products and sums in index order, `exp(x - max)` over the allowed positions, a quotient by their sum). `rug` is not
here; the system's libmpfr.so.6 (4.2.1, no headers) is, and ctypes reaches it. This module restates those primitives and
the Llama decoder of examples/coverage/llama.psk over it, for shapes of a few thousand values: about a million
multiply-adds take seconds.

TEST INFRASTRUCTURE: nothing under presk_b200/ imports this module.
"""
import ctypes as C

import numpy as np

PREC = 256  # the reference's default precision of the exact interpreter (presk-interp/tests/run.rs: `run(.., 256)`)
_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL("libmpfr.so.6")
        _lib.mpfr_get_d.restype = C.c_double
        _lib.mpfr_set_d.argtypes = [C.c_void_p, C.c_double, C.c_int]
        _lib.mpfr_set_str.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int]
    return _lib


def new(x=None):
    """One MPFR number of PREC bits; a float is taken exactly, a string as the decimal it spells."""
    m = C.create_string_buffer(32)  # __mpfr_struct: precision, sign, exponent, limbs
    lib().mpfr_init2(m, PREC)
    if isinstance(x, str):
        lib().mpfr_set_str(m, x.encode(), 10, 0)
    else:
        lib().mpfr_set_d(m, 0.0 if x is None else float(x), 0)
    return m


def to_float(m):
    return lib().mpfr_get_d(m, 0)


class T:
    """A tensor of MPFR numbers, row-major."""

    def __init__(self, shape, data):
        self.shape, self.data = tuple(shape), data

    @staticmethod
    def of(array):
        a = np.asarray(array, dtype=np.float64)
        return T(a.shape, [new(x) for x in a.reshape(-1)])

    def numpy(self):
        return np.array([to_float(m) for m in self.data], dtype=np.float64).reshape(self.shape)


def _bin(fn, a, b):
    r = new()
    fn(r, a, b, 0)
    return r


def _un(fn, a):
    r = new()
    fn(r, a, 0)
    return r


def matmul(x, w):
    """x[n, k] · w[k, m]: each sum in index order from zero (prims.rs:820-879)."""
    L = lib()
    n, k = x.shape
    k2, m = w.shape
    assert k == k2
    fma = L.mpfr_fma
    out = []
    cols = [[w.data[kk * m + j] for kk in range(k)] for j in range(m)]
    for i in range(n):
        row = x.data[i * k:(i + 1) * k]
        for j in range(m):
            acc = new()
            for a, b in zip(row, cols[j]):
                fma(acc, a, b, acc, 0)
            out.append(acc)
    return T((n, m), out)


def softmax_rows(rows, allowed=None):
    """softmax over each list of `rows`; with `allowed` (lists of booleans) the masked one: the maximum and the sum
    over the allowed positions, a refused position gives 0 (prims.rs:881-924)."""
    L = lib()
    out = []
    for r, row in enumerate(rows):
        ok = allowed[r] if allowed is not None else [True] * len(row)
        live = [x for x, a in zip(row, ok) if a]
        if not live:
            out.append([new() for _ in row])
            continue
        mx = live[0]
        for x in live[1:]:
            if L.mpfr_cmp(x, mx) > 0:
                mx = x
        es, z = [], new()
        for x, a in zip(row, ok):
            if a:
                e = _un(L.mpfr_exp, _bin(L.mpfr_sub, x, mx))
                L.mpfr_add(z, z, e, 0)
                es.append(e)
            else:
                es.append(None)
        out.append([_bin(L.mpfr_div, e, z) if e is not None else new() for e in es])
    return out


def llama(params, c, ids, y=None):
    """examples/coverage/llama.psk over MPFR: the logits [B, T, V] as float64 (each the nearest double of the exact
    value at PREC bits), or the loss when labels are given. RMSNorm eps 1e-5, rope base 1e4."""
    L = lib()
    D, H, NL, V = c["D"], c["H"], c["L"], c["V"]
    G = c.get("G", H)
    HD, P = D // H, H // G
    B, Tn = ids.shape
    N = B * Tn
    add, sub, mul, div = L.mpfr_add, L.mpfr_sub, L.mpfr_mul, L.mpfr_div
    tok = T.of(params["tok"])
    x = T((N, D), [tok.data[int(i) * D + j] for i in ids.reshape(-1) for j in range(D)])
    eps = new("1e-5")
    dn = new(float(D))

    def rms(gamma, x):
        g = T.of(gamma).data
        out = []
        for i in range(N):
            row = x.data[i * D:(i + 1) * D]
            s = new()
            for a in row:
                L.mpfr_fma(s, a, a, s, 0)
            root = _un(L.mpfr_sqrt, _bin(add, _bin(div, s, dn), eps))
            out.extend(_bin(mul, _bin(div, a, root), gj) for a, gj in zip(row, g))
        return T((N, D), out)

    # angles: phi[t, r] = t * exp(-(2 r / HD) * ln 10000)
    half = HD // 2
    ln_base = _un(L.mpfr_log, new(1e4))
    freq = [_un(L.mpfr_exp, _un(L.mpfr_neg, _bin(mul, _bin(div, new(2.0 * r), new(float(HD))), ln_base))) for r in range(half)]
    cs = [[_un(L.mpfr_cos, _bin(mul, new(float(t)), f)) for f in freq] for t in range(Tn)]
    sn = [[_un(L.mpfr_sin, _bin(mul, new(float(t)), f)) for f in freq] for t in range(Tn)]

    def rope(vec, t):
        x0, x1 = vec[:half], vec[half:]
        lo = [_bin(sub, _bin(mul, a, cc), _bin(mul, b, ss)) for a, b, cc, ss in zip(x0, x1, cs[t], sn[t])]
        hi = [_bin(add, _bin(mul, b, cc), _bin(mul, a, ss)) for a, b, cc, ss in zip(x0, x1, cs[t], sn[t])]
        return lo + hi

    rt = _un(L.mpfr_sqrt, new(float(HD)))
    for l in range(NL):
        h = rms(params["blocks.n1.γ"][l], x)
        q = matmul(h, T.of(params["blocks.attn.wq"][l]))  # [N, D]: (g, p, hd)
        k = matmul(h, T.of(params["blocks.attn.wk"][l]))  # [N, G·HD]
        v = matmul(h, T.of(params["blocks.attn.wv"][l]))
        o = [None] * (N * D)
        for b in range(B):
            for g in range(G):
                ks = [rope(k.data[(b * Tn + t) * G * HD + g * HD:(b * Tn + t) * G * HD + (g + 1) * HD], t) for t in range(Tn)]
                vs = [v.data[(b * Tn + t) * G * HD + g * HD:(b * Tn + t) * G * HD + (g + 1) * HD] for t in range(Tn)]
                for p in range(P):
                    hq = g * P + p
                    rows, ok = [], []
                    for s in range(Tn):
                        qs = rope(q.data[(b * Tn + s) * D + hq * HD:(b * Tn + s) * D + (hq + 1) * HD], s)
                        row = []
                        for t in range(Tn):
                            acc = new()
                            for a, bb in zip(qs, ks[t]):
                                L.mpfr_fma(acc, a, bb, acc, 0)
                            row.append(_bin(div, acc, rt))
                        rows.append(row)
                        ok.append([t <= s for t in range(Tn)])
                    att = softmax_rows(rows, ok)
                    for s in range(Tn):
                        for d in range(HD):
                            acc = new()
                            for t in range(Tn):
                                L.mpfr_fma(acc, att[s][t], vs[t][d], acc, 0)
                            o[(b * Tn + s) * D + hq * HD + d] = acc
        proj = matmul(T((N, D), o), T.of(params["blocks.attn.wo"][l]))
        x = T((N, D), [_bin(add, a, b) for a, b in zip(x.data, proj.data)])
        h = rms(params["blocks.n2.γ"][l], x)
        gate = matmul(h, T.of(params["blocks.ff.gate.w"][l]))
        up = matmul(h, T.of(params["blocks.ff.up.w"][l]))
        one = new(1.0)
        act = []
        for a, u in zip(gate.data, up.data):
            sig = _bin(div, one, _bin(add, one, _un(L.mpfr_exp, _un(L.mpfr_neg, a))))
            act.append(_bin(mul, _bin(mul, a, sig), u))
        down = matmul(T(gate.shape, act), T.of(params["blocks.ff.down.w"][l]))
        x = T((N, D), [_bin(add, a, b) for a, b in zip(x.data, down.data)])
    logits = matmul(rms(params["norm.γ"], x), T.of(params["head"]))
    if y is None:
        return logits.numpy().reshape(B, Tn, V)
    # cross_entropy = ln z + m - x[y], then the mean
    total = new()
    for i, yi in enumerate(y.reshape(-1)):
        row = logits.data[i * V:(i + 1) * V]
        mx = row[0]
        for a in row[1:]:
            if L.mpfr_cmp(a, mx) > 0:
                mx = a
        z = new()
        for a in row:
            L.mpfr_add(z, z, _un(L.mpfr_exp, _bin(sub, a, mx)), 0)
        L.mpfr_add(total, total, _bin(sub, _bin(add, _un(L.mpfr_log, z), mx), row[int(yi)]), 0)
    return to_float(_bin(div, total, new(float(N))))
