"""psk_describe: the reference's kernel text (presk-kernel/src/ir.rs:495-596) read into a launch.

The first listing is the reference's own (crates/presk-kernel/tests/snapshots/conformance__linear_kernels.snap, a
row-wise `dot` and an `add`, kept in tests/golden/reference_vectors.json); the others are written in the same
grammar from the lowerings they name (crates/presk-kernel/src/lower.rs). Each goes text -> psk_launch -> an
executor and is compared with numpy; on the CPU the executor is the oracle, and the GPU test at the end runs the
same launches through psk_exec_run and asks for the oracle's bits."""
import json
import os

import numpy as np
import pytest

from presk_b200 import PreskError, abi
from presk_b200.api import describe

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.json")))

FUSED = """kernel fused 3 steps (%0 : f32[batch: 3, model: 8], %1 : f32[batch: 3], %2 : f32[model: 8]) -> %3 : f32[batch: 3, model: 8] {
  for i0 in 0..3 {
    for i1 in 0..8 {
      %3[i0, i1] = select((((%0[i0, i1] / %1[i0]) * %2[i1]) < 0), 0, ((%0[i0, i1] / %1[i0]) * %2[i1]))
    }
  }
}
"""

SILU = """kernel fused 2 steps (%0 : bf16[seq: 5, 16]) -> %1 : bf16[seq: 5, 16] {
  for i0 in 0..5 {
    for i1 in 0..16 {
      %1[i0, i1] = (%0[i0, i1] * (1 / (1 + exp(neg(%0[i0, i1])))))
    }
  }
}
"""

# lower.rs:586-636: the generic `ein`, operands relabelled: q[b, g, s, h] and k[b, g, t, h] into [b, g, s, t], one
# scalar accumulator, the product written (1 * x0) * x1
EIN = """kernel ein[batch, groups, seq, seq2] (%0 : f32[batch: 2, groups: 3, seq: 4, hd: 8], %1 : f32[batch: 2, groups: 3, seq: 5, hd: 8]) -> %2 : f32[batch: 2, groups: 3, seq: 4, seq2: 5] {
  for i0 in 0..2 {
    for i1 in 0..3 {
      for i2 in 0..4 {
        for i3 in 0..5 {
          s0 = 0
          for i4 in 0..8 {
            s0 = (s0 + ((1 * %0[i0, i1, i2, i4]) * %1[i0, i1, i3, i4]))
          }
          %2[i0, i1, i2, i3] = s0
        }
      }
    }
  }
}
"""

# lower.rs:1368-1419: the masked softmax in three passes, the mask read in selections only
MASKED_SOFTMAX = """kernel softmax axis seq2 where (%0 : f32[batch: 2, seq: 4, seq2: 4], %1 : i64[seq: 4, seq2: 4]) -> %2 : f32[batch: 2, seq: 4, seq2: 4] {
  for i0 in 0..2 {
    for i1 in 0..4 {
      s2 = 1
      s0 = 0
      for i2 in 0..4 {
        s0 = select((real(%1[i1, i2]) > 0.5), select((s2 > 0.5), %0[i0, i1, i2], select((%0[i0, i1, i2] > s0), %0[i0, i1, i2], s0)), s0)
        s2 = select((real(%1[i1, i2]) > 0.5), 0, s2)
      }
      s1 = 0
      for i2 in 0..4 {
        s1 = (s1 + select((real(%1[i1, i2]) > 0.5), exp((%0[i0, i1, i2] - s0)), 0))
      }
      for i2 in 0..4 {
        %2[i0, i1, i2] = select((real(%1[i1, i2]) > 0.5), (exp((%0[i0, i1, i2] - s0)) / s1), 0)
      }
    }
  }
}
"""

MEAN = """kernel mean axis model (%0 : f32[batch: 3, model: 6, 2]) -> %1 : f32[batch: 3, 2] {
  for i0 in 0..3 {
    for i1 in 0..2 {
      s0 = 0
      for i2 in 0..6 {
        s0 = (s0 + %0[i0, i2, i1])
      }
      %1[i0, i1] = (s0 / 6)
    }
  }
}
"""

XENT = """kernel cross_entropy (%0 : f32[batch: 4, 7], %1 : i64[batch: 4]) -> %2 : f32[batch: 4] {
  for i0 in 0..4 {
    s0 = %0[i0, 0]
    for i1 in 0..7 {
      if (%0[i0, i1] > s0) {
        s0 = %0[i0, i1]
      }
    }
    s1 = 0
    for i1 in 0..7 {
      s1 = (s1 + exp((%0[i0, i1] - s0)))
    }
    %2[i0] = ((log(s1) + s0) - %0[i0, %1[i0]])
  }
}
"""

EMBED = """kernel embed (%0 : f32[9, 4], %1 : i64[batch: 2, seq: 3]) -> %2 : f32[batch: 2, seq: 3, 4] {
  for i0 in 0..2 {
    for i1 in 0..3 {
      for i2 in 0..4 {
        %2[i0, i1, i2] = %0[%1[i0, i1], i2]
      }
    }
  }
}
"""

SLICE = """kernel slice pair: 1..2 (%0 : f32[seq: 3, pair: 2, 4]) -> %1 : f32[seq: 3, pair: 1, 4] {
  for i0 in 0..3 {
    for i1 in 0..1 {
      for i2 in 0..4 {
        %1[i0, i1, i2] = %0[i0, (i1 + 1), i2]
      }
    }
  }
}
"""

# a `dot` in a laned form (lower.rs:906-1139, one row by eight columns): recognised by its name and buffers
TILED_DOT = """kernel dot (%0 : f32[batch: 4, 6], %1 : f32[6, 8]) -> %2 : f32[batch: 4, 8] {
  for i0 in 0..4 {
    for i1 in 0..1 {
      v0 = splat(0)
      for i2 in 0..6 {
        v0 = (v0 + (splat(%0[i0, i2]) * %1[i2, (i1 * 8)]<v>)<v>)<v>
      }
      %2[i0, (i1 * 8)] <v= v0
    }
  }
}
"""


def np_dtype(code):
    return {abi.F32: np.float32, abi.I64: np.int64}[code]


def run_listing(run, text, arrays, out_shape, out_dtype=np.float32):
    """Every kernel of `text` in turn: kernel k's inputs are `arrays[k]`; returns the outputs."""
    outs = []
    for (name, l), ins in zip(describe(text), arrays):
        out = np.full(out_shape, -77, dtype=out_dtype)
        run(l, [np.ascontiguousarray(a) for a in ins], out)
        outs.append((name, out))
    return outs


@pytest.fixture
def on_oracle(oracle):
    def run(l, ins, out):
        oracle.run(l, ins + [out])
    return run


def check_all(run):
    rng = np.random.default_rng(0)
    # the reference's own listing: dot [4, 3] x [3, 2], then add of a bias [2]
    x, w, b = rng.standard_normal((4, 3)).astype(np.float32), rng.standard_normal((3, 2)).astype(np.float32), rng.standard_normal(2).astype(np.float32)
    (n0, l0), (n1, l1) = describe(GOLD["linear_kernels_text"])
    assert (n0, l0.op, l0.n_outer, l0.n_inner, list(l0.dims[:3])) == ("dot", abi.OP_CONTRACT, 2, 1, [4, 2, 3])
    assert (n1, l1.op, l1.n_steps, l1.steps[0].prim) == ("add", abi.OP_FUSED, 1, abi.ADD)
    y = np.zeros((4, 2), np.float32)
    run(l0, [x, w], y)
    want = np.zeros((4, 2), np.float32)
    for k in range(3):  # the nest's order of additions: k = 0, 1, 2 from +0, products rounded before they are added
        want = want + x[:, k:k + 1] * w[k:k + 1, :]
    assert np.array_equal(y, want)
    z = np.zeros((4, 2), np.float32)
    run(l1, [y, b], z)
    assert np.array_equal(z, y + b)

    # a fusion group of three steps (div, mul, relu) with two broadcasts
    a, r, g = rng.standard_normal((3, 8)).astype(np.float32), (rng.random(3) + 0.5).astype(np.float32), rng.standard_normal(8).astype(np.float32)
    (name, l), = describe(FUSED)
    assert (l.op, l.n_steps, [l.steps[i].prim for i in range(3)]) == (abi.OP_FUSED, 3, [abi.DIV, abi.MUL, abi.RELU])
    out = np.zeros((3, 8), np.float32)
    run(l, [a, r, g], out)
    t = (a / r[:, None]) * g[None, :]
    assert np.array_equal(out, np.where(t < 0, np.float32(0), t))

    # the generic ein with relabelled axes
    q, k = rng.standard_normal((2, 3, 4, 8)).astype(np.float32), rng.standard_normal((2, 3, 5, 8)).astype(np.float32)
    (name, l), = describe(EIN)
    assert (name, l.op, l.n_outer, l.n_inner) == ("ein[batch, groups, seq, seq2]", abi.OP_CONTRACT, 4, 1)
    out = np.zeros((2, 3, 4, 5), np.float32)
    run(l, [q, k], out)
    want = np.zeros((2, 3, 4, 5), np.float32)
    for h in range(8):
        want = want + q[:, :, :, None, h] * k[:, :, None, :, h]
    assert np.array_equal(out, want)

    # the masked softmax: the causal mask over (seq, seq2), broadcast over the batch
    s = rng.standard_normal((2, 4, 4)).astype(np.float32)
    mask = np.tril(np.ones((4, 4), np.int64))
    (name, l), = describe(MASKED_SOFTMAX)
    assert (l.op, l.masked, l.n_outer, l.n_inner) == (abi.OP_SOFTMAX, 1, 2, 1)
    out = np.zeros((2, 4, 4), np.float32)
    run(l, [s, mask], out)
    sm = np.where(mask.astype(bool), s.astype(np.float64), -np.inf)
    e = np.exp(sm - sm.max(-1, keepdims=True))
    np.testing.assert_allclose(out, e / e.sum(-1, keepdims=True), rtol=2e-6, atol=0)
    assert np.all(out[:, 0, 1:] == 0)

    # a mean over a middle axis
    m = rng.standard_normal((3, 6, 2)).astype(np.float32)
    (name, l), = describe(MEAN)
    assert (l.op, l.kind, l.iparam[0]) == (abi.OP_REDUCE, abi.REDUCE_MEAN, 6)
    out = np.zeros((3, 2), np.float32)
    run(l, [m], out)
    acc = np.zeros((3, 2), np.float32)
    for j in range(6):
        acc = acc + m[:, j, :]
    assert np.array_equal(out, acc / np.float32(6))

    # cross-entropy, embed, a slice as a copy
    lg, yy = rng.standard_normal((4, 7)).astype(np.float32), rng.integers(0, 7, size=4, dtype=np.int64)
    (name, l), = describe(XENT)
    out = np.zeros(4, np.float32)
    run(l, [lg, yy], out)
    l64 = lg.astype(np.float64)
    np.testing.assert_allclose(out, np.log(np.exp(l64 - l64.max(1, keepdims=True)).sum(1)) + l64.max(1) - l64[np.arange(4), yy], rtol=2e-6)
    tab, ids = rng.standard_normal((9, 4)).astype(np.float32), rng.integers(0, 9, size=(2, 3), dtype=np.int64)
    (name, l), = describe(EMBED)
    out = np.zeros((2, 3, 4), np.float32)
    run(l, [tab, ids], out)
    assert np.array_equal(out, tab[ids])
    p = rng.standard_normal((3, 2, 4)).astype(np.float32)
    (name, l), = describe(SLICE)
    assert (name, l.op) == ("slice pair: 1..2", abi.OP_COPY)
    out = np.zeros((3, 1, 4), np.float32)
    run(l, [p], out)
    assert np.array_equal(out, p[:, 1:2, :])

    # `dot` in a laned form: by its name and buffers
    x, w = rng.standard_normal((4, 6)).astype(np.float32), rng.standard_normal((6, 8)).astype(np.float32)
    (name, l), = describe(TILED_DOT)
    out = np.zeros((4, 8), np.float32)
    run(l, [x, w], out)
    want = np.zeros((4, 8), np.float32)
    for k in range(6):
        want = want + x[:, k:k + 1] * w[k:k + 1, :]
    assert np.array_equal(out, want)


def test_listings_run_on_the_oracle(on_oracle):
    check_all(on_oracle)


def test_bf16_group_keeps_the_sites_rounding(oracle):
    """silu on bf16 codes: the launch's type is the kernel's, the step list is [sigmoid, mul]."""
    (name, l), = describe(SILU)
    assert (l.dtype, l.n_steps, l.steps[0].prim, l.steps[1].prim) == (abi.BF16, 2, abi.SIGMOID, abi.MUL)
    x = np.random.default_rng(1).standard_normal((5, 16)).astype(np.float32)
    xb = oracle.convert(x, abi.BF16)
    out = np.zeros(5 * 16 * 2, np.uint8)
    oracle.run(l, [xb, out])
    xv = oracle.widen(xb, abi.BF16, 80).astype(np.float64)
    got = oracle.widen(out, abi.BF16, 80)
    np.testing.assert_allclose(got, xv / (1 + np.exp(-xv)), rtol=2.0**-8, atol=1e-30)


def test_what_has_no_launch_is_refused():
    """E7005 with a message, never a guess: a laned nest that is not `dot`, `erf` by itself, a product of three
    operands, formats of the kernel interpreter, an index that is not a loop; E7001 for text outside the grammar."""
    cases = {
        "laned": TILED_DOT.replace("kernel dot", "kernel dot_vjp_l"),
        "erf": "kernel erf (%0 : f32[4]) -> %1 : f32[4] {\n  for i0 in 0..4 {\n    %1[i0] = erf(%0[i0])\n  }\n}\n",
        "three": EIN.replace("((1 * %0[i0, i1, i2, i4]) * %1[i0, i1, i3, i4])", "(((1 * %0[i0, i1, i2, i4]) * %1[i0, i1, i3, i4]) * %1[i0, i1, i3, i4])"),
        "formats": GOLD["linear_kernels_text"].replace("-> %2 : f32[batch: 4, 2] {", "-> %2 : f32[batch: 4, 2] arith f32 product i32 accum i32 {", 1),
        "index": "kernel odd (%0 : f32[8]) -> %1 : f32[4] {\n  for i0 in 0..4 {\n    %1[i0] = neg(%0[(i0 * 2)])\n  }\n}\n",
        "literal": "kernel scale (%0 : f32[4]) -> %1 : f32[4] {\n  for i0 in 0..4 {\n    %1[i0] = (%0[i0] * 0.5)\n  }\n}\n",
    }
    for what, text in cases.items():
        with pytest.raises(PreskError) as e:
            describe(text)
        assert e.value.code == 7005, (what, str(e.value))
    for text in ("kernel broken (%0 : f32[4]) -> %1 : f32[4] {\n  for i0 in 0..4 {\n    %1[i0] = neg(%0[i0]\n  }\n}\n", "kernel unclosed (%0 : f32[4]) -> %1 : f32[4] {\n  for i0 in 0..4 {\n"):
        with pytest.raises(PreskError) as e:
            describe(text)
        assert e.value.code == 7001


@pytest.mark.gpu
def test_listings_run_on_the_gpu_with_the_oracles_bits(cuda, oracle):
    """The same listings through psk_exec_run: every output the oracle's, bit for bit (sequential order)."""
    def both(l, ins, out):
        dev = [cuda.upload(a) for a in ins]
        pout = cuda.alloc(max(out.nbytes, 1))
        cuda.run(l, dev + [pout])
        cuda.sync()
        got = cuda.download(pout, out.nbytes)
        for p in dev + [pout]:
            cuda.free(p)
        want = out.copy()
        oracle.run(l, ins + [want])
        assert np.array_equal(got, want.view(np.uint8).reshape(-1)), l.name
        out[...] = want

    check_all(both)
