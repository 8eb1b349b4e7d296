"""The reference's `chunked(size)` order (presk-rt/src/lib.rs:264-269; the nest at presk-kernel/src/lower.rs:424-457):
a contraction over one summed axis adds `size` consecutive terms from zero in index order, then the chunks' sums in
order from zero, the last chunk shorter. The construction is that of the reference's own test
(crates/presk-kernel/tests/formats.rs:342-408): [2, 20] x [20, 3] at chunks of 1, 3, 8, the whole axis and more,
against the sum written out; a chunk of the whole axis or more is the sequential sum; `ein` takes it and sums in the
same chunks as `dot`; a sum over two axes refuses it."""
import numpy as np
import pytest

import models
from presk_b200 import Host, PreskError, abi, launch_desc


def chunked_dot_f32(x, w, size):
    """sum_k x[i, k]·w[k, j] in f32: products rounded, chunks of `size` from zero, then the chunks from zero."""
    i, kk = x.shape
    j = w.shape[1]
    out = np.zeros((i, j), np.float32)
    for c0 in range(0, kk, size):
        part = np.zeros((i, j), np.float32)
        for t in range(c0, min(kk, c0 + size)):
            part = part + x[:, t:t + 1] * w[t:t + 1, :]
        out = out + part
    return out


def dot_launch(i, kk, j, order, size, ein=False):
    l = launch_desc(abi.OP_CONTRACT, abi.F32, [i, j], [kk], order=order, name=b"ein[i, j]" if ein else b"dot")
    l.order_size = size
    l.n_inputs = 2
    l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = abi.F32, i * kk, kk, 1
    l.inputs[1].dtype, l.inputs[1].numel, l.inputs[1].stride[1], l.inputs[1].stride[2] = abi.F32, kk * j, 1, j
    l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = abi.F32, i * j, j, 1
    return l


def case(seed=0x180003, i=2, kk=20, j=3):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((i, kk)).astype(np.float32), rng.standard_normal((kk, j)).astype(np.float32)


def test_a_chunked_order_sums_in_chunks_on_the_oracle(oracle):
    x, w = case()
    seq = np.zeros((2, 3), np.float32)
    oracle.run(dot_launch(2, 20, 3, abi.ORDER_SEQUENTIAL, 0), [x, w, seq])
    for size in (1, 3, 8, 20, 32):
        got = np.zeros((2, 3), np.float32)
        oracle.run(dot_launch(2, 20, 3, abi.ORDER_CHUNKED, size), [x, w, got])
        assert np.array_equal(got.view(np.uint32), chunked_dot_f32(x, w, size).view(np.uint32)), size
        if size >= 20:
            assert np.array_equal(got.view(np.uint32), seq.view(np.uint32))
    # a sum over two axes is refused, as the reference refuses it (lower.rs:429-431)
    l = launch_desc(abi.OP_CONTRACT, abi.F32, [3], [2, 4], order=abi.ORDER_CHUNKED)
    l.order_size, l.n_inputs = 4, 2
    with pytest.raises(RuntimeError):
        oracle.run(l, [np.zeros(8, np.float32), np.zeros(24, np.float32), np.zeros(3, np.float32)])


def test_a_realization_states_the_chunked_order(oracle):
    """`"order": {"kind": "chunked", "size": 8}` through the host: the MLP's two `dot`s sum in chunks of 8 (784 and 256
    terms), every other launch keeps the sequential order; Llama's output projection sums over three axes and is
    refused, as the reference's `ein` refuses it."""
    p = models.mlp_params()
    x, _ = models.mlp_inputs(16)
    h = models.give(Host(oracle.vtable(), {"default": "f32", "order": {"kind": "chunked", "size": 8}}).prepare("mlp"), p)
    got = h.call("apply", [x], (16, 10))
    hid = chunked_dot_f32(x, p["l1.w"], 8) + p["l1.b"]
    hid = np.where(hid < 0, np.float32(0), hid)
    want = chunked_dot_f32(hid, p["l2.w"], 8) + p["l2.b"]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    seq = models.give(Host(oracle.vtable(), "f32").prepare("mlp"), p).call("apply", [x], (16, 10))
    assert not np.array_equal(got.view(np.uint32), seq.view(np.uint32))  # it does reassociate
    c = models.LLAMA_TINY
    hl = models.give(Host(oracle.vtable(), {"default": "f32", "order": {"kind": "chunked", "size": 4}}).prepare("llama", **c), models.llama_params(c))
    with pytest.raises(PreskError, match="E7005.*over 3 axes"):
        hl.call("apply", [np.zeros((1, 4), np.int64)], (1, 4, c["V"]))
    with pytest.raises(PreskError, match="size"):
        Host(oracle.vtable(), {"default": "f32", "order": {"kind": "chunked"}})


@pytest.mark.gpu
def test_a_chunked_order_on_the_gpu_gives_the_oracles_bits(cuda, oracle):
    """The scalar contraction kernels run the order natively: the oracle's bits at the reference's small shape and at
    one that spans several tiles and a ragged last chunk; `ein` (a generic contraction) sums in the same chunks."""
    for (i, kk, j), sizes in (((2, 20, 3), (1, 3, 8, 20, 32)), ((150, 333, 70), (7, 64, 100, 333))):
        x, w = case(i + kk, i, kk, j)
        dev = [cuda.upload(x), cuda.upload(w)]
        pout = cuda.alloc(i * j * 4)
        for size in sizes:
            l = dot_launch(i, kk, j, abi.ORDER_CHUNKED, size)
            cuda.run(l, dev + [pout])
            cuda.sync()
            got = cuda.download(pout, i * j * 4).view(np.float32).reshape(i, j)
            want = np.zeros((i, j), np.float32)
            oracle.run(l, [x, w, want])
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (i, kk, j, size)
            if kk <= 20:
                assert np.array_equal(got.view(np.uint32), chunked_dot_f32(x, w, size).view(np.uint32))
        for p in dev + [pout]:
            cuda.free(p)
    # the host's MLP under the order, on the GPU
    p = models.mlp_params()
    xin, _ = models.mlp_inputs(64)
    rz = {"default": "f32", "order": {"kind": "chunked", "size": 8}}
    got = models.give(Host(cuda, rz).prepare("mlp"), p).call("apply", [xin], (64, 10))
    want = models.give(Host(oracle.vtable(), rz).prepare("mlp"), p).call("apply", [xin], (64, 10))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
