"""The reverse-mode program of examples/coverage/llama.psk `loss` over the CPU oracle, every leaf of the gradient
against an independent float64 statement of the model differentiated by torch's autograd."""
import numpy as np
import pytest
import torch

import models
from presk_b200 import Host


def llama_torch_grads(p, c, ids, y):
    """Llama in float64 torch, straight from examples/coverage/llama.psk (the numpy statement of tests/models.py
    with tensors that carry gradients); returns the loss and d loss / d parameter for every parameter."""
    D, H, L = c["D"], c["H"], c["L"]
    G = c.get("G", H)
    HD, P = D // H, H // G
    B, T = ids.shape
    t = {k: torch.tensor(np.asarray(v, np.float32).astype(np.float64), requires_grad=True) for k, v in p.items()}
    x = t["tok"][torch.tensor(ids)]
    rms = lambda g, x: x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * g
    freq = torch.exp(-2.0 * torch.arange(HD // 2, dtype=torch.float64) / HD * np.log(1e4))
    phi = torch.arange(T, dtype=torch.float64)[:, None] * freq[None, :]
    cs, sn = torch.cos(phi), torch.sin(phi)

    def rope(x):  # [..., T, HD]
        x0, x1 = x[..., : HD // 2], x[..., HD // 2:]
        return torch.cat([x0 * cs - x1 * sn, x1 * cs + x0 * sn], -1)

    mask = torch.tril(torch.ones((T, T), dtype=torch.bool))
    for l in range(L):
        h = rms(t["blocks.n1.γ"][l], x)
        q = (h @ t["blocks.attn.wq"][l]).reshape(B, T, G, P, HD).permute(0, 2, 3, 1, 4)
        k = (h @ t["blocks.attn.wk"][l]).reshape(B, T, G, HD).permute(0, 2, 1, 3)
        v = (h @ t["blocks.attn.wv"][l]).reshape(B, T, G, HD)
        q, k = rope(q), rope(k)
        s = torch.einsum("bgpsh,bgth->bgpst", q, k) / np.sqrt(HD)
        a = torch.softmax(s.masked_fill(~mask, -np.inf), -1)
        o = torch.einsum("bgpst,btgh->bsgph", a, v).reshape(B, T, D)
        x = x + o @ t["blocks.attn.wo"][l]
        h = rms(t["blocks.n2.γ"][l], x)
        g = h @ t["blocks.ff.gate.w"][l]
        x = x + ((g * torch.sigmoid(g)) * (h @ t["blocks.ff.up.w"][l])) @ t["blocks.ff.down.w"][l]
    logits = rms(t["norm.γ"], x) @ t["head"]
    loss = torch.nn.functional.cross_entropy(logits.reshape(B * T, -1), torch.tensor(y).reshape(-1))
    loss.backward()
    return float(loss.detach()), {k: v.grad.numpy() for k, v in t.items()}


@pytest.mark.parametrize("c", [models.LLAMA_TINY, dict(V=50, D=32, H=4, G=2, FF=48, L=3)], ids=["mha", "gqa"])
def test_llama_gradient_against_float64_autograd(oracle, c):
    p = models.llama_params(c, seed=4, std=0.2)
    rng = np.random.default_rng(6)
    for k in ("norm.γ", "blocks.n1.γ", "blocks.n2.γ"):
        p[k] = (1.0 + 0.1 * rng.standard_normal(p[k].shape)).astype(np.float32)
    ids = rng.integers(0, c["V"] // 2, size=(2, 12), dtype=np.int64)  # repeated tokens: rows of tok summed in embed_vjp
    y = rng.integers(0, c["V"], size=(2, 12), dtype=np.int64)
    want_loss, want = llama_torch_grads(p, c, ids, y)
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), p)
    assert float(h.call("loss", [ids, y], ())) == pytest.approx(want_loss, rel=2e-6)
    h.set_logging(True)
    h.call("loss_grad", [ids, y], p["tok"].shape)
    log = h.launch_log()
    assert log.count("cross_entropy_vjp") == 1 and log.count("embed_vjp") == 1 and log.count("scatter_params") == 9 * c["L"]
    for k, w in want.items():
        got = h.result(k, w.shape)
        assert np.abs(w).max() > 0, k
        np.testing.assert_allclose(got, w, rtol=0, atol=3e-5 * np.abs(w).max(), err_msg=k)
    # rows of tokens the batch does not hold stay zero
    absent = np.setdiff1d(np.arange(c["V"]), ids)
    assert not h.result("tok", p["tok"].shape)[absent].any()


def test_llama_training_steps_lower_the_loss(oracle):
    """loss_grad + adamw.step on the small Llama: the loss falls step after step."""
    c = models.LLAMA_TINY
    p = models.llama_params(c, seed=4, std=0.1)
    rng = np.random.default_rng(7)
    ids = rng.integers(0, c["V"], size=(2, 12), dtype=np.int64)
    y = np.roll(ids, -1, axis=1)
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), p).adamw(lr=3e-3, weight_decay=0.01, grad_clip=1.0)
    losses = []
    for t in range(1, 9):
        losses.append(float(h.call("loss", [ids, y], ())))
        h.call("loss_grad", [ids, y], p["tok"].shape)
        h.adamw_step(t, 8)
    assert all(b < a for a, b in zip(losses, losses[1:])) and losses[-1] < 0.9 * losses[0], losses
