"""The optimizer functions over the CPU oracle, against the known answers of the reference's own test
(crates/presk-interp/tests/run.rs `optimizer_schedule_and_step`) and a float64 statement of AdamW."""
import numpy as np
import pytest

from presk_b200 import Host, PreskError


def test_cosine_schedule_known_answers(oracle):
    """run.rs:222-227: cosine(warmup = 2000), lr = 3e-4 at chosen steps (there to 1e-18 in exact arithmetic; here
    in f32, where min(1, x) = 1 - relu(1 - x) costs x an absolute 2^-24 and f32(π) is not π: within lr · 2^-22)."""
    h = Host(oracle.vtable(), "f32").prepare("tower", D=3, L=1).adamw(lr=3e-4, schedule="cosine", warmup=2000)
    tol = 3e-4 * 2.0**-22
    assert abs(h.adamw_lr(1, 4000) - 1.5e-7) <= tol
    assert abs(h.adamw_lr(2000, 4000) - 3e-4) <= tol
    assert abs(h.adamw_lr(3000, 4000) - 1.5e-4) <= tol
    assert abs(h.adamw_lr(4000, 4000)) <= tol
    assert abs(h.adamw_lr(5000, 4000)) <= tol  # past the horizon the rate stays at 0
    lin = Host(oracle.vtable(), "f32").prepare("tower", D=3, L=1).adamw(lr=1e-2, schedule="linear", warmup=10)
    assert abs(lin.adamw_lr(5, 110) - 5e-3) <= 1e-2 * 2.0**-22
    assert abs(lin.adamw_lr(60, 110) - 5e-3) <= 1e-2 * 2.0**-22
    assert Host(oracle.vtable(), "f32").prepare("tower", D=3, L=1).adamw(lr=2e-3).adamw_lr(7, 9) == pytest.approx(2e-3, rel=1e-7)


def test_one_step_from_zero_moments_known_answer(oracle):
    """run.rs:229-253: θ = 1, m = v = 0, g = 0.5, t = 1 of 10, the block's defaults (lr 1e-3, betas (0.9, 0.999),
    eps 1e-8, no decay): m' = 0.05, v' = 0.00025, θ' = 1 - 1e-3 · 0.5 / (0.5 + 1e-8)."""
    h = Host(oracle.vtable(), "f32").prepare("tower", D=4, L=2).adamw()
    h.set_param("blocks.w", np.ones((2, 4, 4)))
    h.set_param("blocks.b", np.ones((2, 4)))
    h.set_result("blocks.w", np.full((2, 4, 4), 0.5))
    h.set_result("blocks.b", np.full((2, 4), 0.5))
    h.set_logging(True)
    h.adamw_step(1, 10)
    assert h.launch_log() == ["sub", "sub", "fused 4 steps", "fused 4 steps"] + ["fused 3 steps", "fused 4 steps", "fused 9 steps"] * 2
    expected = 1.0 - 1e-3 * 0.5 / (0.5 + 1e-8)
    for path, shape in (("blocks.w", (2, 4, 4)), ("blocks.b", (2, 4))):
        np.testing.assert_allclose(h.result("m:" + path, shape), 0.05, rtol=3e-7)
        np.testing.assert_allclose(h.result("v:" + path, shape), 0.00025, rtol=1e-4)  # 1 - f32(0.999) is 0.001 to 6e-5
        np.testing.assert_allclose(h.result(path, shape), expected, rtol=2e-7)


def test_training_steps_follow_float64_adamw_and_lower_the_loss(oracle):
    """Ten steps of loss_grad + adamw.step on the tower (decay, cosine schedule with warm-up): parameters within f32
    accumulation of a float64 AdamW run on the same gradients' formula, and the loss goes down."""
    d, L, b = 8, 2, 16
    rng = np.random.default_rng(5)
    w, bias = rng.uniform(-1, 1, (L, d, d)) * np.sqrt(3.0 / d), rng.standard_normal((L, d)) * 0.5
    x, scale = rng.standard_normal((b, d)), np.float64(0.7)
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, schedule="cosine", warmup=3)
    h = Host(oracle.vtable(), "f32").prepare("tower", D=d, L=L).adamw(**hp)
    h.set_param("blocks.w", w)
    h.set_param("blocks.b", bias)
    theta = {"blocks.w": w.astype(np.float32).astype(np.float64), "blocks.b": bias.astype(np.float32).astype(np.float64)}
    m = {k: np.zeros_like(v) for k, v in theta.items()}
    v2 = {k: np.zeros_like(v) for k, v in theta.items()}
    losses = []
    total = 10
    for t in range(1, total + 1):
        losses.append(float(h.call("loss", [x, scale], ())))
        h.call("loss_grad", [x, scale], (L, d, d))
        g = {k: h.result(k, theta[k].shape).astype(np.float64) for k in theta}
        lr = hp["lr"] * min(1.0, t / 3) * 0.5 * (1 + np.cos(np.pi * min(1.0, max(0.0, (t - 3) / max(total - 3, 1)))))
        assert abs(h.adamw_lr(t, total) - lr) <= 1e-2 * 2.0**-21
        h.adamw_step(t, total)
        for k in theta:
            m[k] = 0.9 * m[k] + 0.1 * g[k]
            v2[k] = 0.95 * v2[k] + 0.05 * g[k] ** 2
            theta[k] = theta[k] - lr * (m[k] / (1 - 0.9**t) / (np.sqrt(v2[k] / (1 - 0.95**t)) + 1e-8) + 0.1 * theta[k])
            np.testing.assert_allclose(h.result(k, theta[k].shape), theta[k], rtol=0, atol=2e-5, err_msg=f"{k} at step {t}")
    assert all(b < a for a, b in zip(losses, losses[1:])) and losses[-1] < 0.9 * losses[0], losses


def test_optimizer_errors(oracle):
    h = Host(oracle.vtable(), "f32").prepare("tower", D=3, L=1)
    with pytest.raises(PreskError, match="E7001"):
        h.adamw(momentum=0.9)
    h.adamw()
    h.set_param("blocks.w", np.ones((1, 3, 3)))
    h.set_param("blocks.b", np.ones((1, 3)))
    with pytest.raises(PreskError, match="no leaf"):
        h.adamw_step(1, 10)


@pytest.mark.parametrize("clip", [0.05, 100.0])
def test_gradient_clipping_to_the_global_norm(oracle, clip):
    """`grad_clip = c`: g · min(1, c / (‖g‖₂ + 1e-6)) over all leaves before the moments (optim.rs:166-178); a bound
    below the norm scales the step, one far above leaves it alone."""
    rng = np.random.default_rng(8)
    g = {"blocks.w": rng.standard_normal((2, 4, 4)), "blocks.b": rng.standard_normal((2, 4))}
    norm = np.sqrt(sum((v.astype(np.float32).astype(np.float64) ** 2).sum() for v in g.values()))
    factor = min(1.0, clip / (norm + 1e-6))
    outs = []
    for hp, scale in ((dict(grad_clip=clip), 1.0), (dict(), factor)):
        h = Host(oracle.vtable(), "f32").prepare("tower", D=4, L=2).adamw(lr=1e-2, **hp)
        h.set_param("blocks.w", np.ones((2, 4, 4)))
        h.set_param("blocks.b", np.ones((2, 4)))
        for k, v in g.items():
            h.set_result(k, v.astype(np.float32).astype(np.float64) * scale)
        h.set_logging(True)
        h.adamw_step(1, 10)
        if hp:
            assert h.launch_log()[:5] == ["sum_squares", "sum_squares", "fused 6 steps", "mul", "mul"]
        outs.append({k: h.result("m:" + k, v.shape) for k, v in g.items()})
    for k in g:
        np.testing.assert_allclose(outs[0][k], outs[1][k], rtol=2e-5, atol=1e-9)  # min(1, x) = 1 - relu(1 - x) keeps x to 2^-24 absolute
    assert (factor < 1.0) == (clip < norm)
