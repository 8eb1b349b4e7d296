"""Budgets against the exact evaluator.

A realization is acceptable when every output stays within its error budget of the exact value: gap = the largest
absolute difference, budget_abs = budget x max |y| (crates/presk-driver/src/gap.rs:35-64). The exact value here is
tests/exact_mpfr.py (MPFR at 256 bits, the reference's exact interpreter's arithmetic) at the reference's own small
constants (presk-cranelift/tests/codes.rs:397: V=100 D=32 H=2 G=2 FF=64 L=2, B=2, T=16). No solved realization file
can be produced here (`presk solve` is Rust), so the budgets below are stated per realization, an order of
magnitude above what the storage types' roundings give at this depth, and the tests assert them for the CPU oracle
and, on a GPU, for the CUDA executor under both orders."""
import numpy as np
import pytest

import exact_mpfr
import models
from presk_b200 import Host

C_TINY = models.LLAMA_TINY
BUDGET = {"f32": 2e-6, "bf16": 3e-2, "f16": 4e-3, "e8m15": 1e-4}


@pytest.fixture(scope="module")
def exact_case():
    p = models.llama_params(C_TINY)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, C_TINY["V"], size=(2, 16), dtype=np.int64)
    y = rng.integers(0, C_TINY["V"], size=(2, 16), dtype=np.int64)
    return p, ids, y, exact_mpfr.llama(p, C_TINY, ids), exact_mpfr.llama(p, C_TINY, ids, y)


def gap(got, exact):
    d = np.abs(np.asarray(got, np.float64) - exact)
    return float(np.inf if not np.isfinite(d).all() else d.max())


def test_the_float64_statement_is_the_exact_model_to_twelve_digits(exact_case):
    """tests/models.py `llama_numpy` (float64) is what the larger shapes are held against, where MPFR would take
    hours: at the small constants it agrees with the exact evaluator to 1e-12 of the logits' scale."""
    p, ids, y, logits, loss = exact_case
    got = models.llama_numpy(p, C_TINY, ids)
    assert gap(got, logits) <= 1e-12 * np.abs(logits).max()
    assert abs(models.llama_numpy(p, C_TINY, ids, y) - loss) <= 1e-12 * abs(loss)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16", "e8m15"])
def test_oracle_within_the_budget_of_the_exact_evaluator(oracle, exact_case, dtype):
    p, ids, y, logits, loss = exact_case
    h = models.give(Host(oracle.vtable(), dtype).prepare("llama", **C_TINY), p)
    got = h.call("apply", [ids], logits.shape)
    assert gap(got, logits) <= BUDGET[dtype] * np.abs(logits).max(), (dtype, gap(got, logits), np.abs(logits).max())
    assert abs(float(h.call("loss", [ids, y], ())) - loss) <= BUDGET[dtype] * abs(loss)


@pytest.mark.gpu
@pytest.mark.parametrize("order", ["sequential", "device"])
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16", "e8m15"])
def test_gpu_within_the_budget_of_the_exact_evaluator(cuda, exact_case, dtype, order):
    """Every output of the CUDA executor inside the declared budget of the exact evaluator, under the reference's
    order and under the device order (tensor-core contractions, tree sums)."""
    p, ids, y, logits, loss = exact_case
    rz = {"default": dtype, "order": {"kind": order}}
    h = models.give(Host(cuda, rz).prepare("llama", **C_TINY), p)
    got = h.call("apply", [ids], logits.shape)
    assert gap(got, logits) <= BUDGET[dtype] * np.abs(logits).max(), (dtype, order, gap(got, logits), np.abs(logits).max())
    assert abs(float(h.call("loss", [ids, y], ())) - loss) <= BUDGET[dtype] * abs(loss)
