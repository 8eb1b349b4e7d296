"""psk_comm_*: the exchange step of a sharded call over NCCL, one process a GPU. Needs two GPUs; on a box with one
the test is skipped (the same logic over gloo on the CPU is tests/test_shard_gloo.py)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import models
from presk_b200 import Host

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def gpus():
    import torch
    return torch.cuda.device_count()


def test_two_ranks_exchange_loss_and_envelope(tmp_path, oracle):
    if gpus() < 2:
        pytest.skip("one GPU: the exchange step needs two")
    n = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "support", "comm_rank.py"), str(r), str(n), str(tmp_path / "id"), str(tmp_path / f"out{r}.json")], env=env) for r in range(n)]
    # A rank that fails leaves its peer waiting in the communicator's set-up or in an all-reduce for an arrival
    # that will never come: whatever happens here, no rank outlives the test.
    try:
        codes = [p.wait(timeout=300) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
                p.wait()
    assert codes == [0] * n
    outs = [json.load(open(tmp_path / f"out{r}.json")) for r in range(n)]
    assert outs[0]["sum"] == outs[1]["sum"] == [2.0 * i + 10.0 for i in range(8)]
    assert outs[0]["max"] == outs[1]["max"] == [2, 100, 0xFFFFFFF1, 7]
    # the whole batch on the oracle: the same loss (a mean of equal shards' means) and the same envelope
    c = models.LLAMA_TINY
    params = models.llama_params(c)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, c["V"], size=(2 * n, 16), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(2 * n, 16), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), params)
    h.set_calibrating(True)
    want = float(h.call("loss", [ids, y], ()))
    assert outs[0]["loss"] == outs[1]["loss"]
    assert abs(outs[0]["loss"] - want) <= 2e-6 * abs(want)
    whole = h.envelope()
    assert outs[0]["envelope"] == outs[1]["envelope"]
    for site, got in outs[0]["envelope"].items():
        if site.startswith("loss/"):
            continue  # the loss's own sites are per-rank means; they are what mean_over_ranks combines
        np.testing.assert_allclose(got, whole[site], rtol=1e-6, err_msg=site)
    # the data-parallel training step: both ranks hold the whole batch's gradient and take its AdamW step
    ht = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), params).adamw(lr=1e-2, weight_decay=0.1)
    ht.call("loss_grad", [ids, y], params["tok"].shape)
    want_g = ht.result("head", params["head"].shape).astype(np.float64)
    assert outs[0]["grad_head"] == outs[1]["grad_head"]
    assert np.abs(np.array(outs[0]["grad_head"]) - want_g).max() <= 1e-5 * np.abs(want_g).max()
    ht.adamw_step(1, 2)
    want_p = ht.result("head", params["head"].shape).astype(np.float64)
    assert outs[0]["head_after"] == outs[1]["head_after"]
    assert np.abs(np.array(outs[0]["head_after"]) - want_p).max() <= 2e-3 * np.abs(want_p).max()
