"""The multi-rank path on the CPU: two gloo ranks, each running the host program over the CPU
oracle on its shard of the batch, then the loss exchange of presk_b200/shard.py. The sharded
loss must be the whole batch's."""
import os
import subprocess
import sys
import textwrap

import numpy as np

import models
from presk_b200 import Host, shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rows_partition():
    for n, world in [(8, 1), (8, 2), (8, 4), (10, 4), (3, 8), (0, 2)]:
        spans = [shard.shard_rows(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1


WORKER = textwrap.dedent("""
    import os, sys, json
    import numpy as np
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
    import torch.distributed as dist
    import models, oracle_lib
    from presk_b200 import Host, shard
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
    rank, world = dist.get_rank(), dist.get_world_size()
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    rng = np.random.default_rng(9)
    ids = rng.integers(0, c["V"], size=(6, 16), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(6, 16), dtype=np.int64)
    lo, hi = shard.shard_rows(6, rank, world)
    h = models.give(Host(oracle_lib.load().vtable(), "f32").prepare("llama", **c), p)
    h.set_calibrating(True)
    local = float(h.call("loss", [ids[lo:hi], y[lo:hi]], ()))
    env = shard.combine_envelopes(h.envelope())
    total = shard.combine_mean(local, (hi - lo) * 16)
    slowest = shard.max_over_ranks(rank + 1.0)
    dist.barrier()
    if rank == 0:
        print(json.dumps({{"loss": total, "slowest": slowest, "envelope": env}}))
    dist.destroy_process_group()
""")


def test_two_ranks_give_the_whole_batch_loss(oracle, tmp_path):
    port = 29500 + os.getpid() % 2000
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    import json
    got = json.loads(outs[0][0].strip().splitlines()[-1])
    c = models.LLAMA_TINY
    p = models.llama_params(c)
    rng = np.random.default_rng(9)
    ids = rng.integers(0, c["V"], size=(6, 16), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(6, 16), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), p)
    h.set_calibrating(True)
    whole = float(h.call("loss", [ids, y], ()))
    assert abs(got["loss"] - whole) <= 2e-6 * abs(whole)
    # calibrate's max-magnitude reduction: the merged envelope of the two shards is the whole batch's,
    # at every site whose values do not depend on how the batch is cut (all but the final mean)
    whole_env = h.envelope()
    for site, v in whole_env.items():
        if site == "loss/%6":
            continue
        assert tuple(got["envelope"][site]) == v, site
    assert got["slowest"] == 2.0


TRAIN_WORKER = textwrap.dedent("""
    import os, sys, json
    import numpy as np
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
    import torch.distributed as dist
    import models, oracle_lib
    from presk_b200 import Host, shard
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
    rank, world = dist.get_rank(), dist.get_world_size()
    c = models.LLAMA_TINY
    p = models.llama_params(c, seed=4, std=0.1)
    rng = np.random.default_rng(11)
    ids = rng.integers(0, c["V"], size=(4, 12), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(4, 12), dtype=np.int64)
    lo, hi = shard.shard_rows(4, rank, world)
    h = models.give(Host(oracle_lib.load().vtable(), "f32").prepare("llama", **c), p).adamw(lr=1e-2, weight_decay=0.1, grad_clip=1.0)
    for t in (1, 2):
        h.call("loss_grad", [ids[lo:hi], y[lo:hi]], p["tok"].shape)
        mine = {{k: h.result(k, np.shape(v), np.float64) for k, v in p.items()}}
        for k, g in shard.combine_gradients(mine, (hi - lo) * 12).items():
            h.set_result(k, g)
        h.adamw_step(t, 2)
    after = {{k: h.result(k, np.shape(v), np.float64).tolist() for k, v in p.items()}}
    with open(sys.argv[2], "w") as f:  # not through a pipe: the parent reads the ranks one after the other
        json.dump(after, f)
    dist.barrier()
    dist.destroy_process_group()
""")


def test_two_ranks_take_the_whole_batch_s_training_steps(oracle, tmp_path):
    """Two data-parallel ranks, each with half the rows: gradients combined by `shard.combine_gradients`, the same
    AdamW step on both. After two steps both ranks hold the same parameters, and they are the parameters one
    process reaches on the whole batch (to the accuracy of f32 gradients summed in another order)."""
    port = 31500 + os.getpid() % 2000
    script = tmp_path / "train_worker.py"
    script.write_text(TRAIN_WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(tmp_path / f"rank{r}.json")], stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    import json
    ranks = [json.load(open(tmp_path / f"rank{r}.json")) for r in range(2)]
    c = models.LLAMA_TINY
    p = models.llama_params(c, seed=4, std=0.1)
    rng = np.random.default_rng(11)
    ids = rng.integers(0, c["V"], size=(4, 12), dtype=np.int64)
    y = rng.integers(0, c["V"], size=(4, 12), dtype=np.int64)
    h = models.give(Host(oracle.vtable(), "f32").prepare("llama", **c), p).adamw(lr=1e-2, weight_decay=0.1, grad_clip=1.0)
    for t in (1, 2):
        h.call("loss_grad", [ids, y], p["tok"].shape)
        h.adamw_step(t, 2)
    for k, v in p.items():
        a, b = np.array(ranks[0][k]), np.array(ranks[1][k])
        assert np.array_equal(a, b), k
        whole = h.result(k, np.shape(v), np.float64)
        assert np.abs(a - whole).max() <= 2e-3 * max(np.abs(whole).max(), 1e-3), (k, np.abs(a - whole).max())
        assert np.abs(whole - np.asarray(v, np.float64)).max() > 0, k
