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
