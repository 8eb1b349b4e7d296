"""One rank of tests/test_gpu_comm.py: `python comm_rank.py RANK NRANKS ID_FILE OUT_FILE`.
Rank 0 writes the communicator's id to ID_FILE; every rank all-reduces a few buffers through psk_comm_*
and runs a small sharded loss and calibration through the host program, then writes what it saw as JSON."""
import json
import os
import sys
import threading
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import models  # noqa: E402
from presk_b200 import Comm, Executor, Host, abi  # noqa: E402

rank, nranks, id_file, out_file = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]

# The rank's own deadline: if the exchange has not finished by then (a peer died before its all-reduce), the
# process ends itself, and with it whatever of its work still waits on the GPU for that peer.
DEADLINE_S = 240


def _give_up():
    sys.stderr.write(f"comm_rank {rank}: not finished after {DEADLINE_S} s; exiting\n")
    sys.stderr.flush()
    os._exit(3)


_watchdog = threading.Timer(DEADLINE_S, _give_up)
_watchdog.daemon = True
_watchdog.start()
ex = Executor(rank)
if rank == 0:
    uid = Comm.unique_id()
    with open(id_file + ".tmp", "wb") as f:
        f.write(uid)
    os.replace(id_file + ".tmp", id_file)
else:
    deadline = time.time() + 120
    while not os.path.exists(id_file):
        if time.time() > deadline:
            raise SystemExit("no communicator id appeared")
        time.sleep(0.05)
    uid = open(id_file, "rb").read()
comm = Comm(ex, nranks, rank, uid)
out = {}
x = np.arange(8, dtype=np.float32) + 10 * rank
p = ex.upload(x)
comm.allreduce(p, 8, abi.F32, abi.COMM_SUM)
ex.sync()
out["sum"] = ex.download(p, 32).view(np.float32).tolist()
w = np.array([rank + 1, 100 - rank, 0xFFFFFFF0 + rank, 7], dtype=np.uint32)
q = ex.upload(w)
comm.allreduce(q, 4, abi.COMM_U32, abi.COMM_MAX)
ex.sync()
out["max"] = ex.download(q, 16).view(np.uint32).tolist()
# a sharded loss: each rank its rows of one batch; the mean over ranks of the per-rank means
c = models.LLAMA_TINY
params = models.llama_params(c)
rng = np.random.default_rng(5)
ids = rng.integers(0, c["V"], size=(2 * nranks, 16), dtype=np.int64)
y = rng.integers(0, c["V"], size=(2 * nranks, 16), dtype=np.int64)
mine = slice(2 * rank, 2 * rank + 2)
h = models.give(Host(ex, "f32").prepare("llama", **c), params)
h.set_calibrating(True)
ids_d, y_d = ex.upload(np.ascontiguousarray(ids[mine])), ex.upload(np.ascontiguousarray(y[mine]))
ptr, dt, n = h.call_device("loss", [(ids_d, abi.I64, (2, 16)), (y_d, abi.I64, (2, 16))])
out["loss"] = h.mean_over_ranks(comm, ptr, dt)
h.envelope_allreduce(comm)
env = h.envelope()
out["envelope"] = {k: list(v) for k, v in sorted(env.items())[:40]}
# a data-parallel training step: each rank's gradient on its rows, averaged over the ranks, the same AdamW step
ht = models.give(Host(ex, "f32").prepare("llama", **c), params).adamw(lr=1e-2, weight_decay=0.1)
ht.call("loss_grad", [ids[mine], y[mine]], params["tok"].shape)
ht.grads_allreduce(comm)
out["grad_head"] = ht.result("head", params["head"].shape).astype(np.float64).tolist()
ht.adamw_step(1, 2)
out["head_after"] = ht.result("head", params["head"].shape).astype(np.float64).tolist()
comm.close()
with open(out_file, "w") as f:
    json.dump(out, f)
_watchdog.cancel()
